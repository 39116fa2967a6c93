// Paged-KV block allocator of an attention worker.
//
// Blocks are handed out from a LIFO free list (recently released blocks are still warm in L2). Every sequence
// also owns one ROW of the device-resident block table; the manager records each (row, column, block) change so
// that the executor can patch the device table incrementally instead of re-uploading it every step.
//
// Reference behaviour covered: csrc/include/block_manager.h:13-65, csrc/engine/block_manager.cpp:11-193
// (can_allocate keeps `reserved_blocks` free for decode growth; allocate / append_block / append_tokens / release
// / batch_release / num_free_blocks; update_block_table; prepare_block_table; prepare_batch_infos).
#pragma once
#include "types.h"

namespace dmoe {

struct BlockTableUpdate {
  int row, col, block;
};

class BlockManager {
 public:
  BlockManager(int block_size, int num_blocks, int reserved_blocks, int max_rows = 0);

  int block_size() const { return block_size_; }
  int num_total_blocks() const { return num_blocks_ + reserved_blocks_; }
  int num_free_blocks();
  bool can_allocate(int seq_len);
  bool can_append();
  void allocate(int seq_id, int seq_len);
  void append_block(int seq_id);
  // Grows the sequence so that `num_tokens` more tokens fit after `context_len` cached ones.
  void append_tokens(int seq_id, int context_len, int num_tokens);
  void release(int seq_id);
  void batch_release(const std::vector<int>& seq_ids);
  bool has_seq_block_list(int seq_id);
  std::vector<int> get_seq_block_list(int seq_id);
  int row_of(int seq_id);
  int num_seqs();

  // Allocates for sequences seen for the first time (prefill rows) and grows every row's sequence so that
  // position `positions[i]` has a slot. Returns nothing; changes are queued as table updates.
  void update_block_table(const AttentionBatchMetadata& meta, const std::vector<int>& context_lens);
  // Flat KV slot of token position `pos` of a sequence.
  int64_t slot_of(int seq_id, int pos);
  // Flat int32 buffer: n*m block-table entries (row-major, -1 padded) followed by n slot ids of the last token.
  std::vector<int> prepare_block_table(const AttentionBatchMetadata& meta, const std::vector<int>& seq_lens,
                                       int* out_max_blocks = nullptr);
  // One decode step for many sequences at once: grows sequence i so that position lengths[i] has a slot and
  // returns its table row and flat slot as [rows..., slots...] (2 * n entries).
  std::vector<int64_t> step_decode(const std::vector<int>& seq_ids, const std::vector<int>& lengths);
  // Table patches since the previous call.
  std::vector<BlockTableUpdate> drain_updates();

 private:
  int take_block_locked();
  void note_locked(int row, int col, int block) { updates_.push_back({row, col, block}); }
  struct Seq {
    std::vector<int> blocks;
    int row;
  };
  int block_size_, num_blocks_, reserved_blocks_;
  std::mutex mu_;
  std::vector<int> free_;       // LIFO
  std::vector<int> free_rows_;  // LIFO
  int next_row_ = 0;
  std::unordered_map<int, Seq> seqs_;
  std::vector<BlockTableUpdate> updates_;
};

// seq_lens | context_lens (= seq_len - 1) | seq_start_loc (exclusive prefix sums, n + 1 entries), back to back.
std::vector<int> prepare_batch_infos(const AttentionBatchMetadata& meta, const std::vector<int>& seq_lens);

}  // namespace dmoe
