// Serving scheduler of one attention group on the fused (device-driven) data plane: request admission, micro-batch
// formation with mixed prompt / decode rows, chunked prefill under a per-iteration prompt budget, KV growth reserved
// at admission. Pure host logic next to the BlockManager it drives; the per-iteration plan is written straight
// into the pinned staging arrays that the engine uploads.
//
// It plays, for the fused path, the part that the pools + layer schedulers + sampler bookkeeping play for the
// host-scheduled path (reference: csrc/engine/scheduler.cpp:35-84, csrc/muhelper/embedding.cpp:96-169,
// disagmoe/scheduler/dpscheduler.py:50-129): which tokens run next, and when a request is finished.
//
// Rules (one iteration = one pass of every micro-batch through all layers):
//   * a running sequence whose prompt is fully cached contributes its next decode token;
//   * a prompt contributes rows up to two budgets per micro-batch: max_tokens rows in total and max_prefill prompt
//     rows; a prompt that does not fit is cut into chunks over several iterations (never fewer than MIN_CHUNK rows
//     unless that finishes it); only the last chunk samples a token;
//   * admission is in arrival order, into the micro-batch with more room, and only while the KV pool keeps enough
//     free blocks for every running sequence to reach its maximum length (no preemption exists).
#pragma once
#include <map>
#include <memory>
#include <tuple>

#include "block_manager.h"

namespace dmoe {

struct FusedSeq {
  int req_id = 0;
  std::vector<int> prompt;
  int max_new_tokens = 0;
  double t_arrival = 0.0;
  int mb = -1;
  int length = 0;          // tokens whose K / V are cached
  int last_token = 0;
  std::vector<int> outputs;
  std::vector<double> t_tokens;
};
using fused_seq_t = std::shared_ptr<FusedSeq>;

struct FusedPlan {
  std::vector<int> ids, pos, rows;
  std::vector<int64_t> slots;
  // (row in the micro-batch or -1, sequence, tokens this step adds to its cache): row >= 0 produces the sequence's
  // next token; row == -1 is a prompt chunk that is not the last one (the cache grows, nothing is sampled)
  std::vector<std::tuple<int, fused_seq_t, int>> emit;
  int size() const { return static_cast<int>(ids.size()); }
  // ids / positions / positions + 1 / block-table rows / slots into int32 (int64 for slots) arrays at `offset`
  void copy_to(int32_t* ids_out, int32_t* pos_out, int32_t* ctx_out, int32_t* row_out, int64_t* slot_out) const;
};

class FusedScheduler {
 public:
  static constexpr int MIN_CHUNK = 16;

  FusedScheduler(std::shared_ptr<BlockManager> bm, int block_size, int n_mb, int max_seqs_per_mb, int max_tokens_per_mb,
                 int max_prefill_tokens_per_mb, bool ignore_eos);

  void add_request(int req_id, std::vector<int> prompt, int max_new_tokens, double t_arrival);
  int num_unfinished() const;
  bool has_work(double now) const;
  std::vector<FusedPlan> build(double now);
  // next_ids[m][row]: token sampled for row `row` of micro-batch m. Returns the (request, token) pairs produced.
  std::vector<std::pair<int, int>> commit(const std::vector<FusedPlan>& plans, const std::vector<std::vector<int>>& next_ids,
                                          double now);

  // state, in the order the policy uses it (snapshots / inspection)
  const std::vector<fused_seq_t>& waiting() const { return waiting_; }
  const std::vector<std::vector<fused_seq_t>>& running() const { return running_; }
  const std::map<int, fused_seq_t>& finished() const { return finished_; }
  void restore_running(int mb, fused_seq_t s);      // resume from a snapshot: the sequence's KV blocks exist already
  void restore_finished(fused_seq_t s);
  int pool_blocks() const { return pool_blocks_; }
  int max_tokens() const { return max_tokens_; }
  int max_seqs() const { return max_seqs_; }
  int max_prefill() const { return max_prefill_; }

 private:
  int blocks_for(int tokens) const { return (tokens + block_size_ - 1) / block_size_; }
  int growth_reserve();
  int add_prompt_rows(FusedPlan& p, const fused_seq_t& s, int budget);

  std::shared_ptr<BlockManager> bm_;
  int block_size_, n_mb_, max_seqs_, max_tokens_, max_prefill_;
  bool ignore_eos_;
  int pool_blocks_;
  std::vector<fused_seq_t> waiting_;                 // arrival order
  std::vector<std::vector<fused_seq_t>> running_;    // per micro-batch, admission order
  std::map<int, fused_seq_t> finished_;
};

}  // namespace dmoe
