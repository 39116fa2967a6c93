#include "block_manager.h"

namespace dmoe {

BlockManager::BlockManager(int block_size, int num_blocks, int reserved_blocks, int max_rows)
    : block_size_(block_size), num_blocks_(num_blocks), reserved_blocks_(reserved_blocks) {
  DMOE_CHECK(block_size > 0 && num_blocks >= 0 && reserved_blocks >= 0, "bad block manager sizes");
  const int total = num_blocks + reserved_blocks;
  free_.reserve(total);
  for (int b = total - 1; b >= 0; --b) free_.push_back(b);  // block 0 is handed out first
  (void)max_rows;
}

int BlockManager::num_free_blocks() {
  std::lock_guard<std::mutex> lk(mu_);
  return static_cast<int>(free_.size());
}

int BlockManager::num_seqs() {
  std::lock_guard<std::mutex> lk(mu_);
  return static_cast<int>(seqs_.size());
}

bool BlockManager::can_allocate(int seq_len) {
  const int need = (seq_len + block_size_ - 1) / block_size_;
  return num_free_blocks() >= need + reserved_blocks_;
}

bool BlockManager::can_append() { return num_free_blocks() > 0; }

int BlockManager::take_block_locked() {
  DMOE_CHECK(!free_.empty(), "out of KV blocks");
  const int b = free_.back();
  free_.pop_back();
  return b;
}

void BlockManager::allocate(int seq_id, int seq_len) {
  std::lock_guard<std::mutex> lk(mu_);
  DMOE_CHECK(seqs_.find(seq_id) == seqs_.end(), "sequence " << seq_id << " already has blocks");
  const int need = std::max(1, (seq_len + block_size_ - 1) / block_size_);
  DMOE_CHECK(static_cast<int>(free_.size()) >= need + reserved_blocks_,
             "cannot allocate " << need << " blocks (" << free_.size() << " free, " << reserved_blocks_ << " reserved)");
  Seq s;
  if (!free_rows_.empty()) {
    s.row = free_rows_.back();
    free_rows_.pop_back();
  } else {
    s.row = next_row_++;
  }
  s.blocks.reserve(need);
  for (int i = 0; i < need; ++i) {
    s.blocks.push_back(take_block_locked());
    note_locked(s.row, i, s.blocks.back());
  }
  seqs_.emplace(seq_id, std::move(s));
}

void BlockManager::append_block(int seq_id) {
  std::lock_guard<std::mutex> lk(mu_);
  auto it = seqs_.find(seq_id);
  DMOE_CHECK(it != seqs_.end(), "unknown sequence " << seq_id);
  it->second.blocks.push_back(take_block_locked());
  note_locked(it->second.row, static_cast<int>(it->second.blocks.size()) - 1, it->second.blocks.back());
}

void BlockManager::append_tokens(int seq_id, int context_len, int num_tokens) {
  DMOE_CHECK(num_tokens >= 1 && context_len >= 0, "append_tokens arguments");
  std::lock_guard<std::mutex> lk(mu_);
  auto it = seqs_.find(seq_id);
  DMOE_CHECK(it != seqs_.end(), "unknown sequence " << seq_id);
  const int need = (context_len + num_tokens + block_size_ - 1) / block_size_;
  while (static_cast<int>(it->second.blocks.size()) < need) {
    it->second.blocks.push_back(take_block_locked());
    note_locked(it->second.row, static_cast<int>(it->second.blocks.size()) - 1, it->second.blocks.back());
  }
}

void BlockManager::release(int seq_id) {
  std::lock_guard<std::mutex> lk(mu_);
  auto it = seqs_.find(seq_id);
  DMOE_CHECK(it != seqs_.end(), "release of unknown sequence " << seq_id);
  for (auto b = it->second.blocks.rbegin(); b != it->second.blocks.rend(); ++b) free_.push_back(*b);
  free_rows_.push_back(it->second.row);
  seqs_.erase(it);
}

void BlockManager::batch_release(const std::vector<int>& seq_ids) {
  for (int s : seq_ids) release(s);
}

bool BlockManager::has_seq_block_list(int seq_id) {
  std::lock_guard<std::mutex> lk(mu_);
  return seqs_.count(seq_id) > 0;
}

std::vector<int> BlockManager::get_seq_block_list(int seq_id) {
  std::lock_guard<std::mutex> lk(mu_);
  auto it = seqs_.find(seq_id);
  DMOE_CHECK(it != seqs_.end(), "unknown sequence " << seq_id);
  return it->second.blocks;
}

int BlockManager::row_of(int seq_id) {
  std::lock_guard<std::mutex> lk(mu_);
  auto it = seqs_.find(seq_id);
  DMOE_CHECK(it != seqs_.end(), "unknown sequence " << seq_id);
  return it->second.row;
}

int64_t BlockManager::slot_of(int seq_id, int pos) {
  std::lock_guard<std::mutex> lk(mu_);
  auto it = seqs_.find(seq_id);
  DMOE_CHECK(it != seqs_.end(), "unknown sequence " << seq_id);
  const int b = pos / block_size_;
  DMOE_CHECK(b < static_cast<int>(it->second.blocks.size()), "position " << pos << " has no block");
  return static_cast<int64_t>(it->second.blocks[b]) * block_size_ + pos % block_size_;
}

void BlockManager::update_block_table(const AttentionBatchMetadata& meta, const std::vector<int>& context_lens) {
  const size_t n = meta.seq_ids.size();
  DMOE_CHECK(context_lens.size() == n, "context_lens size");
  for (size_t i = 0; i < n; ++i) {
    const int seq = meta.seq_ids[i];
    if (!has_seq_block_list(seq)) {
      const int plen = meta.init_prefill_lens[i];
      DMOE_CHECK(plen >= 0, "decode token of unknown sequence " << seq);
      allocate(seq, std::max(plen, context_lens[i] + 1));
    }
    append_tokens(seq, context_lens[i], 1);
  }
}

std::vector<int> BlockManager::prepare_block_table(const AttentionBatchMetadata& meta, const std::vector<int>& seq_lens,
                                                   int* out_max_blocks) {
  const int n = static_cast<int>(meta.seq_ids.size());
  DMOE_CHECK(static_cast<int>(seq_lens.size()) == n, "seq_lens size");
  std::lock_guard<std::mutex> lk(mu_);
  size_t m = 0;
  for (int i = 0; i < n; ++i) {
    auto it = seqs_.find(meta.seq_ids[i]);
    DMOE_CHECK(it != seqs_.end(), "sequence " << meta.seq_ids[i] << " has no blocks");
    m = std::max(m, it->second.blocks.size());
  }
  std::vector<int> flat(static_cast<size_t>(n) * m + n, -1);
  for (int i = 0; i < n; ++i) {
    const auto& blocks = seqs_[meta.seq_ids[i]].blocks;
    std::copy(blocks.begin(), blocks.end(), flat.begin() + static_cast<size_t>(i) * m);
    const int last = seq_lens[i] - 1;
    DMOE_CHECK(last >= 0 && last / block_size_ < static_cast<int>(blocks.size()), "sequence length out of range");
    flat[static_cast<size_t>(n) * m + i] = blocks[last / block_size_] * block_size_ + last % block_size_;
  }
  if (out_max_blocks != nullptr) *out_max_blocks = static_cast<int>(m);
  return flat;
}

std::vector<int64_t> BlockManager::step_decode(const std::vector<int>& seq_ids, const std::vector<int>& lengths) {
  const size_t n = seq_ids.size();
  DMOE_CHECK(lengths.size() == n, "lengths size");
  std::vector<int64_t> out(2 * n);
  std::lock_guard<std::mutex> lk(mu_);
  for (size_t i = 0; i < n; ++i) {
    auto it = seqs_.find(seq_ids[i]);
    DMOE_CHECK(it != seqs_.end(), "unknown sequence " << seq_ids[i]);
    auto& s = it->second;
    const int pos = lengths[i];
    const int need = pos / block_size_ + 1;
    while (static_cast<int>(s.blocks.size()) < need) {
      s.blocks.push_back(take_block_locked());
      note_locked(s.row, static_cast<int>(s.blocks.size()) - 1, s.blocks.back());
    }
    out[i] = s.row;
    out[n + i] = static_cast<int64_t>(s.blocks[pos / block_size_]) * block_size_ + pos % block_size_;
  }
  return out;
}

std::vector<BlockTableUpdate> BlockManager::drain_updates() {
  std::lock_guard<std::mutex> lk(mu_);
  std::vector<BlockTableUpdate> out;
  out.swap(updates_);
  return out;
}

std::vector<int> prepare_batch_infos(const AttentionBatchMetadata& meta, const std::vector<int>& seq_lens) {
  const size_t n = meta.seq_ids.size();
  DMOE_CHECK(seq_lens.size() == n, "seq_lens size");
  std::vector<int> out(3 * n + 1, 0);
  for (size_t i = 0; i < n; ++i) {
    out[i] = seq_lens[i];
    out[n + i] = seq_lens[i] - 1;
    out[2 * n + i + 1] = out[2 * n + i] + seq_lens[i];
  }
  return out;
}

}  // namespace dmoe
