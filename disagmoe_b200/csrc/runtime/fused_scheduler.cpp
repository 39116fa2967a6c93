#include "fused_scheduler.h"

#include <algorithm>
#include <numeric>

namespace dmoe {

void FusedPlan::copy_to(int32_t* ids_out, int32_t* pos_out, int32_t* ctx_out, int32_t* row_out, int64_t* slot_out) const {
  const size_t n = ids.size();
  for (size_t i = 0; i < n; ++i) {
    ids_out[i] = ids[i];
    pos_out[i] = pos[i];
    ctx_out[i] = pos[i] + 1;
    row_out[i] = rows[i];
    slot_out[i] = slots[i];
  }
}

FusedScheduler::FusedScheduler(std::shared_ptr<BlockManager> bm, int block_size, int n_mb, int max_seqs_per_mb,
                               int max_tokens_per_mb, int max_prefill_tokens_per_mb, bool ignore_eos)
    : bm_(std::move(bm)), block_size_(block_size), n_mb_(n_mb), max_seqs_(max_seqs_per_mb), max_tokens_(max_tokens_per_mb),
      max_prefill_(max_prefill_tokens_per_mb > 0 ? max_prefill_tokens_per_mb : max_tokens_per_mb), ignore_eos_(ignore_eos),
      running_(n_mb) {
  DMOE_CHECK(n_mb >= 1 && block_size >= 1, "bad scheduler shape");
  DMOE_CHECK(max_tokens_ > max_seqs_, "a micro-batch must have room for prompt rows next to its decode rows");
  pool_blocks_ = bm_->num_free_blocks();   // the scheduler is created on an empty pool
}

void FusedScheduler::add_request(int req_id, std::vector<int> prompt, int max_new_tokens, double t_arrival) {
  DMOE_CHECK(!prompt.empty() && max_new_tokens >= 1, "a request needs a prompt and at least one new token");
  if (blocks_for(static_cast<int>(prompt.size()) + max_new_tokens) > pool_blocks_)
    throw std::invalid_argument("request " + std::to_string(req_id) + " needs more KV blocks than the pool has");
  auto s = std::make_shared<FusedSeq>();
  s->req_id = req_id;
  s->prompt = std::move(prompt);
  s->max_new_tokens = max_new_tokens;
  s->t_arrival = t_arrival;
  waiting_.push_back(std::move(s));
}

int FusedScheduler::num_unfinished() const {
  size_t n = waiting_.size();
  for (auto& r : running_) n += r.size();
  return static_cast<int>(n);
}

bool FusedScheduler::has_work(double now) const {
  for (auto& r : running_)
    if (!r.empty()) return true;
  return !waiting_.empty() && waiting_.front()->t_arrival <= now;
}

// KV blocks the running sequences will still take before they finish. Admission leaves them free, so that a decode
// step can never find the pool empty.
int FusedScheduler::growth_reserve() {
  int total = 0;
  for (auto& r : running_)
    for (auto& s : r) {
      const int need = blocks_for(static_cast<int>(s->prompt.size()) + s->max_new_tokens);
      const int have = static_cast<int>(bm_->get_seq_block_list(s->req_id).size());
      total += std::max(0, need - have);
    }
  return total;
}

// Appends the next prompt rows of `s` (at most `budget`) to the plan; returns how many.
int FusedScheduler::add_prompt_rows(FusedPlan& p, const fused_seq_t& s, int budget) {
  const int n = static_cast<int>(s->prompt.size()), done = s->length;
  const int take = std::min(n - done, budget);
  if (take <= 0 || (take < MIN_CHUNK && take < n - done)) return 0;
  const int row = bm_->row_of(s->req_id);
  const auto blocks = bm_->get_seq_block_list(s->req_id);
  for (int i = done; i < done + take; ++i) {
    p.ids.push_back(s->prompt[i]);
    p.pos.push_back(i);
    p.rows.push_back(row);
    p.slots.push_back(static_cast<int64_t>(blocks[i / block_size_]) * block_size_ + i % block_size_);
  }
  const bool last = done + take == n;
  p.emit.emplace_back(last ? p.size() - 1 : -1, s, take);
  return take;
}

std::vector<FusedPlan> FusedScheduler::build(double now) {
  std::vector<FusedPlan> plans(n_mb_);
  std::vector<int> prefill(n_mb_, 0);
  auto budget = [&](int m) { return std::min(max_tokens_ - plans[m].size(), max_prefill_ - prefill[m]); };
  for (int m = 0; m < n_mb_; ++m) {
    std::vector<fused_seq_t> seqs;    // fully prefilled: one decode token each
    for (auto& s : running_[m])
      if (s->length >= static_cast<int>(s->prompt.size())) seqs.push_back(s);
    if (!seqs.empty()) {
      std::vector<int> ids, lens;
      for (auto& s : seqs) { ids.push_back(s->req_id); lens.push_back(s->length); }
      const auto rs = bm_->step_decode(ids, lens);
      const size_t n = seqs.size();
      auto& p = plans[m];
      for (size_t i = 0; i < n; ++i) {
        p.ids.push_back(seqs[i]->last_token);
        p.pos.push_back(lens[i]);
        p.rows.push_back(static_cast<int>(rs[i]));
        p.slots.push_back(rs[n + i]);
        p.emit.emplace_back(static_cast<int>(i), seqs[i], 1);
      }
    }
    // prompts that are part-way through, oldest first
    for (auto& s : running_[m])
      if (s->length < static_cast<int>(s->prompt.size())) prefill[m] += add_prompt_rows(plans[m], s, budget(m));
  }
  // admission in arrival order; a request goes to the micro-batch with more room this iteration
  while (!waiting_.empty() && waiting_.front()->t_arrival <= now) {
    auto s = waiting_.front();
    const int n = static_cast<int>(s->prompt.size());
    std::vector<int> order(n_mb_);
    std::iota(order.begin(), order.end(), 0);
    std::stable_sort(order.begin(), order.end(), [&](int a, int b) {
      return std::make_tuple(-budget(a), plans[a].size(), running_[a].size()) <
             std::make_tuple(-budget(b), plans[b].size(), running_[b].size());
    });
    int pick = -1;
    for (int m : order)
      if (static_cast<int>(running_[m].size()) < max_seqs_ && budget(m) >= std::min(n, MIN_CHUNK)) { pick = m; break; }
    if (pick < 0 || bm_->num_free_blocks() - growth_reserve() < blocks_for(n + s->max_new_tokens)) break;
    waiting_.erase(waiting_.begin());
    bm_->allocate(s->req_id, n + 1);
    s->mb = pick;
    running_[pick].push_back(s);
    prefill[pick] += add_prompt_rows(plans[pick], s, budget(pick));
  }
  return plans;
}

std::vector<std::pair<int, int>> FusedScheduler::commit(const std::vector<FusedPlan>& plans,
                                                        const std::vector<std::vector<int>>& next_ids, double now) {
  std::vector<std::pair<int, int>> out;
  for (size_t m = 0; m < plans.size(); ++m) {
    for (auto& e : plans[m].emit) {
      const int row = std::get<0>(e);
      const auto& s = std::get<1>(e);
      s->length += std::get<2>(e);
      if (row < 0) continue;
      DMOE_CHECK(m < next_ids.size() && row < static_cast<int>(next_ids[m].size()), "commit: missing sampled token");
      const int tok = next_ids[m][row];
      s->outputs.push_back(tok);
      s->t_tokens.push_back(now);
      s->last_token = tok;
      out.emplace_back(s->req_id, tok);
      if (static_cast<int>(s->outputs.size()) >= s->max_new_tokens || (!ignore_eos_ && tok == kEosTokenId)) {
        bm_->release(s->req_id);
        auto& r = running_[m];
        r.erase(std::remove(r.begin(), r.end(), s), r.end());
        finished_[s->req_id] = s;
      }
    }
  }
  return out;
}

void FusedScheduler::restore_running(int mb, fused_seq_t s) {
  DMOE_CHECK(mb >= 0 && mb < n_mb_, "restore_running: bad micro-batch");
  s->mb = mb;
  running_[mb].push_back(std::move(s));
}

void FusedScheduler::restore_finished(fused_seq_t s) { finished_[s->req_id] = std::move(s); }

}  // namespace dmoe
