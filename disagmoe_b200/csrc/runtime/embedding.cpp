#include "embedding.h"

namespace dmoe {

Tokenizer::Tokenizer(int device_id, std::vector<Endpoint> endpoints, std::map<int, int> attn_peer)
    : MuDispatcher({}, device_id, ParallelConfig{}, std::move(endpoints)), attn_peer_(std::move(attn_peer)) {}

void Tokenizer::put_request(int req_id, const std::vector<int>& prompt_ids, int dp_rank) {
  DMOE_CHECK(!prompt_ids.empty(), "empty prompt");
  auto m = std::make_shared<Metadata>();
  const int n = static_cast<int>(prompt_ids.size());
  m->shape = {n, 0};
  m->layer_id = 0;
  m->tok.req_ids.assign(n, req_id);
  m->tok.attn_dp_ranks.assign(n, dp_rank);
  m->tok.init_prefill_lens.assign(n, n);
  m->tok.positions.resize(n);
  std::iota(m->tok.positions.begin(), m->tok.positions.end(), 0);
  m->tok.token_ids = prompt_ids;
  put(TensorBatch{torch::Tensor(), m}, 0);
}

void Tokenizer::send_once(const TensorBatch& batch, int) {
  const int dp = batch.metadata->tok.attn_dp_ranks.empty() ? 0 : batch.metadata->tok.attn_dp_ranks[0];
  auto it = attn_peer_.find(dp);
  DMOE_CHECK(it != attn_peer_.end(), "no layer-0 attention worker for dp rank " << dp);
  Endpoint* ep = endpoint_of(it->second);
  DMOE_CHECK(ep != nullptr, "tokenizer has no edge to device " << it->second);
  send_batch(*ep, torch::Tensor(), *batch.metadata, MSG_TOKEN_IDS);
}

Sampler::Sampler(int device_id, std::vector<Endpoint> endpoints, std::map<int, int> attn_peer, int min_output_len,
                 int max_output_len, bool ignore_eos, unsigned seed)
    : MuDispatcher({}, device_id, ParallelConfig{}, std::move(endpoints)), attn_peer_(std::move(attn_peer)),
      min_len_(min_output_len), max_len_(std::max(max_output_len, min_output_len + 1)), ignore_eos_(ignore_eos),
      rng_(seed) {
  mailbox_.bind(get_zmq_addr(device_id_, false, 0));
}

void Sampler::start_all() {
  start();
  if (!recv_thread_.joinable()) recv_thread_ = std::thread([this] { recv_loop(); });
}

void Sampler::stop_all() {
  terminate();
  if (recv_thread_.joinable()) recv_thread_.join();
}

void Sampler::recv_loop() {
  Recorder::instance().create("sampler.recv");
  while (!end_flag_.load()) {
    Frames f;
    if (!mailbox_.recv(f, 50)) continue;
    if (f.size() < 2) continue;
    MsgHeader h;
    from_bytes(f[0], h);
    if (h.kind == MSG_STOP) continue;
    if (seq_filter_.seen(h.sender, h.seq)) continue;   // a duplicated message must not count a token twice
    Metadata meta;
    from_bytes(f[1], meta);
    try {
      process_batch(meta);
    } catch (const std::exception& e) {
      DMOE_LOG(ERROR) << "sampler: " << e.what();
    }
  }
}

void Sampler::set_request_output_len(int req_id, int n) {
  std::lock_guard<std::mutex> lk(result_mu_);
  required_lens_[req_id] = n;
}

bool Sampler::check_finished(int token, int req_id) {
  if (!ignore_eos_ && token == kEosTokenId) return true;
  return output_lens_[req_id] >= required_lens_[req_id];
}

int Sampler::process_batch(const Metadata& meta) {
  const int n = static_cast<int>(meta.tok.size());
  auto next = std::make_shared<Metadata>();
  next->shape = {0, 0};
  next->layer_id = 0;
  int counted = 0;
  {
    std::lock_guard<std::mutex> lk(result_mu_);
    const int64_t now = wall_us();
    for (int i = 0; i < n; ++i) {
      const int rid = meta.tok.req_ids[i];
      const int pos = meta.tok.positions.empty() ? 0 : meta.tok.positions[i];
      if (!token_arrived(rid, pos)) continue;
      const int token = meta.tok.token_ids.empty() ? 0 : meta.tok.token_ids[i];
      ++counted;
      if (slo_stats_.find(rid) == slo_stats_.end()) {
        SloStat s;
        s.req_id = rid;
        s.t_prefill = now;       // the first generated token has arrived
        s.t_prefill_std = now;
        slo_stats_[rid] = s;
        if (!required_lens_.count(rid))
          required_lens_[rid] = min_len_ + static_cast<int>(rng_() % static_cast<unsigned>(max_len_ - min_len_));
      }
      ++output_lens_[rid];
      outputs_[rid].push_back(token);
      slo_stats_[rid].t_tokens.push_back(now);
      if (check_finished(token, rid)) {
        slo_stats_[rid].t_decode = now;
        finished_.insert(rid);
        finished_stats_[rid] = slo_stats_[rid];
        slo_stats_.erase(rid);
        output_lens_.erase(rid);
        required_lens_.erase(rid);
        continue;
      }
      next->tok.req_ids.push_back(rid);
      next->tok.attn_dp_ranks.push_back(meta.tok.attn_dp_ranks.empty() ? 0 : meta.tok.attn_dp_ranks[i]);
      next->tok.init_prefill_lens.push_back(-1);
      next->tok.positions.push_back(pos + 1);
      next->tok.token_ids.push_back(token);
    }
    step_infos_.push_back(SamplerStepInfo{counted, now});
  }
  next->shape[0] = static_cast<int64_t>(next->tok.size());
  if (next->tok.size() > 0) put(TensorBatch{torch::Tensor(), next}, 0);
  return counted;
}

void Sampler::send_once(const TensorBatch& batch, int) {
  // continuing tokens go back to layer 0 of the replica that owns the sequence
  const Metadata& meta = *batch.metadata;
  std::map<int, std::vector<int>> by_dp;
  for (size_t i = 0; i < meta.tok.size(); ++i) by_dp[meta.tok.attn_dp_ranks[i]].push_back(static_cast<int>(i));
  for (auto& [dp, rows] : by_dp) {
    auto it = attn_peer_.find(dp);
    DMOE_CHECK(it != attn_peer_.end(), "no layer-0 attention worker for dp rank " << dp);
    Endpoint* ep = endpoint_of(it->second);
    DMOE_CHECK(ep != nullptr, "sampler has no edge to device " << it->second);
    send_batch(*ep, torch::Tensor(), meta.at(rows), MSG_TOKEN_IDS);
  }
}

std::vector<SloStat> Sampler::fetch_finished_slo_stats() {
  std::lock_guard<std::mutex> lk(result_mu_);
  std::vector<SloStat> out;
  for (int r : finished_) out.push_back(finished_stats_[r]);
  finished_.clear();
  return out;
}

std::vector<SamplerStepInfo> Sampler::fetch_step_infos() {
  std::lock_guard<std::mutex> lk(result_mu_);
  std::vector<SamplerStepInfo> out;
  out.swap(step_infos_);
  return out;
}

std::map<int, SloStat> Sampler::wait_slo_stats(int n_request) {
  std::lock_guard<std::mutex> lk(result_mu_);
  if (static_cast<int>(finished_stats_.size()) < n_request) return {};
  return finished_stats_;
}

std::vector<int> Sampler::get_output_tokens(int req_id) {
  std::lock_guard<std::mutex> lk(result_mu_);
  auto it = outputs_.find(req_id);
  return it == outputs_.end() ? std::vector<int>{} : it->second;
}

int Sampler::num_finished() {
  std::lock_guard<std::mutex> lk(result_mu_);
  return static_cast<int>(finished_stats_.size());
}

void Sampler::reset() {
  std::lock_guard<std::mutex> lk(result_mu_);
  output_lens_.clear();
  required_lens_.clear();
  outputs_.clear();
  slo_stats_.clear();
  finished_.clear();
  finished_stats_.clear();
  step_infos_.clear();
}

}  // namespace dmoe
