#include "muhelper.h"

#include <dlfcn.h>

#include <algorithm>

namespace dmoe {

// ------------------------------------------------------------------------------------------------ batches
namespace {
// dmoe_gather_ptrs of the package's kernel library (lib/libdmoe_kernels.so next to this module): dst[i] = the bf16 row
// at device address ptrs[i]. Resolved once; nullptr when the library is not there (CPU-only installs).
typedef int (*gather_ptrs_fn)(const void*, void*, long long, int, int, void*);
}  // namespace

// A symbol of the package's kernel library (lib/libdmoe_kernels.so next to this module), or nullptr.
void* kernel_library_symbol(const char* name) {
  static void* handle = [] {
    Dl_info info;
    if (dladdr(reinterpret_cast<void*>(&set_helper_error), &info) == 0 || info.dli_fname == nullptr)
      return static_cast<void*>(nullptr);
    std::string dir(info.dli_fname);
    const auto slash = dir.rfind('/');
    dir = slash == std::string::npos ? std::string(".") : dir.substr(0, slash);
    for (const char* rel : {"/lib/libdmoe_kernels.so", "/../../lib/libdmoe_kernels.so"})
      if (void* h = dlopen((dir + rel).c_str(), RTLD_NOW | RTLD_LOCAL)) return h;
    return static_cast<void*>(nullptr);
  }();
  return handle != nullptr ? dlsym(handle, name) : nullptr;
}

namespace {
gather_ptrs_fn kernel_gather() {
  static gather_ptrs_fn fn = reinterpret_cast<gather_ptrs_fn>(kernel_library_symbol("dmoe_gather_ptrs"));
  return fn;
}
}  // namespace

static torch::Tensor gather_rows(const std::vector<TensorBatch>& batches, const std::vector<int>& order_src_of_dst) {
  // order_src_of_dst[r] = index (in the concatenation of all batches) of the row that lands at r
  std::vector<torch::Tensor> parts;
  for (auto& b : batches)
    if (b.data.defined() && b.data.size(0) > 0) parts.push_back(b.data);
  if (parts.empty()) return torch::Tensor();
  const auto& first = parts[0];
  bool device_rows = first.is_cuda() && first.scalar_type() == torch::kBFloat16 && first.dim() == 2 &&
                     first.size(1) % 8 == 0 && kernel_gather() != nullptr;
  for (auto& p : parts)
    device_rows = device_rows && p.is_cuda() && p.scalar_type() == torch::kBFloat16 && p.dim() == 2 &&
                  p.size(1) == first.size(1) && p.stride(1) == 1 && p.get_device() == first.get_device();
  if (device_rows) {
    // Row gather by the package's own kernel from a table of row addresses: no concatenated copy of all batches and
    // no host synchronisation (the reference builds the same table but waits for the stream, csrc/cuda_ops/permute.cu:
    // 144-152). The table goes up through pinned memory on the engine thread's (default) stream, where the kernel runs.
    const int64_t n = static_cast<int64_t>(order_src_of_dst.size());
    const int64_t H = first.size(1);
    std::vector<int64_t> start(parts.size() + 1, 0);
    for (size_t i = 0; i < parts.size(); ++i) start[i + 1] = start[i] + parts[i].size(0);
    auto table = torch::empty({n}, torch::TensorOptions().dtype(torch::kInt64).pinned_memory(true));
    int64_t* tp = table.data_ptr<int64_t>();
    for (int64_t r = 0; r < n; ++r) {
      const int64_t src = order_src_of_dst[r];
      const size_t b = std::upper_bound(start.begin(), start.end(), src) - start.begin() - 1;
      tp[r] = reinterpret_cast<int64_t>(parts[b].data_ptr()) + (src - start[b]) * parts[b].stride(0) * 2;
    }
    auto table_dev = table.to(first.device(), /*non_blocking=*/true);
    auto out = torch::empty({n, H}, first.options());
    const int rc = kernel_gather()(table_dev.data_ptr(), out.data_ptr(), H, static_cast<int>(n), static_cast<int>(H), nullptr);
    DMOE_CHECK(rc == 0, "dmoe_gather_ptrs failed with code " + std::to_string(rc));
    return out;
  }
  auto all = parts.size() == 1 ? parts[0] : torch::cat(parts, 0);
  auto idx = torch::tensor(std::vector<int64_t>(order_src_of_dst.begin(), order_src_of_dst.end()),
                           torch::TensorOptions().dtype(torch::kInt64))
                 .to(all.device());
  return all.index_select(0, idx);
}

TensorBatch TensorBatch::merge(const std::vector<TensorBatch>& batches) {
  DMOE_CHECK(!batches.empty(), "merge of nothing");
  if (batches.size() == 1) {
    // a single batch arrives already expert-sorted from the attention dispatcher
    const auto& e = batches[0].metadata->tok.exp_ids;
    if (std::is_sorted(e.begin(), e.end())) return batches[0];
  }
  std::vector<metadata_t> metas;
  for (auto& b : batches) metas.push_back(b.metadata);
  std::vector<int> mapping;
  auto meta = Metadata::merge_by_exp_ids(metas, mapping);
  std::vector<int> src_of_dst(mapping.size());
  for (size_t i = 0; i < mapping.size(); ++i) src_of_dst[mapping[i]] = static_cast<int>(i);
  return TensorBatch{gather_rows(batches, src_of_dst), meta};
}

TensorBatch TensorBatch::concat(const std::vector<TensorBatch>& batches) {
  std::vector<metadata_t> metas;
  std::vector<torch::Tensor> parts;
  for (auto& b : batches) {
    metas.push_back(b.metadata);
    if (b.data.defined()) parts.push_back(b.data);
  }
  return TensorBatch{parts.empty() ? torch::Tensor() : torch::cat(parts, 0), Metadata::concat(metas)};
}

// ------------------------------------------------------------------------------------------------ MuHelper
namespace {
std::mutex g_err_mu;
std::string g_helper_error;
}  // namespace

void set_helper_error(const std::string& what) {
  std::lock_guard<std::mutex> lk(g_err_mu);
  if (g_helper_error.empty()) g_helper_error = what;
}

std::string helper_error() {
  std::lock_guard<std::mutex> lk(g_err_mu);
  return g_helper_error;
}

void MuHelper::start() {
  if (thread_.joinable()) return;
  end_flag_.store(false);
  thread_ = std::thread([this] {
    Recorder::instance().create(std::string(name()) + "@" + std::to_string(device_id_));
    try {
      run();
    } catch (const std::exception& e) {
      DMOE_LOG(ERROR) << name() << "@" << device_id_ << " stopped: " << e.what();
      set_helper_error(std::string(name()) + "@" + std::to_string(device_id_) + " stopped: " + e.what());
    }
  });
}

void MuHelper::terminate() {
  end_flag_.store(true);
  if (thread_.joinable()) thread_.join();
}

// ------------------------------------------------------------------------------------------------ dispatchers
MuDispatcher::MuDispatcher(std::vector<int> layer_ids, int device_id, ParallelConfig cfg, std::vector<Endpoint> endpoints)
    : MuHelper(std::move(layer_ids), device_id), cfg_(std::move(cfg)), endpoints_(std::move(endpoints)) {}

void MuDispatcher::put(const TensorBatch& batch, int kind) {
  {
    std::lock_guard<std::mutex> lk(mu_);
    queue_.emplace_back(batch, kind);
  }
  cv_.notify_one();
}

size_t MuDispatcher::pending() {
  std::lock_guard<std::mutex> lk(mu_);
  return queue_.size();
}

Endpoint* MuDispatcher::endpoint_of(int peer) {
  for (auto& e : endpoints_)
    if (e.peer == peer) return &e;
  return nullptr;
}

void MuDispatcher::connect_all() {
  if (connected_) return;
  for (auto& e : endpoints_) {
    if (!e.mq) e.mq = std::make_shared<PushSocket>();
    if (!e.mq->connected()) e.mq->connect(get_zmq_addr(e.peer, !is_embedding_node(e.peer), 0));
  }
  connected_ = true;
}

void MuDispatcher::run() {
  connect_all();
  while (!end_flag_.load()) {
    std::pair<TensorBatch, int> item;
    {
      std::unique_lock<std::mutex> lk(mu_);
      if (!cv_.wait_for(lk, std::chrono::milliseconds(50), [&] { return !queue_.empty(); })) continue;
      item = std::move(queue_.front());
      queue_.pop_front();
    }
    DMOE_RANGE("dispatch");
    send_once(item.first, item.second);
  }
}

void MuDispatcher::send_batch(Endpoint& ep, const torch::Tensor& rows, const Metadata& meta, int msg_kind, int dst_role) {
  MsgHeader h;
  h.sender = device_id_;
  h.kind = msg_kind;
  h.dst_role = dst_role;
  const bool has_rows = rows.defined() && rows.numel() > 0;
  const bool inline_payload = !ep.channel || ep.channel->inline_payload();
  h.has_payload = (has_rows && inline_payload) ? 1 : 0;
  h.seq = next_message_seq();
  if (has_rows && !inline_payload) h.ticket = ep.channel->stash(rows);
  std::unique_lock<std::mutex> pair_lock;
  if (ep.channel) pair_lock = std::unique_lock<std::mutex>(ep.channel->send_mutex());
  Frames f{to_bytes(h), to_bytes(meta)};
  if (h.has_payload) f.push_back(tensor_to_bytes(rows));
  ep.mq->send(f);
  if (has_rows && !inline_payload && h.ticket == 0) ep.channel->send(rows.contiguous(), meta);
}

MuAttnDispatcher::MuAttnDispatcher(std::vector<int> layer_ids, int device_id, ParallelConfig cfg,
                                   std::vector<Endpoint> endpoints, std::map<int, std::map<int, int>> next_attn_peer,
                                   int sampler_peer)
    : MuDispatcher(std::move(layer_ids), device_id, std::move(cfg), std::move(endpoints)),
      next_attn_peer_(std::move(next_attn_peer)), sampler_peer_(sampler_peer) {
  for (auto& e : endpoints_)
    for (auto& [layer, expert] : e.info.expert_ids) exp_peer_[layer][cfg_.rank_of(layer, expert)] = e.peer;
}

void MuAttnDispatcher::send_once(const TensorBatch& batch, int kind) {
  const Metadata& meta = *batch.metadata;
  const int n = static_cast<int>(meta.tok.size());
  if (kind == 2) {   // sampled token ids -> sampler
    Endpoint* ep = endpoint_of(sampler_peer_);
    DMOE_CHECK(ep != nullptr, "no edge to the sampler from device " << device_id_);
    send_batch(*ep, torch::Tensor(), meta, MSG_SAMPLED);
    return;
  }
  if (kind == 1) {   // residual part -> the attention worker of the next layer, per dp rank
    std::map<int, std::vector<int>> by_dp;
    for (int i = 0; i < n; ++i) by_dp[meta.tok.attn_dp_ranks.empty() ? 0 : meta.tok.attn_dp_ranks[i]].push_back(i);
    for (auto& [dp, rows] : by_dp) {
      auto lit = next_attn_peer_.find(meta.layer_id);
      DMOE_CHECK(lit != next_attn_peer_.end(), "no attention worker known for layer " << meta.layer_id);
      auto pit = lit->second.find(dp);
      if (pit == lit->second.end()) pit = lit->second.begin();
      Endpoint* ep = endpoint_of(pit->second);
      DMOE_CHECK(ep != nullptr, "no edge " << device_id_ << " -> " << pit->second);
      if (static_cast<int>(rows.size()) == n) {
        send_batch(*ep, batch.data, meta, MSG_TOKENS);
      } else {
        auto idx = torch::tensor(std::vector<int64_t>(rows.begin(), rows.end()), torch::kInt64).to(batch.data.device());
        send_batch(*ep, batch.data.index_select(0, idx), meta.at(rows), MSG_TOKENS);
      }
    }
    return;
  }
  // expert rows, sorted by expert id: contiguous runs that share an EP rank go out as one slice
  int l = 0;
  while (l < n) {
    const int rank = cfg_.rank_of(meta.layer_id, meta.tok.exp_ids[l]);
    int r = l + 1;
    while (r < n && cfg_.rank_of(meta.layer_id, meta.tok.exp_ids[r]) == rank) ++r;
    auto lit = exp_peer_.find(meta.layer_id);
    DMOE_CHECK(lit != exp_peer_.end() && lit->second.count(rank), "no expert worker for layer " << meta.layer_id
                                                                                                << " rank " << rank);
    Endpoint* ep = endpoint_of(lit->second[rank]);
    send_batch(*ep, batch.data.slice(0, l, r), meta.slice(l, r), MSG_TOKENS, /*dst_role=*/1);
    l = r;
  }
}

MuExpertDispatcher::MuExpertDispatcher(std::vector<int> layer_ids, int device_id, ParallelConfig cfg,
                                       std::vector<Endpoint> endpoints, std::map<int, std::map<int, int>> attn_peer)
    : MuDispatcher(std::move(layer_ids), device_id, std::move(cfg), std::move(endpoints)), attn_peer_(std::move(attn_peer)) {}

void MuExpertDispatcher::send_once(const TensorBatch& batch, int kind) {
  (void)kind;
  const Metadata& meta = *batch.metadata;   // layer_id already points at the next layer
  const int n = static_cast<int>(meta.tok.size());
  auto lit = attn_peer_.find(meta.layer_id);
  DMOE_CHECK(lit != attn_peer_.end(), "no attention worker known for layer " << meta.layer_id);
  int l = 0;
  while (l < n) {
    const int dp = meta.tok.attn_dp_ranks.empty() ? 0 : meta.tok.attn_dp_ranks[l];
    int r = l + 1;
    while (r < n && (meta.tok.attn_dp_ranks.empty() ? 0 : meta.tok.attn_dp_ranks[r]) == dp) ++r;
    auto pit = lit->second.find(dp);
    DMOE_CHECK(pit != lit->second.end(), "layer " << meta.layer_id << " has no attention replica " << dp);
    Endpoint* ep = endpoint_of(pit->second);
    DMOE_CHECK(ep != nullptr, "no edge " << device_id_ << " -> " << pit->second);
    send_batch(*ep, batch.data.slice(0, l, r), meta.slice(l, r), MSG_TOKENS);
    l = r;
  }
}

// ------------------------------------------------------------------------------------------------ MuPool
MuPool::MuPool(std::vector<int> layer_ids, int device_id, std::map<int, channel_t> in_channels,
               LayerSchedulePolicy policy, int num_groups, bool is_attn, torch::Device device, bool bind_mailbox)
    : MuHelper(std::move(layer_ids), device_id), in_channels_(std::move(in_channels)), device_(device),
      num_groups_(std::max(1, num_groups)), is_attn_(is_attn), owns_mailbox_(bind_mailbox) {
  const int L = static_cast<int>(layer_ids_.size());
  for (int i = 0; i < L; ++i) layer_to_local_[layer_ids_[i]] = i;
  queues_.resize(static_cast<size_t>(L) * num_groups_);
  tokens_per_cell_.assign(static_cast<size_t>(L) * num_groups_, 0);
  switch (policy) {
    case LayerSchedulePolicy::BASE:
      DMOE_CHECK(num_groups_ == 1, "the base policy has one group");
      layer_scheduler_ = std::make_shared<LayerScheduler>(L, LayerScheduler::Policy::MBFLFS);
      break;
    case LayerSchedulePolicy::ADVANCED:
      DMOE_CHECK(num_groups_ == 1, "the advanced policy has one group");
      layer_scheduler_ = std::make_shared<AdvancedLayerScheduler>(L, 0);
      break;
    case LayerSchedulePolicy::GROUP:
      layer_scheduler_ = std::make_shared<GroupLayerScheduler>(L, num_groups_);
      break;
  }
  // the mailbox is bound here (not in the thread) so that peers can connect as soon as the object exists
  if (owns_mailbox_) mailbox_.bind(get_zmq_addr(device_id_, true, 0));
}

int MuPool::local_layer(int layer_id) const {
  auto it = layer_to_local_.find(layer_id);
  DMOE_CHECK(it != layer_to_local_.end(), "device " << device_id_ << " does not run layer " << layer_id);
  return it->second;
}

void MuPool::set_layer_schedule_type(const std::string& type) {
  std::lock_guard<std::mutex> lk(batch_mu_);
  layer_scheduler_->set_schedule_type(type);
}
void MuPool::set_scheduler_block(int step) {
  std::lock_guard<std::mutex> lk(batch_mu_);
  layer_scheduler_->set_block_size(step);
}

void MuPool::notify() { batch_cv_.notify_all(); }

bool MuPool::wait_for_tokens(int timeout_ms) {
  std::unique_lock<std::mutex> lk(batch_mu_);
  auto any = [&] {
    for (int t : layer_scheduler_->get_tokens_per_layer())
      if (t > 0) return true;
    return false;
  };
  if (any()) return true;
  return batch_cv_.wait_for(lk, std::chrono::milliseconds(timeout_ms), any);
}

void MuPool::run() {
  if (!owns_mailbox_) return;   // fed by the other role's receive loop
  while (!end_flag_.load()) {
    Frames f;
    if (!mailbox_.recv(f, 50)) continue;
    DMOE_CHECK(f.size() >= 2, "short mailbox message");
    MsgHeader h;
    from_bytes(f[0], h);
    if (h.kind == MSG_STOP) continue;
    if (seq_filter_.seen(h.sender, h.seq)) {
      DMOE_LOG(WARN) << "pool@" << device_id_ << ": duplicate message " << h.seq << " from " << h.sender << " dropped";
      continue;
    }
    auto meta = std::make_shared<Metadata>();
    from_bytes(f[1], *meta);
    torch::Tensor t;
    if (h.has_payload) {
      DMOE_CHECK(f.size() == 3, "payload frame missing");
      t = tensor_from_bytes(f[2], *meta);
      if (device_.type() != torch::kCPU) t = t.to(device_, /*non_blocking=*/false);
    } else if (meta->num_tokens() > 0 && meta->token_hidden_dim() > 0 && h.kind == MSG_TOKENS) {
      auto it = in_channels_.find(h.sender);
      DMOE_CHECK(it != in_channels_.end(), "device " << device_id_ << " has no channel from " << h.sender);
      if (h.ticket != 0) {
        t = it->second->claim(h.ticket);
      } else {
        it->second->recv(t, *meta);
        it->second->sync();
      }
    }
    DMOE_RANGE("pool.process_batch");
    const int my_role = is_attn_ ? 0 : 1;
    if (h.dst_role != my_role && forward_) forward_->process_batch(t, meta, h.kind);
    else process_batch(t, meta, h.kind);
  }
}

void MuPool::process_batch(torch::Tensor tensor, metadata_t meta, int kind) {
  (void)kind;
  const int local = local_layer(meta->layer_id);
  const int n = static_cast<int>(meta->num_tokens());
  int group = 0;
  if (num_groups_ > 1 && !meta->tok.attn_dp_ranks.empty()) group = meta->tok.attn_dp_ranks[0] % num_groups_;
  const int cell = local * num_groups_ + group;
  {
    std::lock_guard<std::mutex> lk(batch_mu_);
    queues_[cell].push_back(TensorBatch{tensor, meta, now_ms()});
    tokens_per_cell_[cell] += n;
    layer_scheduler_->add_tokens_to_layer(cell, n);
  }
  notify();
}

std::vector<TensorBatch> MuPool::fetch_largest_batch(int* layer_out) {
  std::lock_guard<std::mutex> lk(batch_mu_);
  const int cell = layer_scheduler_->schedule();
  if (layer_out != nullptr) *layer_out = cell < 0 ? -1 : global_layer(cell / num_groups_);
  std::vector<TensorBatch> out;
  if (cell < 0) return out;
  auto& q = queues_[cell];
  int taken = 0;
  while (!q.empty()) {
    const int n = static_cast<int>(q.front().metadata->num_tokens());
    if (!out.empty() && taken + n > max_batch_size_) break;
    taken += n;
    out.push_back(std::move(q.front()));
    q.pop_front();
  }
  if (!out.empty()) last_delay_ms_.store(static_cast<float>(now_ms() - out.front().t_queued_ms));   // FIFO: oldest first
  tokens_per_cell_[cell] -= taken;
  if (tokens_per_cell_[cell] > 0) layer_scheduler_->add_tokens_to_layer(cell, tokens_per_cell_[cell]);
  return out;
}

std::vector<int> MuPool::get_pool_snapshot() {
  std::lock_guard<std::mutex> lk(batch_mu_);
  return layer_scheduler_->get_tokens_per_layer();
}

int MuPool::tokens_in_layer(int layer_id) {
  std::lock_guard<std::mutex> lk(batch_mu_);
  const int local = local_layer(layer_id);
  int s = 0;
  const auto t = layer_scheduler_->get_tokens_per_layer();
  for (int g = 0; g < num_groups_; ++g) s += t[local * num_groups_ + g];
  return s;
}

// ------------------------------------------------------------------------------------------------ attention pool
MuAttentionPool::MuAttentionPool(std::vector<int> layer_ids, int device_id, std::map<int, channel_t> in_channels,
                                 std::map<int, int> parts_needed, LayerSchedulePolicy policy, torch::Device device)
    : MuPool(std::move(layer_ids), device_id, std::move(in_channels), policy, 1, true, device),
      parts_needed_(std::move(parts_needed)) {
  partial_.resize(layer_ids_.size());
  ready_.resize(layer_ids_.size());
  next_pos_.resize(layer_ids_.size());
}

void MuAttentionPool::release_seqs(const std::vector<int>& seq_ids) {
  std::lock_guard<std::mutex> lk(batch_mu_);
  for (auto& m : next_pos_)
    for (int s : seq_ids) m.erase(s);
}

void MuAttentionPool::process_batch(torch::Tensor tensor, metadata_t meta, int kind) {
  const int local = local_layer(meta->layer_id);
  const int n = static_cast<int>(meta->tok.size());
  auto nit = parts_needed_.find(meta->layer_id);
  const int needed = nit == parts_needed_.end() ? 1 : nit->second;
  int completed = 0;
  {
    std::lock_guard<std::mutex> lk(batch_mu_);
    for (int i = 0; i < n; ++i) {
      const TokenMetadata tm = meta->info_at(i);
      if (kind == MSG_TOKEN_IDS) {
        TokenTopKInfo info;
        info.seq_id = tm.req_id; info.position = tm.position; info.init_prefill_len = tm.init_prefill_len;
        info.attn_dp_rank = tm.attn_dp_rank; info.token_id = meta->tok.token_ids.at(i);
        info.t_ready_ms = now_ms();
        ready_[local].push_back(std::move(info));
        ++completed;
        continue;
      }
      const auto key = std::make_pair(tm.req_id, tm.position);
      auto& info = partial_[local][key];
      if (info.parts.empty()) {
        info.seq_id = tm.req_id; info.position = tm.position; info.init_prefill_len = tm.init_prefill_len;
        info.attn_dp_rank = tm.attn_dp_rank;
      }
      info.parts.emplace_back(tm.topk_slot, tensor[i]);
      if (info.count() >= needed) {
        info.t_ready_ms = now_ms();
        ready_[local].push_back(std::move(info));
        partial_[local].erase(key);
        ++completed;
      }
    }
    if (completed > 0) layer_scheduler_->add_tokens_to_layer(local, completed);
  }
  if (completed > 0) notify();
}

int MuAttentionPool::num_pending_tokens() {
  std::lock_guard<std::mutex> lk(batch_mu_);
  int s = 0;
  for (auto& m : partial_) s += static_cast<int>(m.size());
  return s;
}

AttentionBatch MuAttentionPool::pack(int local, std::vector<TokenTopKInfo>& toks) {
  // prefill rows first (by sequence, position), decode rows after (by sequence)
  std::stable_sort(toks.begin(), toks.end(), [](const TokenTopKInfo& a, const TokenTopKInfo& b) {
    const int da = a.init_prefill_len < 0, db = b.init_prefill_len < 0;
    return std::make_tuple(da, a.seq_id, a.position) < std::make_tuple(db, b.seq_id, b.position);
  });
  AttentionBatch out;
  auto m = std::make_shared<AttentionBatchMetadata>();
  m->layer_id = global_layer(local);
  const int n = static_cast<int>(toks.size());
  int parts = 0;
  bool with_ids = false;
  std::vector<torch::Tensor> rows;
  for (auto& t : toks) {
    m->seq_ids.push_back(t.seq_id);
    m->init_prefill_lens.push_back(t.init_prefill_len);
    m->positions.push_back(t.position);
    m->attn_dp_ranks.push_back(t.attn_dp_rank);
    if (t.token_id >= 0) with_ids = true;
    m->token_ids.push_back(t.token_id);
    std::sort(t.parts.begin(), t.parts.end(), [](auto& a, auto& b) { return a.first < b.first; });
    if (!t.parts.empty()) {
      DMOE_CHECK(parts == 0 || parts == t.count(), "tokens of one batch carry different numbers of parts");
      parts = t.count();
      for (auto& p : t.parts) rows.push_back(p.second);
    }
  }
  if (!with_ids) m->token_ids.clear();
  if (!rows.empty()) {
    DMOE_CHECK(static_cast<int>(rows.size()) == n * parts, "a batch mixes token-id rows and hidden rows");
    auto stacked = torch::stack(rows, 0);   // [n * parts, H]
    out.data = stacked.view({n, parts, stacked.size(1)});
    m->shape = {n, stacked.size(1)};
    m->dtype = dtype_to_string(stacked.scalar_type());
  } else {
    m->shape = {n, 0};
  }
  m->recount();
  out.metadata = m;
  out.num_parts = parts;
  return out;
}

AttentionBatch MuAttentionPool::fetch_attention_batch() {
  std::vector<TokenTopKInfo> toks;
  int local;
  {
    std::lock_guard<std::mutex> lk(batch_mu_);
    local = layer_scheduler_->schedule();
    if (local < 0) return AttentionBatch{};
    auto& q = ready_[local];
    // a batch holds either token-id rows (to be embedded) or hidden rows, never both; prompt tokens are taken in
    // position order per sequence, a token whose predecessors have not run at this layer yet stays queued
    std::vector<TokenTopKInfo> all(std::make_move_iterator(q.begin()), std::make_move_iterator(q.end()));
    q.clear();
    std::stable_sort(all.begin(), all.end(), [](const TokenTopKInfo& a, const TokenTopKInfo& b) {
      return std::make_pair(a.seq_id, a.position) < std::make_pair(b.seq_id, b.position);
    });
    bool have_kind = false, ids_kind = false;
    auto& next = next_pos_[local];
    for (auto& t : all) {
      const bool is_ids = t.token_id >= 0;
      bool ok = static_cast<int>(toks.size()) < max_batch_size_ && (!have_kind || is_ids == ids_kind);
      if (ok && t.init_prefill_len >= 0 && !unordered_.count(local)) {
        auto it = next.find(t.seq_id);
        const int expect = it == next.end() ? 0 : it->second;
        ok = t.position == expect;
        if (ok) next[t.seq_id] = expect + 1;
      }
      if (ok) {
        have_kind = true;
        ids_kind = is_ids;
        toks.push_back(std::move(t));
      } else {
        q.push_back(std::move(t));
      }
    }
    if (!q.empty()) layer_scheduler_->add_tokens_to_layer(local, static_cast<int>(q.size()));
  }
  if (toks.empty()) return AttentionBatch{};
  double oldest = toks.front().t_ready_ms;
  for (auto& t : toks) oldest = std::min(oldest, t.t_ready_ms);
  last_delay_ms_.store(static_cast<float>(now_ms() - oldest));
  return pack(local, toks);
}

AttentionBatch MuAttentionPool::fetch_batch_from(int layer_id, const std::vector<std::pair<int, int>>& tokens,
                                                 int timeout_ms) {
  const int local = local_layer(layer_id);
  std::set<std::pair<int, int>> want(tokens.begin(), tokens.end());
  std::vector<TokenTopKInfo> toks;
  std::unique_lock<std::mutex> lk(batch_mu_);
  auto have_all = [&] {
    size_t c = 0;
    for (auto& t : ready_[local]) c += want.count({t.seq_id, t.position});
    return c >= want.size();
  };
  DMOE_CHECK(batch_cv_.wait_for(lk, std::chrono::milliseconds(timeout_ms), have_all),
             "TP worker did not receive the tokens the driver scheduled for layer " << layer_id);
  std::deque<TokenTopKInfo> rest;
  for (auto& t : ready_[local]) {
    if (want.count({t.seq_id, t.position})) toks.push_back(std::move(t)); else rest.push_back(std::move(t));
  }
  ready_[local] = std::move(rest);
  layer_scheduler_->remove_tokens_from_layer(local, static_cast<int>(toks.size()));
  lk.unlock();
  return pack(local, toks);
}

// ------------------------------------------------------------------------------------------------ schedulers
Scheduler::Scheduler(std::shared_ptr<MuPool> pool, std::vector<int> layer_ids, std::string policy)
    : pool_(std::move(pool)), layer_ids_(std::move(layer_ids)) {
  (void)policy;
}

TensorBatch Scheduler::schedule() {
  DMOE_AUTO_RANGE;
  auto batches = pool_->fetch_largest_batch();
  if (batches.empty()) return TensorBatch{};
  return TensorBatch::merge(batches);
}

AttentionScheduler::AttentionScheduler(std::shared_ptr<MuAttentionPool> pool, std::vector<int> layer_ids,
                                       std::string policy)
    : pool_(std::move(pool)), layer_ids_(std::move(layer_ids)) {
  (void)policy;
}

AttentionBatch AttentionScheduler::schedule() {
  DMOE_AUTO_RANGE;
  return pool_->fetch_attention_batch();
}

AttentionBatch AttentionDriverScheduler::schedule() {
  AttentionBatch b = pool_->fetch_attention_batch();
  if (!b.metadata) return b;
  ScheduleDecision d{b.metadata->layer_id, static_cast<int>(b.metadata->seq_ids.size())};
  for (size_t i = 0; i < b.metadata->seq_ids.size(); ++i) {
    d.push_back(b.metadata->seq_ids[i]);
    d.push_back(b.metadata->positions[i]);
  }
  bcast_(d);
  return b;
}

AttentionBatch AttentionWorkerScheduler::schedule() {
  ScheduleDecision d;
  bcast_(d);
  if (d.size() < 2 || d[1] <= 0) return AttentionBatch{};
  std::vector<std::pair<int, int>> toks;
  for (int i = 0; i < d[1]; ++i) toks.emplace_back(d[2 + 2 * i], d[3 + 2 * i]);
  return pool_->fetch_batch_from(d[0], toks);
}

}  // namespace dmoe
