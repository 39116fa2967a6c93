#include "engine.h"

namespace dmoe {

namespace {
LayerSchedulePolicy parse_pool_policy(const std::string& s) {
  if (s == "base") return LayerSchedulePolicy::BASE;
  if (s == "advanced") return LayerSchedulePolicy::ADVANCED;
  if (s == "group") return LayerSchedulePolicy::GROUP;
  throw RuntimeError("unknown pool policy " + s);
}

// One channel per edge: same device -> local queue, embedding nodes and edges without an NCCL id -> socket
// transport (payload rides in the mailbox message), otherwise a 2-rank NCCL communicator.
channel_t make_channel(int local, int peer, bool sender, const std::map<int, std::string>& nccl_ids,
                       std::map<int, channel_t>& shared_local) {
  if (peer == local) {
    auto& c = shared_local[local];
    if (!c) c = create_local_channel(local);
    return c;
  }
  auto it = nccl_ids.find(peer);
  if (is_embedding_node(peer) || it == nccl_ids.end()) return nullptr;   // inline payload, no channel object needed
  (void)sender;
  return create_channel(local, peer, it->second);
}

std::vector<Endpoint> make_endpoints(const EngineArgs& a, std::map<int, channel_t>& shared_local,
                                     std::vector<channel_t>& to_instantiate) {
  std::vector<Endpoint> eps;
  DMOE_CHECK(a.out_channel_infos.size() == a.out_device_ids.size(), "one ChannelInfo per out device");
  for (size_t i = 0; i < a.out_device_ids.size(); ++i) {
    Endpoint e;
    e.peer = a.out_device_ids[i];
    e.info = a.out_channel_infos[i];
    e.channel = make_channel(a.local_id, e.peer, true, a.out_nccl_ids, shared_local);
    if (e.channel && e.peer != a.local_id) to_instantiate.push_back(e.channel);
    eps.push_back(std::move(e));
  }
  return eps;
}

std::map<int, channel_t> make_in_channels(const EngineArgs& a, std::map<int, channel_t>& shared_local,
                                          std::vector<channel_t>& to_instantiate) {
  std::map<int, channel_t> in;
  for (int peer : a.in_device_ids) {
    auto c = make_channel(a.local_id, peer, false, a.in_nccl_ids, shared_local);
    if (!c) continue;
    in[peer] = c;
    if (peer != a.local_id) to_instantiate.push_back(c);
  }
  return in;
}
}  // namespace

static EngineHandles build(const EngineArgs& a, bool colocate) {
  DMOE_CHECK(colocate ? (a.has_attn && a.has_expert) : (a.has_attn != a.has_expert),
             "a worker runs attention or experts; use init_engine_colocate for both");
  EngineHandles h;
  std::map<int, channel_t> shared_local;
  std::vector<channel_t> pending;
  auto endpoints = make_endpoints(a, shared_local, pending);
  auto in_channels = make_in_channels(a, shared_local, pending);
  instantiate_channels(pending);
  const torch::Device dev(a.device);
  if (a.has_attn) {
    h.attn_pool = std::make_shared<MuAttentionPool>(a.attn_layer_ids, a.local_id, in_channels, a.parts_needed,
                                                    parse_pool_policy(a.attn_policy), dev);
    h.attn_scheduler = std::make_shared<AttentionScheduler>(h.attn_pool, a.attn_layer_ids);
    h.attn_dispatcher = std::make_shared<MuAttnDispatcher>(a.attn_layer_ids, a.local_id, a.cfg, endpoints, a.attn_peer,
                                                          a.sampler_id);
  }
  if (a.has_expert) {
    const auto pol = parse_pool_policy(a.expert_policy);
    h.expert_pool = std::make_shared<MuPool>(a.expert_layer_ids, a.local_id, in_channels, pol,
                                             pol == LayerSchedulePolicy::GROUP ? a.num_dp_groups : 1, false, dev,
                                             /*bind_mailbox=*/!colocate);
    h.scheduler = std::make_shared<Scheduler>(h.expert_pool, a.expert_layer_ids);
    h.expert_dispatcher = std::make_shared<MuExpertDispatcher>(a.expert_layer_ids, a.local_id, a.cfg, endpoints,
                                                              a.attn_peer);
  }
  if (colocate) h.attn_pool->set_forward_pool(h.expert_pool);
  return h;
}

EngineHandles init_engine(const EngineArgs& args) { return build(args, false); }
EngineHandles init_engine_colocate(const EngineArgs& args) { return build(args, true); }

void start_engine(EngineHandles& h) {
  if (h.attn_pool) h.attn_pool->start();
  if (h.expert_pool) h.expert_pool->start();
  if (h.attn_dispatcher) h.attn_dispatcher->start();
  if (h.expert_dispatcher) h.expert_dispatcher->start();
}

void stop_engine(EngineHandles& h) {
  if (h.attn_dispatcher) h.attn_dispatcher->terminate();
  if (h.expert_dispatcher) h.expert_dispatcher->terminate();
  if (h.attn_pool) h.attn_pool->terminate();
  if (h.expert_pool) h.expert_pool->terminate();
}

static std::vector<Endpoint> plain_endpoints(const std::vector<int>& outs) {
  std::vector<Endpoint> eps;
  for (int d : outs) {
    Endpoint e;
    e.peer = d;
    eps.push_back(std::move(e));
  }
  return eps;
}

std::shared_ptr<Sampler> init_sampler(int device_id, int min_output_len, int max_output_len, int top_k,
                                      const std::vector<int>& out_device_ids, const std::map<int, int>& attn_peer,
                                      bool ignore_eos, bool topk_partials) {
  if (topk_partials && top_k > 1)
    return std::make_shared<TopKSampler>(device_id, plain_endpoints(out_device_ids), attn_peer, min_output_len,
                                         max_output_len, top_k, ignore_eos);
  return std::make_shared<Sampler>(device_id, plain_endpoints(out_device_ids), attn_peer, min_output_len, max_output_len,
                                   ignore_eos);
}

std::shared_ptr<Tokenizer> init_tokenizer(int device_id, const std::vector<int>& out_device_ids,
                                          const std::map<int, int>& attn_peer) {
  return std::make_shared<Tokenizer>(device_id, plain_endpoints(out_device_ids), attn_peer);
}

}  // namespace dmoe
