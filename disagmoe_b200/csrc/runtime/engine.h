// Engine factory: builds the channels, pool, scheduler and dispatcher of one worker from its placement slice.
// Reference behaviour covered: csrc/include/engine.h, csrc/engine/engine.cpp:14-342 (init_all_channels, init_engine,
// init_engine_colocate, start_engine, init_sampler, init_tokenizer, set_hosts).
#pragma once
#include "block_manager.h"
#include "embedding.h"

namespace dmoe {

struct EngineArgs {
  int local_id = 0;
  int top_k = 1;
  bool has_attn = false, has_expert = false;
  ParallelConfig cfg;
  std::vector<int> attn_layer_ids;     // attention layers run here (num_layers = the LM-head step, if hosted)
  std::vector<int> expert_layer_ids;   // layers whose experts (an EP shard) run here
  std::vector<int> in_device_ids, out_device_ids;
  std::vector<ChannelInfo> out_channel_infos;          // one per out device
  std::map<int, std::string> in_nccl_ids, out_nccl_ids;  // peer -> 128-byte unique id; no entry = socket transport
  std::map<int, std::map<int, int>> attn_peer;         // layer -> dp rank -> attention device (layer L = head step)
  std::map<int, int> parts_needed;                     // attention layer -> partial rows per token
  int sampler_id = kSamplerDevId;
  int num_dp_groups = 1;                               // expert pool groups
  std::string device = "cpu";
  std::string attn_policy = "base", expert_policy = "group";
};

struct EngineHandles {
  std::shared_ptr<Scheduler> scheduler;                // expert role
  std::shared_ptr<AttentionScheduler> attn_scheduler;  // attention role
  std::shared_ptr<MuAttnDispatcher> attn_dispatcher;
  std::shared_ptr<MuExpertDispatcher> expert_dispatcher;
  std::shared_ptr<MuPool> expert_pool;
  std::shared_ptr<MuAttentionPool> attn_pool;
};

EngineHandles init_engine(const EngineArgs& args);
// Both roles on one device (one mailbox, rows for the expert role are forwarded inside the process).
EngineHandles init_engine_colocate(const EngineArgs& args);
void start_engine(EngineHandles& h);
void stop_engine(EngineHandles& h);
std::shared_ptr<Sampler> init_sampler(int device_id, int min_output_len, int max_output_len, int top_k,
                                      const std::vector<int>& out_device_ids, const std::map<int, int>& attn_peer,
                                      bool ignore_eos, bool topk_partials = false);
std::shared_ptr<Tokenizer> init_tokenizer(int device_id, const std::vector<int>& out_device_ids,
                                          const std::map<int, int>& attn_peer);

}  // namespace dmoe
