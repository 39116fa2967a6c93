// The per-worker helper threads and batch formers ("muhelper"): receive pool, layer scheduling, dispatchers.
//
//   MuHelper            thread base: start / terminate (always joinable: every blocking wait has a timeout)
//   Endpoint            one outgoing edge = mailbox PUSH socket of the peer + tensor channel
//   MuDispatcher        send queue + thread; MuAttnDispatcher (attention -> experts by EP rank, and the residual part
//                       -> next layer's attention); MuExpertDispatcher (experts -> attention replica by dp rank, or
//                       the LM-head step / sampler after the last layer)
//   MuPool              receive loop + per-(layer, group) queues of expert batches
//   MuAttentionPool     per-layer accumulation of partial rows (top-k expert outputs + residual part) until a token
//                       is complete, then it becomes schedulable
//   Scheduler / AttentionScheduler         pick a layer (LayerScheduler policy) and merge its queue into one batch
//   AttentionDriverScheduler / AttentionWorkerScheduler   TP group: rank 0 decides and broadcasts the decision
//
// Reference behaviour covered: csrc/include/muhelper.h:14-336, csrc/muhelper/muhelper.cpp:27-985,
// csrc/include/scheduler.h:20-131, csrc/engine/scheduler.cpp:12-189, csrc/include/datatypes.hpp:503-584,841-953.
#pragma once
#include <atomic>
#include <functional>
#include <set>

#include "channel.h"
#include "layer_scheduler.h"

namespace dmoe {

enum MsgKind : int { MSG_TOKENS = 0, MSG_TOKEN_IDS = 1, MSG_SAMPLED = 2, MSG_STOP = 3 };

struct MsgHeader {
  int sender = 0;
  int kind = MSG_TOKENS;
  int has_payload = 0;
  int dst_role = 0;   // 0 = attention role, 1 = expert role of the receiving device (colocated workers run both)
  uint64_t ticket = 0;  // same-process edges: the tensor waits in the LocalChannel under this ticket
  uint64_t seq = 0;     // process-wide message number of the sender; receivers drop a (sender, seq) seen before
  template <class A>
  void io(A& a) { a(sender, kind, has_payload, dst_role, ticket, seq); }
};

struct TensorBatch {
  torch::Tensor data;     // [tokens, hidden] (undefined for token-id batches)
  metadata_t metadata;
  double t_queued_ms = 0;  // steady-clock time at which a pool queued the batch (0: never queued)
  // Merges batches of one layer into one expert-sorted batch (stable counting sort + row gather).
  static TensorBatch merge(const std::vector<TensorBatch>& batches);
  static TensorBatch concat(const std::vector<TensorBatch>& batches);
};

struct AttentionBatch {
  torch::Tensor data;          // [tokens, parts, hidden] partial rows to be summed, or undefined for layer-0 input
  attn_metadata_t metadata;
  int num_parts = 0;
};

// First exception that ended a helper thread of this process (empty while all of them run).
void set_helper_error(const std::string& what);
// A symbol of the package's kernel library (lib/libdmoe_kernels.so next to this module), or nullptr (CPU-only installs).
void* kernel_library_symbol(const char* name);
std::string helper_error();

class MuHelper {
 public:
  MuHelper(std::vector<int> layer_ids, int device_id) : layer_ids_(std::move(layer_ids)), device_id_(device_id) {}
  virtual ~MuHelper() { terminate(); }
  void start();
  void terminate();
  bool running() const { return thread_.joinable() && !end_flag_.load(); }
  int device_id() const { return device_id_; }

 protected:
  virtual void run() = 0;
  virtual const char* name() const { return "muhelper"; }
  std::vector<int> layer_ids_;
  int device_id_;
  std::atomic<bool> end_flag_{false};
  std::thread thread_;
};

// One outgoing edge.
struct Endpoint {
  int peer = -1;
  std::shared_ptr<PushSocket> mq;
  channel_t channel;
  ChannelInfo info;
};

class MuDispatcher : public MuHelper {
 public:
  MuDispatcher(std::vector<int> layer_ids, int device_id, ParallelConfig cfg, std::vector<Endpoint> endpoints);
  // Queues a batch; `kind` distinguishes expert-bound rows (0), the residual part (1) and sampled ids (2).
  void put(const TensorBatch& batch, int kind = 0);
  size_t pending();
  void connect_all();

 protected:
  void run() override;
  virtual void send_once(const TensorBatch& batch, int kind) = 0;
  void send_batch(Endpoint& ep, const torch::Tensor& rows, const Metadata& meta, int msg_kind, int dst_role = 0);
  Endpoint* endpoint_of(int peer);
  ParallelConfig cfg_;
  std::vector<Endpoint> endpoints_;
  std::mutex mu_;
  std::condition_variable cv_;
  std::deque<std::pair<TensorBatch, int>> queue_;
  bool connected_ = false;
};

class MuAttnDispatcher : public MuDispatcher {
 public:
  // next_attn_peer[layer][dp rank] -> device that runs attention layer `layer` (layer == num_layers: LM head step)
  MuAttnDispatcher(std::vector<int> layer_ids, int device_id, ParallelConfig cfg, std::vector<Endpoint> endpoints,
                   std::map<int, std::map<int, int>> next_attn_peer, int sampler_peer);

 protected:
  const char* name() const override { return "attn_dispatcher"; }
  void send_once(const TensorBatch& batch, int kind) override;

 private:
  std::map<int, std::map<int, int>> exp_peer_;   // layer -> ep rank -> peer device
  std::map<int, std::map<int, int>> next_attn_peer_;
  int sampler_peer_;
};

class MuExpertDispatcher : public MuDispatcher {
 public:
  MuExpertDispatcher(std::vector<int> layer_ids, int device_id, ParallelConfig cfg, std::vector<Endpoint> endpoints,
                     std::map<int, std::map<int, int>> attn_peer);

 protected:
  const char* name() const override { return "expert_dispatcher"; }
  void send_once(const TensorBatch& batch, int kind) override;

 private:
  std::map<int, std::map<int, int>> attn_peer_;  // layer -> dp rank -> peer device
};

enum class LayerSchedulePolicy { BASE, ADVANCED, GROUP };

class MuPool : public MuHelper {
 public:
  MuPool(std::vector<int> layer_ids, int device_id, std::map<int, channel_t> in_channels,
         LayerSchedulePolicy policy = LayerSchedulePolicy::BASE, int num_groups = 1, bool is_attn = false,
         torch::Device device = torch::kCPU, bool bind_mailbox = true);
  // Colocated workers: messages addressed to the other role of this device are handed to `other`.
  void set_forward_pool(std::shared_ptr<MuPool> other) { forward_ = std::move(other); }
  // Picks a (layer, group) cell by the layer-scheduling policy and drains its queue. Empty when idle.
  std::vector<TensorBatch> fetch_largest_batch(int* layer_out = nullptr);
  std::vector<int> get_pool_snapshot();
  int tokens_in_layer(int layer_id);
  void set_max_batch_size(int n) { max_batch_size_ = n; }
  void set_layer_schedule_type(const std::string& type);
  void set_scheduler_block(int step);
  // Blocks (GIL-free when called through the binding) until tokens are queued or the timeout passes.
  bool wait_for_tokens(int timeout_ms);
  // Test hook: injects a batch as if it had been received.
  virtual void process_batch(torch::Tensor tensor, metadata_t meta, int kind);
  // How long the oldest row of the most recently fetched batch had been runnable in this pool (milliseconds).
  float last_queueing_delay_ms() const { return last_delay_ms_.load(); }
  int local_layer(int layer_id) const;
  int global_layer(int local) const { return layer_ids_.at(local); }
  int num_local_layers() const { return static_cast<int>(layer_ids_.size()); }

 protected:
  void run() override;
  const char* name() const override { return "pool"; }
  void notify();
  std::map<int, channel_t> in_channels_;
  PullSocket mailbox_;
  torch::Device device_;
  int num_groups_;
  bool is_attn_;
  int max_batch_size_ = 1 << 30;
  std::shared_ptr<LayerScheduler> layer_scheduler_;
  std::mutex batch_mu_;
  std::condition_variable batch_cv_;
  std::vector<std::deque<TensorBatch>> queues_;   // [local layer * groups + group]
  std::vector<int> tokens_per_cell_;
  std::map<int, int> layer_to_local_;
  std::shared_ptr<MuPool> forward_;
  SeqFilter seq_filter_;
  std::atomic<float> last_delay_ms_{0.f};
  bool owns_mailbox_ = true;
};

// A token whose partial rows are still arriving.
struct TokenTopKInfo {
  int seq_id = 0, position = 0, init_prefill_len = -1, attn_dp_rank = 0, token_id = -1;
  std::vector<std::pair<int, torch::Tensor>> parts;   // (slot, row [hidden])
  double t_ready_ms = 0;                                // when the last part arrived and the token became runnable
  int count() const { return static_cast<int>(parts.size()); }
};

class MuAttentionPool : public MuPool {
 public:
  // parts_needed(layer) = rows that must arrive before a token of that layer is complete (top_k + 1 residual
  // part; 1 after a dense layer; 0 for token-id input of layer 0).
  MuAttentionPool(std::vector<int> layer_ids, int device_id, std::map<int, channel_t> in_channels,
                  std::map<int, int> parts_needed, LayerSchedulePolicy policy = LayerSchedulePolicy::BASE,
                  torch::Device device = torch::kCPU);
  void process_batch(torch::Tensor tensor, metadata_t meta, int kind) override;
  // Drains the complete tokens of the scheduled layer (at most max_batch_size), prefill rows first.
  AttentionBatch fetch_attention_batch();
  // The TP worker side: takes exactly the tokens (seq id, position) the driver scheduled for `layer_id`.
  AttentionBatch fetch_batch_from(int layer_id, const std::vector<std::pair<int, int>>& tokens, int timeout_ms = 30000);
  int num_pending_tokens();
  // Forgets the per-sequence prefill progress of finished sequences.
  void release_seqs(const std::vector<int>& seq_ids);
  // A layer whose step has no dependency between the tokens of a prompt (the LM-head step) takes tokens in any order.
  void set_unordered_layer(int layer_id) { unordered_.insert(local_layer(layer_id)); }

 private:
  AttentionBatch pack(int local_layer, std::vector<TokenTopKInfo>& toks);
  // Causal order inside a prompt: prompt token i of a sequence may run at a layer only after tokens 0..i-1 ran there
  // (their K/V must be in the cache). next_pos_[layer][seq] is the next prompt position that may be scheduled.
  std::vector<std::map<int, int>> next_pos_;
  std::set<int> unordered_;
  std::map<int, int> parts_needed_;
  // per local layer: incomplete tokens keyed by (seq, position); complete tokens in arrival order
  std::vector<std::map<std::pair<int, int>, TokenTopKInfo>> partial_;
  std::vector<std::deque<TokenTopKInfo>> ready_;
};

class Scheduler {
 public:
  Scheduler(std::shared_ptr<MuPool> pool, std::vector<int> layer_ids, std::string policy = "mbfs");
  TensorBatch schedule();
  bool wait_for_new_requests(int timeout_ms = 100) { return pool_->wait_for_tokens(timeout_ms); }
  std::vector<int> get_pool_snapshot() { return pool_->get_pool_snapshot(); }
  // Queueing delay (ms) of the batch the last schedule() returned (reference: Scheduler::get_cur_queueing_delay,
  // csrc/include/scheduler.h:54, where the measurement itself is commented out and the value stays 0).
  float get_cur_queueing_delay() const { return pool_->last_queueing_delay_ms(); }
  void set_max_batch_size(int n) { pool_->set_max_batch_size(n); }
  void set_schedule_policy(const std::string& p) { pool_->set_layer_schedule_type(p); }
  void set_schedule_block(int step) { pool_->set_scheduler_block(step); }
  void start() { pool_->start(); }

 protected:
  std::shared_ptr<MuPool> pool_;
  std::vector<int> layer_ids_;
};

class AttentionScheduler {
 public:
  AttentionScheduler(std::shared_ptr<MuAttentionPool> pool, std::vector<int> layer_ids, std::string policy = "mbfs");
  virtual ~AttentionScheduler() = default;
  virtual AttentionBatch schedule();
  bool wait_for_new_requests(int timeout_ms = 100) { return pool_->wait_for_tokens(timeout_ms); }
  std::vector<int> get_pool_snapshot() { return pool_->get_pool_snapshot(); }
  float get_cur_queueing_delay() const { return pool_->last_queueing_delay_ms(); }
  void set_max_batch_size(int n) { pool_->set_max_batch_size(n); }
  void set_schedule_policy(const std::string& p) { pool_->set_layer_schedule_type(p); }
  void set_schedule_block(int step) { pool_->set_scheduler_block(step); }
  void start() { pool_->start(); }
  std::shared_ptr<MuAttentionPool> pool() { return pool_; }

 protected:
  std::shared_ptr<MuAttentionPool> pool_;
  std::vector<int> layer_ids_;
};

// Decision shared inside a TP group: [layer_id, n, (seq, pos) * n].
using ScheduleDecision = std::vector<int>;
using DecisionBcast = std::function<void(ScheduleDecision&)>;   // root sends, others receive (in place)

class AttentionDriverScheduler : public AttentionScheduler {
 public:
  AttentionDriverScheduler(std::shared_ptr<MuAttentionPool> pool, std::vector<int> layer_ids, DecisionBcast bcast)
      : AttentionScheduler(std::move(pool), std::move(layer_ids)), bcast_(std::move(bcast)) {}
  AttentionBatch schedule() override;

 private:
  DecisionBcast bcast_;
};

class AttentionWorkerScheduler : public AttentionScheduler {
 public:
  AttentionWorkerScheduler(std::shared_ptr<MuAttentionPool> pool, std::vector<int> layer_ids, DecisionBcast bcast)
      : AttentionScheduler(std::move(pool), std::move(layer_ids)), bcast_(std::move(bcast)) {}
  AttentionBatch schedule() override;

 private:
  DecisionBcast bcast_;
};

}  // namespace dmoe
