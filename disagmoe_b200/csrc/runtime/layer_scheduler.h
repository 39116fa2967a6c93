// Layer schedulers: which layer's queued tokens does a worker run next?
//
// Policies (behaviour and constants of csrc/include/scheduler.h:139-287, csrc/engine/scheduler.cpp:191-451):
//   mbfs    max-batch-first: the layer with the most queued tokens
//   flfs    first-layer-first: the lowest layer that has tokens
//   bin     same pick as flfs
//   mbflfs  layers are grouped in blocks of `block_size` (default 8); take the block with the most tokens, then
//           its first non-empty layer (block_size 1 = mbfs, block_size n_layers = flfs)
//   mbtfs   most queued batches, ties broken by tokens
// AdvancedLayerScheduler: per-layer state machine IDLE -> HOLD -> READY -> URGENT. A layer with fewer than 256
//   queued tokens is held for `hold_steps` scheduling rounds; a READY layer older than 30 ms becomes URGENT
//   (oldest first); READY layers are ranked by the look-ahead score sum_{j<4} tokens[(l+j) mod L] * 0.8^j.
// GroupLayerScheduler: the same look-ahead score over (layer, dp-group) cells.
// All schedulers expect the caller to serialise calls (the pool's queue lock).
#pragma once
#include <functional>

#include "core.h"

namespace dmoe {

class LayerScheduler {
 public:
  enum class Policy { MBFS, FLFS, MBFLFS, MBTFS, BIN };
  explicit LayerScheduler(int n_layers, Policy p = Policy::MBFS)
      : n_layers_(n_layers), policy_(p), tokens_(n_layers, 0), batches_(n_layers, 0) {}
  virtual ~LayerScheduler() = default;

  // Picks a layer (or cell) and clears its counters; -1 when nothing is queued.
  virtual int schedule();
  virtual void add_tokens_to_layer(int layer_id, int num_tokens);
  void remove_tokens_from_layer(int layer_id, int num_tokens);
  void set_schedule_type(const std::string& name);
  void set_block_size(int b) { block_size_ = std::max(1, b); }
  std::vector<int> get_tokens_per_layer() const { return tokens_; }
  static Policy parse_policy(const std::string& name);

 protected:
  void clear(int i) { tokens_[i] = 0; batches_[i] = 0; }
  float lookahead_score(int layer, int stride, int offset) const;
  int n_layers_;
  Policy policy_;
  int block_size_ = 8;
  std::vector<int> tokens_, batches_;
};

class AdvancedLayerScheduler : public LayerScheduler {
 public:
  static constexpr int kReadyThreshold = 256;
  static constexpr double kUrgentAfterMs = 30.0;
  AdvancedLayerScheduler(int n_layers, int hold_steps = 2);
  int schedule() override;
  void add_tokens_to_layer(int layer_id, int num_tokens) override;
  // Test hook: replaces the clock (milliseconds).
  void set_clock(std::function<double()> clk) { clock_ = std::move(clk); }

 private:
  enum class State { IDLE, HOLD, READY, URGENT };
  void to_ready(int l) { state_[l] = State::READY; ready_at_[l] = clock_(); }
  int hold_steps_;
  std::vector<State> state_;
  std::vector<int> hold_left_;
  std::vector<double> ready_at_;
  std::function<double()> clock_;
};

class GroupLayerScheduler : public LayerScheduler {
 public:
  GroupLayerScheduler(int n_layers, int n_groups)
      : LayerScheduler(n_layers * n_groups), layers_(n_layers), groups_(n_groups) {}
  using LayerScheduler::add_tokens_to_layer;
  void add_tokens_to_layer(int layer_id, int group_id, int num_tokens) {
    LayerScheduler::add_tokens_to_layer(cell(layer_id, group_id), num_tokens);
  }
  // Returns the cell id layer * n_groups + group, or -1.
  int schedule() override;
  int cell(int layer, int group) const { return layer * groups_ + group; }
  int n_groups() const { return groups_; }

 private:
  int layers_, groups_;
};

}  // namespace dmoe
