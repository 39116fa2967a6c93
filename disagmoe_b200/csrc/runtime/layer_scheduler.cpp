#include "layer_scheduler.h"

#include <algorithm>

namespace dmoe {

LayerScheduler::Policy LayerScheduler::parse_policy(const std::string& name) {
  if (name == "mbfs") return Policy::MBFS;
  if (name == "flfs") return Policy::FLFS;
  if (name == "mbflfs") return Policy::MBFLFS;
  if (name == "mbtfs") return Policy::MBTFS;
  if (name == "bin") return Policy::BIN;
  throw RuntimeError(name + " schedule not implemented");
}

void LayerScheduler::set_schedule_type(const std::string& name) { policy_ = parse_policy(name); }

void LayerScheduler::add_tokens_to_layer(int layer_id, int num_tokens) {
  DMOE_CHECK(layer_id >= 0 && layer_id < static_cast<int>(tokens_.size()), "layer " << layer_id);
  tokens_[layer_id] += num_tokens;
  batches_[layer_id] += 1;
}

void LayerScheduler::remove_tokens_from_layer(int layer_id, int num_tokens) {
  DMOE_CHECK(layer_id >= 0 && layer_id < static_cast<int>(tokens_.size()), "layer " << layer_id);
  tokens_[layer_id] = std::max(0, tokens_[layer_id] - num_tokens);
}

float LayerScheduler::lookahead_score(int layer, int stride, int offset) const {
  // tokens of `layer` and the 3 layers after it (wrapping), discounted by 0.8 per step
  const int L = static_cast<int>(tokens_.size()) / stride;
  float score = 0.f, decay = 1.f;
  for (int j = 0; j < 4; ++j) {
    score += tokens_[((layer + j) % L) * stride + offset] * decay;
    decay *= 0.8f;
  }
  return score;
}

int LayerScheduler::schedule() {
  const int n = static_cast<int>(tokens_.size());
  int pick = -1;
  switch (policy_) {
    case Policy::MBFS: {
      int best = 0;
      for (int i = 0; i < n; ++i)
        if (tokens_[i] > best) { best = tokens_[i]; pick = i; }
      break;
    }
    case Policy::FLFS:
    case Policy::BIN: {
      for (int i = 0; i < n && pick < 0; ++i)
        if (tokens_[i] > 0) pick = i;
      break;
    }
    case Policy::MBFLFS: {
      int best_sum = 0, best_block = -1;
      for (int b = 0; b < n; b += block_size_) {
        int sum = 0;
        for (int j = b; j < std::min(n, b + block_size_); ++j) sum += tokens_[j];
        if (sum > best_sum) { best_sum = sum; best_block = b; }
      }
      if (best_block >= 0)
        for (int j = best_block; j < std::min(n, best_block + block_size_) && pick < 0; ++j)
          if (tokens_[j] > 0) pick = j;
      break;
    }
    case Policy::MBTFS: {
      int bb = 0, bt = 0;
      for (int i = 0; i < n; ++i)
        if (batches_[i] > bb || (batches_[i] == bb && tokens_[i] > bt)) { pick = i; bb = batches_[i]; bt = tokens_[i]; }
      break;
    }
  }
  if (pick >= 0) clear(pick);
  return pick;
}

AdvancedLayerScheduler::AdvancedLayerScheduler(int n_layers, int hold_steps)
    : LayerScheduler(n_layers), hold_steps_(hold_steps), state_(n_layers, State::IDLE), hold_left_(n_layers, 0),
      ready_at_(n_layers, 0.0), clock_([] { return now_ms(); }) {}

void AdvancedLayerScheduler::add_tokens_to_layer(int l, int num_tokens) {
  DMOE_CHECK(l >= 0 && l < n_layers_, "layer " << l);
  tokens_[l] += num_tokens;
  batches_[l] += 1;
  if (state_[l] == State::IDLE) {
    if (tokens_[l] >= kReadyThreshold || hold_steps_ == 0) {
      to_ready(l);
    } else {
      state_[l] = State::HOLD;
      hold_left_[l] = hold_steps_;
    }
  } else if (state_[l] == State::HOLD && tokens_[l] >= kReadyThreshold) {
    to_ready(l);
  }
}

int AdvancedLayerScheduler::schedule() {
  const double now = clock_();
  int pick = -1;
  // 1. urgent layers, oldest first (READY layers that waited too long are promoted here)
  double oldest = 0;
  for (int l = 0; l < n_layers_; ++l) {
    if (state_[l] == State::READY && now - ready_at_[l] > kUrgentAfterMs) state_[l] = State::URGENT;
    if (state_[l] == State::URGENT && (pick < 0 || ready_at_[l] < oldest)) { pick = l; oldest = ready_at_[l]; }
  }
  // 2. ready layers by look-ahead score
  if (pick < 0) {
    float best = 0.f;
    for (int l = 0; l < n_layers_; ++l) {
      if (state_[l] != State::READY) continue;
      const float s = lookahead_score(l, 1, 0);
      if (s > best) { best = s; pick = l; }
    }
  }
  // 3. otherwise the first held layer
  if (pick < 0)
    for (int l = 0; l < n_layers_ && pick < 0; ++l)
      if (state_[l] == State::HOLD) pick = l;
  if (pick < 0) return -1;
  // every other held layer gets one step closer to READY
  for (int l = 0; l < n_layers_; ++l) {
    if (l == pick || state_[l] != State::HOLD) continue;
    if (--hold_left_[l] <= 0) to_ready(l);
  }
  clear(pick);
  state_[pick] = State::IDLE;
  return pick;
}

int GroupLayerScheduler::schedule() {
  int pick = -1;
  float best = 0.f;
  for (int l = 0; l < layers_; ++l)
    for (int g = 0; g < groups_; ++g) {
      const float s = lookahead_score(l, groups_, g);
      // only cells that hold tokens themselves are candidates
      if (tokens_[cell(l, g)] > 0 && s > best) { best = s; pick = cell(l, g); }
    }
  if (pick >= 0) clear(pick);
  return pick;
}

}  // namespace dmoe
