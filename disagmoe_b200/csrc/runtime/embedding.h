// The two CPU "embedding nodes" that close the autoregressive loop.
//
//   Tokenizer   injects a request: one row per prompt token (token id, position) goes to the layer-0 attention
//               worker of the request's DP replica, where the embedding lookup happens on the GPU.
//   Sampler     receives the greedy token id the LM-head step produced for every sequence, keeps per-request output
//               lengths, output tokens and SLO timestamps, decides finish (EOS or the request's output length) and
//               sends every continuing token back to layer 0 as a decode token.
//   TopKSampler same bookkeeping for workers that deliver k partial results per token: a token counts once all k
//               have arrived.
//
// Reference behaviour covered: csrc/include/embedding.h, csrc/muhelper/embedding.cpp:48-356 (the reference's
// tokenizer sends random hidden vectors and its sampler returns a constant token; here real ids travel).
#pragma once
#include <random>

#include "muhelper.h"

namespace dmoe {

class Tokenizer : public MuDispatcher {
 public:
  // attn_peer[dp rank] -> device of the layer-0 attention worker
  Tokenizer(int device_id, std::vector<Endpoint> endpoints, std::map<int, int> attn_peer);
  void put_request(int req_id, const std::vector<int>& prompt_ids, int dp_rank);

 protected:
  const char* name() const override { return "tokenizer"; }
  void send_once(const TensorBatch& batch, int kind) override;

 private:
  std::map<int, int> attn_peer_;
};

class Sampler : public MuDispatcher {
 public:
  Sampler(int device_id, std::vector<Endpoint> endpoints, std::map<int, int> attn_peer, int min_output_len,
          int max_output_len, bool ignore_eos = true, unsigned seed = 0);
  void start_all();   // receive loop + send loop
  void stop_all();
  // Fixes the number of tokens to generate for one request (otherwise uniform in [min, max)).
  void set_request_output_len(int req_id, int n);
  int process_batch(const Metadata& meta);
  std::vector<SloStat> fetch_finished_slo_stats();
  std::vector<SamplerStepInfo> fetch_step_infos();
  std::map<int, SloStat> wait_slo_stats(int n_request);
  std::vector<int> get_output_tokens(int req_id);
  int num_finished();
  void reset();

 protected:
  const char* name() const override { return "sampler"; }
  void send_once(const TensorBatch& batch, int kind) override;
  virtual bool token_arrived(int req_id, int position) { (void)req_id; (void)position; return true; }
  bool check_finished(int token, int req_id);
  void recv_loop();

  std::map<int, int> attn_peer_;
  int min_len_, max_len_;
  bool ignore_eos_;
  std::mt19937 rng_;
  PullSocket mailbox_;
  SeqFilter seq_filter_;
  std::thread recv_thread_;
  std::mutex result_mu_;
  std::map<int, int> output_lens_, required_lens_;
  std::map<int, std::vector<int>> outputs_;
  std::map<int, SloStat> slo_stats_;
  std::set<int> finished_;
  std::map<int, SloStat> finished_stats_;
  std::vector<SamplerStepInfo> step_infos_;
};

class TopKSampler : public Sampler {
 public:
  TopKSampler(int device_id, std::vector<Endpoint> endpoints, std::map<int, int> attn_peer, int min_output_len,
              int max_output_len, int top_k, bool ignore_eos = true)
      : Sampler(device_id, std::move(endpoints), std::move(attn_peer), min_output_len, max_output_len, ignore_eos),
        top_k_(top_k) {}

 protected:
  bool token_arrived(int req_id, int position) override {
    return ++arrivals_[{req_id, position}] >= top_k_ ? (arrivals_.erase({req_id, position}), true) : false;
  }

 private:
  int top_k_;
  std::map<std::pair<int, int>, int> arrivals_;
};

}  // namespace dmoe
