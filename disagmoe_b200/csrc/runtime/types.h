// Wire / data types of the host runtime.
//
// A batch travelling between workers is a [tokens, hidden] tensor plus a Metadata record. Metadata is a small
// header (shape, dtype, layer) and a column-oriented token table: one entry per row in each column. All
// structural operations (slice, gather, concatenate, stable sorts) are written once over the columns.
//
// Layout rules that hold everywhere: rows duplicated for top-k routing are TOKEN-MAJOR (row i*k + j is slot j of
// token i); a prefill contributes one row per prompt token (init_prefill_len = prompt length, position = index
// in the prompt) and a decode step one row (init_prefill_len = -1).
//
// Reference behaviour covered: csrc/include/datatypes.hpp:51-129 (ChannelInfo, TokenMetadata, TokenTopKInfo),
// :135-501 (Metadata), :503-584 (TensorBatch), :590-953 (AttentionBatchMetadata, AttentionBatch), :955-975
// (SloStat, ParallelConfig).
#pragma once
#include <algorithm>
#include <numeric>
#include <tuple>

#include "core.h"

namespace dmoe {

using ExpertId = std::pair<int, int>;  // (layer id, expert id)

constexpr int kTokenizerDevId = 81;
constexpr int kSamplerDevId = 82;
constexpr int kEosTokenId = 2;
inline bool is_embedding_node(int dev) { return dev == kTokenizerDevId || dev == kSamplerDevId; }

struct ChannelInfo {
  std::vector<ExpertId> expert_ids;
  std::vector<int> attn_layer_ids;
  int attn_dp_rank = 0;
  ChannelInfo() = default;
  ChannelInfo(std::vector<ExpertId> e, std::vector<int> a, int dp)
      : expert_ids(std::move(e)), attn_layer_ids(std::move(a)), attn_dp_rank(dp) {}
  bool is_sampler_channel() const { return expert_ids.empty() && attn_layer_ids.empty(); }
  template <class A>
  void io(A& a) { a(expert_ids, attn_layer_ids, attn_dp_rank); }
};

struct TokenMetadata {
  int req_id = 0;
  int exp_id = -1;
  int attn_dp_rank = 0;
  int init_prefill_len = -1;
  float topk_weight = 0.f;
  int position = 0;
  int topk_slot = 0;
};

struct ParallelConfig {
  int tp = 1, ep = 1, dp = 1, n_exp_per_rank = 1;
  std::vector<std::tuple<int, int, int>> expert_ranks;  // (layer, expert, ep rank)
  int rank_of(int layer, int expert) const {
    for (auto& t : expert_ranks)
      if (std::get<0>(t) == layer && std::get<1>(t) == expert) return std::get<2>(t);
    return n_exp_per_rank > 0 ? expert / n_exp_per_rank : 0;
  }
};

// Per-request service-level record. Timestamps are wall-clock microseconds (CPS = 1e6).
struct SloStat {
  int req_id = 0;
  int64_t t_prefill = 0;      // arrival of the first generated token
  int64_t t_prefill_std = 0;  // admission time
  int64_t t_decode = 0;       // completion time
  std::vector<int64_t> t_tokens;  // arrival time of every generated token
  template <class A>
  void io(A& a) { a(req_id, t_prefill, t_prefill_std, t_decode, t_tokens); }
};

struct SamplerStepInfo {
  int num_tokens = 0;
  int64_t time_stamp = 0;
  template <class A>
  void io(A& a) { a(num_tokens, time_stamp); }
};

template <class T>
std::vector<T> slice_vec(const std::vector<T>& v, int l, int r) {
  if (v.empty()) return {};
  if (r < 0) r = static_cast<int>(v.size());
  DMOE_CHECK(0 <= l && l <= r && r <= static_cast<int>(v.size()), "slice [" << l << "," << r << ") of " << v.size());
  return std::vector<T>(v.begin() + l, v.begin() + r);
}
template <class T>
std::vector<T> gather_vec(const std::vector<T>& v, const std::vector<int>& idx) {
  if (v.empty()) return {};
  std::vector<T> out(idx.size());
  for (size_t i = 0; i < idx.size(); ++i) {
    DMOE_CHECK(idx[i] >= 0 && idx[i] < static_cast<int>(v.size()), "gather index " << idx[i]);
    out[i] = v[idx[i]];
  }
  return out;
}
template <class T>
void extend_vec(std::vector<T>& a, const std::vector<T>& b) { a.insert(a.end(), b.begin(), b.end()); }

// Column-oriented per-row token information. A column is either empty (unused) or has one entry per row.
struct TokenTable {
  std::vector<int> req_ids, exp_ids, attn_dp_ranks, init_prefill_lens, positions, topk_slots, token_ids;
  std::vector<float> topk_weights;

  size_t size() const { return req_ids.size(); }
  template <class F>
  void for_each_int(F f) {
    f(req_ids); f(exp_ids); f(attn_dp_ranks); f(init_prefill_lens); f(positions); f(topk_slots); f(token_ids);
  }
  TokenTable slice(int l, int r) const {
    TokenTable t;
    t.req_ids = slice_vec(req_ids, l, r); t.exp_ids = slice_vec(exp_ids, l, r);
    t.attn_dp_ranks = slice_vec(attn_dp_ranks, l, r); t.init_prefill_lens = slice_vec(init_prefill_lens, l, r);
    t.positions = slice_vec(positions, l, r); t.topk_slots = slice_vec(topk_slots, l, r);
    t.token_ids = slice_vec(token_ids, l, r); t.topk_weights = slice_vec(topk_weights, l, r);
    return t;
  }
  // row i of the result = row idx[i] of this
  TokenTable gather(const std::vector<int>& idx) const {
    TokenTable t;
    t.req_ids = gather_vec(req_ids, idx); t.exp_ids = gather_vec(exp_ids, idx);
    t.attn_dp_ranks = gather_vec(attn_dp_ranks, idx); t.init_prefill_lens = gather_vec(init_prefill_lens, idx);
    t.positions = gather_vec(positions, idx); t.topk_slots = gather_vec(topk_slots, idx);
    t.token_ids = gather_vec(token_ids, idx); t.topk_weights = gather_vec(topk_weights, idx);
    return t;
  }
  // Appends `o`; a column missing on one side is padded with `fill` so columns stay row-aligned.
  void append(const TokenTable& o) {
    const size_t n0 = size(), n1 = o.size();
    auto cat_i = [&](std::vector<int>& a, const std::vector<int>& b, int fill) {
      if (a.empty() && b.empty()) return;
      if (a.empty()) a.assign(n0, fill);
      if (b.empty()) a.insert(a.end(), n1, fill); else extend_vec(a, b);
    };
    // req_ids last: it defines size()
    cat_i(exp_ids, o.exp_ids, -1); cat_i(attn_dp_ranks, o.attn_dp_ranks, 0);
    cat_i(init_prefill_lens, o.init_prefill_lens, -1); cat_i(positions, o.positions, 0);
    cat_i(topk_slots, o.topk_slots, 0); cat_i(token_ids, o.token_ids, 0);
    if (!(topk_weights.empty() && o.topk_weights.empty())) {
      if (topk_weights.empty()) topk_weights.assign(n0, 0.f);
      if (o.topk_weights.empty()) topk_weights.insert(topk_weights.end(), n1, 0.f);
      else extend_vec(topk_weights, o.topk_weights);
    }
    extend_vec(req_ids, o.req_ids);
  }
  // Repeats every row k times, token-major; slot column = 0..k-1.
  TokenTable repeat(int k) const {
    std::vector<int> idx(size() * k);
    for (size_t i = 0; i < idx.size(); ++i) idx[i] = static_cast<int>(i / k);
    TokenTable t = gather(idx);
    t.topk_slots.resize(idx.size());
    for (size_t i = 0; i < idx.size(); ++i) t.topk_slots[i] = static_cast<int>(i % k);
    return t;
  }
  TokenMetadata info_at(int i) const {
    TokenMetadata m;
    m.req_id = req_ids[i];
    if (!exp_ids.empty()) m.exp_id = exp_ids[i];
    if (!attn_dp_ranks.empty()) m.attn_dp_rank = attn_dp_ranks[i];
    if (!init_prefill_lens.empty()) m.init_prefill_len = init_prefill_lens[i];
    if (!topk_weights.empty()) m.topk_weight = topk_weights[i];
    if (!positions.empty()) m.position = positions[i];
    if (!topk_slots.empty()) m.topk_slot = topk_slots[i];
    return m;
  }
  template <class A>
  void io(A& a) {
    a(req_ids, exp_ids, attn_dp_ranks, init_prefill_lens, positions, topk_slots, token_ids, topk_weights);
  }
};

struct Metadata;
using metadata_t = std::shared_ptr<Metadata>;

struct Metadata {
  std::vector<int64_t> shape;   // [tokens, hidden]
  std::string dtype = "bf16";   // "bf16" | "fp16" | "fp32"
  int layer_id = 0;
  TokenTable tok;

  // accessors kept for API parity with the reference's flat vectors
  std::vector<int>& req_ids() { return tok.req_ids; }
  std::vector<int>& exp_ids() { return tok.exp_ids; }
  std::vector<int>& attn_dp_ranks() { return tok.attn_dp_ranks; }
  std::vector<int>& init_prefill_lens() { return tok.init_prefill_lens; }
  std::vector<float>& topk_weights() { return tok.topk_weights; }

  size_t num_tokens() const { return shape.empty() ? 0 : static_cast<size_t>(shape[0]); }
  size_t token_hidden_dim() const { return shape.size() > 1 ? static_cast<size_t>(shape[1]) : 0; }
  size_t num_element() const {
    size_t n = 1;
    for (auto s : shape) n *= static_cast<size_t>(s);
    return shape.empty() ? 0 : n;
  }
  size_t element_size() const { return dtype == "fp32" ? 4 : 2; }
  size_t nbytes() const { return num_element() * element_size(); }

  Metadata slice(int l, int r) const {
    Metadata m{shape, dtype, layer_id, tok.slice(l, r)};
    m.shape[0] = r - l;
    return m;
  }
  Metadata at(const std::vector<int>& ids) const {
    Metadata m{shape, dtype, layer_id, tok.gather(ids)};
    m.shape[0] = static_cast<int64_t>(ids.size());
    return m;
  }
  TokenMetadata info_at(int i) const { return tok.info_at(i); }
  void step_layer() { ++layer_id; }

  // Per-expert row counts, experts indexed by GLOBAL id < n_expert.
  std::vector<int> get_expert_batch_sizes(int n_expert) const {
    std::vector<int> c(n_expert, 0);
    for (int e : tok.exp_ids) {
      DMOE_CHECK(e >= 0 && e < n_expert, "expert id " << e);
      ++c[e];
    }
    return c;
  }
  // Row offsets [len(local_experts) + 1] of the given global expert ids in an expert-sorted batch.
  std::vector<int> get_expert_offsets(int n_expert, const std::vector<int>& local_experts) const {
    auto c = get_expert_batch_sizes(n_expert);
    std::vector<int> o(local_experts.size() + 1, 0);
    for (size_t i = 0; i < local_experts.size(); ++i) o[i + 1] = o[i] + c[local_experts[i]];
    return o;
  }

  // Replaces the expert column and/or re-orders the rows: new row mapping[i] = old row i.
  void update_exp_ids(const std::vector<int>& new_exp_ids, const std::vector<int>& mapping) {
    if (!new_exp_ids.empty()) tok.exp_ids = new_exp_ids;
    if (!mapping.empty()) permute_token_infos(mapping);
  }
  void permute_token_infos(const std::vector<int>& mapping) {
    DMOE_CHECK(mapping.size() == tok.size(), "mapping size");
    std::vector<int> inv(mapping.size());
    for (size_t i = 0; i < mapping.size(); ++i) inv[mapping[i]] = static_cast<int>(i);
    tok = tok.gather(inv);
  }
  // Token-major duplication for top-k dispatch; the tensor rows are duplicated the same way by the permute op.
  void duplicate_topk(int k) {
    tok = tok.repeat(k);
    if (!shape.empty()) shape[0] *= k;
  }
  // Inverse bookkeeping after the attention side summed the k partial rows of every token.
  void shrink_topk(int k) {
    DMOE_CHECK(k > 0 && tok.size() % k == 0, "shrink_topk");
    std::vector<int> idx(tok.size() / k);
    for (size_t i = 0; i < idx.size(); ++i) idx[i] = static_cast<int>(i * k);
    tok = tok.gather(idx);
    tok.topk_weights.clear();
    tok.topk_slots.clear();
    if (!shape.empty()) shape[0] /= k;
  }
  // Orders rows by (attention dp rank, prefill before decode, request id, position); returns the mapping
  // old row -> new row, so each attention replica gets one contiguous slice.
  std::vector<int> sort_by_prefill_order() {
    const size_t n = tok.size();
    std::vector<int> order(n);
    std::iota(order.begin(), order.end(), 0);
    auto key = [&](int i) {
      const int dp = tok.attn_dp_ranks.empty() ? 0 : tok.attn_dp_ranks[i];
      const int decode = (tok.init_prefill_lens.empty() || tok.init_prefill_lens[i] < 0) ? 1 : 0;
      const int pos = tok.positions.empty() ? 0 : tok.positions[i];
      const int slot = tok.topk_slots.empty() ? 0 : tok.topk_slots[i];
      return std::make_tuple(dp, decode, tok.req_ids[i], pos, slot);
    };
    std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return key(a) < key(b); });
    std::vector<int> mapping(n);
    for (size_t r = 0; r < n; ++r) mapping[order[r]] = static_cast<int>(r);
    tok = tok.gather(order);
    return mapping;
  }
  // Stable counting sort of several batches by expert id. mapping[i] = destination row of the i-th input row
  // (inputs taken in order of `metas`).
  static metadata_t merge_by_exp_ids(const std::vector<metadata_t>& metas, std::vector<int>& mapping) {
    DMOE_CHECK(!metas.empty(), "merge of nothing");
    auto out = std::make_shared<Metadata>();
    out->shape = metas[0]->shape;
    out->dtype = metas[0]->dtype;
    out->layer_id = metas[0]->layer_id;
    TokenTable all;
    for (auto& m : metas) all.append(m->tok);
    const size_t n = all.size();
    out->shape[0] = static_cast<int64_t>(n);
    std::vector<int> order(n);
    std::iota(order.begin(), order.end(), 0);
    std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return all.exp_ids[a] < all.exp_ids[b]; });
    mapping.assign(n, 0);
    for (size_t r = 0; r < n; ++r) mapping[order[r]] = static_cast<int>(r);
    out->tok = all.gather(order);
    return out;
  }
  static metadata_t concat(const std::vector<metadata_t>& metas) {
    auto out = std::make_shared<Metadata>();
    out->shape = metas[0]->shape;
    out->dtype = metas[0]->dtype;
    out->layer_id = metas[0]->layer_id;
    for (auto& m : metas) out->tok.append(m->tok);
    out->shape[0] = static_cast<int64_t>(out->tok.size());
    return out;
  }
  // Splits into rows [0, p) and [p, n).
  std::pair<metadata_t, metadata_t> split(int p) const {
    return {std::make_shared<Metadata>(slice(0, p)), std::make_shared<Metadata>(slice(p, static_cast<int>(num_tokens())))};
  }
  template <class A>
  void io(A& a) { a(shape, dtype, layer_id, tok); }
  std::string str() const {
    std::ostringstream os;
    os << "Metadata{layer=" << layer_id << ", tokens=" << num_tokens() << ", dtype=" << dtype << "}";
    return os.str();
  }
};

// Batch description on the attention side: prefill rows first (ordered by sequence id, then position), decode rows after.
struct AttentionBatchMetadata;
using attn_metadata_t = std::shared_ptr<AttentionBatchMetadata>;

struct AttentionBatchMetadata {
  int layer_id = 0;
  std::vector<int64_t> shape;
  std::string dtype = "bf16";
  int num_prefill_seqs = 0;
  int num_prefill_tokens = 0;
  int num_decode_tokens = 0;
  std::vector<int> seq_ids;            // per row
  std::vector<int> init_prefill_lens;  // per row (prompt length, -1 for decode rows)
  std::vector<int> positions;          // per row
  std::vector<int> token_ids;          // per row, only for layer-0 input that still has to be embedded
  std::vector<int> expert_ids;         // per row, filled after routing
  std::vector<float> topk_weights;
  std::vector<int> attn_dp_ranks;      // per row

  size_t num_tokens() const { return seq_ids.size(); }

  static attn_metadata_t from_metadata(const Metadata& m) {
    auto a = std::make_shared<AttentionBatchMetadata>();
    a->layer_id = m.layer_id;
    a->shape = m.shape;
    a->dtype = m.dtype;
    a->seq_ids = m.tok.req_ids;
    a->init_prefill_lens = m.tok.init_prefill_lens;
    if (a->init_prefill_lens.empty()) a->init_prefill_lens.assign(a->seq_ids.size(), -1);
    a->positions = m.tok.positions;
    if (a->positions.empty()) a->positions.assign(a->seq_ids.size(), 0);
    a->token_ids = m.tok.token_ids;
    a->attn_dp_ranks = m.tok.attn_dp_ranks;
    if (a->attn_dp_ranks.empty()) a->attn_dp_ranks.assign(a->seq_ids.size(), 0);
    a->recount();
    return a;
  }
  void recount() {
    num_prefill_tokens = num_decode_tokens = num_prefill_seqs = 0;
    int last = -1;
    std::vector<int> seen;
    for (size_t i = 0; i < seq_ids.size(); ++i) {
      if (init_prefill_lens[i] >= 0) {
        ++num_prefill_tokens;
        if (seq_ids[i] != last && std::find(seen.begin(), seen.end(), seq_ids[i]) == seen.end()) {
          seen.push_back(seq_ids[i]);
          ++num_prefill_seqs;
        }
        last = seq_ids[i];
      } else {
        ++num_decode_tokens;
      }
    }
  }
  // Order that puts prefill rows first (by sequence, position) and decode rows after (by sequence).
  std::vector<int> prefill_first_order() const {
    std::vector<int> order(seq_ids.size());
    std::iota(order.begin(), order.end(), 0);
    std::stable_sort(order.begin(), order.end(), [&](int a, int b) {
      const int da = init_prefill_lens[a] < 0, db = init_prefill_lens[b] < 0;
      return std::make_tuple(da, seq_ids[a], positions[a]) < std::make_tuple(db, seq_ids[b], positions[b]);
    });
    return order;
  }
  AttentionBatchMetadata gather(const std::vector<int>& idx) const {
    AttentionBatchMetadata a;
    a.layer_id = layer_id; a.shape = shape; a.dtype = dtype;
    if (!a.shape.empty()) a.shape[0] = static_cast<int64_t>(idx.size());
    a.seq_ids = gather_vec(seq_ids, idx); a.init_prefill_lens = gather_vec(init_prefill_lens, idx);
    a.positions = gather_vec(positions, idx); a.token_ids = gather_vec(token_ids, idx);
    a.expert_ids = gather_vec(expert_ids, idx); a.topk_weights = gather_vec(topk_weights, idx);
    a.attn_dp_ranks = gather_vec(attn_dp_ranks, idx);
    a.recount();
    return a;
  }
  static attn_metadata_t merge(const std::vector<attn_metadata_t>& batches, std::vector<int>& order) {
    auto all = std::make_shared<AttentionBatchMetadata>();
    DMOE_CHECK(!batches.empty(), "merge of nothing");
    all->layer_id = batches[0]->layer_id; all->shape = batches[0]->shape; all->dtype = batches[0]->dtype;
    for (auto& b : batches) {
      extend_vec(all->seq_ids, b->seq_ids); extend_vec(all->init_prefill_lens, b->init_prefill_lens);
      extend_vec(all->positions, b->positions); extend_vec(all->attn_dp_ranks, b->attn_dp_ranks);
      extend_vec(all->token_ids, b->token_ids);
    }
    if (all->token_ids.size() != all->seq_ids.size()) all->token_ids.clear();
    order = all->prefill_first_order();
    auto out = std::make_shared<AttentionBatchMetadata>(all->gather(order));
    return out;
  }
  // The Metadata that leaves the attention worker (one row per token, before top-k duplication).
  metadata_t to_metadata() const {
    auto m = std::make_shared<Metadata>();
    m->shape = shape; m->dtype = dtype; m->layer_id = layer_id;
    m->tok.req_ids = seq_ids; m->tok.init_prefill_lens = init_prefill_lens; m->tok.positions = positions;
    m->tok.attn_dp_ranks = attn_dp_ranks; m->tok.exp_ids = expert_ids; m->tok.topk_weights = topk_weights;
    if (m->tok.exp_ids.empty()) m->tok.exp_ids.assign(seq_ids.size(), -1);
    return m;
  }
  template <class A>
  void io(A& a) {
    a(layer_id, shape, dtype, num_prefill_seqs, num_prefill_tokens, num_decode_tokens, seq_ids, init_prefill_lens,
      positions, token_ids, expert_ids, topk_weights, attn_dp_ranks);
  }
};

}  // namespace dmoe
