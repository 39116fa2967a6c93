// C ABI of libdmoe_kernels.so: hand-written sm_100a kernels of the serving engine.
// Every function takes raw device pointers and a CUDA stream handle and returns 0 on success, a positive
// cudaError_t, or a negative argument error. Nothing here allocates device memory unless it says so.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// ---- GEMM (gemm.cu) -------------------------------------------------------------------------------
// Y[t, f] = sum_k X[t, k] * W[g][f, k] for t in group g. bf16 inputs, fp32 accumulation.
enum { DMOE_EPI_PLAIN = 0, DMOE_EPI_SWIGLU = 1, DMOE_EPI_COMBINE = 2 };

typedef struct DmoeGemm {
  const void* W;      // [G, rows, K] bf16; rows = F (plain / combine) or 2F (SwiGLU: gate rows then up rows)
  const void* X;      // [T, K] bf16, row stride ldx (0 = K)
  void* Y;            // [T, F] bf16 (or fp32 when y_f32), row stride ldy; unused for combine
  const void* R;      // optional residual [T, F] bf16, row stride ldr (plain epilogue only)
  const int* offs;    // [G+1] device token offsets of the groups, or NULL for one dense group
  const void* recs;   // combine: [T] int4 {dst_rank, dst_row (<0 = drop), weight as fp32 bits, 0}
  const void* bases;  // combine: device array of destination base pointers (bf16 rows of stride ldy), one per rank
  void* ws;           // split-K workspace (fp32), ws_bytes >= dmoe_gemm_workspace_bytes(...)
  int* counters;      // split-K tile counters, zero-initialised once; the kernel leaves them zero
  int* status;        // optional device status word (0 = ok)
  // --- multi-GPU fusion (all optional, zero / NULL when unused) ---
  const int* seg_cnt;   // [S, G] rows that source s delivered for group g; region s = rows [s*seg_cap, (s+1)*seg_cap)
  const int* wait_flags;  // [n_wait] arrival flags written by peers; the kernel waits for *wait_epoch + 1
  int* wait_epoch;
  const void* signal_ptrs;  // device array of n_signal flag-array pointers (peer memory); slot signal_slot is written
  int* signal_epoch;
  int* done_ticket;     // one zero-initialised int of scratch (required with wait_flags or signal_ptrs)
  long long ldx, ldy, ldr, ws_bytes;
  int S, seg_cap, n_wait, n_signal, signal_slot;
  int group_regions;    // 1: group g owns rows [g*seg_cap, (g+1)*seg_cap) and seg_cnt[g] is its row count (S unused)
  int clear_n;          // the last CTA zeroes clear_ptr[0..clear_n) before it signals (the dispatch cursors)
  int* clear_ptr;
  int fanout;           // combine: every row is stored to the `fanout` consecutive ranks of the sender's TP group (0/1 = one)
  int G, T, F, K;
  int epi;            // DMOE_EPI_*
  int bn;             // token tile: 32/64/128/256, 0 = pick from T/G
  int splitk;         // >= 1; > 1 only for dense plain / combine GEMMs
  int y_f32;
  // --- tensor-parallel attention fusion (plain epilogue with 16-byte aligned Y; all optional) ---
  // all-gather prologue: rows [s * shard_rows, (s + 1) * shard_rows) of X are pushed by peer s, which then sets
  // wait_flags[s]; a token tile is fetched as soon as the shards it covers have landed (n_wait = number of shards)
  int shard_rows;
  // reduce-scatter epilogue: row t is stored to row rs_slot * rs_cap + t % rs_rows of buffer rs_bases[t / rs_rows]
  // (device array of peer pointers, row stride ldy) instead of Y
  const void* rs_bases;
  int rs_rows, rs_slot, rs_cap;
  // QKV epilogue: neox RoPE on the n_q + n_kv leading heads of head size hd (64 / 128) from rope_table
  // ([rope_max_pos][hd / 2] float2 = (cos, sin), see dmoe_rope_table), K / V rows appended to the paged caches
  // ([blocks, block_size, n_kv, hd]) at slots[t] (< 0: skip); only the q columns are written to Y. F = (n_q + 2 n_kv) hd.
  const void* rope_table;
  const int* positions;
  const long long* slots;
  void* kcache;
  void* vcache;
  int n_q, n_kv, hd, rope_max_pos;
  // --- work distribution ---
  // streamk != 0 (with splitk <= 1, ws and counters given): the K-block iterations of all tiles are dealt out in one
  // equal contiguous share per CTA instead of whole tiles, so no SM idles in a last partial wave; tiles that straddle
  // a share boundary are reduced through ws (2 slots of 128 x bn fp32 per accumulator and CTA). n_counters: ints
  // available at `counters` (0 = 4096); one per tile is needed.
  int streamk, n_counters;
  // pair != 0: clusters of two CTAs compute tiles of 256 weight rows x bn tokens with tcgen05.mma.cta_group::2 (each
  // CTA stages its 128 weight rows and half of the token tile). bn = 128 or 256 (SwiGLU too), whole tiles only.
  int pair;
  // combine epilogue: != 0 states that every destination base in `bases` is 16-byte aligned (with F and ldy multiples
  // of 8 the rows then move as 16-byte segments); 0 keeps 2-byte stores
  int combine_vec;
  // != 0: W is stored tile by tile, [group][128-row tile][K / 64][128][64] (see ops/gemm.py: block_weight), so that
  // every 16 KB box the kernel fetches is one contiguous run of HBM; needs F % 128 == 0 and K % 64 == 0
  int w_blocked;
  // profiling aid, normally null: 16 x uint64 of device memory that CTA 0 fills with %globaltimer stamps (entry, set-up
  // done, first TMA issued, first stage landed, last MMA committed, accumulator seen by the epilogue, epilogue done,
  // tear-down reached, then five points inside the first epilogue chunk and three inside the producer's start)
  void* trace;
} DmoeGemm;

int dmoe_gemm(const DmoeGemm* desc, void* stream);
int dmoe_gemm_pick_bn(int tokens_per_group_hint, int epi);
long long dmoe_gemm_workspace_bytes(int T, int F, int bn, int splitk);

// ---- row kernels (elementwise.cu) -------------------------------------------------------------------
// resid_out = resid_in + sum of n_add partial rows; y = rmsnorm(resid_out) * w. resid_in / resid_out / y may be NULL.
int dmoe_add_rmsnorm(const void* resid_in, const void* add, int n_add, long long add_row_stride,
                     long long add_part_stride, const void* w, float eps, void* resid_out, void* y, int T, int H,
                     long long ld_in, long long ld_out, long long ld_y, void* stream);
// neox RoPE on the q and k heads of qkv rows [q | k | v] in place, then K/V append at slots[t] (slot < 0: no append).
int dmoe_rope_kv_append(void* qkv, long long ld, const int* positions, const long long* slots, void* kcache,
                        void* vcache, int T, int n_q, int n_kv, int hd, float theta, void* stream);
// (cos, sin) of pos * theta^(-2 d / hd) for pos < max_pos, d < hd / 2: the table the QKV epilogue rotates with.
int dmoe_rope_table(void* table, int max_pos, int hd, float theta, void* stream);
int dmoe_embed(const int* ids, const void* table, void* out, int T, int H, int vocab, long long ld_out, void* stream);
int dmoe_argmax(const void* logits, int is_f32, long long ld, int T, int V, int* ids, void* stream);
int dmoe_permute_rows(const void* src, long long ld_src, void* dst, long long ld_dst, const int* map, int n, int H,
                      int repeat, int gather, void* stream);
int dmoe_gather_ptrs(const void* ptrs, void* dst, long long ld_dst, int n, int H, void* stream);
// Debug kernel of the launch / overlap tests: out[i] = in[i] + 1 (fp32).
int dmoe_add_one(const float* in, float* out, long long n, void* stream);

// ---- attention (attention.cu) -----------------------------------------------------------------------
long long dmoe_paged_attention_workspace_floats(int T, int n_q, int hd, int splits);
int dmoe_paged_attention(const void* q, long long ld_q, const void* kcache, const void* vcache,
                         const int* block_tables, int max_blocks, const int* bt_row, const int* ctx_len, int block_size,
                         int T, int n_q, int n_kv, int hd, float scale, int splits, void* out, long long ld_out,
                         float* workspace, void* stream);

// Tiled causal attention for prompt tokens: CTA column i handles tiles[i] = int4 {first row in q / out, tokens
// (<= dmoe_prefill_tile_tokens), block-table row, position of the first token}; the tokens of a tile are consecutive
// rows at consecutive positions of one sequence, whose K / V (own tokens included) are already in the paged cache.
int dmoe_prefill_tile_tokens(int n_q, int n_kv);
int dmoe_prefill_attention(const void* q, long long ld_q, const void* kcache, const void* vcache,
                           const int* block_tables, int max_blocks, const void* tiles, int n_tiles, int block_size,
                           int n_q, int n_kv, int hd, float scale, void* out, long long ld_out, void* stream);

// ---- routing (moe.cu) -------------------------------------------------------------------------------
// (RMSNorm ->) gate -> softmax -> top-k (-> renormalise); counts[e] += tokens routed to e (may be NULL).
int dmoe_route(const void* x, long long ld_x, const void* norm_w, float eps, const void* gate_w, int T, int H, int E,
               int K, int renorm, void* y, long long ld_y, int* topk_ids, float* topk_w, float* logits_out, int* counts,
               const float* logit_bias, void* stream);
int dmoe_route_ex(const void* x, long long ld_x, const void* norm_w, float eps, const void* gate_w, int T, int H, int E,
                  int K, int renorm, void* y, long long ld_y, int* topk_ids, float* topk_w, int* counts,
                  const void* add_ptrs, int n_add, long long ld_add, void* resid_out, long long ld_resid, int count_lo,
                  int count_hi, const float* logit_bias, void* stream);
// Sort-by-expert copy of the routed rows plus their 16-byte records; ws = ints [counts E | cursor E | ticket].
int dmoe_dispatch_local(const void* y, long long ld_y, const int* topk_ids, const float* topk_w, int T, int K, int H,
                        int E, int experts_per_rank, int my_rank, int* ws, int* offs, const void* x_bases,
                        long long ld_dst, const void* rec_bases, int dst_capacity, int* status, void* stream);

// ---- peer-memory dispatch (comm.cu) -----------------------------------------------------------------
// Stores every routed (token, k) row of this attention rank into its region on the expert GPU that owns the
// expert ([experts_per_rank, region_cap] rows per destination), with 16-byte records and a release flag (*epoch + 1);
// row blocks are reserved on the destinations' per-expert cursors (cnt_bases) with system-scope atomics. x_bases /
// rec_bases / cnt_bases / flag_bases are device arrays of n_dst peer pointers. ws = ints [counts E | cursor E |
// ticket, 7 pad | row_base E], counts filled by dmoe_route; cleared for the next launch.
int dmoe_dispatch_remote(const void* y, long long ld_y, const int* topk_ids, const float* topk_w, int T, int K, int H,
                         int E, int experts_per_rank, int n_dst, int my_rank, int region_cap, int* ws,
                         const void* x_bases, long long ld_dst, const void* rec_bases, const void* cnt_bases,
                         const void* flag_bases, int* epoch, int* status, int tok_lo, int tok_hi, void* stream);
// ---- fused attention-side senders (sender.cu) --------------------------------------------------------
// [wait] resid_out = resid_in + sum of n_add partial rows; y = rmsnorm(resid_out) * w is stored to row dst_row0 + t of
// EVERY buffer in dst_ptrs (device array of n_dst pointers: this GPU's and, for a tensor-parallel group, its peers'
// QKV staging buffers); then slot signal_slot of every flag array in signal_ptrs gets *signal_epoch + 1.
// The wait (flags[i] >= *wait_epoch + 1 for i < n_wait, bounded) runs inside the kernel. ticket: one zeroed int.
typedef struct DmoeNormGather {
  const void* resid_in; const void* add; const void* w; void* resid_out; const void* dst_ptrs;
  const int* wait_flags; int* wait_epoch; const void* signal_ptrs; int* signal_epoch; int* ticket; int* status;
  long long ld_in, add_row_stride, add_part_stride, ld_out, dst_row0, ld_dst;
  float eps;
  int n_add, n_dst, T, H, n_wait, n_signal, signal_slot;
} DmoeNormGather;
int dmoe_norm_gather(const DmoeNormGather* desc, void* stream);

// [wait] resid += sum of the n_add partial-row slots (add + s * add_slot_stride, row stride ld_add); y = rmsnorm(resid);
// gate -> softmax -> top-k; every (token, k) pair reserves a row in its expert's region on the owning GPU (atomic on
// cnt_bases[dst][local expert]) and stores row + record there; the last CTA sets flag_bases[d][my_rank] = *disp_epoch + 1
// for every d. gate_w == NULL: reduction and normalisation only. x_bases == NULL: route without dispatching.
typedef struct DmoeRouteDispatch {
  void* resid; const void* add; const void* norm_w; const void* gate_w; const float* logit_bias; void* y;
  int* topk_ids; float* topk_w; const void* x_bases; const void* rec_bases; const void* cnt_bases;
  const void* flag_bases; int* disp_epoch; const int* wait_flags; int* wait_epoch; int* ticket; int* status;
  long long ld_resid, add_slot_stride, ld_add, ld_y, ld_dst;
  float eps;
  int n_add, T, H, E, K, renorm, experts_per_rank, n_dst, my_rank, region_cap, n_wait;
  // rank written into the records as the owner the experts return the rows to, where that is not the sender itself
  // (pipeline-parallel attention: the stage that owns the next layer); 0 with ret_rank_set == 0 means my_rank
  int ret_rank, ret_rank_set;
} DmoeRouteDispatch;
int dmoe_route_dispatch(const DmoeRouteDispatch* desc, void* stream);
// dst_ptrs[d][dst0 + i] = src[i] (i < n) for every d < n_dst, then signal_ptrs[d][signal_slot] = *signal_epoch + 1.
int dmoe_ids_gather(const int* src, int n, const void* dst_ptrs, int n_dst, int dst0, const void* signal_ptrs,
                    int signal_slot, int* signal_epoch, void* stream);

// Waits (bounded) until flags[i] >= *epoch + 1 for i < n, then advances *epoch.
int dmoe_wait_flags(const int* flags, int n, int* epoch, int* status, void* stream);
// Cycle budget of every peer-flag wait in kernels launched from now on (<= 0: the default, about 4 s).
void dmoe_set_flag_wait_cycles(long long cycles);
int dmoe_enable_peer_access(int peer_device);
// Peer arena: a zeroed cudaMalloc block + its 64-byte CUDA IPC handle; dmoe_peer_open maps a peer's block into
// this process for kernels of the CURRENT device (peer access is enabled lazily by the driver).
int dmoe_peer_alloc(long long nbytes, void** ptr, void* handle64);
int dmoe_peer_open(const void* handle64, void** ptr);
int dmoe_peer_close(void* ptr);
int dmoe_peer_free(void* ptr);

#ifdef __cplusplus
}
#endif
