// Paged attention for sm_100a: one kernel serves decode tokens and prefill tokens.
//
// Every query token t attends to the first ctx_len[t] tokens of the paged KV cache of its sequence
// (block table row bt_row[t]); a decode token has ctx_len = sequence length, prompt token i of a prefill has
// ctx_len = i + 1 (causal), its K/V having been appended to the cache by rope_kv_append before this kernel runs.
// So mixed prefill + decode batches need no second code path.
//
// The work of one CTA is (token, kv head, kv split): the GQ query heads that share the kv head are processed
// together, so every K/V byte is read once per group. It is a bandwidth problem (256 B of K and of V per
// cached token and kv head), so the kernel is built around wide loads kept in flight rather than around
// CUDA-core FLOPs: K/V rows stream through per-warp cp.async rings in shared memory and the GQ x 16-token score and
// output tiles run on the tensor cores (mma.sync m16n8k16: the group is far too small for a tcgen05 tile); softmax is online (base 2); the 16 (warp, lane-group) partial states are merged through
// shared memory. With splits > 1 ("flash decoding") partial outputs + log-sum-exp go to a workspace and a
// second kernel merges them.
//
// Cache layout: K and V each [num_blocks, block_size, kv_heads, head_dim] bf16.
// Reference behaviour covered: vLLM paged attention / flash_attn_with_kvcache reached from
// disagmoe/models/attention.py:150-155,219 with metadata built at disagmoe/frontend/engine.py:429-485.
#include "dmoe_kernels.h"
#include "sm100.cuh"

namespace dmoe {

constexpr int kAttnThreads = 128;
constexpr int kAttnParts = 16;  // 4 warps x 4 lane groups

struct alignas(16) bf16x8a {
  __nv_bfloat162 v[4];
};

__device__ __forceinline__ void cvt8(const bf16x8a& p, float* f) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(p.v[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  // src-size 0 zero-fills the 16 destination bytes (rows past the end of the context)
  const int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz) : "memory");
}
// The decode kernel reads every K / V byte once per step: an evict-first L2 policy keeps that stream from pushing the
// small hot tensors of the neighbouring kernels (residual rows, norm and gate weights, staged activations) out of L2.
__device__ __forceinline__ uint64_t l2_stream_policy() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ void cp_async16_stream(uint32_t dst, const void* src, bool valid, uint64_t policy) {
  const int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global.L2::cache_hint [%0], [%1], 16, %2, %3;" ::"r"(dst), "l"(src), "r"(sz), "l"(policy)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
// D (16x8 fp32) += A (16x16 bf16, row) * B (16x8 bf16, col)
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

constexpr int kAttnStages = 3;     // cp.async ring depth, per warp
constexpr int kAttnStageTok = 16;  // cached tokens per stage and warp (block_size must be a multiple of it)
constexpr int kAttnWarps = kAttnThreads / 32;

// Tensor-core formulation: the GQ query heads of one kv head are the (zero padded) 16 rows of an m16n8k16 tile.
// Each warp owns every 4th chunk of 16 cached tokens and streams them through its private cp.async ring
// (swizzled so that ldmatrix is bank-conflict free): S = Q K^T (2 n-tiles), online softmax on the accumulator
// fragments, P re-used in place as the A operand of O += P V (V read with ldmatrix.trans).
template <int HD, int GQ>
__global__ void __launch_bounds__(kAttnThreads)
paged_attn_kernel(const __nv_bfloat16* __restrict__ q, long long ld_q, const __nv_bfloat16* __restrict__ kcache,
                  const __nv_bfloat16* __restrict__ vcache, const int* __restrict__ block_tables, int max_blocks,
                  const int* __restrict__ bt_row, const int* __restrict__ ctx_len, int block_size, int n_kv,
                  float scale_log2, int splits, __nv_bfloat16* __restrict__ out, long long ld_out,
                  float* __restrict__ part_o, float* __restrict__ part_lse) {
  static_assert(GQ <= 8, "the query group must fit the first 8 rows of the MMA tile");
  constexpr int ROWB = HD * 2;                       // bytes of one cached row of one kv head
  constexpr int NCH = HD / 8;                        // 16-byte chunks per row
  constexpr int TILEB = kAttnStageTok * ROWB;        // K (or V) tile of one stage
  constexpr int STAGEB = 2 * TILEB;
  constexpr int WARPB = kAttnStages * STAGEB;
  constexpr int CPL = kAttnStageTok * NCH / 32;      // 16-byte copies per lane per tile
  constexpr int KS = HD / 16;                        // k-steps of Q K^T
  constexpr int NT = HD / 8;                         // n-tiles of the output
  __shared__ float s_m[kAttnWarps][8];
  __shared__ float s_l[kAttnWarps][8];
  extern __shared__ __align__(128) uint8_t s_dyn[];  // per-warp rings; reused as [warps][GQ][HD] floats at the end

  pdl_trigger();
  pdl_wait();      // q, the new K / V rows and the sequence tables come from the kernels before this one
  const int t = blockIdx.x, hkv = blockIdx.y, split = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, tq = lane & 3;            // accumulator row / column-pair of this lane
  const int n_q = n_kv * GQ;

  const int len = ctx_len[t];
  const int row = bt_row != nullptr ? bt_row[t] : t;
  const int* bt = block_tables + static_cast<long long>(row) * max_blocks;
  const int nblk = (len + block_size - 1) / block_size;
  const int blk_per = (nblk + splits - 1) / splits;
  const int c0 = min(len, split * blk_per * block_size);
  const int c1 = min(len, (split + 1) * blk_per * block_size);
  const int nchunk = (c1 - c0 + kAttnStageTok - 1) / kAttnStageTok;
  const int my_chunks = nchunk > warp ? (nchunk - warp + kAttnWarps - 1) / kAttnWarps : 0;
  const long long tok_stride = static_cast<long long>(n_kv) * HD;
  const uint32_t ring = smem_u32(s_dyn) + warp * WARPB;
  const uint64_t stream_policy = l2_stream_policy();

  auto issue = [&](int j) {
    if (j < my_chunks) {
      const int tok0 = c0 + (warp + j * kAttnWarps) * kAttnStageTok;
      const long long blk = bt[tok0 / block_size];
      const long long slot0 = blk * block_size + tok0 % block_size;
      const uint32_t dst0 = ring + (j % kAttnStages) * STAGEB;
#pragma unroll
      for (int i = 0; i < CPL; ++i) {
        const int id = lane + i * 32;
        const int r = id / NCH, c = id % NCH;
        const bool valid = tok0 + r < c1;
        const long long off = valid ? (slot0 + r) * tok_stride + hkv * HD + c * 8 : 0;
        const uint32_t d = dst0 + r * ROWB + ((c ^ (r & 7)) << 4);
        cp_async16_stream(d, kcache + off, valid, stream_policy);
        cp_async16_stream(d + TILEB, vcache + off, valid, stream_policy);
      }
    }
    cp_async_commit();
  };
#pragma unroll
  for (int j = 0; j < kAttnStages - 1; ++j) issue(j);

  // Q fragments (rows >= GQ are zero)
  uint32_t qa[KS][4];
  {
    const __nv_bfloat16* qp = q + static_cast<long long>(t) * ld_q + (hkv * GQ + g) * HD;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      qa[ks][0] = g < GQ ? *reinterpret_cast<const uint32_t*>(qp + ks * 16 + 2 * tq) : 0u;
      qa[ks][2] = g < GQ ? *reinterpret_cast<const uint32_t*>(qp + ks * 16 + 8 + 2 * tq) : 0u;
      qa[ks][1] = 0u;
      qa[ks][3] = 0u;
    }
  }
  float o[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  float m = -INFINITY, l = 0.f;

  // ldmatrix lane roles
  const int lm_mi = lane >> 3, lm_r = lane & 7;
  for (int j = 0; j < my_chunks; ++j) {
    issue(j + kAttnStages - 1);
    cp_async_wait<kAttnStages - 1>();
    __syncwarp();
    const uint32_t kb = ring + (j % kAttnStages) * STAGEB;
    const uint32_t vb = kb + TILEB;
    const int tok0 = c0 + (warp + j * kAttnWarps) * kAttnStageTok;
    float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
    {
      const int r = (lm_mi >> 1) * 8 + lm_r;          // token row this lane addresses
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        const int c = 2 * ks + (lm_mi & 1);
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4(kb + r * ROWB + ((c ^ (r & 7)) << 4), b0, b1, b2, b3);
        mma_bf16_16816(s0, qa[ks], b0, b1);
        mma_bf16_16816(s1, qa[ks], b2, b3);
      }
    }
    // row g: tokens tok0 + 2 tq + {0, 1} (s0) and tok0 + 8 + 2 tq + {0, 1} (s1)
    const int tk = tok0 + 2 * tq;
    float p00 = tk < c1 ? s0[0] * scale_log2 : -INFINITY;
    float p01 = tk + 1 < c1 ? s0[1] * scale_log2 : -INFINITY;
    float p10 = tk + 8 < c1 ? s1[0] * scale_log2 : -INFINITY;
    float p11 = tk + 9 < c1 ? s1[1] * scale_log2 : -INFINITY;
    float mx = fmaxf(fmaxf(p00, p01), fmaxf(p10, p11));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float mn = fmaxf(m, mx);                     // finite: token tok0 itself is always valid
    const float corr = exp2f(m - mn);
    p00 = exp2f(p00 - mn); p01 = exp2f(p01 - mn); p10 = exp2f(p10 - mn); p11 = exp2f(p11 - mn);
    float ls = p00 + p01 + p10 + p11;
    ls += __shfl_xor_sync(0xffffffffu, ls, 1);
    ls += __shfl_xor_sync(0xffffffffu, ls, 2);
    l = l * corr + ls;
    m = mn;
#pragma unroll
    for (int i = 0; i < NT; ++i) { o[i][0] *= corr; o[i][1] *= corr; }
    uint32_t pa[4] = {pack_bf16(p00, p01), 0u, pack_bf16(p10, p11), 0u};
    {
      const int r = (lm_mi & 1) * 8 + lm_r;
#pragma unroll
      for (int dp = 0; dp < NT / 2; ++dp) {
        const int c = 2 * dp + (lm_mi >> 1);
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4_trans(vb + r * ROWB + ((c ^ (r & 7)) << 4), b0, b1, b2, b3);
        mma_bf16_16816(o[2 * dp], pa, b0, b1);
        mma_bf16_16816(o[2 * dp + 1], pa, b2, b3);
      }
    }
    __syncwarp();   // every lane is done with this ring slot before it is refilled
  }
  cp_async_wait<0>();
  __syncthreads();

  // merge the warps' partial states
  float* s_acc = reinterpret_cast<float*>(s_dyn);   // [warps][GQ][HD]
  if (g < GQ) {
    if (tq == 0) { s_m[warp][g] = m; s_l[warp][g] = l; }
#pragma unroll
    for (int i = 0; i < NT; ++i) {
      s_acc[(warp * GQ + g) * HD + i * 8 + 2 * tq] = o[i][0];
      s_acc[(warp * GQ + g) * HD + i * 8 + 2 * tq + 1] = o[i][1];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < GQ * HD; idx += kAttnThreads) {
    const int gg = idx / HD, d = idx % HD;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) M = fmaxf(M, s_m[w][gg]);
    float L = 0.f, O = 0.f;
    if (M > -INFINITY) {
#pragma unroll
      for (int w = 0; w < kAttnWarps; ++w) {
        const float wgt = exp2f(s_m[w][gg] - M);
        L += s_l[w][gg] * wgt;
        O += s_acc[(w * GQ + gg) * HD + d] * wgt;
      }
    }
    const float val = L > 0.f ? O / L : 0.f;
    const int head = hkv * GQ + gg;
    if (splits == 1) {
      out[static_cast<long long>(t) * ld_out + head * HD + d] = __float2bfloat16(val);
    } else {
      const long long pi = (static_cast<long long>(t) * n_q + head) * splits + split;
      part_o[pi * HD + d] = val;
      if (d == 0) part_lse[pi] = L > 0.f ? M + log2f(L) : -INFINITY;
    }
  }
}

// out[t, head] = sum_s softmax_s(lse) * part_o[t, head, s]
template <int HD>
__global__ void attn_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_lse, int splits,
                                  int n_q, __nv_bfloat16* __restrict__ out, long long ld_out) {
  const int t = blockIdx.x, head = blockIdx.y, d = threadIdx.x;
  const long long pi = (static_cast<long long>(t) * n_q + head) * splits;
  float M = -INFINITY;
  for (int s = 0; s < splits; ++s) M = fmaxf(M, part_lse[pi + s]);
  float L = 0.f, O = 0.f;
  if (M > -INFINITY) {
    for (int s = 0; s < splits; ++s) {
      const float w = exp2f(part_lse[pi + s] - M);
      L += w;
      O += w * part_o[(pi + s) * HD + d];
    }
  }
  out[static_cast<long long>(t) * ld_out + head * HD + d] = __float2bfloat16(L > 0.f ? O / L : 0.f);
}

// ---------------------------------------------------------------------------------------------------------------
// Tiled causal attention for prompt tokens (prefill, whole prompts or chunks of them).
//
// The per-token kernel above streams a prompt row's whole prefix for every row: O(n^2) K/V bytes per prompt with no
// reuse. Here a CTA owns a tile of 64 query rows = (64 / GQ consecutive prompt tokens) x (the GQ query heads of one kv
// head) and streams the sequence's K/V pages ONCE for the tile, 64 keys at a time, through a double-buffered
// cp.async ring shared by its four warps; each warp holds 16 query rows as mma.sync A fragments, computes S = Q K^T
// for the 64 keys, applies the causal mask (key position <= query position; the chunk's own K/V are already in the
// cache), runs the online softmax on the accumulator fragments and reuses P in registers as the A operand of O += P V.
// A chunk that continues a prompt attends to the cached prefix and to itself, so chunked prefill needs nothing else.
//
// tiles: one int4 per CTA column = {first row of the tile in q / out, tokens in the tile (<= 64 / GQ), block-table
// row of the sequence, position of the tile's first token}.
constexpr int kPreKeys = 64;       // keys per pipeline stage
constexpr int kPreRows = 64;       // query rows per CTA (4 warps x 16)

template <int HD, int GQ>
__global__ void __launch_bounds__(128)
prefill_attn_kernel(const __nv_bfloat16* __restrict__ q, long long ld_q, const __nv_bfloat16* __restrict__ kcache,
                    const __nv_bfloat16* __restrict__ vcache, const int* __restrict__ block_tables, int max_blocks,
                    const int4* __restrict__ tiles, int block_size, int n_kv, float scale_log2,
                    __nv_bfloat16* __restrict__ out, long long ld_out) {
  constexpr int ROWB = HD * 2;
  constexpr int NCH = HD / 8;                       // 16-byte chunks per K / V row
  constexpr int TILEB = kPreKeys * ROWB;
  constexpr int STAGEB = 2 * TILEB;                 // K tile then V tile
  constexpr int CPT = kPreKeys * NCH / 128;         // 16-byte copies per thread per tile
  constexpr int KS = HD / 16;                       // k-steps of Q K^T
  constexpr int NT = HD / 8;                        // n-tiles of the output
  extern __shared__ __align__(128) uint8_t s_pre[];

  const int4 tile = tiles[blockIdx.x];
  const int row0 = tile.x, ntok = tile.y, pos0 = tile.w;
  const int hkv = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, tq = lane & 3;
  const int* bt = block_tables + static_cast<long long>(tile.z) * max_blocks;
  const int kmax = pos0 + ntok;                     // keys [0, kmax) exist for the last token of the tile
  const int nkb = (kmax + kPreKeys - 1) / kPreKeys;
  const long long tok_stride = static_cast<long long>(n_kv) * HD;
  const uint32_t sbase = smem_u32(s_pre);

  auto issue = [&](int kb) {
    if (kb < nkb) {
      const uint32_t dst0 = sbase + (kb & 1) * STAGEB;
#pragma unroll
      for (int i = 0; i < CPT; ++i) {
        const int id = threadIdx.x + i * 128;
        const int r = id / NCH, c = id % NCH;
        const int key = kb * kPreKeys + r;
        const bool valid = key < kmax;
        long long off = 0;
        if (valid) {
          const long long blk = bt[key / block_size];
          off = (blk * block_size + key % block_size) * tok_stride + hkv * HD + c * 8;
        }
        const uint32_t d = dst0 + r * ROWB + ((c ^ (r & 7)) << 4);
        cp_async16(d, kcache + off, valid);
        cp_async16(d + TILEB, vcache + off, valid);
      }
    }
    cp_async_commit();
  };
  issue(0);

  // Q fragments: this warp's rows R0 = warp * 16 + g and R0 + 8; row R = (token R / GQ, head R % GQ)
  const int R0 = warp * 16 + g, R1 = R0 + 8;
  const int t0 = R0 / GQ, t1 = R1 / GQ;
  const bool v0 = t0 < ntok, v1 = t1 < ntok;
  const int qpos0 = pos0 + t0, qpos1 = pos0 + t1;
  uint32_t qa[KS][4];
  {
    const __nv_bfloat16* q0 = q + static_cast<long long>(row0 + t0) * ld_q + (hkv * GQ + R0 % GQ) * HD;
    const __nv_bfloat16* q1 = q + static_cast<long long>(row0 + t1) * ld_q + (hkv * GQ + R1 % GQ) * HD;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      qa[ks][0] = v0 ? *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + 2 * tq) : 0u;
      qa[ks][1] = v1 ? *reinterpret_cast<const uint32_t*>(q1 + ks * 16 + 2 * tq) : 0u;
      qa[ks][2] = v0 ? *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + 8 + 2 * tq) : 0u;
      qa[ks][3] = v1 ? *reinterpret_cast<const uint32_t*>(q1 + ks * 16 + 8 + 2 * tq) : 0u;
    }
  }
  float o[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  const int lm_mi = lane >> 3, lm_r = lane & 7;
  // the warp's last query position: key blocks entirely behind it are skipped by this warp (causal)
  const int wlast = pos0 + min(ntok - 1, (warp * 16 + 15) / GQ);

  for (int kb = 0; kb < nkb; ++kb) {
    issue(kb + 1);
    cp_async_wait<1>();
    __syncthreads();
    const uint32_t kbuf = sbase + (kb & 1) * STAGEB;
    const uint32_t vbuf = kbuf + TILEB;
    const int key0 = kb * kPreKeys;
    if (key0 <= wlast && warp * 16 / GQ < ntok) {
      float s[8][4];
#pragma unroll
      for (int i = 0; i < 8; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
#pragma unroll
      for (int kg = 0; kg < 4; ++kg) {
        const int r = kg * 16 + (lm_mi >> 1) * 8 + lm_r;       // key row this lane addresses
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
          const int c = 2 * ks + (lm_mi & 1);
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4(kbuf + r * ROWB + ((c ^ (r & 7)) << 4), b0, b1, b2, b3);
          mma_bf16_16816(s[2 * kg], qa[ks], b0, b1);
          mma_bf16_16816(s[2 * kg + 1], qa[ks], b2, b3);
        }
      }
      // mask + online softmax. s[nt][0..1]: row R0, keys key0 + nt * 8 + 2 tq + {0, 1}; s[nt][2..3]: row R1
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        const int k0 = key0 + nt * 8 + 2 * tq;
        s[nt][0] = (v0 && k0 <= qpos0) ? s[nt][0] * scale_log2 : -INFINITY;
        s[nt][1] = (v0 && k0 + 1 <= qpos0) ? s[nt][1] * scale_log2 : -INFINITY;
        s[nt][2] = (v1 && k0 <= qpos1) ? s[nt][2] * scale_log2 : -INFINITY;
        s[nt][3] = (v1 && k0 + 1 <= qpos1) ? s[nt][3] * scale_log2 : -INFINITY;
        mx0 = fmaxf(mx0, fmaxf(s[nt][0], s[nt][1]));
        mx1 = fmaxf(mx1, fmaxf(s[nt][2], s[nt][3]));
      }
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
      // a row with nothing visible yet keeps -inf: subtract 0 instead so that exp2 gives 0, not NaN
      const float sub0 = mn0 == -INFINITY ? 0.f : mn0, sub1 = mn1 == -INFINITY ? 0.f : mn1;
      const float corr0 = exp2f(m0 - sub0), corr1 = exp2f(m1 - sub1);
      float ls0 = 0.f, ls1 = 0.f;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        s[nt][0] = exp2f(s[nt][0] - sub0); s[nt][1] = exp2f(s[nt][1] - sub0);
        s[nt][2] = exp2f(s[nt][2] - sub1); s[nt][3] = exp2f(s[nt][3] - sub1);
        ls0 += s[nt][0] + s[nt][1];
        ls1 += s[nt][2] + s[nt][3];
      }
      ls0 += __shfl_xor_sync(0xffffffffu, ls0, 1);
      ls0 += __shfl_xor_sync(0xffffffffu, ls0, 2);
      ls1 += __shfl_xor_sync(0xffffffffu, ls1, 1);
      ls1 += __shfl_xor_sync(0xffffffffu, ls1, 2);
      l0 = l0 * corr0 + ls0;
      l1 = l1 * corr1 + ls1;
      m0 = mn0;
      m1 = mn1;
#pragma unroll
      for (int i = 0; i < NT; ++i) { o[i][0] *= corr0; o[i][1] *= corr0; o[i][2] *= corr1; o[i][3] *= corr1; }
      // O += P V, 16 keys per k-step: P re-used in place as the A operand
#pragma unroll
      for (int kg = 0; kg < 4; ++kg) {
        const uint32_t pa[4] = {pack_bf16(s[2 * kg][0], s[2 * kg][1]), pack_bf16(s[2 * kg][2], s[2 * kg][3]),
                                pack_bf16(s[2 * kg + 1][0], s[2 * kg + 1][1]), pack_bf16(s[2 * kg + 1][2], s[2 * kg + 1][3])};
        const int r = kg * 16 + (lm_mi & 1) * 8 + lm_r;
#pragma unroll
        for (int dp = 0; dp < NT / 2; ++dp) {
          const int c = 2 * dp + (lm_mi >> 1);
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4_trans(vbuf + r * ROWB + ((c ^ (r & 7)) << 4), b0, b1, b2, b3);
          mma_bf16_16816(o[2 * dp], pa, b0, b1);
          mma_bf16_16816(o[2 * dp + 1], pa, b2, b3);
        }
      }
    }
    __syncthreads();   // every warp is done with this stage before it is refilled
  }
  cp_async_wait<0>();

  const float inv0 = l0 > 0.f ? 1.f / l0 : 0.f, inv1 = l1 > 0.f ? 1.f / l1 : 0.f;
  if (v0) {
    __nv_bfloat16* op = out + static_cast<long long>(row0 + t0) * ld_out + (hkv * GQ + R0 % GQ) * HD;
#pragma unroll
    for (int i = 0; i < NT; ++i)
      *reinterpret_cast<uint32_t*>(op + i * 8 + 2 * tq) = pack_bf16(o[i][0] * inv0, o[i][1] * inv0);
  }
  if (v1) {
    __nv_bfloat16* op = out + static_cast<long long>(row0 + t1) * ld_out + (hkv * GQ + R1 % GQ) * HD;
#pragma unroll
    for (int i = 0; i < NT; ++i)
      *reinterpret_cast<uint32_t*>(op + i * 8 + 2 * tq) = pack_bf16(o[i][2] * inv1, o[i][3] * inv1);
  }
}

template <int HD, int GQ>
static int launch_prefill(const void* q, long long ld_q, const void* kc, const void* vc, const int* bt, int max_blocks,
                          const void* tiles, int n_tiles, int block_size, int n_kv, float scale, void* out,
                          long long ld_out, cudaStream_t stream) {
  const size_t smem = 2 * 2 * static_cast<size_t>(kPreKeys) * HD * 2;
  static PerDeviceOnce configured;
  const int crc = configured.run([] {
    return static_cast<int>(cudaFuncSetAttribute(prefill_attn_kernel<HD, GQ>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 96 * 1024));
  });
  if (crc != 0) return crc;
  dim3 grid(n_tiles, n_kv);
  prefill_attn_kernel<HD, GQ><<<grid, 128, smem, stream>>>(
      static_cast<const __nv_bfloat16*>(q), ld_q, static_cast<const __nv_bfloat16*>(kc),
      static_cast<const __nv_bfloat16*>(vc), bt, max_blocks, static_cast<const int4*>(tiles), block_size, n_kv,
      scale * 1.4426950408889634f, static_cast<__nv_bfloat16*>(out), ld_out);
  return static_cast<int>(cudaGetLastError());
}

template <int HD, int GQ>
static int launch_attn(const void* q, long long ld_q, const void* kc, const void* vc, const int* bt, int max_blocks,
                       const int* bt_row, const int* ctx_len, int block_size, int T, int n_kv, float scale, int splits,
                       void* out, long long ld_out, float* part_o, float* part_lse, cudaStream_t stream) {
  const size_t merge_b = static_cast<size_t>(kAttnWarps) * GQ * HD * sizeof(float);
  const size_t ring_b = static_cast<size_t>(kAttnWarps) * kAttnStages * 2 * kAttnStageTok * HD * 2;
  const size_t smem = merge_b > ring_b ? merge_b : ring_b;
  static PerDeviceOnce configured;
  const int crc = configured.run([] {
    return static_cast<int>(cudaFuncSetAttribute(paged_attn_kernel<HD, GQ>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 160 * 1024));
  });
  if (crc != 0) return crc;
  dim3 grid(T, n_kv, splits);
  cudaError_t e = launch_kernel(paged_attn_kernel<HD, GQ>, grid, dim3(kAttnThreads), smem, stream,
      static_cast<const __nv_bfloat16*>(q), ld_q, static_cast<const __nv_bfloat16*>(kc),
      static_cast<const __nv_bfloat16*>(vc), bt, max_blocks, bt_row, ctx_len, block_size, n_kv,
      scale * 1.4426950408889634f, splits, static_cast<__nv_bfloat16*>(out), ld_out, part_o, part_lse);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (splits > 1) {
    dim3 g2(T, n_kv * GQ);
    attn_merge_kernel<HD><<<g2, HD, 0, stream>>>(part_o, part_lse, splits, n_kv * GQ,
                                                  static_cast<__nv_bfloat16*>(out), ld_out);
    e = cudaGetLastError();
  }
  return static_cast<int>(e);
}

}  // namespace dmoe

using namespace dmoe;

extern "C" long long dmoe_paged_attention_workspace_floats(int T, int n_q, int hd, int splits) {
  if (splits <= 1) return 0;
  return static_cast<long long>(T) * n_q * splits * (hd + 1);
}

extern "C" int dmoe_paged_attention(const void* q, long long ld_q, const void* kcache, const void* vcache,
                                    const int* block_tables, int max_blocks, const int* bt_row, const int* ctx_len,
                                    int block_size, int T, int n_q, int n_kv, int hd, float scale, int splits, void* out,
                                    long long ld_out, float* workspace, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (T == 0) return 0;
  if (n_kv < 1 || n_q % n_kv != 0 || splits < 1 || splits > 65535 || n_kv > 65535 || block_size % kAttnStageTok != 0) return -10;
  if (splits > 1 && workspace == nullptr) return -12;
  const int gq = n_q / n_kv;
  float* part_o = workspace;
  float* part_lse = workspace != nullptr ? workspace + static_cast<long long>(T) * n_q * splits * hd : nullptr;
#define DMOE_ATTN(HD_, GQ_)                                                                                        \
  return launch_attn<HD_, GQ_>(q, ld_q, kcache, vcache, block_tables, max_blocks, bt_row, ctx_len, block_size, T, \
                               n_kv, scale, splits, out, ld_out, part_o, part_lse, stream)
  if (hd == 128) {
    switch (gq) {
      case 1: DMOE_ATTN(128, 1);
      case 2: DMOE_ATTN(128, 2);
      case 4: DMOE_ATTN(128, 4);
      case 8: DMOE_ATTN(128, 8);
    }
  } else if (hd == 64) {
    switch (gq) {
      case 1: DMOE_ATTN(64, 1);
      case 2: DMOE_ATTN(64, 2);
      case 4: DMOE_ATTN(64, 4);
      case 8: DMOE_ATTN(64, 8);
    }
  }
#undef DMOE_ATTN
  return -11;
}

// Tokens per tile of dmoe_prefill_attention for a query group of n_q / n_kv heads.
extern "C" int dmoe_prefill_tile_tokens(int n_q, int n_kv) {
  if (n_kv < 1 || n_q % n_kv != 0) return 0;
  const int gq = n_q / n_kv;
  return (gq == 1 || gq == 2 || gq == 4 || gq == 8) ? kPreRows / gq : 0;
}

extern "C" int dmoe_prefill_attention(const void* q, long long ld_q, const void* kcache, const void* vcache,
                                      const int* block_tables, int max_blocks, const void* tiles, int n_tiles,
                                      int block_size, int n_q, int n_kv, int hd, float scale, void* out, long long ld_out,
                                      void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (n_tiles == 0) return 0;
  if (n_kv < 1 || n_q % n_kv != 0 || n_kv > 65535 || n_tiles < 0 || block_size < 1 || tiles == nullptr) return -10;
  const int gq = n_q / n_kv;
#define DMOE_PRE(HD_, GQ_)                                                                                     \
  return launch_prefill<HD_, GQ_>(q, ld_q, kcache, vcache, block_tables, max_blocks, tiles, n_tiles, block_size, \
                                  n_kv, scale, out, ld_out, stream)
  if (hd == 128) {
    switch (gq) {
      case 1: DMOE_PRE(128, 1);
      case 2: DMOE_PRE(128, 2);
      case 4: DMOE_PRE(128, 4);
      case 8: DMOE_PRE(128, 8);
    }
  } else if (hd == 64) {
    switch (gq) {
      case 1: DMOE_PRE(64, 1);
      case 2: DMOE_PRE(64, 2);
      case 4: DMOE_PRE(64, 4);
      case 8: DMOE_PRE(64, 8);
    }
  }
#undef DMOE_PRE
  return -11;
}
