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
// tensor cores: K/V rows stream through a 4-deep cp.async ring in shared memory (16 cached tokens per stage),
// a warp covers 4 cached tokens at a time, 8 lanes per token, 16-byte reads; scores are reduced with 3 shuffles; softmax is online (base 2); the 16 (warp, lane-group) partial states are merged through
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

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

constexpr int kAttnStages = 4;     // cp.async ring depth
constexpr int kAttnStageTok = 16;  // cached tokens per stage (block_size must be a multiple of it)

template <int HD, int GQ>
__global__ void __launch_bounds__(kAttnThreads)
paged_attn_kernel(const __nv_bfloat16* __restrict__ q, long long ld_q, const __nv_bfloat16* __restrict__ kcache,
                  const __nv_bfloat16* __restrict__ vcache, const int* __restrict__ block_tables, int max_blocks,
                  const int* __restrict__ bt_row, const int* __restrict__ ctx_len, int block_size, int n_kv,
                  float scale_log2, int splits, __nv_bfloat16* __restrict__ out, long long ld_out,
                  float* __restrict__ part_o, float* __restrict__ part_lse) {
  constexpr int CH = HD / 64;     // 16-byte chunks per lane (8 lanes cover one row)
  constexpr int EL = CH * 8;      // elements per lane
  constexpr int ROWB = HD * 2;    // bytes of one cached row of one kv head
  constexpr int STAGEB = 2 * kAttnStageTok * ROWB;  // K rows then V rows
  constexpr int CPT = (kAttnStageTok * (HD / 8)) / kAttnThreads;  // 16-byte copies per thread per stage, K or V
  __shared__ float s_m[kAttnParts][GQ];
  __shared__ float s_l[kAttnParts][GQ];
  extern __shared__ __align__(16) uint8_t s_dyn[];  // cp.async ring; reused as [kAttnParts][GQ][HD] floats at the end
  float* s_acc = reinterpret_cast<float*>(s_dyn);

  const int t = blockIdx.x, hkv = blockIdx.y, split = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int grp = lane >> 3, sub = lane & 7;
  const int part = warp * 4 + grp;
  const int n_q = n_kv * GQ;

  const int len = ctx_len[t];
  const int row = bt_row != nullptr ? bt_row[t] : t;
  const int* bt = block_tables + static_cast<long long>(row) * max_blocks;
  // split the context in block-aligned chunks
  const int nblk = (len + block_size - 1) / block_size;
  const int blk_per = (nblk + splits - 1) / splits;
  const int c0 = min(len, split * blk_per * block_size);
  const int c1 = min(len, (split + 1) * blk_per * block_size);
  const int nst = (c1 - c0 + kAttnStageTok - 1) / kAttnStageTok;
  const long long tok_stride = static_cast<long long>(n_kv) * HD;
  const uint32_t ring = smem_u32(s_dyn);

  // stage s holds cached tokens [c0 + 16 s, c0 + 16 s + 16) of this kv head: K rows, then V rows
  auto issue = [&](int s) {
    if (s < nst) {
      const int tok0 = c0 + s * kAttnStageTok;
      const long long blk = bt[tok0 / block_size];
      const long long slot0 = blk * block_size + tok0 % block_size;
      const uint32_t dst0 = ring + (s % kAttnStages) * STAGEB;
#pragma unroll
      for (int i = 0; i < CPT; ++i) {
        const int id = threadIdx.x + i * kAttnThreads;
        const int r = id / (HD / 8), c = id % (HD / 8);
        if (tok0 + r < c1) {
          const long long off = (slot0 + r) * tok_stride + hkv * HD + c * 8;
          cp_async16(dst0 + r * ROWB + c * 16, kcache + off);
          cp_async16(dst0 + kAttnStageTok * ROWB + r * ROWB + c * 16, vcache + off);
        }
      }
    }
    cp_async_commit();
  };
#pragma unroll
  for (int s = 0; s < kAttnStages - 1; ++s) issue(s);

  float qr[GQ][EL];
#pragma unroll
  for (int g = 0; g < GQ; ++g) {
    const __nv_bfloat16* qp = q + static_cast<long long>(t) * ld_q + (hkv * GQ + g) * HD;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      cvt8(*reinterpret_cast<const bf16x8a*>(qp + (c * 8 + sub) * 8), &qr[g][c * 8]);
    }
#pragma unroll
    for (int i = 0; i < EL; ++i) qr[g][i] *= scale_log2;
  }

  float m[GQ], l[GQ], acc[GQ][EL];
#pragma unroll
  for (int g = 0; g < GQ; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int i = 0; i < EL; ++i) acc[g][i] = 0.f;
  }

  const unsigned gmask = 0xFFu << (grp * 8);  // the 8 lanes that share one cached token
  for (int s = 0; s < nst; ++s) {
    issue(s + kAttnStages - 1);
    cp_async_wait<kAttnStages - 1>();
    __syncthreads();
    if (c0 + s * kAttnStageTok + part < c1) {   // uniform across the 8 lanes of a group
      const uint8_t* kb = s_dyn + (s % kAttnStages) * STAGEB + part * ROWB;
      const uint8_t* vb = kb + kAttnStageTok * ROWB;
      float kf[EL], vf[EL];
#pragma unroll
      for (int c = 0; c < CH; ++c) cvt8(*reinterpret_cast<const bf16x8a*>(kb + (c * 8 + sub) * 16), &kf[c * 8]);
#pragma unroll
      for (int c = 0; c < CH; ++c) cvt8(*reinterpret_cast<const bf16x8a*>(vb + (c * 8 + sub) * 16), &vf[c * 8]);
#pragma unroll
      for (int g = 0; g < GQ; ++g) {
        float sc = 0.f;
#pragma unroll
        for (int i = 0; i < EL; ++i) sc += qr[g][i] * kf[i];
        sc += __shfl_xor_sync(gmask, sc, 1);
        sc += __shfl_xor_sync(gmask, sc, 2);
        sc += __shfl_xor_sync(gmask, sc, 4);
        const float mn = fmaxf(m[g], sc);
        const float corr = exp2f(m[g] - mn);
        const float p = exp2f(sc - mn);
        m[g] = mn;
        l[g] = l[g] * corr + p;
#pragma unroll
        for (int i = 0; i < EL; ++i) acc[g][i] = acc[g][i] * corr + p * vf[i];
      }
    }
    __syncthreads();  // the ring slot is free for the copy issued at the top of the next iteration
  }
  cp_async_wait<0>();
  __syncthreads();

#pragma unroll
  for (int g = 0; g < GQ; ++g) {
    if (sub == 0) { s_m[part][g] = m[g]; s_l[part][g] = l[g]; }
#pragma unroll
    for (int c = 0; c < CH; ++c)
#pragma unroll
      for (int i = 0; i < 8; ++i) s_acc[(part * GQ + g) * HD + (c * 8 + sub) * 8 + i] = acc[g][c * 8 + i];
  }
  __syncthreads();

  for (int o = threadIdx.x; o < GQ * HD; o += kAttnThreads) {
    const int g = o / HD, d = o % HD;
    float M = -INFINITY;
#pragma unroll
    for (int p = 0; p < kAttnParts; ++p) M = fmaxf(M, s_m[p][g]);
    float L = 0.f, O = 0.f;
    if (M > -INFINITY) {
#pragma unroll
      for (int p = 0; p < kAttnParts; ++p) {
        const float w = exp2f(s_m[p][g] - M);
        L += s_l[p][g] * w;
        O += s_acc[(p * GQ + g) * HD + d] * w;
      }
    }
    const float val = L > 0.f ? O / L : 0.f;
    const int head = hkv * GQ + g;
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

template <int HD, int GQ>
static int launch_attn(const void* q, long long ld_q, const void* kc, const void* vc, const int* bt, int max_blocks,
                       const int* bt_row, const int* ctx_len, int block_size, int T, int n_kv, float scale, int splits,
                       void* out, long long ld_out, float* part_o, float* part_lse, cudaStream_t stream) {
  const size_t merge_b = static_cast<size_t>(kAttnParts) * GQ * HD * sizeof(float);
  const size_t ring_b = static_cast<size_t>(kAttnStages) * 2 * kAttnStageTok * HD * 2;
  const size_t smem = merge_b > ring_b ? merge_b : ring_b;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(paged_attn_kernel<HD, GQ>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  dim3 grid(T, n_kv, splits);
  paged_attn_kernel<HD, GQ><<<grid, kAttnThreads, smem, stream>>>(
      static_cast<const __nv_bfloat16*>(q), ld_q, static_cast<const __nv_bfloat16*>(kc),
      static_cast<const __nv_bfloat16*>(vc), bt, max_blocks, bt_row, ctx_len, block_size, n_kv,
      scale * 1.4426950408889634f, splits, static_cast<__nv_bfloat16*>(out), ld_out, part_o, part_lse);
  cudaError_t e = cudaGetLastError();
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
