// MoE routing on the device, with no host round trip between the router and the expert GEMMs.
//
//   route_kernel    (optional residual add +) RMSNorm -> gate logits -> softmax -> top-k (-> renormalise),
//                   and a per-expert histogram. One CTA per token.
//   dispatch_kernel exclusive scan of the histogram -> expert offsets; every (token, k) pair reserves a slot in
//                   its expert's segment, copies the normalised row there and writes a 16-byte token record
//                   {dst_rank, dst_row, router weight, token} next to it. The destination of a row may be this
//                   GPU's buffer or a peer GPU's buffer (table of base pointers), which is how the attention ->
//                   expert dispatch leaves the GPU without NCCL.
//
// Reference behaviour covered: disagmoe/models/attention.py:221-231 (post-attention norm, gate, fused_topk with
// renormalize), disagmoe/frontend/engine.py:667-677 (tolist + Python counting sort + permute_tokens),
// disagmoe/ops/memory.py:33-54 (mapping from expert ids), csrc/include/datatypes.hpp:228-247 (expert batch sizes).
#include "dmoe_kernels.h"
#include "sm100.cuh"

namespace dmoe {

struct alignas(16) bf16x8m {
  __nv_bfloat162 v[4];
};

constexpr int kRouteThreads = 256;
constexpr int kRouteMaxVec = 4;   // H <= 8192
constexpr int kMaxExperts = 256;
constexpr int kMaxTopK = 8;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__global__ void __launch_bounds__(kRouteThreads)
route_kernel(const __nv_bfloat16* __restrict__ x, long long ld_x, const __nv_bfloat16* __restrict__ norm_w, float eps,
             const __nv_bfloat16* __restrict__ gate_w, int H, int E, int K, int renorm,
             __nv_bfloat16* __restrict__ y, long long ld_y, int* __restrict__ topk_ids, float* __restrict__ topk_w,
             float* __restrict__ logits_out, int* __restrict__ counts, const void* const* __restrict__ add_ptrs, int n_add,
             long long ld_add, __nv_bfloat16* __restrict__ resid_out, long long ld_resid, int count_lo, int count_hi,
             const float* __restrict__ logit_bias) {
  extern __shared__ float srow[];            // [H] normalised row (fp32, as rounded to bf16)
  __shared__ float red[32];
  __shared__ float slog[kMaxExperts];
  const long long t = blockIdx.x;
  const int nvec = H / 8;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = kRouteThreads / 32;

  float xr[kRouteMaxVec][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < kRouteMaxVec; ++i) {
    const int v = threadIdx.x + i * kRouteThreads;
    if (v < nvec) {
      const bf16x8m p = *reinterpret_cast<const bf16x8m*>(x + t * ld_x + v * 8);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(p.v[j]);
        xr[i][2 * j] = f.x;
        xr[i][2 * j + 1] = f.y;
      }
      // tensor-parallel attention: the o_proj partial sums of all TP ranks (peer memory) are reduced here, so the
      // all-reduce costs no kernel of its own
      for (int a = 0; a < n_add; ++a) {
        const bf16x8m q = *reinterpret_cast<const bf16x8m*>(static_cast<const __nv_bfloat16*>(add_ptrs[a]) + t * ld_add + v * 8);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(q.v[j]);
          xr[i][2 * j] += f.x;
          xr[i][2 * j + 1] += f.y;
        }
      }
      if (n_add > 0) {
        bf16x8m r;   // the residual stream is stored in bf16: round once, and normalise what is stored
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          r.v[j] = __floats2bfloat162_rn(xr[i][2 * j], xr[i][2 * j + 1]);
          const float2 f = __bfloat1622float2(r.v[j]);
          xr[i][2 * j] = f.x;
          xr[i][2 * j + 1] = f.y;
        }
        if (resid_out != nullptr) *reinterpret_cast<bf16x8m*>(resid_out + t * ld_resid + v * 8) = r;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += xr[i][j] * xr[i][j];
    }
  }
  float inv = 1.f;
  if (norm_w != nullptr) {
    ss = warp_sum(ss);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    float tot = lane < nw ? red[lane] : 0.f;
    tot = warp_sum(tot);
    inv = rsqrtf(tot / static_cast<float>(H) + eps);
  }
#pragma unroll
  for (int i = 0; i < kRouteMaxVec; ++i) {
    const int v = threadIdx.x + i * kRouteThreads;
    if (v < nvec) {
      bf16x8m o;
      if (norm_w != nullptr) {
        const bf16x8m wv = *reinterpret_cast<const bf16x8m*>(norm_w + v * 8);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 wf = __bfloat1622float2(wv.v[j]);
          o.v[j] = __floats2bfloat162_rn(xr[i][2 * j] * inv * wf.x, xr[i][2 * j + 1] * inv * wf.y);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) o.v[j] = __floats2bfloat162_rn(xr[i][2 * j], xr[i][2 * j + 1]);
      }
      if (y != nullptr) *reinterpret_cast<bf16x8m*>(y + t * ld_y + v * 8) = o;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(o.v[j]);
        srow[v * 8 + 2 * j] = f.x;
        srow[v * 8 + 2 * j + 1] = f.y;
      }
    }
  }
  __syncthreads();
  if (gate_w == nullptr) return;   // reduction + normalisation only (a dense-FFN layer has no router)

  // gate logits: warp w takes experts w, w + nw, ...
  for (int e = warp; e < E; e += nw) {
    const __nv_bfloat16* wr = gate_w + static_cast<long long>(e) * H;
    float acc = 0.f;
    for (int v = lane; v < nvec; v += 32) {
      const bf16x8m p = *reinterpret_cast<const bf16x8m*>(wr + v * 8);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(p.v[j]);
        acc += f.x * srow[v * 8 + 2 * j] + f.y * srow[v * 8 + 2 * j + 1];
      }
    }
    acc = warp_sum(acc);
    // the optional bias skews expert popularity (synthetic load-imbalance experiments); it enters the softmax too
    if (lane == 0) slog[e] = acc + (logit_bias != nullptr ? logit_bias[e] : 0.f);
  }
  __syncthreads();

  if (warp == 0) {
    // softmax over E, then K rounds of arg-max (lowest index wins ties)
    float mx = -INFINITY;
    for (int e = lane; e < E; e += 32) mx = fmaxf(mx, slog[e]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) sum += __expf(slog[e] - mx);
    sum = warp_sum(sum);
    if (logits_out != nullptr)
      for (int e = lane; e < E; e += 32) logits_out[t * E + e] = slog[e];
    float wsel[kMaxTopK];
    int isel[kMaxTopK];
    float wtot = 0.f;
    for (int k = 0; k < K; ++k) {
      float best = -INFINITY;
      int bi = 0x7fffffff;
      for (int e = lane; e < E; e += 32) {
        const float v = slog[e];
        if (v > best) { best = v; bi = e; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
      }
      if (bi >= E) {
        // no finite logit left (NaN activations): fall back to the lowest expert not chosen yet with weight 0, so
        // that the ids stay valid and the damage stays visible in the output instead of corrupting the dispatch
        bi = 0;
        for (bool again = true; again;) {
          again = false;
          for (int j = 0; j < k; ++j)
            if (isel[j] == bi) { ++bi; again = true; }
        }
        wsel[k] = 0.f;
      } else {
        wsel[k] = __expf(best - mx) / sum;
      }
      isel[k] = bi;
      wtot += wsel[k];
      __syncwarp();
      if (lane == 0) slog[bi] = -INFINITY;
      __syncwarp();
    }
    if (lane == 0) {
      for (int k = 0; k < K; ++k) {
        topk_ids[t * K + k] = isel[k];
        topk_w[t * K + k] = (renorm && wtot > 0.f) ? wsel[k] / wtot : wsel[k];
        if (counts != nullptr && t >= count_lo && t < count_hi) atomicAdd(&counts[isel[k]], 1);
      }
    }
  }
}

// Workspace layout (ints): counts[E] | cursor[E] | ticket | pad... ; offs[E+1] is a separate output.
// dst of expert e's segment: rank = e / experts_per_rank, buffer rows [offs_local ...]. For a single-GPU
// (colocated) engine experts_per_rank = E and bases[0] is the local sorted-token buffer.
//
// Row placement: row_base[e] + slot, where row_base[e] is the exclusive prefix of counts restricted to the
// experts of the same destination rank (so every rank's buffer is packed from row 0) -- when `rank_packed` --
// or the global exclusive prefix otherwise.
__global__ void __launch_bounds__(256)
dispatch_kernel(const __nv_bfloat16* __restrict__ y, long long ld_y, const int* __restrict__ topk_ids,
                const float* __restrict__ topk_w, int T, int K, int H, int E, int experts_per_rank, int my_rank,
                int* __restrict__ ws, int* __restrict__ offs, void* const* __restrict__ x_bases, long long ld_dst,
                void* const* __restrict__ rec_bases, int dst_capacity, int* __restrict__ status) {
  __shared__ int s_base[kMaxExperts + 1];
  int* counts = ws;
  int* cursor = ws + E;
  int* ticket = ws + 2 * E;
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < E; ++e) {
      if (e % experts_per_rank == 0) run = 0;  // every destination rank's buffer starts at row 0
      s_base[e] = run;
      run += counts[e];
    }
  }
  __syncthreads();
  if (blockIdx.x == 0 && offs != nullptr) {
    // offsets of the local (rank-0-relative) view: global exclusive scan, used by a colocated engine
    if (threadIdx.x == 0) {
      int run = 0;
      for (int e = 0; e < E; ++e) { offs[e] = run; run += counts[e]; }
      offs[E] = run;
    }
  }
  const int nvec = H / 8;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const int npairs = T * K;
  for (int p = blockIdx.x * nw + warp; p < npairs; p += gridDim.x * nw) {
    const int e = topk_ids[p];
    if (e < 0 || e >= E) {
      if (lane == 0 && status != nullptr) atomicCAS(status, kStatusOk, kStatusBadIndex);
      continue;
    }
    int slot = 0;
    if (lane == 0) slot = atomicAdd(&cursor[e], 1);
    slot = __shfl_sync(0xffffffffu, slot, 0);
    const int rank = e / experts_per_rank;
    const int row = s_base[e] + slot;
    if (row >= dst_capacity) {
      if (lane == 0 && status != nullptr) atomicCAS(status, kStatusOk, kStatusCapacity);
      continue;
    }
    const int t = p / K;
    const bf16x8m* sp = reinterpret_cast<const bf16x8m*>(y + static_cast<long long>(t) * ld_y);
    bf16x8m* dp = reinterpret_cast<bf16x8m*>(static_cast<__nv_bfloat16*>(x_bases[rank]) + static_cast<long long>(row) * ld_dst);
    for (int v = lane; v < nvec; v += 32) dp[v] = sp[v];
    if (lane == 0) {
      int4 rec;
      rec.x = my_rank;
      rec.y = p;                       // destination row of the combine: [T, K, H] partial-output buffer
      rec.z = __float_as_int(topk_w[p]);
      rec.w = e;
      reinterpret_cast<int4*>(rec_bases[rank])[row] = rec;
    }
  }
  // the last CTA to finish clears the histogram and cursors for the next layer
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const int old = atomicAdd(ticket, 1);
    if (old == static_cast<int>(gridDim.x) - 1) {
      for (int e = 0; e < E; ++e) { counts[e] = 0; cursor[e] = 0; }
      *ticket = 0;
      __threadfence();
    }
  }
}

}  // namespace dmoe

using namespace dmoe;

// route_kernel keeps one fp32 row in dynamic shared memory (up to 32 KB): opt in once per device.
static int configure_route() {
  static PerDeviceOnce once;
  return once.run([] {
    return static_cast<int>(cudaFuncSetAttribute(route_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 8192 * 4));
  });
}

extern "C" int dmoe_route(const void* x, long long ld_x, const void* norm_w, float eps, const void* gate_w, int T, int H,
                          int E, int K, int renorm, void* y, long long ld_y, int* topk_ids, float* topk_w,
                          float* logits_out, int* counts, const float* logit_bias, void* stream) {
  if (H % 8 != 0 || H > kRouteThreads * kRouteMaxVec * 8 || E > kMaxExperts || K > kMaxTopK || K > E) return -10;
  if (T == 0) return 0;
  if (const int rc = configure_route()) return rc;
  route_kernel<<<T, kRouteThreads, H * sizeof(float), static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), ld_x, static_cast<const __nv_bfloat16*>(norm_w), eps,
      static_cast<const __nv_bfloat16*>(gate_w), H, E, K, renorm, static_cast<__nv_bfloat16*>(y), ld_y, topk_ids, topk_w,
      logits_out, counts, nullptr, 0, 0, nullptr, 0, 0, T, logit_bias);
  return static_cast<int>(cudaGetLastError());
}

// Same router with the tensor-parallel reduction folded in: x + sum of n_add partial rows (device array of pointers,
// typically the TP peers' o_proj outputs) is written to resid_out and normalised; only tokens in [count_lo, count_hi)
// enter the expert histogram (the slice this rank dispatches). gate_w == nullptr stops after the normalised rows
// (layers with a dense FFN). logit_bias (fp32 [E], optional) is added to the gate logits.
extern "C" int dmoe_route_ex(const void* x, long long ld_x, const void* norm_w, float eps, const void* gate_w, int T,
                             int H, int E, int K, int renorm, void* y, long long ld_y, int* topk_ids, float* topk_w,
                             int* counts, const void* add_ptrs, int n_add, long long ld_add, void* resid_out,
                             long long ld_resid, int count_lo, int count_hi, const float* logit_bias, void* stream) {
  if (H % 8 != 0 || H > kRouteThreads * kRouteMaxVec * 8) return -10;
  if (gate_w != nullptr && (E > kMaxExperts || K > kMaxTopK || K > E)) return -10;
  if (T == 0) return 0;
  if (const int rc = configure_route()) return rc;
  route_kernel<<<T, kRouteThreads, H * sizeof(float), static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), ld_x, static_cast<const __nv_bfloat16*>(norm_w), eps,
      static_cast<const __nv_bfloat16*>(gate_w), H, E, K, renorm, static_cast<__nv_bfloat16*>(y), ld_y, topk_ids, topk_w,
      nullptr, counts, static_cast<const void* const*>(add_ptrs), n_add, ld_add, static_cast<__nv_bfloat16*>(resid_out),
      ld_resid, count_lo, count_hi, logit_bias);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int dmoe_dispatch_local(const void* y, long long ld_y, const int* topk_ids, const float* topk_w, int T, int K,
                                   int H, int E, int experts_per_rank, int my_rank, int* ws, int* offs,
                                   const void* x_bases, long long ld_dst, const void* rec_bases, int dst_capacity,
                                   int* status, void* stream) {
  if (H % 8 != 0 || E > kMaxExperts || experts_per_rank < 1) return -10;
  if (T == 0) return 0;
  const int npairs = T * K;
  int grid = (npairs + 7) / 8;
  if (grid > device_num_sms() * 4) grid = device_num_sms() * 4;
  dispatch_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(y), ld_y, topk_ids, topk_w, T, K, H, E, experts_per_rank, my_rank, ws, offs,
      static_cast<void* const*>(x_bases), ld_dst, static_cast<void* const*>(rec_bases), dst_capacity, status);
  return static_cast<int>(cudaGetLastError());
}
