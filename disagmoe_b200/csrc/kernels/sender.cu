// Attention-side sender kernels of the fused disaggregated pipeline: each one folds the wait for its producers, the
// row math, the transfer over NVLink peer memory and the completion signal into a single launch.
//
//   norm_gather_kernel     [bounded wait for the experts' combine flags] resid += partial rows; y = RMSNorm(resid);
//                          y is stored into the QKV staging buffer of every rank of the tensor-parallel group (the
//                          all-gather that the QKV GEMM's prologue consumes shard by shard); the last CTA releases one
//                          flag per destination. With one destination and no flags it is a plain add + RMSNorm that has
//                          the combine wait folded in.
//   route_dispatch_kernel  [bounded wait for the TP peers' o_proj flags] resid += the o_proj partial rows that the
//                          peers' GEMM epilogues scattered to this rank (ordered local sum: the reduce half of the
//                          reduce-scatter); post-attention RMSNorm; gate logits, softmax, top-k; every (token, k) pair
//                          reserves a row of its expert's receive region on the GPU that owns the expert with one
//                          system-scope atomic and stores the normalised row and a 16-byte record there; the last CTA
//                          releases one flag per expert GPU. One launch replaces router + reservation + dispatch.
//   ids_gather_kernel      the sampled token ids of this rank's rows are stored into every TP rank's id buffer.
//
// Every wait is bounded and reports through the status word; a poisoned run (status != 0) skips its waits.
//
// Reference behaviour covered: disagmoe/models/attention.py:210-231 (norms, gate, fused_topk), the all-reduce of
// disagmoe/models/linear.py:1064-1089 / csrc/muhelper/comm.cpp:399-416, the broadcast of a TP group's inputs
// disagmoe/frontend/engine.py:494-535, and the dispatch path disagmoe/frontend/engine.py:667-677 +
// csrc/muhelper/muhelper.cpp:189-228.
#include <stdlib.h>

#include "dmoe_kernels.h"
#include "sm100.cuh"

namespace dmoe {

struct alignas(16) bf16x8s {
  __nv_bfloat162 v[4];
};

constexpr int kSendThreads = 256;
constexpr int kSendMaxVec = 4;      // H <= 256 * 4 * 8 = 8192
constexpr int kSendMaxExperts = 256;
constexpr int kSendMaxTopK = 8;
constexpr int kSendMaxDst = 16;

__device__ __forceinline__ int ld_acquire_sys_s(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Requests `bytes` at `p` into L2 (the whole CTA takes part, one 128-byte line per thread and round): used for what a
// kernel will need AFTER its flag wait and does not depend on it (weights, this CTA's residual row), so that the HBM
// latency of those reads overlaps the wait instead of following it.
__device__ __forceinline__ void cta_prefetch_l2(const void* p, long long bytes) {
  const char* c = static_cast<const char*>(p);
  for (long long off = static_cast<long long>(threadIdx.x) * 128; off < bytes; off += static_cast<long long>(blockDim.x) * 128)
    asm volatile("prefetch.global.L2 [%0];" ::"l"(c + off));
}

__device__ __forceinline__ float warp_sum_s(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Threads [0, n) wait until flags[i] >= want (bounded); the whole CTA then synchronises.
__device__ __forceinline__ void cta_wait_flags(const int* flags, int n, int want, int* status, long long max_cycles) {
  if (n > 0) {
    if (threadIdx.x < n) {
      const bool poisoned = status != nullptr && *reinterpret_cast<volatile int*>(status) != kStatusOk;
      const long long t0 = clock64();
      while (!poisoned && ld_acquire_sys_s(flags + threadIdx.x) < want) {
        if (clock64() - t0 > max_cycles) {
          if (status != nullptr) atomicCAS(status, kStatusOk, kStatusFlagTimeout);
          break;
        }
        __nanosleep(64);
      }
    }
    __syncthreads();
  }
}

// Completion shared by the sender kernels: every thread's (possibly remote) stores are made visible system-wide, the
// CTA takes a ticket, and the last CTA of the grid releases `n_signal` flags with this launch's epoch and advances the
// device-resident epochs (by then every CTA has read them).
__device__ __forceinline__ void cta_complete(int* ticket, int* const* signal_ptrs, int n_signal, int signal_slot,
                                             int* signal_epoch, int n_wait, int* wait_epoch) {
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int old = atomicAdd(ticket, 1);
    if (old == static_cast<int>(gridDim.x) - 1) {
      __threadfence_system();
      if (n_signal > 0) {
        const int epoch = *signal_epoch + 1;
        for (int i = 0; i < n_signal; ++i) st_relaxed_sys(signal_ptrs[i] + signal_slot, epoch);   // fenced above
        *signal_epoch = epoch;
      }
      if (n_wait > 0) *wait_epoch = *wait_epoch + 1;
      *ticket = 0;
      __threadfence();
    }
  }
}

struct NormGatherArgs {
  const __nv_bfloat16* resid_in;   // [T, H] or null
  long long ld_in;
  const __nv_bfloat16* add;        // partial rows: add[t * add_row_stride + p * add_part_stride], p < n_add
  int n_add;
  long long add_row_stride, add_part_stride;
  const __nv_bfloat16* w;
  float eps;
  __nv_bfloat16* resid_out;        // [T, H] or null
  long long ld_out;
  void* const* dst_ptrs;           // [n_dst] base of the normalised-row buffer on every destination
  int n_dst;
  long long dst_row0, ld_dst;      // row t goes to row dst_row0 + t
  int T, H;
  const int* wait_flags;           // optional gate (the experts' combine flags)
  int n_wait;
  int* wait_epoch;
  int* const* signal_ptrs;         // optional completion flags (one array per destination, slot signal_slot)
  int n_signal, signal_slot;
  int* signal_epoch;
  int* ticket;
  int* status;
  long long max_cycles;
  int prefetch;
};

__global__ void __launch_bounds__(kSendThreads) norm_gather_kernel(const NormGatherArgs a) {
  __shared__ float red[32];
  pdl_trigger();
  if (a.prefetch && blockIdx.x == 0) cta_prefetch_l2(a.w, static_cast<long long>(a.H) * 2);
  pdl_wait();
  const int want = a.n_wait > 0 ? *a.wait_epoch + 1 : 0;
  if (a.prefetch && a.resid_in != nullptr && blockIdx.x < a.T) cta_prefetch_l2(a.resid_in + blockIdx.x * a.ld_in, static_cast<long long>(a.H) * 2);
  cta_wait_flags(a.wait_flags, a.n_wait, want, a.status, a.max_cycles);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = kSendThreads / 32;
  const int nvec = a.H / 8;
  for (long long t = blockIdx.x; t < a.T; t += gridDim.x) {
    float x[kSendMaxVec][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < kSendMaxVec; ++i) {
      const int v = threadIdx.x + i * kSendThreads;
      if (v < nvec) {
        if (a.resid_in != nullptr) {
          const bf16x8s p = *reinterpret_cast<const bf16x8s*>(a.resid_in + t * a.ld_in + v * 8);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(p.v[j]);
            x[i][2 * j] = f.x;
            x[i][2 * j + 1] = f.y;
          }
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) x[i][j] = 0.f;
        }
        for (int p = 0; p < a.n_add; ++p) {
          // the partial rows were written by other GPUs' kernels: read them past L1
          const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(a.add + t * a.add_row_stride + p * a.add_part_stride + v * 8));
          const __nv_bfloat162* q = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(q[j]);
            x[i][2 * j] += f.x;
            x[i][2 * j + 1] += f.y;
          }
        }
        if (a.resid_out != nullptr) {
          bf16x8s r;   // the residual stream is kept in bf16: round once so that the norm sees what is stored
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            r.v[j] = __floats2bfloat162_rn(x[i][2 * j], x[i][2 * j + 1]);
            const float2 f = __bfloat1622float2(r.v[j]);
            x[i][2 * j] = f.x;
            x[i][2 * j + 1] = f.y;
          }
          *reinterpret_cast<bf16x8s*>(a.resid_out + t * a.ld_out + v * 8) = r;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += x[i][j] * x[i][j];
      }
    }
    // the norm weights do not depend on the row: request them before the block-wide reduction, not after it
    bf16x8s wreg[kSendMaxVec];
#pragma unroll
    for (int i = 0; i < kSendMaxVec; ++i) {
      const int v = threadIdx.x + i * kSendThreads;
      if (v < nvec) wreg[i] = *reinterpret_cast<const bf16x8s*>(a.w + v * 8);
    }
    ss = warp_sum_s(ss);
    __syncthreads();               // red[] of the previous row has been read by everyone
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    float tot = lane < nw ? red[lane] : 0.f;
    tot = warp_sum_s(tot);
    const float inv = rsqrtf(tot / static_cast<float>(a.H) + a.eps);
#pragma unroll
    for (int i = 0; i < kSendMaxVec; ++i) {
      const int v = threadIdx.x + i * kSendThreads;
      if (v < nvec) {
        const bf16x8s wv = wreg[i];
        bf16x8s o;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 wf = __bfloat1622float2(wv.v[j]);
          o.v[j] = __floats2bfloat162_rn(x[i][2 * j] * inv * wf.x, x[i][2 * j + 1] * inv * wf.y);
        }
        for (int d = 0; d < a.n_dst; ++d)
          *reinterpret_cast<bf16x8s*>(static_cast<__nv_bfloat16*>(a.dst_ptrs[d]) + (a.dst_row0 + t) * a.ld_dst + v * 8) = o;
      }
    }
  }
  if (a.ticket != nullptr)
    cta_complete(a.ticket, a.signal_ptrs, a.n_signal, a.signal_slot, a.signal_epoch, a.n_wait, a.wait_epoch);
}

struct RouteDispatchArgs {
  __nv_bfloat16* resid;            // [T, H] residual stream of this rank's rows (read, and rewritten when n_add > 0)
  long long ld_resid;
  const __nv_bfloat16* add;        // [n_add][add_slot_rows][H] partial rows scattered here by the TP peers' o_proj
  int n_add;
  long long add_slot_stride, ld_add;
  const __nv_bfloat16* norm_w;
  float eps;
  const __nv_bfloat16* gate_w;     // [E, H]; null: reduction + normalisation only (a layer with a dense FFN)
  const float* logit_bias;         // optional fp32 [E]
  int T, H, E, K, renorm;
  __nv_bfloat16* y;                // optional [T, H] normalised rows kept on this GPU (shared experts, dense FFN)
  long long ld_y;
  int* topk_ids;                   // optional [T, K]
  float* topk_w;                   // optional [T, K]
  // dispatch
  int experts_per_rank, n_dst, my_rank, region_cap;
  int ret_rank;                    // rank named in the records (the rows' owner for the experts' combine)
  void* const* x_bases;            // [n_dst] receive rows ([experts_per_rank * region_cap, H] bf16)
  long long ld_dst;
  void* const* rec_bases;          // [n_dst] records (int4 per row)
  int* const* cnt_bases;           // [n_dst] per-expert row cursors
  int* const* flag_bases;          // [n_dst] arrival flags, slot my_rank
  int* disp_epoch;
  const int* wait_flags;           // optional gate (the TP peers' o_proj completion flags)
  int n_wait;
  int* wait_epoch;
  int* ticket;
  int* status;
  long long max_cycles;
  int prefetch;
};

__global__ void __launch_bounds__(kSendThreads) route_dispatch_kernel(const RouteDispatchArgs a) {
  extern __shared__ float srow[];            // [H] normalised row (fp32 value of what is stored in bf16)
  __shared__ float red[32];
  __shared__ float slog[kSendMaxExperts];
  __shared__ int s_sel[kSendMaxTopK];        // chosen experts
  __shared__ float s_wt[kSendMaxTopK];
  __shared__ long long s_row[kSendMaxTopK];  // destination row (-1: dropped)
  pdl_trigger();
  if (a.prefetch && a.gate_w != nullptr && blockIdx.x < 16) {
    // the gate matrix is shared by all CTAs: the first 16 request one sixteenth each
    const long long slice = (static_cast<long long>(a.E) * a.H * 2 + 15) / 16;
    cta_prefetch_l2(reinterpret_cast<const char*>(a.gate_w) + blockIdx.x * slice,
                    min(slice, static_cast<long long>(a.E) * a.H * 2 - blockIdx.x * slice));
  }
  if (a.prefetch && blockIdx.x == 16 % gridDim.x) cta_prefetch_l2(a.norm_w, static_cast<long long>(a.H) * 2);
  pdl_wait();
  const int want = a.n_wait > 0 ? *a.wait_epoch + 1 : 0;
  if (a.prefetch && blockIdx.x < a.T) cta_prefetch_l2(a.resid + blockIdx.x * a.ld_resid, static_cast<long long>(a.H) * 2);
  cta_wait_flags(a.wait_flags, a.n_wait, want, a.status, a.max_cycles);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = kSendThreads / 32;
  const int nvec = a.H / 8;

  for (long long t = blockIdx.x; t < a.T; t += gridDim.x) {
    float xr[kSendMaxVec][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < kSendMaxVec; ++i) {
      const int v = threadIdx.x + i * kSendThreads;
      if (v < nvec) {
        const bf16x8s p = *reinterpret_cast<const bf16x8s*>(a.resid + t * a.ld_resid + v * 8);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(p.v[j]);
          xr[i][2 * j] = f.x;
          xr[i][2 * j + 1] = f.y;
        }
        for (int s = 0; s < a.n_add; ++s) {
          const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(a.add + s * a.add_slot_stride + t * a.ld_add + v * 8));
          const __nv_bfloat162* q = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(q[j]);
            xr[i][2 * j] += f.x;
            xr[i][2 * j + 1] += f.y;
          }
        }
        if (a.n_add > 0) {
          bf16x8s r;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            r.v[j] = __floats2bfloat162_rn(xr[i][2 * j], xr[i][2 * j + 1]);
            const float2 f = __bfloat1622float2(r.v[j]);
            xr[i][2 * j] = f.x;
            xr[i][2 * j + 1] = f.y;
          }
          *reinterpret_cast<bf16x8s*>(a.resid + t * a.ld_resid + v * 8) = r;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += xr[i][j] * xr[i][j];
      }
    }
    bf16x8s wreg[kSendMaxVec];       // norm weights: requested before the block-wide reduction
#pragma unroll
    for (int i = 0; i < kSendMaxVec; ++i) {
      const int v = threadIdx.x + i * kSendThreads;
      if (v < nvec) wreg[i] = *reinterpret_cast<const bf16x8s*>(a.norm_w + v * 8);
    }
    ss = warp_sum_s(ss);
    __syncthreads();               // shared state of the previous row is no longer read
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    float tot = lane < nw ? red[lane] : 0.f;
    tot = warp_sum_s(tot);
    const float inv = rsqrtf(tot / static_cast<float>(a.H) + a.eps);
    bf16x8s o[kSendMaxVec];
#pragma unroll
    for (int i = 0; i < kSendMaxVec; ++i) {
      const int v = threadIdx.x + i * kSendThreads;
      if (v < nvec) {
        const bf16x8s wv = wreg[i];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 wf = __bfloat1622float2(wv.v[j]);
          o[i].v[j] = __floats2bfloat162_rn(xr[i][2 * j] * inv * wf.x, xr[i][2 * j + 1] * inv * wf.y);
          const float2 f = __bfloat1622float2(o[i].v[j]);
          srow[v * 8 + 2 * j] = f.x;
          srow[v * 8 + 2 * j + 1] = f.y;
        }
        if (a.y != nullptr) *reinterpret_cast<bf16x8s*>(a.y + t * a.ld_y + v * 8) = o[i];
      }
    }
    __syncthreads();
    if (a.gate_w == nullptr) continue;   // CTA-uniform

    // gate logits: warp w takes experts w, w + nw, ...
    for (int e = warp; e < a.E; e += nw) {
      const __nv_bfloat16* wr = a.gate_w + static_cast<long long>(e) * a.H;
      float acc = 0.f;
      for (int v = lane; v < nvec; v += 32) {
        const bf16x8s p = *reinterpret_cast<const bf16x8s*>(wr + v * 8);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(p.v[j]);
          acc += f.x * srow[v * 8 + 2 * j] + f.y * srow[v * 8 + 2 * j + 1];
        }
      }
      acc = warp_sum_s(acc);
      if (lane == 0) slog[e] = acc + (a.logit_bias != nullptr ? a.logit_bias[e] : 0.f);
    }
    __syncthreads();

    if (warp == 0) {
      // softmax over E, then K rounds of arg-max (lowest index wins ties)
      float mx = -INFINITY;
      for (int e = lane; e < a.E; e += 32) mx = fmaxf(mx, slog[e]);
#pragma unroll
      for (int s = 16; s > 0; s >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, s));
      float sum = 0.f;
      for (int e = lane; e < a.E; e += 32) sum += __expf(slog[e] - mx);
      sum = warp_sum_s(sum);
      float wsel[kSendMaxTopK];
      int isel[kSendMaxTopK];
      float wtot = 0.f;
      for (int k = 0; k < a.K; ++k) {
        float best = -INFINITY;
        int bi = 0x7fffffff;
        for (int e = lane; e < a.E; e += 32) {
          const float v = slog[e];
          if (v > best) { best = v; bi = e; }
        }
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) {
          const float ob = __shfl_xor_sync(0xffffffffu, best, s);
          const int oi = __shfl_xor_sync(0xffffffffu, bi, s);
          if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
        }
        if (bi >= a.E) {
          // no finite logit left (NaN activations): the lowest expert not chosen yet, with weight 0, keeps ids valid
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
      // lane k owns pair k: reserve its row on the expert's GPU (one system-scope atomic over NVLink), write the record
      if (lane < a.K) {
        int e = isel[0];
        float w = wsel[0];
#pragma unroll
        for (int k = 1; k < kSendMaxTopK; ++k)
          if (k == lane) { e = isel[k]; w = wsel[k]; }
        if (a.renorm && wtot > 0.f) w /= wtot;
        const long long p = t * a.K + lane;
        if (a.topk_ids != nullptr) a.topk_ids[p] = e;
        if (a.topk_w != nullptr) a.topk_w[p] = w;
        long long row = -1;
        if (a.x_bases != nullptr) {
          const int dst = e / a.experts_per_rank, le = e % a.experts_per_rank;
          if (dst >= a.n_dst) {
            if (a.status != nullptr) atomicCAS(a.status, kStatusOk, kStatusBadIndex);
          } else {
            const int slot = atomicAdd_system(a.cnt_bases[dst] + le, 1);
            if (slot >= a.region_cap) {
              if (a.status != nullptr) atomicCAS(a.status, kStatusOk, kStatusCapacity);
            } else {
              row = static_cast<long long>(le) * a.region_cap + slot;
              int4 rec;
              rec.x = a.ret_rank;
              rec.y = static_cast<int>(p);     // row of the pair in this rank's [T, K, H] partial-output buffer
              rec.z = __float_as_int(w);
              rec.w = e;
              reinterpret_cast<int4*>(a.rec_bases[dst])[row] = rec;
            }
          }
        }
        s_sel[lane] = e;
        s_wt[lane] = w;
        s_row[lane] = row;
      }
    }
    __syncthreads();
    if (a.x_bases != nullptr) {
      for (int k = 0; k < a.K; ++k) {
        const long long row = s_row[k];
        if (row < 0) continue;
        __nv_bfloat16* dp = static_cast<__nv_bfloat16*>(a.x_bases[s_sel[k] / a.experts_per_rank]) + row * a.ld_dst;
#pragma unroll
        for (int i = 0; i < kSendMaxVec; ++i) {
          const int v = threadIdx.x + i * kSendThreads;
          if (v < nvec) *reinterpret_cast<bf16x8s*>(dp + v * 8) = o[i];
        }
      }
    }
  }
  if (a.ticket != nullptr) {
    // the dispatch flags (one per expert GPU, slot = this rank) double as this kernel's completion signal
    cta_complete(a.ticket, a.flag_bases, a.x_bases != nullptr ? a.n_dst : 0, a.my_rank, a.disp_epoch, a.n_wait,
                 a.wait_epoch);
  }
}

// dst[d][dst0 + i] = src[i] for every destination d, then one release flag per destination.
__global__ void ids_gather_kernel(const int* __restrict__ src, int n, int* const* dst_ptrs, int n_dst, int dst0,
                                  int* const* signal_ptrs, int signal_slot, int* signal_epoch) {
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int v = src[i];
    for (int d = 0; d < n_dst; ++d) dst_ptrs[d][dst0 + i] = v;
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0 && signal_ptrs != nullptr) {
    const int epoch = *signal_epoch + 1;
    __threadfence_system();      // release fence of the signalling thread, after the barrier that gathered the CTA's stores
    for (int d = 0; d < n_dst; ++d) st_relaxed_sys(signal_ptrs[d] + signal_slot, epoch);
    *signal_epoch = epoch;
  }
}

}  // namespace dmoe

using namespace dmoe;

// DMOE_SENDER_PREFETCH=0 turns the L2 prefetches of the sender kernels off (read once per process)
static int sender_prefetch() {
  static const int v = [] {
    const char* e = getenv("DMOE_SENDER_PREFETCH");
    return (e != nullptr && e[0] == '0') ? 0 : 1;
  }();
  return v;
}

extern "C" int dmoe_norm_gather(const DmoeNormGather* d, void* stream) {
  if (d->H % 8 != 0 || d->H > kSendThreads * kSendMaxVec * 8 || d->T < 0 || d->n_dst < 1 || d->n_dst > kSendMaxDst ||
      d->dst_ptrs == nullptr || d->w == nullptr || d->n_wait < 0 || d->n_wait > kSendThreads || d->n_signal < 0)
    return -10;
  if ((d->n_wait > 0 && (d->wait_flags == nullptr || d->wait_epoch == nullptr)) ||
      (d->n_signal > 0 && (d->signal_ptrs == nullptr || d->signal_epoch == nullptr)) ||
      ((d->n_wait > 0 || d->n_signal > 0) && d->ticket == nullptr))
    return -11;
  NormGatherArgs a;
  a.resid_in = static_cast<const __nv_bfloat16*>(d->resid_in); a.ld_in = d->ld_in;
  a.add = static_cast<const __nv_bfloat16*>(d->add); a.n_add = d->add != nullptr ? d->n_add : 0;
  a.add_row_stride = d->add_row_stride; a.add_part_stride = d->add_part_stride;
  a.w = static_cast<const __nv_bfloat16*>(d->w); a.eps = d->eps;
  a.resid_out = static_cast<__nv_bfloat16*>(d->resid_out); a.ld_out = d->ld_out;
  a.dst_ptrs = static_cast<void* const*>(d->dst_ptrs); a.n_dst = d->n_dst; a.dst_row0 = d->dst_row0; a.ld_dst = d->ld_dst;
  a.T = d->T; a.H = d->H;
  a.wait_flags = d->wait_flags; a.n_wait = d->n_wait; a.wait_epoch = d->wait_epoch;
  a.signal_ptrs = reinterpret_cast<int* const*>(d->signal_ptrs); a.n_signal = d->n_signal; a.signal_slot = d->signal_slot;
  a.signal_epoch = d->signal_epoch; a.ticket = d->ticket; a.status = d->status; a.max_cycles = g_dmoe_flag_wait_cycles; a.prefetch = sender_prefetch();
  // an empty shard still takes part in the hand-shake (it waits, signals and advances its epochs)
  const int grid = d->T > 0 ? d->T : 1;
  if (launch_kernel(norm_gather_kernel, dim3(grid), dim3(kSendThreads), 0, static_cast<cudaStream_t>(stream), a) != cudaSuccess)
    return static_cast<int>(cudaGetLastError());
  return static_cast<int>(cudaGetLastError());
}

extern "C" int dmoe_route_dispatch(const DmoeRouteDispatch* d, void* stream) {
  if (d->H % 8 != 0 || d->H > kSendThreads * kSendMaxVec * 8 || d->T < 0 || d->resid == nullptr || d->norm_w == nullptr ||
      d->n_wait < 0 || d->n_wait > kSendThreads || d->n_add < 0)
    return -10;
  if (d->gate_w != nullptr && (d->E < 1 || d->E > kSendMaxExperts || d->K < 1 || d->K > kSendMaxTopK || d->K > d->E)) return -10;
  const bool send = d->gate_w != nullptr && d->x_bases != nullptr;
  if (send && (d->experts_per_rank < 1 || d->n_dst < 1 || d->n_dst > kSendMaxDst || d->n_dst * d->experts_per_rank < d->E ||
               (d->n_dst - 1) * d->experts_per_rank >= d->E || d->rec_bases == nullptr || d->cnt_bases == nullptr ||
               d->flag_bases == nullptr || d->disp_epoch == nullptr || d->ticket == nullptr || d->region_cap < 1))
    return -11;
  if (d->n_wait > 0 && (d->wait_flags == nullptr || d->wait_epoch == nullptr || d->ticket == nullptr)) return -11;
  if (d->n_add > 0 && d->add == nullptr) return -11;
  static PerDeviceOnce once;
  const int crc = once.run([] {
    return static_cast<int>(cudaFuncSetAttribute(route_dispatch_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 8192 * 4));
  });
  if (crc != 0) return crc;
  RouteDispatchArgs a;
  a.resid = static_cast<__nv_bfloat16*>(d->resid); a.ld_resid = d->ld_resid;
  a.add = static_cast<const __nv_bfloat16*>(d->add); a.n_add = d->n_add; a.add_slot_stride = d->add_slot_stride;
  a.ld_add = d->ld_add;
  a.norm_w = static_cast<const __nv_bfloat16*>(d->norm_w); a.eps = d->eps;
  a.gate_w = static_cast<const __nv_bfloat16*>(d->gate_w); a.logit_bias = d->logit_bias;
  a.T = d->T; a.H = d->H; a.E = d->E; a.K = d->K; a.renorm = d->renorm;
  a.y = static_cast<__nv_bfloat16*>(d->y); a.ld_y = d->ld_y; a.topk_ids = d->topk_ids; a.topk_w = d->topk_w;
  a.experts_per_rank = d->experts_per_rank; a.n_dst = d->n_dst; a.my_rank = d->my_rank; a.region_cap = d->region_cap;
  a.ret_rank = d->ret_rank_set ? d->ret_rank : d->my_rank;
  a.x_bases = send ? static_cast<void* const*>(d->x_bases) : nullptr; a.ld_dst = d->ld_dst;
  a.rec_bases = static_cast<void* const*>(d->rec_bases); a.cnt_bases = static_cast<int* const*>(d->cnt_bases);
  a.flag_bases = static_cast<int* const*>(d->flag_bases); a.disp_epoch = d->disp_epoch;
  a.wait_flags = d->wait_flags; a.n_wait = d->n_wait; a.wait_epoch = d->wait_epoch;
  a.ticket = (send || d->n_wait > 0) ? d->ticket : nullptr; a.status = d->status; a.max_cycles = g_dmoe_flag_wait_cycles; a.prefetch = sender_prefetch();
  const int grid = d->T > 0 ? d->T : 1;   // an empty slice still publishes its flags
  if (launch_kernel(route_dispatch_kernel, dim3(grid), dim3(kSendThreads), d->H * sizeof(float),
                    static_cast<cudaStream_t>(stream), a) != cudaSuccess)
    return static_cast<int>(cudaGetLastError());
  return static_cast<int>(cudaGetLastError());
}

extern "C" int dmoe_ids_gather(const int* src, int n, const void* dst_ptrs, int n_dst, int dst0, const void* signal_ptrs,
                               int signal_slot, int* signal_epoch, void* stream) {
  if (n < 0 || n_dst < 1 || n_dst > kSendMaxDst || dst_ptrs == nullptr || (signal_ptrs != nullptr && signal_epoch == nullptr))
    return -10;
  ids_gather_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      src, n, static_cast<int* const*>(dst_ptrs), n_dst, dst0, static_cast<int* const*>(signal_ptrs), signal_slot,
      signal_epoch);
  return static_cast<int>(cudaGetLastError());
}
