// Bandwidth-bound row kernels of the decoder: (fused add +) RMSNorm, neox RoPE + paged KV append,
// embedding lookup, greedy argmax, row permute / gather. All bf16 in memory, fp32 in registers,
// 16-byte vector accesses (hidden sizes must be multiples of 8).
//
// Reference behaviour covered: vLLM RMSNorm / fused-add RMSNorm used at disagmoe/models/attention.py:166-167,
// 210-214,221; rotary embedding + reshape_and_cache at attention.py:143-149,218-219; the sampler stub
// csrc/muhelper/embedding.cpp:212-215 (replaced by a real argmax); permute_tokens / gather_tokens of
// csrc/cuda_ops/permute.cu:18-152.
#include "dmoe_kernels.h"
#include "sm100.cuh"

namespace dmoe {

struct alignas(16) bf16x8 {
  __nv_bfloat162 v[4];
};

__device__ __forceinline__ void unpack8(const bf16x8& p, float (&f)[8]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(p.v[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ bf16x8 pack8(const float (&f)[8]) {
  bf16x8 p;
#pragma unroll
  for (int i = 0; i < 4; ++i) p.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return p;
}

__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : 0.f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  __syncthreads();
  return t;
}

// resid_out[t] = resid_in[t] + sum_{p < n_add} add[t * add_row_stride + p * add_part_stride]   (resid_in may be null)
// y[t] = rmsnorm(resid_out[t]) * w.   One CTA per row; the row stays in registers (<= 8 vectors per thread).
constexpr int kNormThreads = 256;
constexpr int kNormMaxVec = 4;  // supports H <= 256 * 4 * 8 = 8192

__global__ void __launch_bounds__(kNormThreads)
add_rmsnorm_kernel(const __nv_bfloat16* __restrict__ resid_in, const __nv_bfloat16* __restrict__ add, int n_add,
                   long long add_row_stride, long long add_part_stride, const __nv_bfloat16* __restrict__ w,
                   float eps, __nv_bfloat16* __restrict__ resid_out, __nv_bfloat16* __restrict__ y, int H,
                   long long ld_in, long long ld_out, long long ld_y) {
  __shared__ float red[32];
  const long long t = blockIdx.x;
  const int nvec = H / 8;
  float x[kNormMaxVec][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < kNormMaxVec; ++i) {
    const int v = threadIdx.x + i * kNormThreads;
    if (v < nvec) {
      if (resid_in != nullptr) {
        unpack8(*reinterpret_cast<const bf16x8*>(resid_in + t * ld_in + v * 8), x[i]);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) x[i][j] = 0.f;
      }
      for (int p = 0; p < n_add; ++p) {
        float a[8];
        unpack8(*reinterpret_cast<const bf16x8*>(add + t * add_row_stride + p * add_part_stride + v * 8), a);
#pragma unroll
        for (int j = 0; j < 8; ++j) x[i][j] += a[j];
      }
      if (resid_out != nullptr) {
        // the residual stream is kept in bf16: round once so that the norm sees what is stored
        const bf16x8 r = pack8(x[i]);
        *reinterpret_cast<bf16x8*>(resid_out + t * ld_out + v * 8) = r;
        unpack8(r, x[i]);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += x[i][j] * x[i][j];
    }
  }
  const float tot = block_sum(ss, red);
  const float inv = rsqrtf(tot / static_cast<float>(H) + eps);
  if (y == nullptr) return;
#pragma unroll
  for (int i = 0; i < kNormMaxVec; ++i) {
    const int v = threadIdx.x + i * kNormThreads;
    if (v < nvec) {
      float wv[8], o[8];
      unpack8(*reinterpret_cast<const bf16x8*>(w + v * 8), wv);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = x[i][j] * inv * wv[j];
      *reinterpret_cast<bf16x8*>(y + t * ld_y + v * 8) = pack8(o);
    }
  }
}

// Neox-style rotary embedding on q and k (rotary_dim = head_dim) followed by the paged KV append.
// qkv row layout: [q heads | k heads | v heads]. Cache layout: [num_blocks, block_size, kv_heads, head_dim]
// for K and V separately; slot = block * block_size + offset, slot < 0 skips the append.
// One CTA per token, one thread per (head, pair-vector).
__global__ void rope_kv_append_kernel(__nv_bfloat16* __restrict__ qkv, long long ld, const int* __restrict__ positions,
                                      const long long* __restrict__ slots, __nv_bfloat16* __restrict__ kcache,
                                      __nv_bfloat16* __restrict__ vcache, int n_q, int n_kv, int hd, float theta_log2) {
  const long long t = blockIdx.x;
  const int half = hd / 2;
  const int vec_per_head = half / 8;  // 8 rotation pairs per thread: elements [8v, 8v+8) and [half + 8v, ...)
  const float pos = static_cast<float>(positions[t]);
  const long long slot = slots != nullptr ? slots[t] : -1;
  __nv_bfloat16* row = qkv + t * ld;
  const int n_rot = (n_q + n_kv) * vec_per_head;
  for (int i = threadIdx.x; i < n_rot; i += blockDim.x) {
    const int head = i / vec_per_head, v = i % vec_per_head;
    __nv_bfloat16* p = row + head * hd + v * 8;
    float a[8], b[8], oa[8], ob[8];
    unpack8(*reinterpret_cast<const bf16x8*>(p), a);
    unpack8(*reinterpret_cast<const bf16x8*>(p + half), b);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int d = v * 8 + j;
      // inv_freq = theta^(-2d/hd)
      const float inv_freq = exp2f(-theta_log2 * (2.f * d) / static_cast<float>(hd));
      float s, c;
      sincosf(pos * inv_freq, &s, &c);
      oa[j] = a[j] * c - b[j] * s;
      ob[j] = b[j] * c + a[j] * s;
    }
    const bf16x8 pa = pack8(oa), pb = pack8(ob);
    *reinterpret_cast<bf16x8*>(p) = pa;
    *reinterpret_cast<bf16x8*>(p + half) = pb;
    if (head >= n_q && slot >= 0) {
      __nv_bfloat16* kc = kcache + (slot * n_kv + (head - n_q)) * hd + v * 8;
      *reinterpret_cast<bf16x8*>(kc) = pa;
      *reinterpret_cast<bf16x8*>(kc + half) = pb;
    }
  }
  if (slot >= 0) {
    const int nv = n_kv * hd / 8;
    const __nv_bfloat16* vsrc = row + (n_q + n_kv) * hd;
    for (int i = threadIdx.x; i < nv; i += blockDim.x) {
      *reinterpret_cast<bf16x8*>(vcache + slot * n_kv * hd + i * 8) = *reinterpret_cast<const bf16x8*>(vsrc + i * 8);
    }
  }
}

// table[pos][d] = (cos, sin)(pos * theta^(-2 d / hd)): the same arithmetic as rope_kv_append_kernel, so that the QKV
// GEMM's rotating epilogue and the stand-alone kernel produce identical bits.
__global__ void rope_table_kernel(float2* __restrict__ table, int max_pos, int hd, float theta_log2) {
  const int half = hd / 2;
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= static_cast<long long>(max_pos) * half) return;
  const int pos = static_cast<int>(i / half), d = static_cast<int>(i % half);
  const float inv_freq = exp2f(-theta_log2 * (2.f * d) / static_cast<float>(hd));
  float s, c;
  sincosf(static_cast<float>(pos) * inv_freq, &s, &c);
  table[i] = make_float2(c, s);
}

// out[t] = table[ids[t]]
__global__ void embed_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                             __nv_bfloat16* __restrict__ out, int H, int vocab, long long ld_out) {
  const long long t = blockIdx.x;
  int id = ids[t];
  if (id < 0 || id >= vocab) id = 0;
  const bf16x8* src = reinterpret_cast<const bf16x8*>(table + static_cast<long long>(id) * H);
  bf16x8* dst = reinterpret_cast<bf16x8*>(out + t * ld_out);
  for (int i = threadIdx.x; i < H / 8; i += blockDim.x) dst[i] = src[i];
}

// ids[t] = argmax_v logits[t, v] (first maximum wins). logits fp32 or bf16.
template <typename T>
__global__ void argmax_kernel(const T* __restrict__ logits, long long ld, int V, int* __restrict__ ids) {
  __shared__ float sv[32];
  __shared__ int si[32];
  const long long t = blockIdx.x;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int v = threadIdx.x; v < V; v += blockDim.x) {
    const float x = static_cast<float>(logits[t * ld + v]);
    if (x > best || (x == best && v < bi)) { best = x; bi = v; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (lane == 0) { sv[warp] = best; si[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    best = lane < nw ? sv[lane] : -INFINITY;
    bi = lane < nw ? si[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    if (lane == 0) ids[t] = bi;
  }
}

// dst[map[i]] = src[i / repeat]   (scatter; repeat > 1 duplicates each source row, e.g. once per top-k slot)
// or dst[i] = src[map[i]]          (gather). map entries < 0 are skipped. Two rows per CTA pass.
__global__ void permute_rows_kernel(const __nv_bfloat16* __restrict__ src, long long ld_src,
                                    __nv_bfloat16* __restrict__ dst, long long ld_dst, const int* __restrict__ map,
                                    int n, int H, int repeat, int gather) {
  const int nvec = H / 8;
  for (long long i = blockIdx.x; i < n; i += gridDim.x) {
    const int m = map[i];
    if (m < 0) continue;
    const long long s = gather ? m : i / repeat;
    const long long d = gather ? i : m;
    const bf16x8* sp = reinterpret_cast<const bf16x8*>(src + s * ld_src);
    bf16x8* dp = reinterpret_cast<bf16x8*>(dst + d * ld_dst);
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) dp[v] = sp[v];
  }
}

// Row gather through a device-resident table of row pointers (the scheduler's batch merge): dst[i] = *ptrs[i].
__global__ void gather_ptrs_kernel(const __nv_bfloat16* const* __restrict__ ptrs, __nv_bfloat16* __restrict__ dst,
                                   long long ld_dst, int n, int H) {
  const int nvec = H / 8;
  for (long long i = blockIdx.x; i < n; i += gridDim.x) {
    const bf16x8* sp = reinterpret_cast<const bf16x8*>(ptrs[i]);
    bf16x8* dp = reinterpret_cast<bf16x8*>(dst + i * ld_dst);
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) dp[v] = sp[v];
  }
}

// Debug kernel of the launch / overlap tests: out[i] = in[i] + 1 (reference: csrc/cuda_ops/test.cu:6-13, one thread per
// block there; 256 here).
__global__ void add_one_kernel(const float* __restrict__ in, float* __restrict__ out, long long n) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) out[i] = in[i] + 1.f;
}

}  // namespace dmoe

using namespace dmoe;

extern "C" int dmoe_add_one(const float* in, float* out, long long n, void* stream) {
  if (n <= 0) return 0;
  add_one_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(in, out, n);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int dmoe_add_rmsnorm(const void* resid_in, const void* add, int n_add, long long add_row_stride,
                                long long add_part_stride, const void* w, float eps, void* resid_out, void* y, int T,
                                int H, long long ld_in, long long ld_out, long long ld_y, void* stream) {
  if (H % 8 != 0 || H > kNormThreads * kNormMaxVec * 8) return -10;
  if (T == 0) return 0;
  add_rmsnorm_kernel<<<T, kNormThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(resid_in), static_cast<const __nv_bfloat16*>(add), n_add, add_row_stride,
      add_part_stride, static_cast<const __nv_bfloat16*>(w), eps, static_cast<__nv_bfloat16*>(resid_out),
      static_cast<__nv_bfloat16*>(y), H, ld_in, ld_out, ld_y);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int dmoe_rope_kv_append(void* qkv, long long ld, const int* positions, const long long* slots, void* kcache,
                                   void* vcache, int T, int n_q, int n_kv, int hd, float theta, void* stream) {
  if (hd % 16 != 0) return -10;
  if (T == 0) return 0;
  rope_kv_append_kernel<<<T, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(qkv), ld, positions, slots, static_cast<__nv_bfloat16*>(kcache),
      static_cast<__nv_bfloat16*>(vcache), n_q, n_kv, hd, log2f(theta));
  return static_cast<int>(cudaGetLastError());
}

extern "C" int dmoe_rope_table(void* table, int max_pos, int hd, float theta, void* stream) {
  if (hd % 16 != 0 || max_pos < 1) return -10;
  const long long n = static_cast<long long>(max_pos) * (hd / 2);
  rope_table_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<float2*>(table), max_pos, hd, log2f(theta));
  return static_cast<int>(cudaGetLastError());
}

extern "C" int dmoe_embed(const int* ids, const void* table, void* out, int T, int H, int vocab, long long ld_out,
                          void* stream) {
  if (H % 8 != 0) return -10;
  if (T == 0) return 0;
  embed_kernel<<<T, 128, 0, static_cast<cudaStream_t>(stream)>>>(ids, static_cast<const __nv_bfloat16*>(table),
                                                                 static_cast<__nv_bfloat16*>(out), H, vocab, ld_out);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int dmoe_argmax(const void* logits, int is_f32, long long ld, int T, int V, int* ids, void* stream) {
  if (T == 0) return 0;
  if (is_f32)
    argmax_kernel<float><<<T, 1024, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const float*>(logits), ld, V, ids);
  else
    argmax_kernel<__nv_bfloat16><<<T, 1024, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(logits), ld, V, ids);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int dmoe_permute_rows(const void* src, long long ld_src, void* dst, long long ld_dst, const int* map, int n,
                                 int H, int repeat, int gather, void* stream) {
  if (H % 8 != 0 || repeat < 1) return -10;
  if (n == 0) return 0;
  const int grid = n < device_num_sms() * 16 ? n : device_num_sms() * 16;
  permute_rows_kernel<<<grid, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(src), ld_src, static_cast<__nv_bfloat16*>(dst), ld_dst, map, n, H, repeat, gather);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int dmoe_gather_ptrs(const void* ptrs, void* dst, long long ld_dst, int n, int H, void* stream) {
  if (H % 8 != 0) return -10;
  if (n == 0) return 0;
  const int grid = n < device_num_sms() * 16 ? n : device_num_sms() * 16;
  gather_ptrs_kernel<<<grid, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16* const*>(ptrs), static_cast<__nv_bfloat16*>(dst), ld_dst, n, H);
  return static_cast<int>(cudaGetLastError());
}
