// Attention -> expert token dispatch over peer memory (NVLink / NVSwitch), issued from the kernel.
//
// dispatch_remote_kernel: every routed (token, k) pair of this attention rank is stored straight into the receive
// region of its expert on the GPU that holds the expert: row copy (16-byte stores), a 16-byte token record {source
// rank, row in the source's partial-output buffer, router weight, expert} next to it, and, once every row of the
// launch is out, a release flag carrying the launch's epoch. Each sender first reserves a block of rows per expert
// with one system-scope atomic add on the expert's cursor (reserve_kernel), so the rows of an expert arrive contiguous
// from all senders and the cursor is the row count the consumer's grouped GEMM reads. No host round trip, no NCCL, no
// TCP message: sizes travel with the data.
//
// wait_flags_kernel: bounded wait on peers' flags (used before an op that reads rows peers combine into this GPU).
// A wait that runs out records kStatusFlagTimeout and returns; later waits of a poisoned run return at once.
//
// Replaces, on the device: disagmoe/frontend/engine.py:667-677 (tolist + counting sort + permute),
// csrc/muhelper/muhelper.cpp:189-228 (per-EP-rank ZMQ metadata message + ncclSend) and the receive side
// csrc/muhelper/muhelper.cpp:485-515 (ZMQ recv + ncclRecv + stream sync).
#include <string.h>

#include "dmoe_kernels.h"
#include "sm100.cuh"

namespace dmoe {

struct alignas(16) bf16x8c {
  __nv_bfloat162 v[4];
};

constexpr int kMaxExpertsComm = 256;
constexpr int kMaxRanksComm = 16;

__device__ __forceinline__ int ld_acquire_sys_i32(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

struct DispatchRemoteArgs {
  const __nv_bfloat16* y;       // [T, H] normalised rows
  long long ld_y;
  const int* topk_ids;          // [T, K]
  const float* topk_w;          // [T, K]
  int T, K, H, E, experts_per_rank, n_dst, my_rank, region_cap;
  int tok_lo, tok_hi;           // this rank dispatches tokens [tok_lo, tok_hi) (a TP rank sends its slice only)
  int* ws;                      // [counts E | cursor E | ticket]
  void* const* x_bases;         // [n_dst] receive-row buffers on the destinations ([n_src * region_cap, H] bf16)
  long long ld_dst;
  void* const* rec_bases;       // [n_dst] record buffers ([n_src * region_cap] int4)
  int* const* cnt_bases;        // [n_dst] per-expert row cursors on the destinations ([experts_per_rank] int)
  const int* row_base;          // [E] first row (inside the expert's region) reserved for this rank by reserve_kernel
  int* const* flag_bases;       // [n_dst] arrival flags ([n_src] int)
  int* epoch;                   // launch counter of this dispatcher (device resident)
  int* status;
};

__global__ void __launch_bounds__(256) dispatch_remote_kernel(const DispatchRemoteArgs a) {
  __shared__ int s_base[kMaxExpertsComm];
  int* counts = a.ws;
  int* cursor = a.ws + a.E;
  int* ticket = a.ws + 2 * a.E;
  // every expert owns one region of region_cap rows on its GPU; this rank's rows start at the offset it reserved
  for (int e = threadIdx.x; e < a.E; e += blockDim.x) s_base[e] = a.row_base[e];
  __syncthreads();
  const int nvec = a.H / 8;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const int npairs = a.tok_hi * a.K;
  for (int p = a.tok_lo * a.K + blockIdx.x * nw + warp; p < npairs; p += gridDim.x * nw) {
    const int e = a.topk_ids[p];
    if (e < 0 || e >= a.E) {
      if (lane == 0 && a.status != nullptr) atomicCAS(a.status, kStatusOk, kStatusBadIndex);
      continue;
    }
    int slot = 0;
    if (lane == 0) slot = atomicAdd(&cursor[e], 1);
    slot = __shfl_sync(0xffffffffu, slot, 0);
    const int dst = e / a.experts_per_rank;
    const int row_in_region = s_base[e] + slot;
    if (row_in_region >= a.region_cap || dst >= a.n_dst) {
      if (lane == 0 && a.status != nullptr) atomicCAS(a.status, kStatusOk, kStatusCapacity);
      continue;
    }
    const long long row = static_cast<long long>(e % a.experts_per_rank) * a.region_cap + row_in_region;
    const int t = p / a.K;
    const bf16x8c* sp = reinterpret_cast<const bf16x8c*>(a.y + static_cast<long long>(t) * a.ld_y);
    bf16x8c* dp = reinterpret_cast<bf16x8c*>(static_cast<__nv_bfloat16*>(a.x_bases[dst]) + row * a.ld_dst);
    for (int v = lane; v < nvec; v += 32) dp[v] = sp[v];
    if (lane == 0) {
      int4 rec;
      rec.x = a.my_rank;
      rec.y = p;                         // row of the (token, k) pair in this rank's [T, K, H] partial buffer
      rec.z = __float_as_int(a.topk_w[p]);
      rec.w = e;
      reinterpret_cast<int4*>(a.rec_bases[dst])[row] = rec;
    }
  }
  // completion: rows and records first (system-scope fence per thread), then counts, then the flag
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int old = atomicAdd(ticket, 1);
    if (old == static_cast<int>(gridDim.x) - 1) {
      __threadfence_system();
      const int epoch = *a.epoch + 1;
      for (int d = 0; d < a.n_dst; ++d) st_relaxed_sys(a.flag_bases[d] + a.my_rank, epoch);
      *a.epoch = epoch;
      for (int e = 0; e < a.E; ++e) { counts[e] = 0; cursor[e] = 0; }
      *ticket = 0;
      __threadfence();
    }
  }
}

// Row reservation of one dispatch launch: for every expert e this rank adds its row count to the expert's cursor on
// the owning GPU (one system-scope atomic over NVLink) and keeps the old value as the first row of its block. Rows of
// an expert therefore arrive contiguous from all senders, so the consumer's GEMM sees one segment per expert.
__global__ void reserve_kernel(const int* counts, int E, int experts_per_rank, int* const* cnt_bases, int* row_base) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= E) return;
  const int c = counts[e];
  row_base[e] = c > 0 ? atomicAdd_system(cnt_bases[e / experts_per_rank] + e % experts_per_rank, c) : 0;
}

// Thread i waits until flags[i] >= *epoch + 1; then *epoch is advanced.
__global__ void wait_flags_kernel(const int* flags, int n, int* epoch, int* status, long long max_cycles) {
  const int want = *epoch + 1;
  if (threadIdx.x < n) {
    const bool poisoned = status != nullptr && *reinterpret_cast<volatile int*>(status) != kStatusOk;
    const long long t0 = clock64();
    while (!poisoned && ld_acquire_sys_i32(flags + threadIdx.x) < want) {
      if (clock64() - t0 > max_cycles) {
        if (status != nullptr) atomicCAS(status, kStatusOk, kStatusFlagTimeout);
        break;
      }
      __nanosleep(100);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) *epoch = want;
}

}  // namespace dmoe

using namespace dmoe;

extern "C" int dmoe_dispatch_remote(const void* y, long long ld_y, const int* topk_ids, const float* topk_w, int T,
                                    int K, int H, int E, int experts_per_rank, int n_dst, int my_rank, int region_cap,
                                    int* ws, const void* x_bases, long long ld_dst, const void* rec_bases,
                                    const void* cnt_bases, const void* flag_bases, int* epoch, int* status,
                                    int tok_lo, int tok_hi, void* stream) {
  if (H % 8 != 0 || E > kMaxExpertsComm || experts_per_rank < 1 || n_dst < 1 || n_dst > kMaxRanksComm ||
      n_dst * experts_per_rank < E || (n_dst - 1) * experts_per_rank >= E || epoch == nullptr)
    return -10;
  DispatchRemoteArgs a;
  a.y = static_cast<const __nv_bfloat16*>(y); a.ld_y = ld_y; a.topk_ids = topk_ids; a.topk_w = topk_w;
  a.T = T; a.K = K; a.H = H; a.E = E; a.experts_per_rank = experts_per_rank; a.n_dst = n_dst; a.my_rank = my_rank;
  a.region_cap = region_cap; a.ws = ws; a.x_bases = static_cast<void* const*>(x_bases); a.ld_dst = ld_dst;
  a.rec_bases = static_cast<void* const*>(rec_bases); a.cnt_bases = static_cast<int* const*>(cnt_bases);
  a.flag_bases = static_cast<int* const*>(flag_bases); a.epoch = epoch; a.status = status;
  a.row_base = ws + 2 * E + 8;
  if (tok_hi <= 0 || tok_hi > T) tok_hi = T;
  if (tok_lo < 0 || tok_lo > tok_hi) tok_lo = 0;
  a.tok_lo = tok_lo; a.tok_hi = tok_hi;
  const int npairs = (tok_hi - tok_lo) * K;
  int grid = (npairs + 7) / 8;
  if (grid > device_num_sms() * 2) grid = device_num_sms() * 2;
  if (grid < 1) grid = 1;   // an empty batch still publishes its flag
  reserve_kernel<<<(E + 63) / 64, 64, 0, static_cast<cudaStream_t>(stream)>>>(ws, E, experts_per_rank, a.cnt_bases,
                                                                               ws + 2 * E + 8);
  dispatch_remote_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(a);
  return static_cast<int>(cudaGetLastError());
}

// Cycle budget of every peer-flag wait of the library (wait_flags, the GEMM's arrival gates, the sender kernels);
// kernels launched later use the new value. <= 0 restores the default of about 4 s.
namespace dmoe {
long long g_dmoe_flag_wait_cycles = 4 * DMOE_WAIT_CYCLES;
}

extern "C" void dmoe_set_flag_wait_cycles(long long cycles) {
  g_dmoe_flag_wait_cycles = cycles > 0 ? cycles : 4 * DMOE_WAIT_CYCLES;
}

extern "C" int dmoe_wait_flags(const int* flags, int n, int* epoch, int* status, void* stream) {
  if (n < 0 || n > 256 || epoch == nullptr) return -10;
  wait_flags_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(flags, n, epoch, status, g_dmoe_flag_wait_cycles);
  return static_cast<int>(cudaGetLastError());
}

// Enables loads / stores from the current device to `peer_device` memory (idempotent).
extern "C" int dmoe_enable_peer_access(int peer_device) {
  int cur = 0;
  cudaGetDevice(&cur);
  if (cur == peer_device) return 0;
  int can = 0;
  cudaError_t e = cudaDeviceCanAccessPeer(&can, cur, peer_device);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (!can) return -20;
  e = cudaDeviceEnablePeerAccess(peer_device, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) {
    cudaGetLastError();
    return 0;
  }
  return static_cast<int>(e);
}

// ---- peer arenas: allocation and CUDA IPC mapping ----------------------------------------------------------
// The arena is a plain cudaMalloc block (so its IPC handle names exactly this block); a peer's handle is opened
// with THIS process's device current, which maps the block for loads / stores issued by kernels of this device.
extern "C" int dmoe_peer_alloc(long long nbytes, void** ptr, void* handle64) {
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, static_cast<size_t>(nbytes));
  if (e != cudaSuccess) return static_cast<int>(e);
  e = cudaMemset(p, 0, static_cast<size_t>(nbytes));
  if (e != cudaSuccess) return static_cast<int>(e);
  cudaIpcMemHandle_t h;
  e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) return static_cast<int>(e);
  static_assert(sizeof(h) == 64, "IPC handle size");
  memcpy(handle64, &h, sizeof(h));
  *ptr = p;
  return static_cast<int>(cudaDeviceSynchronize());
}

extern "C" int dmoe_peer_open(const void* handle64, void** ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return static_cast<int>(e);
  *ptr = p;
  return 0;
}

extern "C" int dmoe_peer_close(void* ptr) { return static_cast<int>(cudaIpcCloseMemHandle(ptr)); }
extern "C" int dmoe_peer_free(void* ptr) { return static_cast<int>(cudaFree(ptr)); }
