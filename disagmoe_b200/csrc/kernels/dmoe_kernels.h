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
  long long ldx, ldy, ldr, ws_bytes;
  int G, T, F, K;
  int epi;            // DMOE_EPI_*
  int bn;             // token tile: 32/64/128/256, 0 = pick from T/G
  int splitk;         // >= 1; > 1 only for dense plain / combine GEMMs
  int y_f32;
} DmoeGemm;

int dmoe_gemm(const DmoeGemm* desc, void* stream);
int dmoe_gemm_pick_bn(int tokens_per_group_hint, int epi);
long long dmoe_gemm_workspace_bytes(int T, int F, int bn, int splitk);

#ifdef __cplusplus
}
#endif
