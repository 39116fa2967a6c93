// An entry point of libdmoe_kernels.so that never allocates device memory.
//
// This function has no counterpart in the reference (USC-NSL/DisagMoE); it exists for callers of this library that
// are not in a position to allocate:
//   * a serving engine that, after its memory-profiling run, has handed every remaining byte of HBM to the KV cache,
//     so that a later cudaMalloc (or a growth of PyTorch's caching allocator) may simply fail;
//   * helper threads of the native runtime, which must not call cudaMalloc / cudaFree (both synchronise the whole
//     device and would stall the decode stream) nor take the framework allocator's lock.
//
// dmoe_linear_noalloc computes Y[T, F] = X[T, K] * W[F, K]^T (bf16 in, fp32 accumulate, bf16 out) with the split-K
// variant of the tcgen05 GEMM. The split-K partial tiles, the per-tile arrival counters and the status word live in
// one file-scope `static __device__` array inside the library instead of in caller-provided or freshly allocated
// memory. The caller passes only the inputs and the output.
//
// Limits and rules:
//   * The scratch array has a fixed size (DMOE_NOALLOC_WS_BYTES of partial tiles, DMOE_NOALLOC_MAX_TILES counters).
//     A problem that needs more is rejected with DMOE_NOALLOC_E_TOO_LARGE before anything is launched;
//     dmoe_noalloc_last_error() then returns a sentence that names the limit. Every GPU that loads the library
//     holds the array until the process exits.
//   * The first call on a device resolves the array's device address (cudaGetSymbolAddress, with that device
//     current). Make that first call before any stream capture begins.
//   * All calls share the one array and it keeps what the previous call left in it. The entry point clears the
//     counters and the status word on the caller's stream before every launch; the partial tiles need no clearing
//     (every element that is read was written by the same call). Two calls that overlap on the GPU (different
//     streams without an ordering between them) race on the array: serialise them.
//   * No cudaMalloc, cudaFree, or allocating library routine (PyTorch's included) is called.
//   * Host threads: the entry points may be called from several host threads (the per-device tables are guarded by a
//     mutex and dmoe_noalloc_last_error() is per thread), but the GPU work of two calls must still not overlap.
//   * dmoe_noalloc_last_status() reads the word on the stream that the last dmoe_linear_noalloc call on the current
//     device was given and synchronises that stream, so it is ordered behind that call whatever kind of stream it is.
//     Do not call it while that stream is being captured.
//   * Every non-zero return fills dmoe_noalloc_last_error(). Besides the three codes below, a positive value is a
//     cudaError_t and other negative values come from the GEMM's own argument checks (for example a tensor-map
//     encoding that the driver refused).
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define DMOE_NOALLOC_WS_BYTES (16ll << 20)
#define DMOE_NOALLOC_MAX_TILES 4096
#define DMOE_NOALLOC_E_TOO_LARGE (-30)
#define DMOE_NOALLOC_E_BAD_ARG (-31)
#define DMOE_NOALLOC_E_SETUP (-32)

// W [F, K] bf16 K-contiguous and 16-byte aligned, X [T, K] bf16, 16-byte aligned, with row stride ldx elements
// (0 = K; >= K and a multiple of 8), Y [T, F] bf16 with row stride ldy (0 = F; >= F). bn: token tile 32/64/128/256 (0 = pick); splitk >= 1 (0 = pick). Returns 0, a positive cudaError_t, or
// one of the negative codes above.
int dmoe_linear_noalloc(const void* W, const void* X, void* Y, int T, int F, int K, long long ldx, long long ldy,
                        int bn, int splitk, void* stream);
// Blocking read of the status word the last call on the current device left (0 = every bounded wait completed),
// ordered behind that call on its stream.
int dmoe_noalloc_last_status(int* status_out);
const char* dmoe_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
