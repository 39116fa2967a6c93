// Grouped / dense bf16 GEMM for sm_100a: TMA -> shared memory -> tcgen05.mma -> TMEM -> epilogue.
//
// Computes, for every group g (an expert, or the single group of a dense linear layer),
//     Y[t, f] = sum_k X[t, k] * W[g][f, k]          t in [offs[g], offs[g+1])
// with W stored [G, rows, K] K-contiguous ("out, in" like F.linear) and X stored [T, K].
//
// Serving is decode heavy: few tokens per expert and large weight matrices, so the kernel is laid out
// "swap-AB": the WEIGHT tile (128 rows) is the M operand of the UMMA and the TOKEN tile (BN = 32..256 rows)
// is the N operand. A CTA therefore never pads a handful of tokens up to 128 MMA rows, and the weight
// stream (the HBM-bound part) is read exactly once. The accumulator lives in TMEM as [128 lanes = features,
// BN columns = tokens]; the epilogue thread that owns lane i owns output feature i of the tile.
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = TMEM owner + MMA issuer, warps 2..5 = epilogue.
// Accumulators are double buffered in TMEM so the epilogue of tile i overlaps the main loop of tile i+1.
// Persistent grid: CTA b runs tiles b, b + gridDim.x, ...; group sizes are read from device memory, so the
// host never needs to know the routing result.
//
// Epilogues: plain (+ optional residual), SwiGLU (two accumulators: gate rows and up rows of the fused w13
// weight; out = silu(gate) * up), combine (row scatter through 16-byte token records with a per-row scale
// and a table of destination base pointers, which may be peer GPUs' buffers), and split-K with a
// last-arriver reduction through an fp32 workspace.
//
// Reference behaviour covered: disagmoe/models/experts.py:81-96 (gmm -> silu*mul -> gmm),
// disagmoe/models/linear.py:131-136 (F.linear), disagmoe/frontend/engine.py:731-734 (weight scale + un-permute).
#include <string.h>

#include "dmoe_kernels.h"
#include "sm100.cuh"
#include "work_walker.cuh"

namespace dmoe {

constexpr int kBM = 128;       // weight rows per tile (UMMA M)
constexpr int kBK = 64;        // K elements per stage: 64 bf16 = 128 bytes = one swizzle span
constexpr int kUmmaK = 16;     // K per tcgen05.mma for 16-bit inputs
constexpr int kThreads = 192;
constexpr int kEpiThreads = 128;
constexpr int kSmemBudget = 220 * 1024;
constexpr int kTailBytes = 10 * 1024;   // barriers + segment table (2 x kMaxSeg ints)
constexpr int kMaxSeg = 1024;            // groups x sources

enum { EPI_PLAIN = 0, EPI_SWIGLU = 1, EPI_COMBINE = 2 };

struct GemmArgs {
  const int* offs;   // [G+1] device token offsets, or nullptr for one dense group of T tokens
  int G, T, F, K;    // F: output features per group
  int w_rows;        // weight rows per group (F, or 2F for SwiGLU)
  void* Y;
  long long ldy;
  int y_f32;
  const __nv_bfloat16* R;  // optional residual [T, F]
  long long ldr;
  const int4* recs;        // combine: per input row {dst_rank, dst_row, weight (fp32 bits), unused}
  void* const* bases;      // combine: destination base pointer per rank
  int splitk;
  int streamk;   // 1: stream-K work distribution (see work_walker.cuh); splitk is then 1
  float* ws;
  int* counters;
  int* status;
  // multi-source input (the expert side of a dispatch): S sources wrote their rows for group g into region s
  // (rows [s * seg_cap, (s + 1) * seg_cap)), packed group after group; seg_cnt[s * G + g] rows each.
  const int* seg_cnt;
  int S;
  int seg_cap;
  // arrival gate: wait until wait_flags[i] >= *wait_epoch + 1 for i < n_wait before reading seg_cnt / rows
  const int* wait_flags;
  int n_wait;
  int* wait_epoch;
  // completion signal: after the last tile, store *signal_epoch + 1 to signal_ptrs[i][signal_slot] for i < n_signal
  int* const* signal_ptrs;
  int n_signal;
  int signal_slot;
  int* signal_epoch;
  int* done_ticket;
  int fanout;   // combine: destinations per row (TP group size of the senders)
  int group_regions;
  int clear_n;
  int* clear_ptr;
  int epi_vec;   // plain epilogue may use 16-byte accesses on Y / R (alignment checked on the host)
  // all-gather prologue: X rows [s * shard_rows, (s + 1) * shard_rows) are pushed by peer s; a token tile is loaded
  // once wait_flags[s] carries this call's epoch for every shard it touches (0 = one gate for the whole launch)
  int shard_rows;
  // reduce-scatter epilogue: row t belongs to rank t / rs_rows and is stored to row rs_slot * rs_cap + t % rs_rows of
  // that rank's buffer rs_bases[t / rs_rows] (row stride ldy); the owner sums the slots
  void* const* rs_bases;
  int rs_rows, rs_slot, rs_cap;
  // QKV epilogue: neox RoPE on the q and k heads from a (cos, sin) table [pos][hd / 2], K / V append to the paged
  // cache at slots[t] (< 0: none); only the q columns are written to Y
  const float2* rope_table;
  const int* positions;
  const long long* slots;
  __nv_bfloat16* kcache;
  __nv_bfloat16* vcache;
  int n_q, n_kv, hd, rope_max_pos;
  long long flag_cycles;   // budget of the peer-flag waits
  // w_blocked: the weights are stored tile by tile ([group][128-row tile][K block][128][64], every 16 KB TMA box one
  // contiguous run of HBM) instead of row-major [group][row][K]
  int w_blocked;
  // optional [16] nanosecond stamps written by CTA 0 (a profiling aid, null in normal launches): 0 entry, 1 set-up done,
  // 2 first TMA issued, 3 first stage landed, 4 last MMA committed, 5 accumulator seen by the epilogue, 6 epilogue done,
  // 7 tear-down reached; 8-12 inside the first epilogue chunk: TMEM read done, staged to shared memory, barrier passed,
  // rows stored, second barrier passed; 13-15 in the producer: work walker initialised, L2 policies made, first stage free
  unsigned long long* trace;
};

// PAIR: the kernel runs as clusters of two CTAs on one tile of 256 weight rows (two m-tiles) x BN tokens with
// tcgen05.mma.cta_group::2: each CTA stages its own 128 weight rows and HALF of the token tile, so the shared-memory
// fill per output (the limiter at 128 and more tokens per expert) drops by a third to a half; each CTA keeps the
// accumulator of its 128 rows in its own TMEM and runs its own epilogue.
template <int BN, int EPI, bool PAIR = false>
struct Cfg {
  static constexpr int kNumA = (EPI == EPI_SWIGLU) ? 2 : 1;
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBRows = PAIR ? BN / 2 : BN;      // token rows this CTA stages
  static constexpr int kBBytes = kBRows * kBK * 2;
  static constexpr int kStageBytes = kNumA * kABytes + kBBytes;
  // plain and combine epilogues (and SwiGLU from 128-token tiles on, where the stage count does not pay for it): one
  // 32-token x 128-feature fp32 chunk is transposed through shared memory, so that Y (and the residual) move as
  // 16-byte row segments instead of one 2-byte element per thread
  static constexpr int kEpiStageBytes =
      (EPI == EPI_PLAIN || EPI == EPI_COMBINE || (EPI == EPI_SWIGLU && BN >= 128)) ? 32 * kBM * 4 : 0;
  static constexpr int kStagesRaw = (kSmemBudget - 1024 - kTailBytes - kEpiStageBytes) / kStageBytes;
  static constexpr int kStages = kStagesRaw > 8 ? 8 : kStagesRaw;
  static constexpr int kAccCols = BN * kNumA;
  // two accumulator buffers (the epilogue of a tile overlaps the next main loop) unless one already fills TMEM
  static constexpr int kAccBufs = (2 * kAccCols <= 512) ? 2 : 1;
  static constexpr int kTmemCols = (kAccBufs * kAccCols) < 32 ? 32 : kAccBufs * kAccCols;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*alignment slack*/ + kTailBytes + kEpiStageBytes;
  static_assert(kTmemCols <= 512, "accumulators do not fit TMEM");
  static_assert((kTmemCols & (kTmemCols - 1)) == 0, "TMEM columns must be a power of two");
  static_assert(kStages >= 3, "pipeline too shallow");
};

__device__ __forceinline__ void trace_stamp(const GemmArgs& a, int i) {
  if (a.trace != nullptr && blockIdx.x == 0) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    a.trace[i] = t;
  }
}

__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

template <int BN, int EPI, bool PAIR>
__global__ void __launch_bounds__(kThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, const GemmArgs a) {
  using C = Cfg<BN, EPI, PAIR>;
  // pair mode: rank of this CTA in its pair (the even CTA issues the MMAs), work is dealt out per pair
  const uint32_t prank = PAIR ? cluster_ctarank() : 0u;
  const bool leader = prank == 0;
  const int work_cta = PAIR ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
  const int work_grid = PAIR ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* tail = smem + C::kStages * C::kStageBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(tail);            // [kStages]
  uint64_t* empty_bar = full_bar + C::kStages;                       // [kStages]
  uint64_t* tfull_bar = empty_bar + C::kStages;                      // [2]
  uint64_t* tempty_bar = tfull_bar + 2;                              // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2); // [1]
  int* abort_word = reinterpret_cast<int*>(tmem_slot + 1);
  int* last_flag = abort_word + 1;
  int* s_start = last_flag + 1;                                      // [S * G]
  int* s_cnt = s_start + kMaxSeg;                                    // [S * G]
  float* epi_stage = reinterpret_cast<float*>(tail + kTailBytes);    // [32][kBM] (plain epilogue only)
  const int S = (a.S > 0 && !a.group_regions) ? a.S : 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int MT1 = (a.F + kBM - 1) / kBM;              // 128-row weight tiles
  const int MT = PAIR ? (MT1 + 1) / 2 : MT1;          // work tiles along M (pairs of them in pair mode)
  const int kblocks = (a.K + kBK - 1) / kBK;
  // the producer may legitimately sit in a peer-flag wait (all-gather prologue): the warps behind it must outlast it
  const long long bar_budget = DMOE_WAIT_CYCLES + (a.shard_rows > 0 ? a.flag_cycles : 0);

  pdl_trigger();
  if (threadIdx.x == 0) {
    trace_stamp(a, 0);
    *abort_word = 0;
    *last_flag = 0;
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&tfull_bar[b]), 1);
      // pair mode: the epilogue threads of BOTH CTAs hand an accumulator buffer back to the even CTA's MMA thread
      mbar_init(smem_u32(&tempty_bar[b]), PAIR ? 2 * kEpiThreads : kEpiThreads);
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmW);
    tma_prefetch_desc(&tmX);
  }
  pdl_wait();      // nothing above reads global data; everything below may read what the previous kernel wrote
  if (a.n_wait > 0 && a.shard_rows == 0) {
    // arrival gate: the senders' rows, counts and records are complete once their flag carries this call's epoch
    if (threadIdx.x < a.n_wait) {
      const int want = *a.wait_epoch + 1;
      const bool poisoned = a.status != nullptr && *reinterpret_cast<volatile int*>(a.status) != kStatusOk;
      const long long t0 = clock64();
      while (!poisoned && ld_acquire_sys(a.wait_flags + threadIdx.x) < want) {
        if (clock64() - t0 > a.flag_cycles) {
          if (a.status != nullptr) atomicCAS(a.status, kStatusOk, kStatusFlagTimeout);
          break;
        }
        __nanosleep(100);
      }
    }
    __syncthreads();
  }
  if (a.seg_cnt != nullptr && a.group_regions) {
    // every group owns a fixed region; its row count is the cursor the senders advanced
    for (int g = threadIdx.x; g < a.G; g += blockDim.x) {
      const int c = __ldcg(a.seg_cnt + g);
      s_start[g] = g * a.seg_cap;
      s_cnt[g] = c < 0 ? 0 : min(c, a.seg_cap);
    }
  } else if (a.seg_cnt != nullptr) {
    // (s, g) -> first row: region s starts at s * seg_cap and is packed group after group
    for (int s = threadIdx.x; s < S; s += blockDim.x) {
      int run = s * a.seg_cap;
      for (int g = 0; g < a.G; ++g) {
        const int c = __ldcg(a.seg_cnt + s * a.G + g);
        s_start[s * a.G + g] = run;
        s_cnt[s * a.G + g] = c < 0 ? 0 : min(c, (s + 1) * a.seg_cap - run);
        run += s_cnt[s * a.G + g];
      }
    }
  } else if (a.offs != nullptr) {
    for (int i = threadIdx.x; i < a.G; i += blockDim.x) {
      const int o0 = a.offs[i], o1 = a.offs[i + 1];
      s_start[i] = o0;
      s_cnt[i] = o1 > o0 ? o1 - o0 : 0;
    }
  } else if (threadIdx.x == 0) {
    s_start[0] = 0;
    s_cnt[0] = a.T;
  }
  if (warp == 1) {
    if (PAIR) {
      tmem_alloc_pair(smem_u32(tmem_slot), C::kTmemCols);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(smem_u32(tmem_slot), C::kTmemCols);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();      // both CTAs' barriers are initialised before either is signalled from outside
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (threadIdx.x == 0) trace_stamp(a, 1);

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      WorkWalker tw;
      tw.init(s_start, s_cnt, a.G, S, MT, BN, kblocks, a.splitk, a.streamk, work_cta, work_grid);
      trace_stamp(a, 13);
      if (a.n_wait > 0) asm volatile("fence.proxy.async;" ::: "memory");  // peers' generic stores -> TMA reads
      const uint64_t pol_w = l2_policy_evict_first();
      const uint64_t pol_x = l2_policy_evict_last();
      trace_stamp(a, 14);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      bool traced = false;
      unsigned long long shard_ready = 0;     // bit s: shard s of X has landed (all-gather prologue)
      const int shard_want = (a.shard_rows > 0) ? *a.wait_epoch + 1 : 0;
      WorkUnit u;
      while (ok && tw.next(u)) {
        const int ntok_ = u.ntok;
        // pair mode: this CTA stages the token rows of its half of the MMA's N extent (the even CTA the first half)
        int n_eff = (u.ntok + 31) & ~31;
        n_eff = n_eff > BN ? BN : n_eff;
        const int xrow = u.row0 + (PAIR ? static_cast<int>(prank) * (n_eff / 2) : 0);
        const int wrow = u.g * a.w_rows + (PAIR ? 2 * u.m + static_cast<int>(prank) : u.m) * kBM;
        const int kb0 = u.kb0, kb1 = u.kb1;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1, abort_word, bar_budget)) { ok = false; break; }
          if (a.trace != nullptr && !traced) trace_stamp(a, 15);
          // pair mode: the bytes of both CTAs are counted on the even CTA's barrier, which its producer arms
          const uint32_t fb = PAIR ? mapa_rank(smem_u32(&full_bar[stage]), 0) : smem_u32(&full_bar[stage]);
          uint8_t* st = smem + stage * C::kStageBytes;
          if (!PAIR) mbar_expect_tx(fb, C::kStageBytes);
          else if (leader) mbar_expect_tx(smem_u32(&full_bar[stage]), 2 * C::kStageBytes);
          auto load = [&](uint32_t dst, const CUtensorMap* m, int x, int y, uint64_t pol) {
            if (PAIR) tma_load_2d_pair(dst, m, x, y, fb, pol);
            else tma_load_2d(dst, m, x, y, fb, pol);
          };
          if (a.w_blocked) {
            // blocked weights: the map is a [tiles * K blocks * 128, 64] matrix, tile (t, kb) starts at row (t * kblocks + kb) * 128
            const int wt = wrow / kBM;
            load(smem_u32(st), &tmW, 0, (wt * kblocks + kb) * kBM, pol_w);
            if (EPI == EPI_SWIGLU) load(smem_u32(st + C::kABytes), &tmW, 0, ((wt + a.F / kBM) * kblocks + kb) * kBM, pol_w);
          } else {
            load(smem_u32(st), &tmW, kb * kBK, wrow, pol_w);
            if (EPI == EPI_SWIGLU) load(smem_u32(st + C::kABytes), &tmW, kb * kBK, wrow + a.F, pol_w);
          }
          if (a.shard_rows > 0 && kb == kb0) {
            // the weight tile is already on its way; the token tile may only be fetched once every peer whose rows
            // it covers has published them (the peers' stores are generic-proxy writes: fence before the TMA read)
            const int s0 = u.row0 / a.shard_rows;
            const int s1 = min((u.row0 + ntok_ - 1) / a.shard_rows, a.n_wait - 1);
            for (int sh = s0; sh <= s1 && ok; ++sh) {
              if ((shard_ready >> sh) & 1ull) continue;
              const long long t0 = clock64();
              while (ld_acquire_sys(a.wait_flags + sh) < shard_want) {
                if (*reinterpret_cast<volatile int*>(abort_word) != 0 || clock64() - t0 > a.flag_cycles ||
                    (a.status != nullptr && *reinterpret_cast<volatile int*>(a.status) != kStatusOk)) {
                  if (a.status != nullptr) atomicCAS(a.status, kStatusOk, kStatusFlagTimeout);
                  *abort_word = 1;
                  ok = false;
                  break;
                }
                __nanosleep(64);
              }
              if (ok) {
                shard_ready |= 1ull << sh;
                asm volatile("fence.proxy.async;" ::: "memory");
              }
            }
            if (!ok) break;
          }
          load(smem_u32(st + C::kNumA * C::kABytes), &tmX, kb * kBK, xrow, pol_x);
          if (a.trace != nullptr && !traced) { trace_stamp(a, 2); traced = true; }
          if (++stage == C::kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (pair mode: the even CTA's only)
    if (lane == 0 && leader) {
      WorkWalker tw;
      tw.init(s_start, s_cnt, a.G, S, MT, BN, kblocks, a.splitk, a.streamk, work_cta, work_grid);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      WorkUnit u;
      for (; ok && tw.next(u); ++it) {
        const int buf = it % C::kAccBufs;
        const uint32_t bphase = (it / C::kAccBufs) & 1;
        if (PAIR) {
          if (!mbar_wait_cluster(smem_u32(&tempty_bar[buf]), bphase ^ 1, abort_word, bar_budget)) { ok = false; break; }
        } else if (!mbar_wait(smem_u32(&tempty_bar[buf]), bphase ^ 1, abort_word, bar_budget)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d0 = tmem_base + buf * C::kAccCols;
        // a ragged token tile only pays for the MMA columns it has (N is a run-time field of the instruction)
        const int nq = PAIR ? 32 : 16;
        int n_eff = (u.ntok + nq - 1) & ~(nq - 1);
        n_eff = n_eff < nq ? nq : (n_eff > BN ? BN : n_eff);
        const uint32_t idesc = umma_idesc_bf16(PAIR ? 2 * kBM : kBM, n_eff);
        const int kb0 = u.kb0, kb1 = u.kb1;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(smem_u32(&full_bar[stage]), phase, abort_word, bar_budget)) { ok = false; break; }
          if (a.trace != nullptr && it == 0 && kb == kb0) trace_stamp(a, 3);
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * C::kStageBytes);
          const uint64_t da = umma_desc_sw128(sa);
          const uint64_t db = umma_desc_sw128(sa + C::kNumA * C::kABytes);
#pragma unroll
          for (int k = 0; k < kBK / kUmmaK; ++k) {
            const uint32_t acc = (kb > kb0 || k > 0) ? 1u : 0u;
            // advancing K by 16 bf16 = 32 bytes inside the 128-byte swizzle span: +2 in the (>>4) address field
            if (PAIR) umma_f16_pair(d0, da + 2 * k, db + 2 * k, idesc, acc);
            else umma_f16(d0, da + 2 * k, db + 2 * k, idesc, acc);
            if (EPI == EPI_SWIGLU) {
              const uint64_t da2 = umma_desc_sw128(sa + C::kABytes);
              if (PAIR) umma_f16_pair(d0 + BN, da2 + 2 * k, db + 2 * k, idesc, acc);
              else umma_f16(d0 + BN, da2 + 2 * k, db + 2 * k, idesc, acc);
            }
          }
          // frees the smem stage when these MMAs retire (pair mode: in both CTAs, one arrival each)
          if (PAIR) {
            umma_commit_pair(mapa_rank(smem_u32(&empty_bar[stage]), 0));
            umma_commit_pair(mapa_rank(smem_u32(&empty_bar[stage]), 1));
          } else {
            umma_commit(smem_u32(&empty_bar[stage]));
          }
          if (++stage == C::kStages) { stage = 0; phase ^= 1; }
        }
        if (ok) {
          if (PAIR) {
            umma_commit_pair(mapa_rank(smem_u32(&tfull_bar[buf]), 0));
            umma_commit_pair(mapa_rank(smem_u32(&tfull_bar[buf]), 1));
          } else {
            umma_commit(smem_u32(&tfull_bar[buf]));
            trace_stamp(a, 4);
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;                 // TMEM lane quarter this warp may read
    const int row = q * 32 + lane;          // accumulator lane = feature within the tile
    const int et = threadIdx.x - 64;        // 0..127
    WorkWalker tw;
    tw.init(s_start, s_cnt, a.G, S, MT, BN, kblocks, a.splitk, a.streamk, work_cta, work_grid);
    constexpr size_t kSlotF4 = static_cast<size_t>(C::kNumA) * (BN / 4) * kBM;   // float4 per workspace slot
    int it = 0;
    bool ok = true;
    WorkUnit u;
    for (; ok && tw.next(u); ++it) {
      const int m = PAIR ? 2 * u.m + static_cast<int>(prank) : u.m, tok_base = u.row0, ntok = u.ntok;
      const int buf = it % C::kAccBufs;
      const uint32_t bphase = (it / C::kAccBufs) & 1;
      if (!mbar_wait(smem_u32(&tfull_bar[buf]), bphase, abort_word, bar_budget)) { ok = false; break; }
      if (et == 0) trace_stamp(a, 5);
      tc_fence_after();
      const uint32_t t0 = tmem_base + buf * C::kAccCols + (static_cast<uint32_t>(q * 32) << 16);
      const int f = m * kBM + row;
      const bool f_ok = f < a.F;
      const int nchunk = (ntok + 31) / 32;        // 32-token chunks that hold valid tokens

      // A tile computed by several units (split-K, or a stream-K share boundary inside the tile): every unit parks
      // its fp32 partial accumulator(s) in its workspace slot; the last one to arrive adds them all up and runs the
      // epilogue. Slot layout: [accumulator (gate, up)][chunk of 4 tokens][feature row] float4.
      const bool shared_tile = u.ncontrib > 1;
      if (shared_tile) {
        float4* wsp = reinterpret_cast<float4*>(a.ws) + static_cast<size_t>(u.slot) * kSlotF4;
#pragma unroll 1
        for (int c = 0; c < nchunk; ++c) {
#pragma unroll
          for (int h = 0; h < C::kNumA; ++h) {
            uint32_t v[32];
            tmem_ld32(t0 + h * BN + c * 32, v);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              float4 o;
              o.x = __uint_as_float(v[4 * j]); o.y = __uint_as_float(v[4 * j + 1]);
              o.z = __uint_as_float(v[4 * j + 2]); o.w = __uint_as_float(v[4 * j + 3]);
              wsp[(static_cast<size_t>(h) * (BN / 4) + c * 8 + j) * kBM + row] = o;
            }
          }
        }
        tc_fence_before();
        if (PAIR) mbar_arrive_cluster(mapa_rank(smem_u32(&tempty_bar[buf]), 0));
        else mbar_arrive(smem_u32(&tempty_bar[buf]));
        __threadfence();
        named_bar_sync(1, kEpiThreads);
        if (et == 0) {
          const int old = atomicAdd(&a.counters[u.tile], 1);
          const int last = (old == u.ncontrib - 1);
          if (last) a.counters[u.tile] = 0;  // self-resetting for the next launch
          *last_flag = last;
        }
        named_bar_sync(1, kEpiThreads);
        const bool reduce_here = (*last_flag != 0);
        named_bar_sync(1, kEpiThreads);      // everyone has read last_flag before the next tile rewrites it
        if (!reduce_here) continue;
        __threadfence();
      }

#pragma unroll 1
      for (int c = 0; c < nchunk; ++c) {             // chunks past the last valid token are never read
        float acc[32];
        const int jmax = min(32, ntok - c * 32);
        // Residual rows of this chunk are requested first, so that they travel together with the partial tiles /
        // the TMEM read below instead of after them. Y may alias R (in-place update of the residual stream): all
        // loads of a chunk are issued before its first store, and chunks cover disjoint tokens.
        float r[32];
        const bool vec = (EPI == EPI_PLAIN || (EPI == EPI_SWIGLU && C::kEpiStageBytes > 0)) && a.epi_vec != 0;
        const bool has_r = (EPI == EPI_PLAIN) && a.R != nullptr && f_ok && !vec;
        if (has_r) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const long long t = tok_base + c * 32 + j;
            r[j] = (j < jmax) ? __bfloat162float(a.R[t * a.ldr + f]) : 0.f;
          }
        }
        if (shared_tile) {
          float up[(EPI == EPI_SWIGLU) ? 32 : 1];
#pragma unroll
          for (int j = 0; j < 32; ++j) acc[j] = 0.f;
          if (EPI == EPI_SWIGLU) {
#pragma unroll
            for (int j = 0; j < 32; ++j) up[j] = 0.f;
          }
          for (int s = 0; s < u.ncontrib; ++s) {
            const float4* w0 = reinterpret_cast<const float4*>(a.ws) + static_cast<size_t>(tw.contrib_slot(u, s)) * kSlotF4;
            float4 o0[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) o0[j] = __ldcg(&w0[(c * 8 + j) * kBM + row]);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              acc[4 * j] += o0[j].x; acc[4 * j + 1] += o0[j].y; acc[4 * j + 2] += o0[j].z; acc[4 * j + 3] += o0[j].w;
            }
            if (EPI == EPI_SWIGLU) {
#pragma unroll
              for (int j = 0; j < 8; ++j) o0[j] = __ldcg(&w0[(static_cast<size_t>(BN / 4) + c * 8 + j) * kBM + row]);
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                up[4 * j] += o0[j].x; up[4 * j + 1] += o0[j].y; up[4 * j + 2] += o0[j].z; up[4 * j + 3] += o0[j].w;
              }
            }
          }
          if (EPI == EPI_SWIGLU) {
#pragma unroll
            for (int j = 0; j < 32; ++j) acc[j] = (acc[j] / (1.f + __expf(-acc[j]))) * up[j];
          }
        } else {
          uint32_t v[32];
          tmem_ld32(t0 + c * 32, v);
          if (EPI == EPI_SWIGLU) {
            uint32_t uu[32];
            tmem_ld32(t0 + BN + c * 32, uu);
            tmem_ld_wait();
            if (et == 0 && c == 0) trace_stamp(a, 8);
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const float g = __uint_as_float(v[j]);
              const float up = __uint_as_float(uu[j]);
              acc[j] = (g / (1.f + __expf(-g))) * up;
            }
          } else {
            tmem_ld_wait();
            if (et == 0 && c == 0) trace_stamp(a, 8);
#pragma unroll
            for (int j = 0; j < 32; ++j) acc[j] = __uint_as_float(v[j]);
          }
          if (c == nchunk - 1) {
            // all of this thread's TMEM reads are done: hand the accumulator buffer back to the MMA warp
            tc_fence_before();
            if (PAIR) mbar_arrive_cluster(mapa_rank(smem_u32(&tempty_bar[buf]), 0));
            else mbar_arrive(smem_u32(&tempty_bar[buf]));
          }
        }
        if ((EPI == EPI_PLAIN || EPI == EPI_SWIGLU) && vec) {
          if (jmax <= 0) continue;                   // uniform over the CTA: no barrier is skipped by some threads only
          // transpose the chunk: thread = feature row writes its 32 token values; then thread (token, 8 features)
          const int fg = et & 15, tk0 = et >> 4;
          const int f0 = m * kBM + fg * 8;
          // QKV epilogue: the positions and cache slots of this thread's four tokens are requested before the
          // transposition, so that their latency overlaps it
          int pos4[4] = {0, 0, 0, 0};
          long long slot4[4] = {-1, -1, -1, -1};
          if (a.rope_table != nullptr && f0 < a.F) {
            const bool kv_tile = f0 / a.hd >= a.n_q;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const int j = tk0 + q * 8;
              if (j < jmax) {
                const long long t = tok_base + c * 32 + j;
                pos4[q] = __ldg(a.positions + t);
                if (kv_tile && a.slots != nullptr) slot4[q] = __ldg(a.slots + t);
              }
            }
          }
          // the residual cells of this thread (the same cells it stores to when Y aliases R) are requested before the
          // transposition as well
          uint4 rr[4];
          if (a.R != nullptr && f0 < a.F) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const int j = tk0 + q * 8;
              const long long t = tok_base + c * 32 + j;
              rr[q] = (j < jmax) ? *reinterpret_cast<const uint4*>(a.R + t * a.ldr + f0) : make_uint4(0, 0, 0, 0);
            }
          }
#pragma unroll
          for (int j = 0; j < 32; ++j) epi_stage[j * kBM + row] = acc[j];
          if (et == 0 && c == 0) trace_stamp(a, 9);
          named_bar_sync(1, kEpiThreads);
          if (et == 0 && c == 0) trace_stamp(a, 10);
          const bool simple = a.rope_table == nullptr && a.R == nullptr && a.rs_bases == nullptr && !a.y_f32;
          if (simple && f0 < a.F) {
            // the common case (bf16 rows straight to Y: SwiGLU activations, plain linears) without any of the
            // variants' branches inside the loop: four independent load -> pack -> store chains
            __nv_bfloat16* ybase = reinterpret_cast<__nv_bfloat16*>(a.Y) + (tok_base + c * 32) * a.ldy + f0;
            float4 x0[4], x1[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const int j = tk0 + q * 8;
              x0[q] = *reinterpret_cast<const float4*>(&epi_stage[j * kBM + fg * 8]);
              x1[q] = *reinterpret_cast<const float4*>(&epi_stage[j * kBM + fg * 8 + 4]);
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const int j = tk0 + q * 8;
              uint4 pk;
              __nv_bfloat162* pp = reinterpret_cast<__nv_bfloat162*>(&pk);
              pp[0] = __floats2bfloat162_rn(x0[q].x, x0[q].y);
              pp[1] = __floats2bfloat162_rn(x0[q].z, x0[q].w);
              pp[2] = __floats2bfloat162_rn(x1[q].x, x1[q].y);
              pp[3] = __floats2bfloat162_rn(x1[q].z, x1[q].w);
              if (j < jmax) *reinterpret_cast<uint4*>(ybase + static_cast<long long>(j) * a.ldy) = pk;
            }
          } else if (f0 < a.F && a.rope_table == nullptr) {
            // residual / fp32 output / reduce-scatter variants, each as four independent load -> combine -> store
            // chains: the variant is chosen outside the loops, stores are predicated on the token being valid
            float o[4][8];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const int j = tk0 + q * 8;
              const float4 x0 = *reinterpret_cast<const float4*>(&epi_stage[j * kBM + fg * 8]);
              const float4 x1 = *reinterpret_cast<const float4*>(&epi_stage[j * kBM + fg * 8 + 4]);
              o[q][0] = x0.x; o[q][1] = x0.y; o[q][2] = x0.z; o[q][3] = x0.w;
              o[q][4] = x1.x; o[q][5] = x1.y; o[q][6] = x1.z; o[q][7] = x1.w;
            }
            if (a.R != nullptr) {
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const __nv_bfloat162* rp = reinterpret_cast<const __nv_bfloat162*>(&rr[q]);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  const float2 rf = __bfloat1622float2(rp[i]);
                  o[q][2 * i] += rf.x;
                  o[q][2 * i + 1] += rf.y;
                }
              }
            }
            if (a.y_f32) {
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const int j = tk0 + q * 8;
                float* yp = reinterpret_cast<float*>(a.Y) + (tok_base + c * 32 + j) * a.ldy + f0;
                if (j < jmax) {
                  *reinterpret_cast<float4*>(yp) = make_float4(o[q][0], o[q][1], o[q][2], o[q][3]);
                  *reinterpret_cast<float4*>(yp + 4) = make_float4(o[q][4], o[q][5], o[q][6], o[q][7]);
                }
              }
            } else {
              __nv_bfloat16* dst[4];
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const int j = tk0 + q * 8;
                const long long t = tok_base + c * 32 + j;
                if (a.rs_bases != nullptr) {
                  // reduce-scatter: the row goes to slot rs_slot of the partial buffer of the rank that owns it
                  const int tt = j < jmax ? static_cast<int>(t) : tok_base;      // keep the table index in range
                  const int owner = tt / a.rs_rows;
                  const long long lrow = static_cast<long long>(a.rs_slot) * a.rs_cap + (tt - owner * a.rs_rows);
                  dst[q] = static_cast<__nv_bfloat16*>(a.rs_bases[owner]) + lrow * a.ldy + f0;
                } else {
                  dst[q] = reinterpret_cast<__nv_bfloat16*>(a.Y) + t * a.ldy + f0;
                }
              }
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                uint4 pk;
                __nv_bfloat162* pp = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
                for (int i = 0; i < 4; ++i) pp[i] = __floats2bfloat162_rn(o[q][2 * i], o[q][2 * i + 1]);
                if (tk0 + q * 8 < jmax) *reinterpret_cast<uint4*>(dst[q]) = pk;
              }
            }
          } else if (f0 < a.F) {
            // QKV epilogue: neox RoPE on the q and k heads, q to Y, K / V into the paged cache. A 128-feature tile
            // holds whole heads (hd = 64 or 128), so the rotation partner of a feature (d +- hd / 2) sits in the same
            // shared-memory chunk. Everything that depends on the thread's features only is computed once.
            const int half = a.hd >> 1;
            const int d0 = f0 % a.hd;                          // first of this thread's 8 features inside its head
            const int head = f0 / a.hd;
            const bool rot = head < a.n_q + a.n_kv;
            const bool lower = d0 < half;
            const int pf = fg * 8 + (lower ? half : -half);     // partner features inside the tile
            const int kvh = head - a.n_q;
            __nv_bfloat16* const cache = kvh < a.n_kv ? a.kcache : a.vcache;
            const int hh = kvh < a.n_kv ? kvh : kvh - a.n_kv;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const int j = tk0 + q * 8;
              const long long t = tok_base + c * 32 + j;
              const float4 x0 = *reinterpret_cast<const float4*>(&epi_stage[j * kBM + fg * 8]);
              const float4 x1 = *reinterpret_cast<const float4*>(&epi_stage[j * kBM + fg * 8 + 4]);
              float o[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
              if (rot) {
                const float4 p0 = *reinterpret_cast<const float4*>(&epi_stage[j * kBM + pf]);
                const float4 p1 = *reinterpret_cast<const float4*>(&epi_stage[j * kBM + pf + 4]);
                const float pr[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
                int pos = pos4[q];
                pos = pos < 0 ? 0 : (pos >= a.rope_max_pos ? a.rope_max_pos - 1 : pos);
                const float4* cs = reinterpret_cast<const float4*>(a.rope_table + static_cast<long long>(pos) * half +
                                                                   (lower ? d0 : d0 - half));
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  const float4 v = __ldg(cs + i);      // (cos, sin) of two consecutive rotation pairs
                  // the accumulator is rounded to bf16 before the rotation, as the unfused path stores and re-reads it
                  const float a0 = __bfloat162float(__float2bfloat16(o[2 * i])), b0 = __bfloat162float(__float2bfloat16(pr[2 * i]));
                  const float a1 = __bfloat162float(__float2bfloat16(o[2 * i + 1])), b1 = __bfloat162float(__float2bfloat16(pr[2 * i + 1]));
                  o[2 * i] = lower ? a0 * v.x - b0 * v.y : a0 * v.x + b0 * v.y;
                  o[2 * i + 1] = lower ? a1 * v.z - b1 * v.w : a1 * v.z + b1 * v.w;
                }
              }
              uint4 pk;
              __nv_bfloat162* pp = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
              for (int i = 0; i < 4; ++i) pp[i] = __floats2bfloat162_rn(o[2 * i], o[2 * i + 1]);
              if (head < a.n_q) {
                if (j < jmax) *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(a.Y) + t * a.ldy + f0) = pk;
              } else {
                const long long slot = slot4[q];
                if (j < jmax && slot >= 0) *reinterpret_cast<uint4*>(cache + (slot * a.n_kv + hh) * a.hd + d0) = pk;
              }
            }
          }
          if (et == 0 && c == 0) trace_stamp(a, 11);
          named_bar_sync(1, kEpiThreads);            // the stage is free again for the next chunk / tile
          if (et == 0 && c == 0) trace_stamp(a, 12);
          continue;
        }
        if (EPI == EPI_COMBINE && a.epi_vec != 0) {
          if (jmax <= 0) continue;                   // uniform over the CTA
          // same transposition as the plain epilogue: thread (token lane, 8 features) scales its 8 values by the
          // row's router weight and stores 16 bytes into the destination row named by the record. The four records
          // of the thread are requested before the transposition, so that their latency overlaps it.
          const int fg = et & 15, tk0 = et >> 4;
          const int f0 = m * kBM + fg * 8;
          int4 rec4[4];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int j = tk0 + q * 8;
            rec4[q] = (j < jmax) ? __ldg(&a.recs[tok_base + c * 32 + j]) : make_int4(0, -1, 0, 0);
          }
#pragma unroll
          for (int j = 0; j < 32; ++j) epi_stage[j * kBM + row] = acc[j];
          named_bar_sync(1, kEpiThreads);
          if (f0 < a.F) {
            uint4 pk[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const int j = tk0 + q * 8;
              const float w = __int_as_float(rec4[q].z);
              const float4 x0 = *reinterpret_cast<const float4*>(&epi_stage[j * kBM + fg * 8]);
              const float4 x1 = *reinterpret_cast<const float4*>(&epi_stage[j * kBM + fg * 8 + 4]);
              __nv_bfloat162* pp = reinterpret_cast<__nv_bfloat162*>(&pk[q]);
              pp[0] = __floats2bfloat162_rn(x0.x * w, x0.y * w);
              pp[1] = __floats2bfloat162_rn(x0.z * w, x0.w * w);
              pp[2] = __floats2bfloat162_rn(x1.x * w, x1.y * w);
              pp[3] = __floats2bfloat162_rn(x1.z * w, x1.w * w);
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              if (rec4[q].y < 0) continue;
              const long long off = static_cast<long long>(rec4[q].y) * a.ldy + f0;
              if (a.fanout <= 1) {
                *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(a.bases[rec4[q].x]) + off) = pk[q];
              } else {
                const int g0 = rec4[q].x / a.fanout * a.fanout;
                for (int i = 0; i < a.fanout; ++i)
                  *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(a.bases[g0 + i]) + off) = pk[q];
              }
            }
          }
          named_bar_sync(1, kEpiThreads);            // the stage is free again for the next chunk / tile
          continue;
        }
        if (!f_ok) continue;
        if (EPI == EPI_COMBINE) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            if (j >= jmax) break;
            const int4 rec = __ldg(&a.recs[tok_base + c * 32 + j]);
            if (rec.y < 0) continue;
            const __nv_bfloat16 val = __float2bfloat16(acc[j] * __int_as_float(rec.z));
            if (a.fanout <= 1) {
              (reinterpret_cast<__nv_bfloat16*>(a.bases[rec.x]) + static_cast<long long>(rec.y) * a.ldy)[f] = val;
            } else {
              // tensor-parallel senders: every member of the sender's TP group keeps the full residual stream
              const int g0 = rec.x / a.fanout * a.fanout;
              for (int i = 0; i < a.fanout; ++i)
                (reinterpret_cast<__nv_bfloat16*>(a.bases[g0 + i]) + static_cast<long long>(rec.y) * a.ldy)[f] = val;
            }
          }
        } else {
          if (has_r) {
#pragma unroll
            for (int j = 0; j < 32; ++j) acc[j] += r[j];
          }
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            if (j >= jmax) break;
            const long long t = tok_base + c * 32 + j;
            const float v = acc[j];
            if (a.y_f32) reinterpret_cast<float*>(a.Y)[t * a.ldy + f] = v;
            else reinterpret_cast<__nv_bfloat16*>(a.Y)[t * a.ldy + f] = __float2bfloat16(v);
          }
        }
      }
    }
  }

  if (threadIdx.x == 64) trace_stamp(a, 6);
  // ---------------------------------------------------------------- completion: signal peers, advance epochs
  if (a.done_ticket != nullptr && warp >= 2) {
    // every epilogue thread makes its (possibly remote) stores visible system-wide, then the CTA takes a ticket.
    // The last CTA of the grid publishes this call's epoch to every destination and advances the gate's epoch
    // (by then every CTA has long read it). A launch that signals nobody (it only advances its gate's epoch) has
    // nothing to publish: its output is consumed in stream order.
    if (a.n_signal > 0) __threadfence_system();
    named_bar_sync(1, kEpiThreads);
    if (threadIdx.x == 64) {
      const int old = atomicAdd(a.done_ticket, 1);
      if (old == static_cast<int>(gridDim.x) - 1) {
        for (int i = 0; i < a.clear_n; ++i) a.clear_ptr[i] = 0;
        __threadfence_system();
        if (a.n_signal > 0) {
          const int epoch = *a.signal_epoch + 1;
          for (int i = 0; i < a.n_signal; ++i) st_relaxed_sys(a.signal_ptrs[i] + a.signal_slot, epoch);   // fenced above
          *a.signal_epoch = epoch;
        }
        if (a.n_wait > 0) *a.wait_epoch = *a.wait_epoch + 1;
        *a.done_ticket = 0;
        __threadfence();
      }
    }
  }

  // ---------------------------------------------------------------- tear-down
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) trace_stamp(a, 7);
  if (*abort_word) {
    if (threadIdx.x == 0 && a.status != nullptr) atomicCAS(a.status, kStatusOk, kStatusBarrierTimeout);
    // give copies that may still be in flight time to land before shared memory is released
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (PAIR) cluster_sync_all();      // neither CTA leaves (or frees TMEM) while the other may still signal or use it
  if (warp == 1) {
    tc_fence_after();
    if (PAIR) tmem_dealloc_pair(tmem_base, C::kTmemCols);
    else tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(p);
    }
  }
  return fn;
}

// Tensor map over a row-major [rows, K] bf16 matrix with a [box_rows, 64] box and the 128-byte swizzle.
static int make_map_2d(CUtensorMap* map, const void* ptr, long long rows, long long K, long long ld_elems,
                       int box_rows) {
  EncodeTiledFn enc = get_encode_fn();
  if (enc == nullptr) return -1;
  cuuint64_t gdim[2] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(rows)};
  cuuint64_t gstride[1] = {static_cast<cuuint64_t>(ld_elems) * 2};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(kBK), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), gdim, gstride, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -2;
}

static int num_sms() { return device_num_sms(); }

template <int BN, int EPI, bool PAIR = false>
static int launch(const CUtensorMap& tmW, const CUtensorMap& tmX, const GemmArgs& a, int max_tiles,
                  cudaStream_t stream) {
  using C = Cfg<BN, EPI, PAIR>;
  static PerDeviceOnce configured;
  const int crc = configured.run([] {
    return static_cast<int>(cudaFuncSetAttribute(gemm_kernel<BN, EPI, PAIR>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 C::kSmemBytes));
  });
  if (crc != 0) return crc;
  if (!PAIR) {
    int grid = num_sms();
    if (max_tiles < grid) grid = max_tiles;
    if (grid < 1) grid = 1;
    return static_cast<int>(launch_kernel(gemm_kernel<BN, EPI, false>, dim3(grid), dim3(kThreads), C::kSmemBytes, stream,
                                          tmW, tmX, a));
  }
  // one cluster of two CTAs (two SMs of a TPC) per work tile
  int pairs = num_sms() / 2;
  if (max_tiles < pairs) pairs = max_tiles;
  if (pairs < 1) pairs = 1;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(2 * pairs, 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = C::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return static_cast<int>(cudaLaunchKernelEx(&cfg, gemm_kernel<BN, EPI, true>, tmW, tmX, a));
}

}  // namespace dmoe

using namespace dmoe;

extern "C" int dmoe_gemm_pick_bn(int tokens_per_group_hint, int epi) {
  const int cap = (epi == EPI_SWIGLU) ? 128 : 256;
  int bn = 32;
  while (bn < tokens_per_group_hint && bn < cap) bn *= 2;
  return bn;
}

extern "C" long long dmoe_gemm_workspace_bytes(int T, int F, int bn, int splitk) {
  if (splitk <= 1) return 0;
  const long long mt = (F + kBM - 1) / kBM;
  const long long nt = (T + bn - 1) / bn;
  return mt * nt * splitk * kBM * bn * 4;
}

extern "C" int dmoe_gemm(const DmoeGemm* d, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (d->G < 1 || d->G > kMaxSeg || d->K % 8 != 0 || d->F < 1 || d->T < 0) return -10;
  if (d->T == 0) return 0;
  const int epi = d->epi;
  int bn = d->bn;
  if (bn == 0) bn = dmoe_gemm_pick_bn((d->T + d->G - 1) / d->G, epi);
  if (bn != 32 && bn != 64 && bn != 128 && bn != 256) return -11;
  const bool pair = d->pair != 0;
  if (pair && (bn < 128 || d->splitk > 1)) return -11;
  int splitk = d->splitk < 1 ? 1 : d->splitk;
  const int kblocks = (d->K + kBK - 1) / kBK;
  if (splitk > kblocks) splitk = kblocks;
  if (splitk > 1) {
    // no split may be empty
    const int per = (kblocks + splitk - 1) / splitk;
    splitk = (kblocks + per - 1) / per;
  }
  if (splitk > 1 && (epi == EPI_SWIGLU || d->offs != nullptr || d->S > 0 || d->group_regions || d->ws == nullptr || d->counters == nullptr)) return -12;
  if (splitk > 1 && dmoe_gemm_workspace_bytes(d->T, d->F, bn, splitk) > d->ws_bytes) return -13;
  // stream-K: one contiguous share of the K-block iterations per CTA; needs two partial-tile slots per CTA and one
  // counter per tile. Where the scratch is too small the launch quietly keeps whole tiles (a performance matter only).
  int streamk = (d->streamk != 0 && !pair && splitk == 1 && d->ws != nullptr && d->counters != nullptr) ? 1 : 0;
  if (epi == EPI_COMBINE && (d->recs == nullptr || d->bases == nullptr)) return -14;

  GemmArgs a;
  a.offs = d->offs;
  a.G = d->G; a.T = d->T; a.F = d->F; a.K = d->K;
  a.w_rows = (epi == EPI_SWIGLU) ? 2 * d->F : d->F;
  a.Y = d->Y; a.ldy = d->ldy; a.y_f32 = d->y_f32;
  a.R = static_cast<const __nv_bfloat16*>(d->R); a.ldr = d->ldr;
  a.recs = static_cast<const int4*>(d->recs);
  a.bases = static_cast<void* const*>(d->bases);
  a.splitk = splitk; a.streamk = 0; a.ws = static_cast<float*>(d->ws); a.counters = d->counters;
  a.status = d->status;
  a.seg_cnt = d->seg_cnt; a.S = d->S; a.seg_cap = d->seg_cap;
  a.wait_flags = d->wait_flags; a.n_wait = d->n_wait; a.wait_epoch = d->wait_epoch;
  a.signal_ptrs = reinterpret_cast<int* const*>(d->signal_ptrs); a.n_signal = d->n_signal;
  a.signal_slot = d->signal_slot; a.signal_epoch = d->signal_epoch; a.done_ticket = d->done_ticket;
  a.fanout = d->fanout; a.group_regions = d->group_regions; a.clear_n = d->clear_n; a.clear_ptr = d->clear_ptr;
  {
    const auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    const long long ymod = d->y_f32 ? 4 : 8;
    a.epi_vec = ((epi == EPI_PLAIN || epi == EPI_SWIGLU) && d->F % 8 == 0 && d->ldy % ymod == 0 && al16(d->Y) &&
                 (d->R == nullptr || (d->ldr % 8 == 0 && al16(d->R)))) ? 1 : 0;
    // combine: the destination bases live in a device table; the caller states that all of them are 16-byte aligned
    if (epi == EPI_COMBINE && d->combine_vec != 0 && d->F % 8 == 0 && d->ldy % 8 == 0) a.epi_vec = 1;
  }
  a.shard_rows = d->shard_rows;
  a.flag_cycles = g_dmoe_flag_wait_cycles;
  a.rs_bases = static_cast<void* const*>(d->rs_bases);
  a.rs_rows = d->rs_rows; a.rs_slot = d->rs_slot; a.rs_cap = d->rs_cap;
  a.rope_table = static_cast<const float2*>(d->rope_table);
  a.positions = d->positions; a.slots = d->slots;
  a.kcache = static_cast<__nv_bfloat16*>(d->kcache); a.vcache = static_cast<__nv_bfloat16*>(d->vcache);
  a.n_q = d->n_q; a.n_kv = d->n_kv; a.hd = d->hd; a.rope_max_pos = d->rope_max_pos;
  if (a.shard_rows < 0 || (a.shard_rows > 0 && (a.n_wait < 1 || a.n_wait > 64 || epi == EPI_SWIGLU || d->offs != nullptr ||
                                                 d->S > 0 || d->group_regions)))
    return -18;
  if (a.rs_bases != nullptr && (!a.epi_vec || d->y_f32 || a.rs_rows < 1 || a.rs_cap < a.rs_rows || a.rs_slot < 0 ||
                                d->R != nullptr || a.rope_table != nullptr))
    return -18;
  if (a.rope_table != nullptr &&
      (!a.epi_vec || d->y_f32 || d->R != nullptr || a.positions == nullptr || a.kcache == nullptr || a.vcache == nullptr ||
       (a.hd != 64 && a.hd != 128) || a.n_q < 1 || a.n_kv < 1 || (a.n_q + 2 * a.n_kv) * a.hd != d->F ||
       a.rope_max_pos < 1 || (reinterpret_cast<uintptr_t>(a.rope_table) & 15) != 0 ||
       (reinterpret_cast<uintptr_t>(a.kcache) & 15) != 0 || (reinterpret_cast<uintptr_t>(a.vcache) & 15) != 0))
    return -19;
  if (a.group_regions && (a.seg_cnt == nullptr || static_cast<long long>(a.G) * a.seg_cap > d->T)) return -16;
  if (!a.group_regions && a.S > 0 && (a.seg_cnt == nullptr || a.S * a.G > kMaxSeg || a.S * a.seg_cap > d->T)) return -16;
  if (a.S == 0 && a.G > kMaxSeg) return -16;
  if ((a.n_wait > 0 || a.n_signal > 0) && a.done_ticket == nullptr) return -17;
  if (a.n_wait > kThreads || (a.n_wait > 0 && (a.wait_flags == nullptr || a.wait_epoch == nullptr))) return -17;
  if (a.n_signal > 0 && (a.signal_ptrs == nullptr || a.signal_epoch == nullptr)) return -17;

  CUtensorMap tmW, tmX;
  const long long ldx = d->ldx > 0 ? d->ldx : d->K;
  a.trace = static_cast<unsigned long long*>(d->trace);
  a.w_blocked = d->w_blocked != 0;
  if (a.w_blocked) {
    // whole 128-row tiles and whole 64-element K blocks only; row coordinates must stay below 2^31
    const long long rows = static_cast<long long>(d->G) * a.w_rows * (d->K / kBK);
    if (d->K % kBK != 0 || d->F % kBM != 0 || rows >= (1ll << 31)) return -22;
    if (make_map_2d(&tmW, d->W, rows, kBK, kBK, kBM) != 0) return -20;
  } else if (make_map_2d(&tmW, d->W, static_cast<long long>(d->G) * a.w_rows, d->K, d->K, kBM) != 0) {
    return -20;
  }
  if (make_map_2d(&tmX, d->X, d->T, d->K, ldx, pair ? bn / 2 : bn) != 0) return -21;

  long long mt = (d->F + kBM - 1) / kBM;
  if (pair) mt = (mt + 1) / 2;
  // upper bound of the tile count (group sizes live on the device): every group may add one ragged tile
  long long max_tiles = mt * ((d->T + bn - 1) / bn + ((d->offs || d->S > 0 || d->group_regions) ? d->G * (d->S > 0 ? d->S : 1) : 0)) * splitk;
  if (max_tiles > (1 << 30)) max_tiles = 1 << 30;
  const int mtiles = static_cast<int>(max_tiles);
  if (streamk) {
    const long long grid = mtiles < num_sms() ? mtiles : num_sms();
    const long long slot_bytes = static_cast<long long>(epi == EPI_SWIGLU ? 2 : 1) * kBM * bn * 4;
    const long long n_counters = d->n_counters > 0 ? d->n_counters : 4096;
    if (grid * 2 * slot_bytes > d->ws_bytes || max_tiles / splitk > n_counters) streamk = 0;
  }
  a.streamk = streamk;

#define DMOE_LAUNCH(BN_, EPI_) return launch<BN_, EPI_>(tmW, tmX, a, mtiles, stream)
#define DMOE_LAUNCH_PAIR(BN_, EPI_) return launch<BN_, EPI_, true>(tmW, tmX, a, mtiles, stream)
  if (pair) {
    if (epi == EPI_PLAIN) {
      if (bn == 128) DMOE_LAUNCH_PAIR(128, EPI_PLAIN);
      DMOE_LAUNCH_PAIR(256, EPI_PLAIN);
    } else if (epi == EPI_SWIGLU) {
      if (bn == 128) DMOE_LAUNCH_PAIR(128, EPI_SWIGLU);
      DMOE_LAUNCH_PAIR(256, EPI_SWIGLU);
    } else if (epi == EPI_COMBINE) {
      if (bn == 128) DMOE_LAUNCH_PAIR(128, EPI_COMBINE);
      DMOE_LAUNCH_PAIR(256, EPI_COMBINE);
    }
    return -15;
  }
  if (epi == EPI_PLAIN) {
    switch (bn) {
      case 32: DMOE_LAUNCH(32, EPI_PLAIN);
      case 64: DMOE_LAUNCH(64, EPI_PLAIN);
      case 128: DMOE_LAUNCH(128, EPI_PLAIN);
      default: DMOE_LAUNCH(256, EPI_PLAIN);
    }
  } else if (epi == EPI_SWIGLU) {
    switch (bn) {
      case 32: DMOE_LAUNCH(32, EPI_SWIGLU);
      case 64: DMOE_LAUNCH(64, EPI_SWIGLU);
      case 128: DMOE_LAUNCH(128, EPI_SWIGLU);
      default: DMOE_LAUNCH(256, EPI_SWIGLU);   // gate + up accumulators fill TMEM: one buffer, epilogue not overlapped
    }
  } else if (epi == EPI_COMBINE) {
    switch (bn) {
      case 32: DMOE_LAUNCH(32, EPI_COMBINE);
      case 64: DMOE_LAUNCH(64, EPI_COMBINE);
      case 128: DMOE_LAUNCH(128, EPI_COMBINE);
      default: DMOE_LAUNCH(256, EPI_COMBINE);
    }
  }
#undef DMOE_LAUNCH
#undef DMOE_LAUNCH_PAIR
  return -15;
}

// ------------------------------------------------------------------------------------------------------------
// Allocation-free entry point (see dmoe_noalloc.h): the split-K scratch is a file-scope device array.
#include <stdio.h>

#include <mutex>

#include "dmoe_noalloc.h"

constexpr long long kNoallocCounterBytes = DMOE_NOALLOC_MAX_TILES * 4ll;
constexpr long long kNoallocBytes = DMOE_NOALLOC_WS_BYTES + kNoallocCounterBytes + 256;
// layout: [partial tiles | tile counters | status word]
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoallocBytes];

namespace {

constexpr int kMaxDevices = kMaxDevicesPerProcess;
std::mutex g_noalloc_mu;                                 // guards the two tables below
unsigned char* g_noalloc_ptr[kMaxDevices] = {nullptr};   // device address of the array, per device
cudaStream_t g_noalloc_stream[kMaxDevices] = {nullptr};  // stream of the last call, per device
thread_local char g_noalloc_error[256] = "";             // message of this thread's last failing call

#define NOALLOC_FAIL(code, ...)                                          \
  do {                                                                   \
    snprintf(g_noalloc_error, sizeof(g_noalloc_error), __VA_ARGS__);     \
    return (code);                                                       \
  } while (0)

// In host code `g_noalloc_scratch` is only a handle of the symbol, not a device address: the address a kernel may
// use has to be asked for, once per device, with that device current.
int noalloc_setup(int dev, unsigned char** out) {
  if (dev < 0 || dev >= kMaxDevices) NOALLOC_FAIL(DMOE_NOALLOC_E_SETUP, "device index %d is out of range", dev);
  std::lock_guard<std::mutex> lock(g_noalloc_mu);
  if (g_noalloc_ptr[dev] == nullptr) {
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr)
      NOALLOC_FAIL(DMOE_NOALLOC_E_SETUP, "cudaGetSymbolAddress failed on device %d: %s", dev, cudaGetErrorString(e));
    g_noalloc_ptr[dev] = static_cast<unsigned char*>(p);
  }
  *out = g_noalloc_ptr[dev];
  return 0;
}
}  // namespace

extern "C" const char* dmoe_noalloc_last_error(void) { return g_noalloc_error; }

extern "C" int dmoe_linear_noalloc(const void* W, const void* X, void* Y, int T, int F, int K, long long ldx,
                                   long long ldy, int bn, int splitk, void* stream_) {
  g_noalloc_error[0] = 0;
  if (W == nullptr || X == nullptr || Y == nullptr || T < 0 || F < 1 || K < 8 || K % 8 != 0)
    NOALLOC_FAIL(DMOE_NOALLOC_E_BAD_ARG, "bad argument (T=%d F=%d K=%d; K must be a multiple of 8)", T, F, K);
  if (ldx <= 0) ldx = K;
  if (ldy <= 0) ldy = F;
  if (ldx < K || ldy < F || ldx % 8 != 0)
    NOALLOC_FAIL(DMOE_NOALLOC_E_BAD_ARG, "bad row stride (ldx=%lld needs >= K=%d and a multiple of 8; ldy=%lld needs >= F=%d)",
                 ldx, K, ldy, F);
  if ((reinterpret_cast<uintptr_t>(W) & 15) != 0 || (reinterpret_cast<uintptr_t>(X) & 15) != 0)
    NOALLOC_FAIL(DMOE_NOALLOC_E_BAD_ARG, "W and X must be 16-byte aligned (TMA)");
  if (T == 0) return 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) NOALLOC_FAIL(DMOE_NOALLOC_E_SETUP, "cudaGetDevice failed");
  unsigned char* base = nullptr;
  const int rc = noalloc_setup(dev, &base);
  if (rc != 0) return rc;
  if (bn == 0) bn = dmoe_gemm_pick_bn(T, DMOE_EPI_PLAIN);
  if (bn != 32 && bn != 64 && bn != 128 && bn != 256)
    NOALLOC_FAIL(DMOE_NOALLOC_E_BAD_ARG, "token tile %d is not one of 32/64/128/256", bn);
  if (splitk < 0) NOALLOC_FAIL(DMOE_NOALLOC_E_BAD_ARG, "splitk=%d is negative", splitk);
  const int kblocks = (K + 63) / 64;
  const long long tiles = static_cast<long long>((F + 127) / 128) * ((T + bn - 1) / bn);
  if (splitk == 0) {
    splitk = 1;
    const int sms = num_sms();
    if (tiles < sms / 2 && kblocks >= 8) {
      splitk = static_cast<int>(sms / tiles);
      if (splitk > kblocks / 4) splitk = kblocks / 4;
      if (splitk > 16) splitk = 16;
      if (splitk < 1) splitk = 1;
    }
  }
  if (splitk > kblocks) splitk = kblocks;
  const long long need = dmoe_gemm_workspace_bytes(T, F, bn, splitk);
  if (need > DMOE_NOALLOC_WS_BYTES || (splitk > 1 && tiles > DMOE_NOALLOC_MAX_TILES))
    NOALLOC_FAIL(DMOE_NOALLOC_E_TOO_LARGE,
                 "problem too large for the built-in scratch: T=%d F=%d tile=%d splitk=%d needs %lld bytes of partial tiles "
                 "and %lld counters; the limits are %lld bytes and %d counters",
                 T, F, bn, splitk, need, tiles, static_cast<long long>(DMOE_NOALLOC_WS_BYTES), DMOE_NOALLOC_MAX_TILES);
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  {
    std::lock_guard<std::mutex> lock(g_noalloc_mu);
    g_noalloc_stream[dev] = stream;
  }
  unsigned char* counters = base + DMOE_NOALLOC_WS_BYTES;
  // the counters and the status word must start at zero; the array keeps whatever the previous call left behind
  cudaError_t e = cudaMemsetAsync(counters, 0, static_cast<size_t>(kNoallocCounterBytes + 256), stream);
  if (e != cudaSuccess) NOALLOC_FAIL(static_cast<int>(e), "cudaMemsetAsync of the counters failed: %s", cudaGetErrorString(e));
  DmoeGemm d;
  memset(&d, 0, sizeof(d));
  d.W = W; d.X = X; d.Y = Y;
  d.ws = base; d.ws_bytes = DMOE_NOALLOC_WS_BYTES;
  d.counters = reinterpret_cast<int*>(counters);
  d.status = reinterpret_cast<int*>(counters + kNoallocCounterBytes);
  d.ldx = ldx;
  d.ldy = ldy;
  d.G = 1; d.T = T; d.F = F; d.K = K;
  d.epi = DMOE_EPI_PLAIN; d.bn = bn; d.splitk = splitk; d.y_f32 = 0;
  const int grc = dmoe_gemm(&d, stream_);
  if (grc > 0) NOALLOC_FAIL(grc, "launch failed: %s", cudaGetErrorString(static_cast<cudaError_t>(grc)));
  if (grc < 0) NOALLOC_FAIL(grc, "the GEMM rejected the problem with code %d (tensor-map encoding or argument check)", grc);
  return 0;
}

extern "C" int dmoe_noalloc_last_status(int* status_out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || status_out == nullptr)
    NOALLOC_FAIL(DMOE_NOALLOC_E_SETUP, "cudaGetDevice failed or status_out is NULL");
  unsigned char* base = nullptr;
  const int rc = noalloc_setup(dev, &base);
  if (rc != 0) return rc;
  cudaStream_t stream;
  {
    std::lock_guard<std::mutex> lock(g_noalloc_mu);
    stream = g_noalloc_stream[dev];
  }
  // read on the stream of the last call, behind its memset and kernel: a copy on the legacy default stream would not
  // be ordered behind work on a non-blocking or per-thread stream
  cudaError_t e = cudaMemcpyAsync(status_out, base + DMOE_NOALLOC_WS_BYTES + kNoallocCounterBytes, sizeof(int),
                                  cudaMemcpyDeviceToHost, stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess) NOALLOC_FAIL(static_cast<int>(e), "status read failed: %s", cudaGetErrorString(e));
  return 0;
}
