// Work distribution of the persistent GEMM: which (tile, K range) units a CTA runs.
//
// Tiles are numbered group after group (a group = an expert, or the one group of a dense GEMM): within a group the
// weight tile m is the slow index and the token tile n the fast one, so neighbouring CTAs work on the same weight
// tile at the same time and the second fetch of it hits L2. A group owns S segments of token rows (one per source);
// its token tiles enumerate the segments one after the other.
//
// Two modes:
//   split-K   every tile is cut into `splitk` equal K ranges (1 = whole tiles); unit i of the flat list (tile-major,
//             split fastest) runs on CTA i mod grid.
//   stream-K  full waves run as whole tiles (tile w * grid + c on CTA c in wave w: the CTAs of a wave work on
//             neighbouring tiles at the same time, so a weight tile that two token tiles need is fetched from HBM
//             once). The tiles of the last, partial wave are not left to a few CTAs: their work, counted in K blocks,
//             is cut into one contiguous share per CTA (equal to within one K block). A tile that straddles a share
//             boundary is computed by two or more CTAs; each parks its fp32 partial accumulator in a workspace slot
//             and the last one to arrive adds them up and runs the epilogue. With fewer tiles than CTAs every tile is
//             in that last wave.
//
// Plain C++ (also compiled for the host by the unit test of the partition arithmetic).
#pragma once

#if defined(__CUDACC__)
#define DMOE_HD __host__ __device__ __forceinline__
#else
#define DMOE_HD inline
#endif

namespace dmoe {

struct WorkUnit {
  int tile;        // tile id over (group, m, n)
  int g, m, n;
  int row0, ntok;  // first token row and number of valid tokens of the tile
  int kb0, kb1;    // K blocks [kb0, kb1) of the tile that this unit covers
  int ncontrib;    // units that together cover the tile (1: this unit is the whole tile)
  int c_first;     // stream-K: first CTA contributing to the tile
  int slot;        // workspace slot where this unit parks its partial accumulator (when ncontrib > 1)
};

struct WorkWalker {
  const int* seg_start;  // [S * G] absolute first row of segment (s, g)
  const int* seg_cnt;    // [S * G]
  int G, S, MT, BN, kblocks, splitk, kb_per, streamk;
  int g, base, ntn;      // group cursor: tiles of group g start at id `base`
  // All counters are 32-bit on purpose (the launcher bounds tiles x splits by 2^30 and the stream-K remainder holds
  // fewer tiles than the grid has CTAs): 64-bit divisions cost a microsecond of every launch's prologue.
  int lin, lin_step;                    // split-K: next flat unit id of this CTA and the stride
  // stream-K: `waves` full waves of whole tiles, then this CTA's share [it_begin, it_end) of the K-block iterations
  // of the remaining tiles (ids from tile0 on); `total` counts the remainder's iterations
  int it, it_end, total, it_begin;
  int active, cta, grid, waves, wave, tile0;

  DMOE_HD static int min_i(int a, int b) { return a < b ? a : b; }

  DMOE_HD void advance_group() {
    ++g;
    ntn = 0;
    if (g < G)
      for (int s = 0; s < S; ++s) ntn += (seg_cnt[s * G + g] + BN - 1) / BN;
  }

  // (products of a CTA index and an iteration count: 64-bit multiply, 32-bit operands, one division each)
  DMOE_HD int share_begin(int c) const { return static_cast<int>(static_cast<long long>(c) * total / active); }
  // CTA whose share holds iteration i: the largest c with share_begin(c) <= i
  DMOE_HD int owner(int i) const {
    return static_cast<int>((static_cast<long long>(i + 1) * active + total - 1) / total) - 1;
  }

  DMOE_HD void init(const int* s_start, const int* s_cnt, int G_, int S_, int MT_, int BN_, int kblocks_, int splitk_,
                    int streamk_, int cta_, int grid_) {
    seg_start = s_start; seg_cnt = s_cnt; G = G_; S = S_; MT = MT_; BN = BN_; kblocks = kblocks_;
    splitk = splitk_ < 1 ? 1 : splitk_; streamk = streamk_; cta = cta_;
    kb_per = (kblocks + splitk - 1) / splitk;
    lin = cta_; lin_step = grid_;
    it = it_end = it_begin = total = 0; active = 1; grid = grid_; waves = wave = tile0 = 0;
    int tiles = 0;
    for (int gg = 0; gg < G; ++gg) {
      int t = 0;
      for (int s = 0; s < S; ++s) t += (seg_cnt[s * G + gg] + BN - 1) / BN;
      tiles += MT * t;
    }
    if (!streamk) {
      // Balanced waves: with u units and w = ceil(u / grid) waves, only ceil(u / w) CTAs take part, each with w (or
      // w - 1) units, so that all of them finish together instead of a few CTAs running a last, nearly empty wave
      // while the rest idle. A memory-bound launch loses nothing (fewer SMs still saturate HBM) and sheds the tail;
      // a compute-bound one takes w unit times either way.
      const int units = tiles * splitk;
      if (units > 0) {
        const int w = (units + grid_ - 1) / grid_;
        const int use = (units + w - 1) / w;
        lin_step = use;
        if (cta_ >= use) lin = units;      // idle CTA: its first unit is already past the end
      }
    }
    if (streamk) {
      waves = tiles / grid_;
      tile0 = waves * grid_;
      total = (tiles - tile0) * kblocks;
      // a share shorter than a few K blocks (or a tile cut into more than 8 pieces) costs more in partial-tile
      // traffic than it wins in balance
      int min_share = kblocks >= 8 ? 4 : kblocks;
      if (min_share < (kblocks + 7) / 8) min_share = (kblocks + 7) / 8;
      int act = total / min_share;
      if (act < 1) act = 1;
      active = act < grid_ ? act : grid_;
      if (total > 0 && cta_ < active) {
        it_begin = it = share_begin(cta_);
        it_end = share_begin(cta_ + 1);
      }
    }
    g = -1; base = 0; ntn = 0;
    advance_group();
  }

  // Positions the group cursor on `tile` (ids must not decrease across calls) and fills g, m, n, row0, ntok.
  DMOE_HD bool locate(int tile, WorkUnit& u) {
    while (g < G) {
      const int ntiles = MT * ntn;
      if (tile < base + ntiles) {
        const int r = tile - base;
        u.tile = tile; u.g = g; u.n = r % ntn; u.m = r / ntn;
        int nl = u.n;
        for (int s = 0; s < S; ++s) {
          const int c = seg_cnt[s * G + g];
          const int t = (c + BN - 1) / BN;
          if (nl < t) {
            u.row0 = seg_start[s * G + g] + nl * BN;
            u.ntok = min_i(BN, c - nl * BN);
            return true;
          }
          nl -= t;
        }
        return false;  // unreachable
      }
      base += ntiles;
      advance_group();
    }
    return false;
  }

  // The next unit of this CTA; false when it has none left.
  DMOE_HD bool next(WorkUnit& u) {
    if (!streamk) {
      const int tile = lin / splitk;
      if (lin < 0 || !locate(tile, u)) return false;
      const int ks = lin - tile * splitk;
      lin += lin_step;
      u.kb0 = ks * kb_per;
      u.kb1 = min_i(kblocks, u.kb0 + kb_per);
      u.ncontrib = splitk;
      u.c_first = 0;
      u.slot = tile * splitk + ks;
      return true;
    }
    if (wave < waves) {
      // full waves: whole tiles, neighbouring CTAs on neighbouring tiles
      if (!locate(wave * grid + cta, u)) return false;
      ++wave;
      u.kb0 = 0; u.kb1 = kblocks; u.ncontrib = 1; u.c_first = cta; u.slot = 0;
      return true;
    }
    if (it >= it_end) return false;
    const int rtile = it / kblocks;                // tile index inside the remainder
    if (!locate(tile0 + rtile, u)) return false;
    const int t0 = rtile * kblocks, t1 = t0 + kblocks;
    const bool first_unit = (it == it_begin);
    u.kb0 = it - t0;
    const int end = it_end < t1 ? it_end : t1;
    u.kb1 = end - t0;
    it = end;
    u.c_first = owner(t0);
    u.ncontrib = owner(t1 - 1) - u.c_first + 1;
    u.slot = cta * 2 + (first_unit ? 0 : 1);
    return true;
  }

  // Workspace slot of contributor j (0 <= j < ncontrib) of unit u's tile.
  DMOE_HD int contrib_slot(const WorkUnit& u, int j) const {
    if (!streamk) return u.tile * splitk + j;
    const int c = u.c_first + j;
    const int first_tile = tile0 + share_begin(c) / kblocks;   // the tile CTA c's share starts in: its slot 0
    return c * 2 + (first_tile == u.tile ? 0 : 1);
  }
};

}  // namespace dmoe
