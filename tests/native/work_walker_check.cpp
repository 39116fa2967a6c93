// Host-side check of the GEMM work partition (csrc/kernels/work_walker.cuh): for random problems, in both modes,
// the units of all CTAs cover every tile's K blocks exactly once, ncontrib counts the units per tile, contrib_slot
// names exactly the slots those units park in, and no two parked units share a slot.
#include <cstdio>
#include <cstdlib>
#include <map>
#include <set>
#include <vector>

#include "work_walker.cuh"

using namespace dmoe;

static unsigned long long rng = 88172645463325252ull;
static int rnd(int n) {
  rng ^= rng << 13; rng ^= rng >> 7; rng ^= rng << 17;
  return static_cast<int>(rng % static_cast<unsigned long long>(n));
}

int main() {
  int cases = 0;
  for (int iter = 0; iter < 4000; ++iter) {
    const int G = 1 + rnd(9), S = 1 + rnd(3), MT = 1 + rnd(40), BN = 32 << rnd(4), kblocks = 1 + rnd(230);
    const int grid = 1 + rnd(148), streamk = rnd(2);
    int splitk = streamk ? 1 : 1 + rnd(5);
    if (splitk > kblocks) splitk = kblocks;
    {  // as the launcher does: no split may be empty
      const int per = (kblocks + splitk - 1) / splitk;
      splitk = (kblocks + per - 1) / per;
    }
    std::vector<int> cnt(S * G), start(S * G);
    int row = 0;
    for (int s = 0; s < S; ++s)
      for (int g = 0; g < G; ++g) {
        cnt[s * G + g] = rnd(4) == 0 ? 0 : rnd(700);
        start[s * G + g] = row;
        row += cnt[s * G + g];
      }
    long long tiles = 0;
    for (int g = 0; g < G; ++g) {
      int t = 0;
      for (int s = 0; s < S; ++s) t += (cnt[s * G + g] + BN - 1) / BN;
      tiles += 1ll * MT * t;
    }
    std::map<int, std::vector<WorkUnit>> by_tile;
    std::set<long long> parked;
    for (int c = 0; c < grid; ++c) {
      WorkWalker w;
      w.init(start.data(), cnt.data(), G, S, MT, BN, kblocks, splitk, streamk, c, grid);
      WorkUnit u;
      int last_tile = -1;
      while (w.next(u)) {
        if (u.tile < last_tile || u.kb0 >= u.kb1 || u.kb1 > kblocks || u.ntok < 1 || u.ntok > BN) {
          printf("bad unit: iter %d cta %d tile %d kb [%d,%d) ntok %d\n", iter, c, u.tile, u.kb0, u.kb1, u.ntok);
          return 1;
        }
        last_tile = u.tile;
        if (u.ncontrib > 1 && !parked.insert(u.slot).second) {
          printf("slot reused: iter %d cta %d tile %d slot %lld\n", iter, c, u.tile, u.slot);
          return 1;
        }
        by_tile[u.tile].push_back(u);
      }
    }
    if (static_cast<long long>(by_tile.size()) != tiles) {
      printf("tile count: iter %d got %zu want %lld (streamk %d)\n", iter, by_tile.size(), tiles, streamk);
      return 1;
    }
    for (auto& kv : by_tile) {
      auto& us = kv.second;
      std::vector<int> cover(kblocks, 0);
      std::set<long long> slots, named;
      for (auto& u : us) {
        for (int k = u.kb0; k < u.kb1; ++k) cover[k]++;
        if (static_cast<int>(us.size()) != u.ncontrib) {
          // split-K cuts every tile into `splitk` units even when some of them are empty tails
          if (!(streamk == 0 && u.ncontrib == splitk)) {
            printf("ncontrib: iter %d tile %d has %zu units, unit says %d\n", iter, kv.first, us.size(), u.ncontrib);
            return 1;
          }
        }
        slots.insert(u.slot);
      }
      for (int k = 0; k < kblocks; ++k)
        if (cover[k] != 1) {
          printf("coverage: iter %d tile %d kb %d covered %d times (streamk %d splitk %d)\n", iter, kv.first, k, cover[k],
                 streamk, splitk);
          return 1;
        }
      if (us[0].ncontrib > 1 && streamk) {
        WorkWalker w;
        w.init(start.data(), cnt.data(), G, S, MT, BN, kblocks, splitk, streamk, 0, grid);
        for (int j = 0; j < us[0].ncontrib; ++j) named.insert(w.contrib_slot(us[0], j));
        if (named != slots) {
          printf("slots: iter %d tile %d\n", iter, kv.first);
          return 1;
        }
      }
    }
    ++cases;
  }
  printf("ok %d\n", cases);
  return 0;
}
