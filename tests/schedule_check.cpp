// Host-side check of the static tile schedules the GEMM kernels walk on the device
// (flash_muon_b200/csrc/tile_schedule.cuh, compiled here as plain C++).  The reference launches one
// Triton program per tile pair and lets the lower-triangle ones exit
// (flash_muon/matmul_transpose_triton.py:43-44); here the lists are enumerated by persistent CTAs,
// so "every output block exactly once" is a property of this arithmetic and is tested as such.
//
// Properties checked:
//   1. single-CTA lists (128 x 128 and 128 x 256 tiles), general and symmetric: every 128 x 128
//      output block that has to be computed is covered by exactly one tile, no block below the
//      diagonal of a symmetric product is covered, every tile lies inside the matrix;
//   2. CTA-pair lists (256 x 256 tiles): the same with 256-blocks, in the column order and in
//      column strips of several widths;
//   3. the balanced tail: over all pairs every (tile, K block) is computed exactly once; a pair
//      deposits at most once and before it gathers; the deposits a finishing pair adds up are
//      exactly those of pairs c_first .. pair-1 (the rule the kernel uses to find them), and the
//      deposit counters stay inside their array.
#include <cstdio>
#include <cstdlib>
#include <map>
#include <set>
#include <vector>

#include "tile_schedule.cuh"

namespace {

struct Sched {
  int M, N, sym, tiles_m, tiles_n, num_tiles, num_kb, strip_w, sk_dp_tiles, sk_per;
  long long sk_total;
};

long long g_checked = 0;

#define REQUIRE(cond, ...)                      \
  do {                                          \
    if (!(cond)) {                              \
      std::fprintf(stderr, "FAILED %s: ", #cond); \
      std::fprintf(stderr, __VA_ARGS__);        \
      std::fprintf(stderr, "\n");               \
      std::exit(1);                             \
    }                                           \
  } while (0)

template <int BN>
void check_single(int M, int N, int sym) {
  Sched p{};
  p.M = M; p.N = N; p.sym = sym;
  p.tiles_m = (M + 127) / 128;
  p.num_tiles = fm::count_tiles<BN>(M, N, sym);
  const int bn = (N + 127) / 128;
  std::vector<int> cover((size_t)p.tiles_m * bn, 0);
  for (int t = 0; t < p.num_tiles; ++t) {
    const fm::Tile tl = fm::decode_tile<BN>(p, t);
    REQUIRE(tl.m0 >= 0 && tl.m0 < M && tl.m0 % 128 == 0, "BN=%d M=%d N=%d sym=%d t=%d m0=%d", BN, M, N, sym, t, tl.m0);
    REQUIRE(tl.n0 >= 0 && tl.n0 < N && tl.n0 % 128 == 0, "BN=%d M=%d N=%d sym=%d t=%d n0=%d", BN, M, N, sym, t, tl.n0);
    REQUIRE(tl.ncols == 128 || tl.ncols == 256, "ncols=%d", tl.ncols);
    REQUIRE(tl.bi == tl.m0 / 128, "bi=%d m0=%d", tl.bi, tl.m0);
    for (int c = 0; c < tl.ncols / 128; ++c) {
      const int bj = tl.n0 / 128 + c;
      if (bj >= bn) {
        // a 256-wide tile may hang over the right edge only by a block that starts outside N
        REQUIRE(bj * 128 >= N, "tile reaches past the matrix");
        continue;
      }
      ++cover[(size_t)tl.bi * bn + bj];
    }
  }
  for (int bi = 0; bi < p.tiles_m; ++bi)
    for (int bj = 0; bj < bn; ++bj) {
      const int want = (sym && bj < bi) ? 0 : 1;
      REQUIRE(cover[(size_t)bi * bn + bj] == want, "BN=%d M=%d N=%d sym=%d block (%d,%d) covered %d times",
              BN, M, N, sym, bi, bj, cover[(size_t)bi * bn + bj]);
    }
  ++g_checked;
}

// 128 x 64 tiles: every 128 x 64 block on or above the diagonal's 128-row block exactly once.
void check_single_64(int M, int N, int sym) {
  Sched p{};
  p.M = M; p.N = N; p.sym = sym;
  p.tiles_m = (M + 127) / 128;
  p.num_tiles = fm::count_tiles<64>(M, N, sym);
  const int bn = (N + 63) / 64;
  std::vector<int> cover((size_t)p.tiles_m * bn, 0);
  for (int t = 0; t < p.num_tiles; ++t) {
    const fm::Tile tl = fm::decode_tile<64>(p, t);
    REQUIRE(tl.m0 >= 0 && tl.m0 < M && tl.m0 % 128 == 0, "BN=64 M=%d N=%d sym=%d t=%d m0=%d", M, N, sym, t, tl.m0);
    REQUIRE(tl.n0 >= 0 && tl.n0 < N && tl.n0 % 64 == 0, "BN=64 M=%d N=%d sym=%d t=%d n0=%d", M, N, sym, t, tl.n0);
    REQUIRE(tl.ncols == 64 && tl.bi == tl.m0 / 128, "ncols=%d bi=%d", tl.ncols, tl.bi);
    ++cover[(size_t)tl.bi * bn + tl.n0 / 64];
  }
  for (int bi = 0; bi < p.tiles_m; ++bi)
    for (int bj = 0; bj < bn; ++bj) {
      const int want = (sym && bj < 2 * bi) ? 0 : 1;
      REQUIRE(cover[(size_t)bi * bn + bj] == want, "BN=64 M=%d N=%d sym=%d block (%d,%d) covered %d times",
              M, N, sym, bi, bj, cover[(size_t)bi * bn + bj]);
    }
  ++g_checked;
}

void check_pair_list(int M, int N, int sym, int strip_w = 0, bool columns_first = false) {
  Sched p{};
  p.M = M; p.N = N; p.sym = sym; p.strip_w = strip_w;
  p.tiles_m = (M + 255) / 256;
  p.tiles_n = (!sym && columns_first) ? (N + 255) / 256 : 0;  // general products: walk along columns first
  p.num_tiles = fm::count_tiles2(M, N, sym);
  const int bn = (N + 255) / 256;
  std::vector<int> cover((size_t)p.tiles_m * bn, 0);
  for (int t = 0; t < p.num_tiles; ++t) {
    const fm::Tile2 tl = fm::decode_tile2(p, t);
    REQUIRE(tl.m0 >= 0 && tl.m0 < M && tl.m0 % 256 == 0, "M=%d N=%d sym=%d t=%d m0=%d", M, N, sym, t, tl.m0);
    REQUIRE(tl.n0 >= 0 && tl.n0 < N && tl.n0 % 256 == 0, "M=%d N=%d sym=%d t=%d n0=%d", M, N, sym, t, tl.n0);
    ++cover[(size_t)(tl.m0 / 256) * bn + tl.n0 / 256];
  }
  for (int bi = 0; bi < p.tiles_m; ++bi)
    for (int bj = 0; bj < bn; ++bj) {
      const int want = (sym && bj < bi) ? 0 : 1;
      REQUIRE(cover[(size_t)bi * bn + bj] == want, "pair list M=%d N=%d sym=%d block (%d,%d) covered %d times",
              M, N, sym, bi, bj, cover[(size_t)bi * bn + bj]);
    }
  ++g_checked;
}

// One launch of the pair kernel on `pairs` CTA pairs.  `force` balances whenever the list has a
// partial last wave, ignoring the profitability rule, so that short K loops are exercised too.
void check_balanced(int num_tiles, int num_kb, int max_pairs, bool force) {
  Sched p{};
  p.num_tiles = num_tiles;
  p.num_kb = num_kb;
  p.sk_dp_tiles = num_tiles;
  int pairs = num_tiles < max_pairs ? num_tiles : max_pairs;
  int dp = 0, per = 0;
  long long total = 0;
  bool on = fm::plan_balance(num_tiles, num_kb, max_pairs, &dp, &per, &total);
  if (!on && force && num_tiles > max_pairs && num_tiles % max_pairs != 0) {
    dp = (num_tiles / max_pairs - 1) * max_pairs;
    total = (long long)(num_tiles - dp) * num_kb;
    per = (int)((total + max_pairs - 1) / max_pairs);
    on = true;
  }
  if (on) {
    p.sk_dp_tiles = dp; p.sk_per = per; p.sk_total = total;
    pairs = max_pairs;
    REQUIRE(dp >= 0 && dp % max_pairs == 0, "dp=%d", dp);
    REQUIRE(num_tiles - dp > max_pairs && num_tiles - dp < 2 * max_pairs, "balanced region of %d tiles on %d pairs", num_tiles - dp, max_pairs);
  }
  std::vector<int> cover((size_t)num_tiles * num_kb, 0);
  std::map<int, std::set<int>> depositors;    // sk_tile -> pairs that deposited a part of it
  std::map<int, int> finisher;                // sk_tile -> pair that gathers
  for (int pair = 0; pair < pairs; ++pair) {
    fm::WorkIter it(p, pair, pairs);
    fm::WorkItem w;
    int deposits = 0, gathers = 0;
    bool region = false;
    while (it.next(p, w)) {
      REQUIRE(w.tile >= 0 && w.tile < num_tiles, "tile %d of %d", w.tile, num_tiles);
      REQUIRE(0 <= w.kb0 && w.kb0 < w.kb1 && w.kb1 <= num_kb, "range [%d,%d) of %d", w.kb0, w.kb1, num_kb);
      for (int kb = w.kb0; kb < w.kb1; ++kb) ++cover[(size_t)w.tile * num_kb + kb];
      if (w.tile < p.sk_dp_tiles) {
        REQUIRE(!region, "a whole-list tile after the balanced region began");
        REQUIRE(w.kb0 == 0 && w.kb1 == num_kb && !w.deposit && !w.gather, "dealt tile is not whole");
        continue;
      }
      region = true;
      REQUIRE(w.sk_tile == w.tile - p.sk_dp_tiles, "sk_tile %d for tile %d", w.sk_tile, w.tile);
      REQUIRE(w.sk_tile * 2 + 1 < 4 * max_pairs, "deposit counter %d outside its array", w.sk_tile * 2 + 1);
      REQUIRE(!(w.deposit && w.gather), "deposit and gather at once");
      if (w.deposit) {
        REQUIRE(gathers == 0, "pair %d deposits after it gathered: it could wait on itself", pair);
        REQUIRE(w.kb1 < num_kb, "a deposit that finishes its tile");
        ++deposits;
        REQUIRE(depositors[w.sk_tile].insert(pair).second, "pair %d deposits twice into one tile", pair);
      } else {
        REQUIRE(w.kb1 == num_kb, "an item with an epilogue that does not finish its tile");
        if (w.kb0 != 0) REQUIRE(w.gather, "finishing a begun tile without gathering");
        if (w.gather) {
          ++gathers;
          REQUIRE(finisher.emplace(w.sk_tile, pair).second, "two finishers for one tile");
        }
      }
    }
    REQUIRE(deposits <= 1, "pair %d deposits %d times but owns one scratch slot", pair, deposits);
    REQUIRE(gathers <= 1, "pair %d gathers %d times", pair, gathers);
  }
  for (size_t i = 0; i < cover.size(); ++i)
    REQUIRE(cover[i] == 1, "T=%d kb=%d P=%d: tile %zu K block %zu computed %d times", num_tiles, num_kb,
            max_pairs, i / num_kb, i % num_kb, cover[i]);
  for (const auto& kv : depositors) {
    const auto f = finisher.find(kv.first);
    REQUIRE(f != finisher.end(), "tile %d has deposits but no finisher", kv.first);
    const int g = f->second;
    const int c_first = (int)(((long long)kv.first * num_kb) / p.sk_per);  // the kernel's rule
    std::set<int> want;
    for (int c = c_first; c < g; ++c) want.insert(c);
    REQUIRE(kv.second == want, "T=%d kb=%d P=%d tile %d: depositors are not pairs %d..%d", num_tiles,
            num_kb, max_pairs, kv.first, c_first, g - 1);
  }
  for (const auto& kv : finisher)
    REQUIRE(depositors.count(kv.first) == 1, "a finisher gathers a tile nobody deposited into");
  ++g_checked;
}

}  // namespace

int main() {
  const int dims[] = {1, 64, 127, 128, 129, 255, 256, 257, 384, 511, 512, 640, 1000, 1024, 1031, 1536,
                      2048, 2500, 4096, 6144, 8192, 14336, 16384};
  for (int m : dims)
    for (int sym = 0; sym < 2; ++sym) {
      if (sym) {
        check_single<128>(m, m, 1);
        check_single<256>(m, m, 1);
        check_single_64(m, m, 1);
        check_pair_list(m, m, 1);
        for (int w : {1, 2, 3, 5, 8, 12, 64}) check_pair_list(m, m, 1, w);   // column strips
      } else {
        for (int n : dims) {
          if ((long long)m * n > 8192LL * 16384) continue;
          check_single<128>(m, n, 0);
          check_single<256>(m, n, 0);
          check_single_64(m, n, 0);
          check_pair_list(m, n, 0);
          check_pair_list(m, n, 0, 0, true);
        }
      }
    }
  // balanced tail: the resident pair counts seen in practice (74 on B200, fewer when shared
  // memory is left to others) and small ones that make every corner frequent
  const int pair_counts[] = {1, 2, 3, 5, 8, 37, 73, 74, 80};
  const int kbs[] = {1, 2, 3, 7, 16, 64, 65, 128, 224, 256};
  for (int P : pair_counts)
    for (int kb : kbs)
      for (int T = 1; T <= 6 * P + 3 && T <= 600; ++T)
        for (int force = 0; force < 2; ++force) check_balanced(T, kb, P, force != 0);
  // the shapes of the benchmarked configurations on 74 pairs
  check_balanced(528, 128, 74, false);   // 8192^2 symmetric product
  check_balanced(136, 224, 74, false);   // 4096 x 14336 symmetric product
  check_balanced(896, 64, 74, false);    // [4096,4096] x [4096,14336]
  std::printf("OK %lld schedules checked\n", g_checked);
  return 0;
}
