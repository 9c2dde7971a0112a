// Static tile schedules of the tensor-core GEMM kernels, kept free of anything device-only so that
// a host program can enumerate them and check that every output tile and every K block is
// computed exactly once (tests/schedule_check.cpp does; it includes this file with a plain C++
// compiler).  The functions are templated on the parameter struct: the kernels pass GemmParams,
// a host check passes any struct with the same schedule fields
//   M, N, sym, tiles_m, tiles_n, num_tiles, num_kb, strip_w, sk_dp_tiles, sk_per, sk_total.
#pragma once
#include <math.h>

#if defined(__CUDACC__)
#define FM_HD __host__ __device__ __forceinline__
#else
#define FM_HD inline
#endif

namespace fm {

// ---------------------------------------------------------------------------------------------
// Single-CTA kernel: 128 x BN tiles (BN = 64, 128 or 256).
// ---------------------------------------------------------------------------------------------
struct Tile {
  int m0;     // first output row
  int n0;     // first output column
  int ncols;  // 64, 128 or 256 (UMMA N)
  int bi;     // 128-row block index (for the diagonal test)
};

// Tiles before column super-tile j of the triangular schedule (R = BN / 128).
template <int R>
FM_HD long long tri_before(long long j) {
  return R == 1 ? j * (j + 1) / 2 : j * (j + 1);
}

// 64-wide tiles (BN = 64), symmetric lists: column tile j holds the row blocks i with
// 128 i <= 64 j + 63, i.e. i <= j / 2.  Tiles before column tile j:
FM_HD long long half_before(long long j) {
  const long long a = j >> 1;
  return (j & 1) ? (a + 1) * (a + 1) : a * (a + 1);
}

// Length of the tile list of the single-CTA kernel.
template <int BN>
FM_HD int count_tiles(long long M, long long N, int sym) {
  constexpr int R = BN / 128;
  const int tiles_m = (int)((M + 127) / 128);
  const int tiles_n = (int)((N + BN - 1) / BN);
  if (!sym) return tiles_m * tiles_n;
  if (BN < 128) return (int)half_before(tiles_n);
  int n = 0;
  for (int j = 0; j < tiles_n; ++j) n += (R * j + R < tiles_m) ? (R * j + R) : tiles_m;
  return n;
}

template <int BN, class P>
FM_HD Tile decode_tile(const P& p, int t) {
  constexpr int R = BN / 128;
  Tile o;
  if (BN < 128) {  // 128 x 64 tiles
    int i, j;
    if (!p.sym) {
      j = t / p.tiles_m;
      i = t - j * p.tiles_m;
    } else {
      j = (int)(2.f * sqrtf((float)t));
      while (half_before(j + 1) <= t) ++j;
      while (half_before(j) > t) --j;
      i = t - (int)half_before(j);
    }
    o.m0 = i * 128;
    o.bi = i;
    o.n0 = j * BN;
    o.ncols = BN;
    return o;
  }
  int nblk0;
  if (!p.sym) {
    const int tn = t / p.tiles_m;
    const int tm = t - tn * p.tiles_m;
    o.m0 = tm * 128;
    o.bi = tm;
    nblk0 = tn * R;
    o.ncols = BN;
  } else {
    // Column super-tile j owns row blocks i in [0, min(R*j + R, tiles_m)); only the last column
    // can be clipped, so tri_before() is exact for every column start.
    int j = R == 1 ? (int)((sqrtf(8.f * (float)t + 1.f) - 1.f) * 0.5f)
                   : (int)((sqrtf(4.f * (float)t + 1.f) - 1.f) * 0.5f);
    while (tri_before<R>(j + 1) <= t) ++j;
    while (tri_before<R>(j) > t) --j;
    const int i = t - (int)tri_before<R>(j);
    o.m0 = i * 128;
    o.bi = i;
    const int sub = (i > R * j) ? (i - R * j) : 0;  // leading 128-column blocks below the diagonal
    nblk0 = R * j + sub;
    o.ncols = BN - sub * 128;
  }
  o.n0 = nblk0 * 128;
  const int left = p.N - o.n0;  // > 0 by construction
  if (left <= 128 && o.ncols > 128) o.ncols = 128;
  return o;
}

// ---------------------------------------------------------------------------------------------
// CTA-pair kernel: 256 x 256 tiles.
// ---------------------------------------------------------------------------------------------
struct Tile2 {
  int m0, n0;  // first row / column of the 256 x 256 tile
};

FM_HD int count_tiles2(long long M, long long N, int sym) {
  const long long tm = (M + 255) / 256, tn = (N + 255) / 256;
  return (int)(sym ? tn * (tn + 1) / 2 : tm * tn);
}

// Symmetric lists come in two orders.  strip_w == 0: column by column, rows 0..j inside column
// j.  strip_w == w > 0: strips of w tile columns; inside a strip row by row (i = 0 .. last
// column of the strip), inside a row the strip's columns j >= i.  The CTA pairs of a launch work
// on consecutive tiles at the same time and advance through K in step, so what a "wave" of them
// reads from DRAM is one K sweep of every distinct 256-row panel its tiles touch, as row or as
// column.  P consecutive tiles of the column order touch about j + P / j panels around column j
// (all 32 of an 8192-row matrix in the last waves); P consecutive tiles of a strip touch about
// w + P / w, e.g. 17 for w = 8 and 74 pairs.
template <class P>
FM_HD long long strip_tiles_before(const P& p, int s) {
  const long long w = p.strip_w;
  return w * w * s * (s - 1) / 2 + (long long)s * w * (w + 1) / 2;
}

template <class P>
FM_HD Tile2 decode_tile2(const P& p, int t) {
  Tile2 o;
  if (!p.sym) {
    // Consecutive tiles (which run at the same time) walk along the dimension with FEWER tiles, so
    // that a wave re-reads the panels of the smaller operand (they stay in L2) and streams the
    // panels of the larger one once; tiles_n > 0 selects the walk along columns.
    if (p.tiles_n > 0) {
      const int tm = t / p.tiles_n;
      const int tn = t - tm * p.tiles_n;
      o.m0 = tm * 256;
      o.n0 = tn * 256;
    } else {
      const int tn = t / p.tiles_m;
      const int tm = t - tn * p.tiles_m;
      o.m0 = tm * 256;
      o.n0 = tn * 256;
    }
  } else if (p.strip_w > 0) {
    const int w = p.strip_w;
    int s = 0;
    while (strip_tiles_before(p, s + 1) <= t) ++s;      // a handful of strips
    const int c0 = s * w;
    const int n = p.tiles_m;                            // tile rows = tile columns
    const int wc = (c0 + w <= n) ? w : (n - c0);        // only the last strip can be narrower
    int r = t - (int)strip_tiles_before(p, s);
    int i, j;
    if (r < c0 * wc) {                                  // rows above the strip's diagonal block
      i = r / wc;
      j = c0 + (r - i * wc);
    } else {                                            // the triangle on the diagonal
      r -= c0 * wc;
      int ii = 0;
      while (r >= wc - ii) {
        r -= wc - ii;
        ++ii;
      }
      i = c0 + ii;
      j = i + r;
    }
    o.m0 = i * 256;
    o.n0 = j * 256;
  } else {
    int j = (int)((sqrtf(8.f * (float)t + 1.f) - 1.f) * 0.5f);
    while ((long long)(j + 1) * (j + 2) / 2 <= t) ++j;
    while ((long long)j * (j + 1) / 2 > t) --j;
    const int i = t - j * (j + 1) / 2;
    o.m0 = i * 256;
    o.n0 = j * 256;
  }
  return o;
}

// Work of one CTA pair.  The first `sk_dp_tiles` tiles of the list are dealt round-robin, one
// whole tile at a time.  The rest (between one and two waves' worth; empty unless the host
// decides that balancing pays, see plan_balance) is cut by K blocks into equal contiguous shares,
// so that every pair finishes at the same time instead of most of them idling through a last
// partial wave.  A pair walks its share from the END: first the range that begins a tile it
// cannot finish -- that partial accumulator is deposited in fp32 scratch right away -- then
// whole tiles, last the range that finishes a tile begun by earlier pairs.  There the deposits
// of those pairs (made at the start of their shares, so long since complete) are added in a
// fixed order to the accumulator and the tile's epilogue runs as usual.  The result does not
// depend on timing; the wait for the deposits is a formality with the usual cycle limit.
struct WorkItem {
  int tile;      // index into the tile list
  int kb0, kb1;  // K-block range
  int sk_tile;   // index of the tile inside the balanced region
  int deposit;   // 1: range stops short of the tile's last K block -> deposit, no epilogue
  int gather;    // 1: range finishes a tile whose first K blocks were done by earlier pairs
};

struct WorkIter {
  int dp_next, dp_step, dp_end;
  long long lo, hi;
  template <class P>
  FM_HD WorkIter(const P& p, int pair, int npairs) {
    dp_next = pair;
    dp_step = npairs;
    dp_end = p.sk_dp_tiles;
    lo = (long long)pair * p.sk_per;
    hi = lo + p.sk_per;
    if (hi > p.sk_total) hi = p.sk_total;
    if (lo > hi) lo = hi;
  }
  template <class P>
  FM_HD bool next(const P& p, WorkItem& w) {
    if (dp_next < dp_end) {
      w.tile = dp_next; w.kb0 = 0; w.kb1 = p.num_kb; w.sk_tile = 0; w.deposit = 0; w.gather = 0;
      dp_next += dp_step;
      return true;
    }
    if (hi > lo) {
      const int rel = (int)((hi - 1) / p.num_kb);
      const long long t_begin = (long long)rel * p.num_kb;
      const long long seg_lo = lo > t_begin ? lo : t_begin;
      w.tile = p.sk_dp_tiles + rel;
      w.sk_tile = rel;
      w.kb0 = (int)(seg_lo - t_begin);
      w.kb1 = (int)(hi - t_begin);
      w.deposit = (w.kb1 != p.num_kb) ? 1 : 0;
      w.gather = (w.kb0 != 0 && !w.deposit) ? 1 : 0;
      hi = seg_lo;
      return true;
    }
    return false;
  }
};

// Decides whether the tail of a list of `num_tiles` tiles of `num_kb` K blocks is cut by K blocks
// on `max_pairs` resident CTA pairs, and how.  Returns false when every tile is dealt whole.
// Worth it only when the idle time of the last partial wave exceeds what the partial sums cost.
// Measured on B200 (same process, alternating): 8192^2 and 6144^2 products gain 7-10 %; lists of
// one or two waves, or tiles with K <= 4096, lose 2-15 %.  Model: a K block of a 256 x 256 tile
// takes ~0.41 us, depositing and re-reading partial accumulators ~12 us per pair, so balance when
// the K blocks saved, num_kb * (P - R) / P, are worth more than ~24 us.
FM_HD bool plan_balance(int num_tiles, int num_kb, int max_pairs, int* dp_tiles, int* per,
                        long long* total) {
  if (num_tiles <= max_pairs) return false;
  const int R = num_tiles % max_pairs;
  if (R == 0) return false;
  if ((long long)num_kb * (max_pairs - R) < 58LL * max_pairs) return false;
  *dp_tiles = (num_tiles / max_pairs - 1) * max_pairs;  // leave between one and two waves to balance
  *total = (long long)(num_tiles - *dp_tiles) * num_kb;
  *per = (int)((*total + max_pairs - 1) / max_pairs);
  return true;
}

}  // namespace fm
