// CTA-pair variant of the tensor-core GEMM family (see gemm_tc.cu for the operation itself):
// two CTAs of a cluster compute one 256 x 256 output tile with tcgen05.mma.cta_group::2.
// Each CTA stages only its own 128 rows of A and its own 128 rows of B per 64-wide K slab
// (32 KiB per stage instead of 48 KiB), so the operand traffic per FLOP from L2 and from shared
// memory drops by a third and a half respectively against the 128 x 256 single-CTA tile, and six
// stages fit.  No load is a multicast: the two CTAs issue plain TMA tile loads into their own
// shared memory; only the completion bytes are counted on the leader's mbarrier, and the MMA
// completion is signalled to both CTAs by tcgen05.commit.
//
// Roles per CTA (192 threads): warp 0 TMA producer (both CTAs), warp 1 MMA issuer (leader CTA
// only; both CTAs take part in the TMEM allocation), warps 2..5 epilogue (both CTAs, each for
// its own 128 accumulator rows).
//
// A launch may carry a batch of problems of identical extents (operands stacked along the rows
// of one tensor map each): the tile list is then the single-problem list repeated per problem,
// so that many small matrices share one launch -- the grouped form Newton-Schulz uses for
// matrices too small to fill the GPU on their own.
//
// Outputs leave through shared memory: each epilogue warp converts its 32 rows x 64 columns,
// writes them row-wise and transposed into two small staging tiles and lets TMA store both (full
// 128- and 64-byte row segments; rows and columns past the matrix edge are clipped by the tensor
// map).  Per-lane global stores (32 scattered 16-byte pieces per instruction) cost 14-23 % of a
// K = 4096 product although they overlap the main loop; tiles on the diagonal of a symmetric
// product, with their element-wise mirror rule, and outputs TMA cannot address keep that path.
//
// The kernel is launched with programmatic stream serialization: its set-up (barriers, TMEM,
// tensor-map prefetch) runs while the previous kernel of the stream drains.  A launch whose CTAs
// all finish together (one wave, or a balanced tail) lets the next kernel be placed as soon as
// every CTA has started its last piece of work; a launch with a ragged last wave does not, because
// SMs that fall idle early are better taken by a kernel of another stream than by a successor
// that can only wait.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"
#include "gemm_common.cuh"
#include "gemm_tc.cuh"
#include "ptx.cuh"
#include "tile_schedule.cuh"

namespace fm {
namespace {

constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int kThreads = 192;
constexpr int kSlabBytes = 128 * BK * 2;      // 16 KiB: 128 rows x 64 columns of 16-bit values
constexpr int kMaxStages = 7;
constexpr int kDefaultStages = 6;
constexpr int kStageBytes = 2 * kSlabBytes;   // this CTA's A slab + B slab
constexpr int kTmemCols = 512;                // two accumulators of 256 fp32 columns
constexpr int kNumBars = 2 * kMaxStages + 4 + 8;  // + two addend barriers per epilogue warp
// staging of the TMA stores: per epilogue warp 32 x 64 values row-wise (4 KiB) and transposed (4 KiB)
constexpr int kStagingBytes = 4 * 8192;
constexpr int kMaxStagesWithStaging = 6;
constexpr int smem_bytes(int stages, bool staging) {
  return stages * kStageBytes + (staging ? kStagingBytes : 0) + kNumBars * 8 + 16 + 1024;
}

// Scratch of the balanced tail: deposit counters first, then one partial accumulator per CTA of
// every pair (128 rows x 256 fp32 columns each: a pair leaves at most one tile unfinished).
constexpr size_t kSkCntBytes = 4096;
constexpr size_t kSkPartBytes = (size_t)128 * 256 * 4;

// Problem and tile of entry `t` of a (possibly batched) tile list.
struct TileRef {
  int g;
  Tile2 tl;
};
__device__ __forceinline__ TileRef locate(const GemmParams& p, int t) {
  TileRef r;
  r.g = 0;
  if (p.batch > 1) {
    r.g = t / p.tiles_per_batch;
    t -= r.g * p.tiles_per_batch;
  }
  r.tl = decode_tile2(p, t);
  return r;
}

// kSplitK: the instantiation that can deposit and gather partial accumulators (balanced tail).
// Launches that deal whole tiles use the other one, whose epilogue spends the registers of the
// partial sums on fetching the addend two 32-column chunks ahead instead of one.
template <typename T, bool kSplitK>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc2_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmT,
                const __grid_constant__ CUtensorMap tmD, const __grid_constant__ GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  // The ring has p.stages slots of one 64-wide K block each; a pipeline stage (one full / empty
  // barrier pair) covers p.kb_per_stage consecutive slots.
  const int kbs = p.kb_per_stage;
  const int kStages = p.stages / kbs;
  const uint32_t smem_base = ptx::smem_u32(smem);
  const int staging_off = p.stages * kStageBytes;  // multiple of 1024: the swizzled tile needs it
  const int bar_off = staging_off + (p.tma_store ? kStagingBytes : 0);
  const uint32_t bar_base = smem_base + bar_off;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + bar_off + kNumBars * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kMaxStages + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * kMaxStages + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * kMaxStages + 2 + a); };
  auto dfull_bar = [&](int q, int b) { return bar_base + 8u * (2 * kMaxStages + 4 + 2 * q + b); };
  auto a_smem = [&](int s) { return smem_base + s * kStageBytes; };
  auto b_smem = [&](int s) { return smem_base + s * kStageBytes + kSlabBytes; };

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = ptx::cluster_ctarank();  // 0 = leader (issues the MMAs)
  const int pair = blockIdx.x >> 1;
  const int npairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(full_bar(s), 1);   // leader's producer arrives once (with the byte count)
      ptx::mbar_init(empty_bar(s), 1);  // one commit arrival per use
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(tfull_bar(a), 1);
      ptx::mbar_init(tempty_bar(a), 8);  // 4 epilogue warps of each of the two CTAs
    }
    for (int q = 0; q < 4; ++q)
      for (int b = 0; b < 2; ++b) ptx::mbar_init(dfull_bar(q, b), 1);
    *abort_flag = 0;
    ptx::mbar_fence_init();
    ptx::prefetch_tmap(&tmA);
    ptx::prefetch_tmap(&tmB);
    if (p.tma_store) {
      if (p.C != nullptr) ptx::prefetch_tmap(&tmC);
      if (p.CT != nullptr) ptx::prefetch_tmap(&tmT);
    }
    if (p.tma_d) ptx::prefetch_tmap(&tmD);
  }
  if (warp == 1) {
    ptx::tmem_alloc_pair(ptx::smem_u32(tmem_slot), kTmemCols);
    ptx::tmem_relinquish_pair();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_sync();  // the peer's barriers exist before anything remote touches them
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Nothing above reads or writes global memory; everything below may depend on the previous
  // kernel of the stream.
  ptx::grid_dep_wait();

  if (warp == 0) {
    // ------------------------------------------------------------- TMA producer (both CTAs)
    // Like the MMA issuer, the whole warp runs the loop convergently and only the TMA and
    // barrier instructions are predicated on the leading lane.
    {
      const uint32_t lead = (lane == 0) ? 1u : 0u;
      const uint32_t expect_lead = (lane == 0 && rank == 0) ? 1u : 0u;
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      WorkIter it(p, pair, npairs);
      WorkItem w, nxt;
      bool have = it.next(p, w);
      if (!have && p.early_trigger && lane == 0) ptx::grid_dep_launch();
      while (ok && have) {
        const bool more = it.next(p, nxt);
        // last piece of work of this CTA: the next kernel of the stream may be placed
        if (!more && p.early_trigger && lane == 0) ptx::grid_dep_launch();
        const TileRef tr = locate(p, w.tile);
        const Tile2 tl = tr.tl;
        const int ya = tr.g * p.a_batch_rows + tl.m0 + (int)rank * 128;
        const int yb = tr.g * p.b_batch_rows + tl.n0 + (int)rank * 128;
        // On a diagonal tile of the symmetric product the B slab is the A slab (same rows of
        // the same matrix): load it once and let the MMA read it through both descriptors.
        const bool same = p.sym && (tl.m0 == tl.n0);
        const uint32_t load_b = same ? 0u : lead;
        for (int kb = w.kb0; kb < w.kb1; kb += kbs) {
          const int nh = (w.kb1 - kb) < kbs ? (w.kb1 - kb) : kbs;  // K blocks of this stage
          if (!ptx::mbar_wait(empty_bar(s), ph ^ 1u, abort_flag)) { ok = false; break; }
          const uint32_t leader_full = ptx::mapa(full_bar(s), 0);
          ptx::mbar_expect_tx_lead(full_bar(s), (uint32_t)nh * (same ? 2u : 4u) * kSlabBytes, expect_lead);
          for (int h = 0; h < nh; ++h) {
            ptx::tma_load_2d_pair_lead(a_smem(s * kbs + h), &tmA, leader_full, (kb + h) * BK, ya, lead);
            ptx::tma_load_2d_pair_lead(b_smem(s * kbs + h), &tmB, leader_full, (kb + h) * BK, yb, load_b);
          }
          if (++s == kStages) { s = 0; ph ^= 1u; }
        }
        w = nxt;
        have = more;
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issuer (leader CTA only)
    // The tensor pipe holds only a few MMAs, so the issuing code is on the critical path:
    // whatever runs between two MMAs (barrier poll, descriptor arithmetic, commit) has to fit
    // under the ones still queued.  The whole warp runs the loop convergently -- addresses and
    // descriptors then stay warp-uniform values -- and only the MMA and commit instructions
    // themselves are predicated on the leading lane; the MMAs of a stage are straight-line code,
    // and the wait for the NEXT stage's data sits in front of the last MMA of the current one.
    if (rank == 0) {
      const uint32_t lead = (lane == 0) ? 1u : 0u;
      int s = 0;
      uint32_t ph = 0;
      int acc = 0;
      uint32_t acc_ph = 0;
      bool ok = true;
      const uint32_t idesc = ptx::make_idesc_f16(Num<T>::kFormat, 256, 256);
      const uint64_t desc_base = ptx::make_kmajor_sw128_desc(a_smem(0));  // slot 0, A slab
      constexpr uint32_t kSlotStep = (uint32_t)(kStageBytes >> 4);        // descriptor units per slot
      WorkIter it(p, pair, npairs);
      WorkItem w;
      while (ok && it.next(p, w)) {
        if (!ptx::mbar_wait_cluster(tempty_bar(acc), acc_ph ^ 1u, abort_flag)) { ok = false; break; }
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * 256);
        const Tile2 tl = locate(p, w.tile).tl;
        const bool same = p.sym && (tl.m0 == tl.n0);
        int kb = w.kb0;
        if (kb < w.kb1 && !ptx::mbar_wait(full_bar(s), ph, abort_flag)) { ok = false; break; }
        while (kb < w.kb1) {
          const int nh = (w.kb1 - kb) < kbs ? (w.kb1 - kb) : kbs;
          const int s_next = (s + 1 == kStages) ? 0 : s + 1;
          const uint32_t ph_next = (s + 1 == kStages) ? (ph ^ 1u) : ph;
          const bool more = kb + nh < w.kb1;
          const uint64_t a0 = desc_base + (uint64_t)((uint32_t)(s * kbs) * kSlotStep);
          const uint64_t b0 = same ? a0 : a0 + (uint64_t)(kSlabBytes >> 4);
          const uint32_t first = (kb != w.kb0) ? 1u : 0u;
          // MMA i of a stage reads K block i / 4 (one slot further on per block) and the 16
          // columns i % 4 of it (32 bytes = 2 in the descriptor's address field)
          if (nh == 1) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              if (i == 3 && more && !ptx::mbar_wait(full_bar(s_next), ph_next, abort_flag)) ok = false;
              ptx::umma_f16_pair_lead(d_tmem, a0 + (uint64_t)(2 * i), b0 + (uint64_t)(2 * i), idesc,
                                      i == 0 ? first : 1u, lead);
            }
          } else if (nh == 2) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              if (i == 7 && more && !ptx::mbar_wait(full_bar(s_next), ph_next, abort_flag)) ok = false;
              const uint64_t off = (uint64_t)((i >> 2) * kSlotStep + (i & 3) * 2);
              ptx::umma_f16_pair_lead(d_tmem, a0 + off, b0 + off, idesc, i == 0 ? first : 1u, lead);
            }
          } else {
#pragma unroll
            for (int i = 0; i < 12; ++i) {
              if (i == 11 && more && !ptx::mbar_wait(full_bar(s_next), ph_next, abort_flag)) ok = false;
              const uint64_t off = (uint64_t)((i >> 2) * kSlotStep + (i & 3) * 2);
              ptx::umma_f16_pair_lead(d_tmem, a0 + off, b0 + off, idesc, i == 0 ? first : 1u, lead);
            }
          }
          ptx::umma_commit_pair_lead(empty_bar(s), 0x3, lead);  // frees the stage in both CTAs
          if (!ok) break;
          kb += nh;
          s = s_next;
          ph = ph_next;
        }
        if (!ok) break;
        ptx::umma_commit_pair_lead(tfull_bar(acc), 0x3, lead);  // accumulator halves complete in both CTAs
        acc ^= 1;
        if (acc == 0) acc_ph ^= 1u;
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------- epilogue (both CTAs)
    const int q = warp & 3;
    int acc = 0;
    uint32_t acc_ph = 0;
    volatile int* sk_flag = reinterpret_cast<volatile int*>(tmem_slot + 2);
    uint8_t* const sC = smem + staging_off + q * 8192;  // this warp's staging tiles
    uint8_t* const sT = sC + 4096;
    WorkIter it(p, pair, npairs);
    WorkItem w;
    while (it.next(p, w)) {
      const TileRef tr = locate(p, w.tile);
      const Tile2 tl = tr.tl;
      const EpiPtrs ep = epilogue_ptrs(p, tr.g, (int)sizeof(T));
      const int row_local = q * 32 + lane;
      const int row = tl.m0 + (int)rank * 128 + row_local;
      const int row0w = row - lane;               // first row of this warp's 32
      const int bi = (tl.m0 >> 7) + (int)rank;
      // tile stores for everything but the diagonal tiles of a symmetric product
      const bool tma_tile = p.tma_store && !(p.sym && tl.m0 == tl.n0);
      const bool deposit = kSplitK && w.deposit;
      const bool gather = kSplitK && w.gather;
      // Addend values of the chunks to come: dq[0] is the chunk being processed, dq[kAhead] the
      // one whose loads go out now.
      constexpr int kAhead = kSplitK ? 1 : 2;  // measured: 3 and 4 are slower again at K = 1024
      alignas(16) T dq[kAhead + 1][32];
      // Addend by TMA (whole-tile instantiation, tiles that leave through tile stores): the
      // warp's two 4 KB staging tiles take turns as landing buffer of the addend's next 32 x 64
      // block; the block is computed on in place and stored from there.
      const bool d_tma = !kSplitK && p.tma_d != 0 && tma_tile && ep.D != nullptr;
      if (d_tma) {
        if (lane == 0) {
          ptx::bulk_wait_read_all();  // stores of the previous tile have let go of the tiles
          ptx::mbar_expect_tx(dfull_bar(q, 0), 4096u);
          ptx::tma_load_2d(ptx::smem_u32(sC), &tmD, dfull_bar(q, 0), tl.n0,
                           tr.g * p.d_batch_rows + row0w);
        }
        __syncwarp();
      } else if (!deposit) {
#pragma unroll
        for (int a = 0; a < kAhead; ++a) epilogue_load_d<T>(p, ep, row, tl.n0 + a * 32, dq[a]);
      }

      // parts of this tile deposited by earlier pairs: pairs c_first .. pair-1
      int c_first = pair;
      unsigned int* cnt = nullptr;
      if (gather) {
        c_first = (int)(((long long)w.sk_tile * p.num_kb) / p.sk_per);
        cnt = p.sk_cnt + (w.sk_tile * 2 + (int)rank);
        if (threadIdx.x == 64) {
          const unsigned int need = (unsigned int)(pair - c_first);
          const long long t0 = clock64();
          int got = 0;
          while (!got) {
            const unsigned int v = *reinterpret_cast<volatile unsigned int*>(cnt);
            got = (v >= need);
            if (!got && (*abort_flag || clock64() - t0 > ptx::kWaitLimitCycles)) {
              *abort_flag = 1;
              break;
            }
          }
          *sk_flag = got;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const int got = *sk_flag;
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (!got) break;
        __threadfence();
      }
      // Deposit layout per (pair, CTA rank): [chunk 0..7][quad 0..7][row 0..127] float4, so that
      // the 32 lanes of a warp (32 consecutive rows) touch 512 contiguous bytes per access.
      auto part_ptr = [&](int c, int ch) {
        return reinterpret_cast<const float4*>(p.sk_ws + ((size_t)(c * 2 + (int)rank) << 15)) +
               (size_t)(ch * 8) * 128 + row_local;
      };
      float psum[32], pnext[32];
      auto load_parts = [&](int ch, float (&dst)[32]) {
#pragma unroll
        for (int j = 0; j < 32; ++j) dst[j] = 0.f;
        for (int c = c_first; c < pair; ++c) {  // fixed order: by contributing pair
          const float4* src = part_ptr(c, ch);
#pragma unroll
          for (int v = 0; v < 8; ++v) {
            const float4 f = __ldcg(src + v * 128);
            dst[4 * v] += f.x; dst[4 * v + 1] += f.y; dst[4 * v + 2] += f.z; dst[4 * v + 3] += f.w;
          }
        }
      };
      if (gather) load_parts(0, psum);

      bool ok = ptx::mbar_wait(tfull_bar(acc), acc_ph, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      ptx::tc_fence_after();
      const uint32_t t_acc = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * 256);
      if (d_tma) {
        EpiPtrs ept = ep;   // the transposed output leaves through per-lane stores
        ept.C = nullptr;
        bool okd = true;
#pragma unroll 1
        for (int jp = 0; jp < 4 && okd; ++jp) {
          const int b = jp & 1;
          uint8_t* const cur = b ? sT : sC;
          uint8_t* const oth = b ? sC : sT;
          if (jp + 1 < 4) {  // the next block of the addend into the other tile
            if (lane == 0) {
              ptx::bulk_wait_read_all();  // the store that read the other tile (if any) is done
              ptx::mbar_expect_tx(dfull_bar(q, b ^ 1), 4096u);
              ptx::tma_load_2d(ptx::smem_u32(oth), &tmD, dfull_bar(q, b ^ 1), tl.n0 + (jp + 1) * 64,
                               tr.g * p.d_batch_rows + row0w);
            }
            __syncwarp();
          }
          // every tile uses each barrier twice: use k of a tile waits for parity k
          okd = ptx::mbar_wait(dfull_bar(q, b), (uint32_t)(jp >> 1), abort_flag);
          okd = __all_sync(0xffffffffu, okd);
          if (!okd) break;
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            const int ch = 2 * jp + half;
            const int c0 = tl.n0 + ch * 32;
            uint32_t raw[32];
            ptx::tmem_ld_32x32(t_acc + (uint32_t)(ch * 32), raw);
            alignas(16) T dv[32];
#pragma unroll
            for (int v = 0; v < 4; ++v)
              reinterpret_cast<uint4*>(dv)[v] = *reinterpret_cast<const uint4*>(
                  cur + lane * 128 + (((half * 4 + v) ^ (lane & 7)) * 16));
            ptx::tmem_ld_wait();
            if (row0w < p.M && c0 < p.N) {  // warp-uniform
              alignas(16) T outv[32];
              epilogue_values<T>(p, ep, raw, dv, outv);
              if (ep.C != nullptr) epilogue_stage<T>(outv, cur, cur, lane, half, true, false);
              if (ep.CT != nullptr) epilogue_store_regs<T>(p, ept, outv, row, c0, bi);
            }
          }
          if (ep.C != nullptr) {
            ptx::fence_proxy_async_smem();
            __syncwarp();
            const int cx = tl.n0 + jp * 64;
            if (lane == 0 && row0w < p.M && cx < p.N) {
              ptx::tma_store_2d(&tmC, ptx::smem_u32(cur), cx, tr.g * p.c_batch_rows + row0w);
              ptx::bulk_commit();
            }
          }
        }
        if (!okd) break;
      } else if (!deposit) {
#pragma unroll 1
        for (int ch = 0; ch < 8; ++ch) {
          uint32_t raw[32];
          ptx::tmem_ld_32x32(t_acc + (uint32_t)(ch * 32), raw);
          if (ch + kAhead < 8) epilogue_load_d<T>(p, ep, row, tl.n0 + (ch + kAhead) * 32, dq[kAhead]);
          if (gather && ch + 1 < 8) load_parts(ch + 1, pnext);
          ptx::tmem_ld_wait();
          if (gather) {
#pragma unroll
            for (int j = 0; j < 32; ++j) raw[j] = __float_as_uint(psum[j] + __uint_as_float(raw[j]));
          }
          const int c0 = tl.n0 + ch * 32;
          if (!tma_tile) {
            epilogue_store<T>(p, ep, raw, dq[0], row, c0, bi);
          } else if (row0w < p.M && (c0 & ~63) < p.N) {  // warp-uniform: something of this 64-column pair is inside
            const int half = ch & 1;
            if (c0 < p.N) {
              alignas(16) T outv[32];
              epilogue_values<T>(p, ep, raw, dq[0], outv);
              if (half == 0) {  // the previous stores of this warp have let go of the staging tiles
                if (lane == 0) ptx::bulk_wait_read_all();
                __syncwarp();
              }
              epilogue_stage<T>(outv, sC, sT, lane, half, ep.C != nullptr, ep.CT != nullptr);
            }
            if (half == 1) {
              ptx::fence_proxy_async_smem();
              __syncwarp();
              if (lane == 0) {
                const int cx = c0 - 32;  // first column of the pair
                if (ep.C != nullptr)
                  ptx::tma_store_2d(&tmC, ptx::smem_u32(sC), cx, tr.g * p.c_batch_rows + row0w);
                if (ep.CT != nullptr)
                  ptx::tma_store_2d(&tmT, ptx::smem_u32(sT), row0w, tr.g * p.t_batch_rows + cx);
                ptx::bulk_commit();
              }
            }
          }
          if (ep.D != nullptr) {
#pragma unroll
            for (int a = 0; a < kAhead; ++a) {
#pragma unroll
              for (int v = 0; v < 4; ++v)
                reinterpret_cast<uint4*>(dq[a])[v] = reinterpret_cast<const uint4*>(dq[a + 1])[v];
            }
          }
          if (gather) {
#pragma unroll
            for (int j = 0; j < 32; ++j) psum[j] = pnext[j];
          }
        }
      } else {
        // deposit this part of the tile (this CTA's 128 rows x 256 fp32 columns)
        uint4* mine = reinterpret_cast<uint4*>(p.sk_ws + ((size_t)(pair * 2 + (int)rank) << 15)) +
                      row_local;
#pragma unroll 1
        for (int ch = 0; ch < 8; ++ch) {
          uint32_t raw[32];
          ptx::tmem_ld_32x32(t_acc + (uint32_t)(ch * 32), raw);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int v = 0; v < 8; ++v)
            mine[(size_t)(ch * 8 + v) * 128] =
                make_uint4(raw[4 * v], raw[4 * v + 1], raw[4 * v + 2], raw[4 * v + 3]);
        }
      }
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive_cluster(ptx::mapa(tempty_bar(acc), 0));
      acc ^= 1;
      if (acc == 0) acc_ph ^= 1u;

      if (deposit) {
        // publish the deposit: all 128 threads' stores first, then one count
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (threadIdx.x == 64) atomicAdd(p.sk_cnt + (w.sk_tile * 2 + (int)rank), 1u);
      }
    }
    // tile stores in flight read this CTA's shared memory and must be performed before the grid
    // counts as complete for its dependents
    if (p.tma_store && lane == 0) ptx::bulk_wait_all();
    __syncwarp();
  }

  // ---------------------------------------------------------------- teardown
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_sync();  // neither CTA frees TMEM or exits while the other may still use it
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc_pair(tmem_base, kTmemCols);
  }
  if (threadIdx.x == 0 && *abort_flag) atomicExch(p.err, 0x47320000u | (unsigned)blockIdx.x);
}

// Ring depth: 6 stages of 32 KiB by default; 4 cost 2-3 % on the large products, 3 cost 12 %.
int pair_stages(bool staging) {
  const int w = options().gemm_stages;
  const int v = (w >= 2 && w <= kMaxStages) ? w : kDefaultStages;
  return (staging && v > kMaxStagesWithStaging) ? kMaxStagesWithStaging : v;
}

// Tile order of a symmetric list: column strips of width w (tile_schedule.cuh has the reasoning:
// fewer distinct panels per wave, hence fewer DRAM reads) or plain column order (0).
int strip_width(const GemmParams& p) {
  if (!p.sym || p.batch > 1) return 0;
  const int w = options().gemm_strip;
  // By size: once the triangle has more tile columns than a wave of CTA pairs can keep in L2 side
  // by side, strips of 8 columns cut the DRAM reads (8192 x 8192: 671 -> 492 MB per launch, same
  // duration); smaller triangles keep the column order.
  if (w < 0) return p.tiles_m >= 24 ? 8 : 0;
  return w <= 64 ? w : 0;
}

// Clusters of two CTAs that can be resident at once on the current device (0 if unknown).
template <typename T>
int max_pairs_for() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  if (cached[dev] == 0) {
    constexpr int kMost = smem_bytes(kMaxStages, false) > smem_bytes(kMaxStagesWithStaging, true)
                              ? smem_bytes(kMaxStages, false)
                              : smem_bytes(kMaxStagesWithStaging, true);
    if (cudaFuncSetAttribute(gemm_tc2_kernel<T, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             kMost) != cudaSuccess ||
        cudaFuncSetAttribute(gemm_tc2_kernel<T, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             kMost) != cudaSuccess)
      return 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem_bytes(kDefaultStages, true);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, gemm_tc2_kernel<T, true>, &cfg) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      n = sm_count() / 2;
    }
    cached[dev] = n;
  }
  return cached[dev];
}

// Whether (and how) a list of `tiles` tiles of `num_kb` K blocks is balanced on `max_pairs` pairs.
// Depends on the extents and the device only, never on what else is running.
bool balance_plan(int tiles, int num_kb, int max_pairs, int batch, int* dp_tiles, int* per,
                  long long* total) {
  if (batch > 1 || !options().gemm_balance || max_pairs <= 0) return false;
  if ((size_t)max_pairs * 4 * sizeof(unsigned int) > kSkCntBytes) return false;
  return plan_balance(tiles, num_kb, max_pairs, dp_tiles, per, total);
}

template <typename T>
int launch2(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmC,
            const CUtensorMap& tmT, const CUtensorMap& tmD, GemmParams& p, int max_pairs,
            void* sk_ws, size_t sk_bytes, cudaStream_t stream) {
  const int T_all = p.num_tiles;
  int pairs = T_all < max_pairs ? T_all : max_pairs;
  p.sk_dp_tiles = T_all;
  p.sk_per = 0;
  p.sk_total = 0;
  p.sk_ws = nullptr;
  p.sk_cnt = nullptr;
  int dp_tiles = 0, per = 0;
  long long total = 0;
  const size_t need = kSkCntBytes + (size_t)max_pairs * 2 * kSkPartBytes;
  if (sk_ws != nullptr && sk_bytes >= need && (reinterpret_cast<uintptr_t>(sk_ws) & 255u) == 0 &&
      balance_plan(T_all, p.num_kb, max_pairs, p.batch, &dp_tiles, &per, &total)) {
    p.sk_dp_tiles = dp_tiles;
    p.sk_total = total;
    p.sk_per = per;
    p.sk_cnt = static_cast<unsigned int*>(sk_ws);
    p.sk_ws = reinterpret_cast<float*>(static_cast<char*>(sk_ws) + kSkCntBytes);
    pairs = max_pairs;
    // the deposit counters start every launch at zero, whatever an earlier launch left behind
    FM_CUDA_CHECK(cudaMemsetAsync(p.sk_cnt, 0, kSkCntBytes, stream));
  }
  {
    const int mode = options().pdl_trigger;  // 0 by schedule, 1 always early, 2 never
    p.early_trigger = mode == 1 || (mode == 0 && (T_all <= max_pairs || p.sk_per > 0));
  }
  p.stages = pair_stages(p.tma_store != 0);
  {
    const int want = options().gemm_kb_per_stage;
    p.kb_per_stage = (want >= 1 && want <= 3 && p.stages / want >= 2) ? want : 1;
  }
  p.stages -= p.stages % p.kb_per_stage;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(2 * pairs));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem_bytes(p.stages, p.tma_store != 0);
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.numAttrs = 1;
  if (options().pdl) {
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.numAttrs = 2;
  }
  cfg.attrs = attr;
  if (p.sk_per > 0) {
    p.tma_d = 0;  // the instantiation with partial sums keeps the per-lane addend loads
    FM_CUDA_CHECK(cudaLaunchKernelEx(&cfg, gemm_tc2_kernel<T, true>, tmA, tmB, tmC, tmT, tmD, p));
  } else {
    FM_CUDA_CHECK(cudaLaunchKernelEx(&cfg, gemm_tc2_kernel<T, false>, tmA, tmB, tmC, tmT, tmD, p));
  }
  return FM_OK;
}

}  // namespace

int gemm_tc2_tiles(int64_t M, int64_t N, int sym) {
  return count_tiles2(M, N, sym);
}

int gemm_tc2_max_pairs(int dtype) {
  return dtype == FM_BF16 ? max_pairs_for<__nv_bfloat16>() : max_pairs_for<__half>();
}

size_t gemm_tc2_sk_bytes(int dtype, int64_t M, int64_t N, int64_t K, int sym) {
  const int max_pairs = gemm_tc2_max_pairs(dtype);
  int dp_tiles = 0, per = 0;
  long long total = 0;
  if (!balance_plan(gemm_tc2_tiles(M, N, sym), (int)((K + BK - 1) / BK), max_pairs, 1, &dp_tiles,
                    &per, &total))
    return 0;
  return kSkCntBytes + (size_t)max_pairs * 2 * kSkPartBytes;
}

// `p` arrives filled except for the schedule fields, which depend on the tile shape.
int gemm_tc2_launch(int dtype, const CUtensorMap& tmA, const CUtensorMap& tmB,
                    const CUtensorMap& tmC, const CUtensorMap& tmT, const CUtensorMap& tmD,
                    GemmParams& p, void* sk_ws, size_t sk_bytes, cudaStream_t stream) {
  p.tiles_m = (p.M + 255) / 256;
  {
    const int tn = (p.N + 255) / 256;
    p.tiles_n = (!p.sym && tn < p.tiles_m) ? tn : 0;
  }
  p.tiles_per_batch = gemm_tc2_tiles(p.M, p.N, p.sym);
  p.num_tiles = p.tiles_per_batch * p.batch;
  p.strip_w = strip_width(p);
  const int max_pairs = gemm_tc2_max_pairs(dtype);
  if (max_pairs <= 0) return fail(FM_ERR_CUDA, "no resident CTA pair possible for the GEMM kernel");
  return dtype == FM_BF16
             ? launch2<__nv_bfloat16>(tmA, tmB, tmC, tmT, tmD, p, max_pairs, sk_ws, sk_bytes, stream)
             : launch2<__half>(tmA, tmB, tmC, tmT, tmD, p, max_pairs, sk_ws, sk_bytes, stream);
}

}  // namespace fm
