// Warp-specialised persistent GEMM engine for sm_100a.
//
//   warp 0      TMA producer   (one elected lane): global -> shared ring of kStages slots
//   warp 1      MMA issuer     (one elected lane): tcgen05.mma, shared -> TMEM accumulator
//   warps 2..   epilogue       (kEpiWarps/4 warps per 32-lane TMEM quarter, interleaved 32-column groups):
//                              TMEM -> registers -> policy
//
// One CTA per SM (the shared-memory request forbids a second one, which also keeps the 512-column
// TMEM allocation from ever blocking).  The accumulator is double buffered (2 x 256 columns) so the
// epilogue of tile t overlaps the main loop of tile t+1.  Every wait is bounded (ptx.cuh).
//
// A policy supplies: operand kind/majorness, the tile -> job mapping and the epilogue.
#pragma once
#include "ptx.cuh"

namespace xmc {

constexpr int kMaxEpiWarps = 16;            // a policy picks 4, 8 or 16 epilogue warps (kEpiWarps)
constexpr int kStages = 4;
constexpr int kTileM = 128;                 // UMMA M = TMEM lanes
constexpr int kTileN = 256;                 // UMMA N upper bound = TMEM columns per accumulator
constexpr int kRowBytes = 128;              // swizzle span: one operand row per k-step
constexpr int kStageABytes = kTileM * kRowBytes;   // 16 KB
constexpr int kStageBBytes = kTileN * kRowBytes;   // 32 KB
constexpr int kStageBytes = kStageABytes + kStageBBytes;
constexpr int kTmemCols = 512;
constexpr int kMnBoxBytes = 64 * kRowBytes;  // MN-major operands arrive as boxes of 64 k-rows x 128 B

struct Job {
  int a0;        // K-major: first row of A;   MN-major: first M index
  int b0;        // K-major: first row of B;   MN-major: first N index
  int k_begin;   // first k-step (one k-step = 128 bytes of K for K-major, 64 k-rows for MN-major)
  int k_steps;
  int n_eff;     // UMMA N of this tile: multiple of 16, <= 256
  int t0, t1, t2;  // policy-defined tile coordinates
};

struct EpiCtx {
  int q;        // TMEM lane quarter: rows q*32 .. q*32+31 of the tile
  int lane;
  int h;        // this warp handles 32-column groups h, h+nsplit, h+2*nsplit, ...
  int nsplit;
  int slot;     // epilogue warp index 0..kEpiWarps-1
};

struct SharedTail {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  Ctl ctl;
  uint32_t bitmap[kTileM * (kTileN / 32)];   // positives of one (label tile, batch tile)
};

constexpr int kSmemBytes = kStages * kStageBytes + (int)sizeof(SharedTail) + 1024;
static_assert(kSmemBytes <= 232448, "exceeds the 227 KB of shared memory a CTA can get");

template <class Policy>
__global__ void __launch_bounds__(64 + 32 * Policy::kEpiWarps, 1)
gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
            const typename Policy::Params p) {
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment: the 128-byte swizzle pattern is a function of address bits [4,10)
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  SharedTail& sh = *reinterpret_cast<SharedTail*>(smem + kStages * kStageBytes);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_tiles = Policy::num_tiles(p);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&sh.full[s]), 1);
      mbar_init(smem_u32(&sh.empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&sh.tmem_full[b]), 1);
      mbar_init(smem_u32(&sh.tmem_empty[b]), 32 * Policy::kEpiWarps);
    }
    sh.ctl.abort = 0;
    fence_barrier_init();
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&sh.tmem_base), kTmemCols);
    tmem_relinquish();
  }
  pdl_launch_dependents();                  // the next kernel may start its prologue as SMs free up
  tc_fence_before();
  __syncthreads();
  pdl_wait();                               // nothing above touches global memory written by earlier kernels
  tc_fence_after();
  const uint32_t tmem_base = sh.tmem_base;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x) {
        Job job;
        Policy::job(p, tile, job);
        for (int k = 0; k < job.k_steps; ++k, ++it) {
          const uint32_t s = it % kStages, ph = (it / kStages) & 1u;
          if (!mbar_wait(smem_u32(&sh.empty[s]), ph ^ 1u, &sh.ctl, p.status, 100 + (int)s)) {
            ok = false;
            break;
          }
          const uint32_t bar = smem_u32(&sh.full[s]);
          const uint32_t sa = smem_u32(smem + s * kStageBytes);
          const uint32_t sb = sa + kStageABytes;
          const int kk = job.k_begin + k;
          if constexpr (!Policy::kMnMajor) {
            mbar_arrive_expect_tx(bar, kStageBytes);
            tma_load_2d(sa, &map_a, bar, kk * Policy::kElemsPerRow, job.a0);
            tma_load_2d(sb, &map_b, bar, kk * Policy::kElemsPerRow, job.b0);
          } else {
            const int nb = (job.n_eff + 63) >> 6;
            mbar_arrive_expect_tx(bar, (2 + nb) * kMnBoxBytes);
            for (int j = 0; j < 2; ++j)
              tma_load_2d(sa + j * kMnBoxBytes, &map_a, bar, job.a0 + 64 * j, kk * 64);
            for (int j = 0; j < nb; ++j)
              tma_load_2d(sb + j * kMnBoxBytes, &map_b, bar, job.b0 + 64 * j, kk * 64);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      uint32_t it = 0, t_local = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x, ++t_local) {
        Job job;
        Policy::job(p, tile, job);
        const uint32_t buf = t_local & 1u, aph = (t_local >> 1) & 1u;
        if (!mbar_wait(smem_u32(&sh.tmem_empty[buf]), aph ^ 1u, &sh.ctl, p.status, 200 + (int)buf)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * kTileN;
        const uint32_t idesc = make_idesc(kTileM, (uint32_t)job.n_eff, Policy::kFmt, Policy::kFmt,
                                          Policy::kMnMajor ? 1u : 0u, Policy::kMnMajor ? 1u : 0u);
        for (int k = 0; k < job.k_steps; ++k, ++it) {
          const uint32_t s = it % kStages, ph = (it / kStages) & 1u;
          if (!mbar_wait(smem_u32(&sh.full[s]), ph, &sh.ctl, p.status, 300 + (int)s)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * kStageBytes);
          const uint32_t sb = sa + kStageABytes;
          if constexpr (!Policy::kMnMajor) {
            // K-major, 128B swizzle: rows of 128 B, 8-row groups 1024 B apart; one UMMA eats 32 B of K
            const uint64_t da = smem_desc_sw128(sa, 16, 1024);
            const uint64_t db = smem_desc_sw128(sb, 16, 1024);
#pragma unroll
            for (int u = 0; u < kRowBytes / 32; ++u) {
              const uint32_t acc = (k | u) != 0 ? 1u : 0u;
              if constexpr (Policy::kFp8) umma_f8(d_tmem, da + 2u * u, db + 2u * u, idesc, acc);
              else umma_f16(d_tmem, da + 2u * u, db + 2u * u, idesc, acc);
            }
          } else {
            // MN-major, 128B swizzle: blocks of 64 MN-elements (128 B) x 64 k-rows; 8-k-row groups
            // 1024 B apart (stride offset), MN blocks 8192 B apart (leading offset); one UMMA eats
            // 16 k-rows = 2048 B
            const uint64_t da = smem_desc_sw128(sa, kMnBoxBytes, 1024);
            const uint64_t db = smem_desc_sw128(sb, kMnBoxBytes, 1024);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const uint32_t acc = (k | u) != 0 ? 1u : 0u;
              umma_f16(d_tmem, da + 128u * u, db + 128u * u, idesc, acc);
            }
          }
          umma_commit(smem_u32(&sh.empty[s]));     // slot is free once these MMAs have read it
        }
        if (ok) umma_commit(smem_u32(&sh.tmem_full[buf]));
      }
    }
  } else {
    // ------------------------------ epilogue ------------------------------
    // No block-level barrier is used in here: a warp that unwinds after a time-out must never
    // leave the others stuck in an unbounded bar.sync.  Warps cooperate through __syncwarp only.
    EpiCtx ec;
    ec.q = warp & 3;                                // TMEM lane quarter this warp may access
    ec.lane = lane;
    ec.h = (warp - 2) >> 2;                         // which of the column-group phases this warp takes
    ec.nsplit = Policy::kEpiWarps / 4;
    ec.slot = warp - 2;
    const int q = ec.q;
    typename Policy::EpilogueState st;
    Policy::epilogue_begin(p, st);
    uint32_t t_local = 0;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++t_local) {
      Job job;
      Policy::job(p, tile, job);
      const uint32_t buf = t_local & 1u, aph = (t_local >> 1) & 1u;
      Policy::epilogue_pre(p, job, sh, ec, st);          // overlaps the tile's main loop
      if (!mbar_wait_relaxed(smem_u32(&sh.tmem_full[buf]), aph, &sh.ctl, p.status, 400 + (int)buf)) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * kTileN;
      Policy::epilogue(p, job, taddr, job.k_steps > 0, sh, ec, st);
      tc_fence_before();
      mbar_arrive(smem_u32(&sh.tmem_empty[buf]));
    }
    Policy::epilogue_end(p, sh, ec, st);
  }

  __syncwarp();
  if (sh.ctl.abort) {
    // unwinding after a time-out: give copies still in flight time to land before the CTA exits
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace xmc
