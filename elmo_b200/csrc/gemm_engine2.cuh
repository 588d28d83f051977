// The GEMM engine on CTA PAIRS (cluster of two, tcgen05 cta_group::2) for K-major operands.
//
// A pair owns a 256 x 256 output tile: CTA r of the pair holds rows [128 r, 128 r + 128) of the
// accumulator in its own TMEM and loads only its own 128 rows of A and its own HALF of the B rows
// (plain TMA into its own shared memory; completion bytes are counted on the leader's barrier).
// One thread of the leader CTA issues every MMA for both SMs.  Compared with the single-CTA engine
// each CTA stages 32 KB instead of 48 KB per k-step for the same tensor work, so the ring holds 6
// stages and the L2 -> shared-memory operand stream shrinks by a third.
//
// Barriers: full[s] lives in the leader (1 arrival + the bytes of both CTAs); empty[s] and
// tmem_full[b] exist in both CTAs and are signalled together by the leader's commits;
// tmem_empty[b] lives in the leader and collects the epilogue threads of both CTAs.
// Policies are the ones of gemm_engine.cuh; their tile -> job mapping must use 256-row M tiles
// (Params::m_rows == 256).
#pragma once
#include "gemm_engine.cuh"

namespace xmc {

constexpr int kStages2 = 6;
constexpr int kStage2Bytes = 2 * kStageABytes;          // A 16 KB + half of B 16 KB
static_assert(kStages2 <= 8, "SharedTail2 holds 8 stage barriers");

struct SharedTail2 {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  Ctl ctl;
  uint32_t bitmap[kTileM * (kTileN / 32)];
};
// the epilogues address `bitmap` through SharedTail: hand the policies a SharedTail view whose
// bitmap member coincides with this one
static_assert(sizeof(SharedTail2) - offsetof(SharedTail2, bitmap) == sizeof(SharedTail) - offsetof(SharedTail, bitmap),
              "tail layouts diverged");

constexpr int kSmem2Bytes = kStages2 * kStage2Bytes + (int)sizeof(SharedTail2) + 1024;
static_assert(kSmem2Bytes <= 232448, "exceeds the 227 KB of shared memory a CTA can get");

template <class Policy>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(64 + 32 * Policy::kEpiWarps, 1)
gemm2_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
             const typename Policy::Params p) {
  static_assert(!Policy::kMnMajor, "CTA pairs are implemented for K-major operands");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  SharedTail2& sh = *reinterpret_cast<SharedTail2*>(smem + kStages2 * kStage2Bytes);
  // view for the policies: same bitmap member
  SharedTail& shp = *reinterpret_cast<SharedTail*>(reinterpret_cast<uint8_t*>(&sh) + offsetof(SharedTail2, bitmap) -
                                                   offsetof(SharedTail, bitmap));
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int n_pairs = (int)gridDim.x >> 1;
  const int pair = (int)blockIdx.x >> 1;
  const int n_tiles = Policy::num_tiles(p);
  constexpr uint32_t kEpiThreads = 32 * Policy::kEpiWarps;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages2; ++s) {
      mbar_init(smem_u32(&sh.full[s]), 1);
      mbar_init(smem_u32(&sh.empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&sh.tmem_full[b]), 1);
      mbar_init(smem_u32(&sh.tmem_empty[b]), 2 * kEpiThreads);
    }
    sh.ctl.abort = 0;
    fence_barrier_init();
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(&sh.tmem_base), kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  cluster_sync_all();                       // both CTAs' barriers exist before anything remote happens
  tc_fence_after();
  const uint32_t tmem_base = sh.tmem_base;

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------------------
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = pair; ok && tile < n_tiles; tile += n_pairs) {
        Job job;
        Policy::job(p, tile, job);
        const int a_row = job.a0 + 128 * (int)rank;
        const int b_row = job.b0 + (int)rank * (job.n_eff >> 1);
        for (int k = 0; k < job.k_steps; ++k, ++it) {
          const uint32_t s = it % kStages2, ph = (it / kStages2) & 1u;
          if (!mbar_wait(smem_u32(&sh.empty[s]), ph ^ 1u, &sh.ctl, p.status, 100 + (int)s)) {
            ok = false;
            break;
          }
          const uint32_t bar_local = smem_u32(&sh.full[s]);
          if (leader) mbar_arrive_expect_tx(bar_local, 2 * kStage2Bytes);      // bytes of both CTAs
          const uint32_t bar = mapa_shared(bar_local, 0);
          const uint32_t sa = smem_u32(smem + s * kStage2Bytes);
          const int kk = job.k_begin + k;
          tma_load_2d_pair(sa, &map_a, bar, kk * Policy::kElemsPerRow, a_row);
          tma_load_2d_pair(sa + kStageABytes, &map_b, bar, kk * Policy::kElemsPerRow, b_row);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (leader CTA only) ------------------------------
    if (lane == 0 && leader) {
      uint32_t it = 0, t_local = 0;
      bool ok = true;
      for (int tile = pair; ok && tile < n_tiles; tile += n_pairs, ++t_local) {
        Job job;
        Policy::job(p, tile, job);
        const uint32_t buf = t_local & 1u, aph = (t_local >> 1) & 1u;
        if (!mbar_wait(smem_u32(&sh.tmem_empty[buf]), aph ^ 1u, &sh.ctl, p.status, 200 + (int)buf)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * kTileN;
        const uint32_t idesc = make_idesc(256, (uint32_t)job.n_eff, Policy::kFmt, Policy::kFmt, 0u, 0u);
        for (int k = 0; k < job.k_steps; ++k, ++it) {
          const uint32_t s = it % kStages2, ph = (it / kStages2) & 1u;
          if (!mbar_wait(smem_u32(&sh.full[s]), ph, &sh.ctl, p.status, 300 + (int)s)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * kStage2Bytes);
          const uint64_t da = smem_desc_sw128(sa, 16, 1024);
          const uint64_t db = smem_desc_sw128(sa + kStageABytes, 16, 1024);
#pragma unroll
          for (int u = 0; u < kRowBytes / 32; ++u) {
            const uint32_t acc = (k | u) != 0 ? 1u : 0u;
            if constexpr (Policy::kFp8) umma_f8_pair(d_tmem, da + 2u * u, db + 2u * u, idesc, acc);
            else umma_f16_pair(d_tmem, da + 2u * u, db + 2u * u, idesc, acc);
          }
          umma_commit_pair(smem_u32(&sh.empty[s]));      // frees slot s in both CTAs
        }
        if (ok) umma_commit_pair(smem_u32(&sh.tmem_full[buf]));
      }
    }
  } else {
    // ------------------------------ epilogue (both CTAs, own 128 rows) ------------------------------
    EpiCtx ec;
    ec.q = warp & 3;
    ec.lane = lane;
    ec.h = (warp - 2) >> 2;
    ec.nsplit = Policy::kEpiWarps / 4;
    ec.slot = warp - 2;
    typename Policy::EpilogueState st;
    Policy::epilogue_begin(p, st);
    uint32_t t_local = 0;
    for (int tile = pair; tile < n_tiles; tile += n_pairs, ++t_local) {
      Job job;
      Policy::job(p, tile, job);
      job.a0 += 128 * (int)rank;
      const uint32_t buf = t_local & 1u, aph = (t_local >> 1) & 1u;
      Policy::epilogue_pre(p, job, shp, ec, st);
      if (!mbar_wait_relaxed(smem_u32(&sh.tmem_full[buf]), aph, &sh.ctl, p.status, 400 + (int)buf)) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(ec.q * 32) << 16) + buf * kTileN;
      Policy::epilogue(p, job, taddr, job.k_steps > 0, shp, ec, st);
      tc_fence_before();
      mbar_arrive_cluster(mapa_shared(smem_u32(&sh.tmem_empty[buf]), 0));
    }
    Policy::epilogue_end(p, shp, ec, st);
  }

  __syncwarp();
  if (sh.ctl.abort) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before();
  cluster_sync_all();                       // the peer may still be reading this CTA's shared memory / TMEM
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

}  // namespace xmc
