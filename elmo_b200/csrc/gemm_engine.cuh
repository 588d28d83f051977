// Warp-specialised persistent GEMM engine for sm_100a.
//
//   warp 0      TMA producer   (one elected lane): global -> shared ring of kStages slots
//   warp 1      MMA issuer     (one elected lane): tcgen05.mma, shared -> TMEM accumulator
//   warps 2..   epilogue       (kEpiWarps/4 warps per 32-lane TMEM quarter, interleaved 32-column groups):
//                              TMEM -> registers -> policy
//   then        4 operand-converter warps (kConv policies) or 1 store warp (kCTile policies)
//
// One CTA per SM (the shared-memory request forbids a second one, which also keeps the 512-column
// TMEM allocation from ever blocking).  The accumulator is double buffered (2 x 256 columns) so the
// epilogue of tile t overlaps the main loop of tile t+1.  Every wait is bounded (ptx.cuh).
//
// A policy supplies: operand kind/majorness, the tile -> job mapping and the epilogue.  A policy with
// kConv = 1 (2) takes its A (B) operand from e4m3 storage although it multiplies in bf16 (the
// "simulated FP8" arithmetic): the producer brings the raw bytes in, four extra warps rewrite them as
// bf16 in the operand's swizzled layout, and the MMA issuer waits for both.  A policy with
// kCTile set also has the producer fetch, per tile, the 128 x 256-byte block of a third tensor (the
// weights the update epilogue reads and rewrites) into a two-deep shared-memory ring while the tile's
// main loop runs; the epilogue rewrites the block in place and a warp of its own stores it back by TMA
// and hands the slot back to the producer, so no epilogue thread ever touches global memory or waits for
// a copy.
//
// PAIR = true runs the same roles on CTA PAIRS (cluster of two, tcgen05 cta_group::2): a pair owns a
// 256 x 256 output tile; CTA r holds rows [128 r, 128 r + 128) of the accumulator in its own TMEM and
// loads only its own 128 rows of A and its own HALF of the B rows (plain TMA into its own shared memory,
// no multicast; the bytes of both CTAs are counted on the leader's barrier).  One elected thread of the
// leader issues every MMA for both SMs.  Per CTA and k-step 32 KB instead of 48 KB are staged and each
// MMA reads 8 KB instead of 12 KB of shared memory for the same tensor work: the shared-memory traffic
// that bounds the single-CTA tile falls by a third, the operand stream from L2 likewise, and the ring
// holds more stages.  Barriers: full[s] lives in the leader; empty[s] and tmem_full[b] exist in both
// CTAs and are signalled together by the leader's commits; tmem_empty[b] lives in the leader and
// collects the epilogue threads of both CTAs.  Everything else (epilogue, weight-tile ring, bitmap)
// is per CTA as before.  A policy's tile -> job mapping uses Params::m_rows (256 for pairs); the
// engine adds 128 * rank to Job::a0.
#pragma once
#include "ptx.cuh"

namespace xmc {

constexpr int kMaxEpiWarps = 16;            // a policy picks 4, 8 or 16 epilogue warps (kEpiWarps)
constexpr int kMaxStages = 8;               // a policy picks its ring depth (kStages / kStagesPair <= kMaxStages)
constexpr int kTileM = 128;                 // UMMA M = TMEM lanes
constexpr int kTileN = 256;                 // UMMA N upper bound = TMEM columns per accumulator
constexpr int kRowBytes = 128;              // swizzle span: one operand row per k-step
constexpr int kStageABytes = kTileM * kRowBytes;   // 16 KB
constexpr int kStageBBytes = kTileN * kRowBytes;   // 32 KB
constexpr int kStageBytes = kStageABytes + kStageBBytes;
constexpr int kTmemCols = 512;
constexpr int kMnBoxBytes = 64 * kRowBytes;  // MN-major operands arrive as boxes of 64 k-rows x 128 B
constexpr int kCHalfBytes = kTileM * 128;    // epilogue-input tile: two 128-byte-swizzled halves of 128 rows x 128 B
constexpr int kCTileBytes = 2 * kCHalfBytes; // 32 KB

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
  uint8_t* ctile;         // this tile's read-modify-write block in shared memory (kCTile policies)
  uint32_t* bitmap;       // kBitmap policies: kTileM x kTileN bits, the positives of one (label tile, batch tile)
};

struct SharedTail {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t raw_full[kMaxStages];   // kConv policies: the raw e4m3 bytes of the stage have landed
  uint64_t conv_full[kMaxStages];  // ... and have been rewritten as bf16 (one arrival per converter warp)
  uint64_t c_full[2];      // epilogue tile landed (kCTile policies)
  uint64_t c_done[2];      // all epilogue warps have rewritten their part of it
  uint64_t c_empty[2];     // it has been stored back and may be refilled
  uint32_t tmem_base;
  Ctl ctl;
};
constexpr int kBitmapBytes = kTileM * (kTileN / 32) * 4;
// roles of a CTA, as bits of Policy::kWaitRoles (who waits for the previous kernels of the stream)
constexpr int kRoleProducer = 1, kRoleMma = 2, kRoleEpilogue = 4, kRoleExtra = 8, kRoleAll = 15;
constexpr int kConvWarps = 4;
template <class Policy>
__host__ __device__ constexpr int conv_rows() { return Policy::kConv == 1 ? kTileM : (Policy::kConv == 2 ? kTileN : 0); }
template <class Policy>
__host__ __device__ constexpr int block_threads() {
  return 64 + 32 * Policy::kEpiWarps + (Policy::kConv ? 32 * kConvWarps : 0) + (Policy::kCTile ? 32 : 0);
}


// ring depth and bytes of one stage (a CTA of a pair stages half of the B rows)
template <class Policy, bool PAIR>
__host__ __device__ constexpr int ring_stages() {
  if constexpr (PAIR) return Policy::kStagesPair;
  else return Policy::kStages;
}
template <bool PAIR>
__host__ __device__ constexpr int stage_bytes() { return PAIR ? kStageABytes + kStageBBytes / 2 : kStageBytes; }

template <class Policy, bool PAIR = false>
__host__ __device__ constexpr int smem_bytes() {
  return ring_stages<Policy, PAIR>() * (stage_bytes<PAIR>() + conv_rows<Policy>() * 64) +
         (Policy::kCTile ? Policy::kCBufs * kCTileBytes : 0) + (Policy::kBitmap ? kBitmapBytes : 0) +
         (int)sizeof(SharedTail) + 1024;
}

// Address of the 8 bytes at byte column `col` (multiple of 8) of row `row` of an epilogue tile, as the
// 128-byte-swizzling TMA copies lay it out (two halves of 128 rows x 128 B; 16-byte pieces XOR row & 7).
__device__ __forceinline__ uint2* ctile_ptr8(uint8_t* tile, int row, int col) {
  uint8_t* rowp = tile + (col >> 7) * kCHalfBytes + row * 128;
  return reinterpret_cast<uint2*>(rowp + (((((col & 127) >> 4) ^ (row & 7)) << 4) | (col & 8)));
}

template <class Policy, bool PAIR = false>
__global__ void __launch_bounds__(block_threads<Policy>(), 1)
gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
            const __grid_constant__ CUtensorMap map_c, const typename Policy::Params p) {
  constexpr int kStages = ring_stages<Policy, PAIR>();
  constexpr int kStageBytes = stage_bytes<PAIR>();          // shadows the single-CTA constant on purpose
  static_assert(kStages >= 2 && kStages <= kMaxStages, "ring depth");
  static_assert(smem_bytes<Policy, PAIR>() <= 232448, "exceeds the 227 KB of shared memory a CTA can get");
  static_assert(!PAIR || (!Policy::kMnMajor && Policy::kConv == 0), "CTA pairs take K-major operands as stored");
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment: the 128-byte swizzle pattern is a function of address bits [4,10)
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  constexpr int kRawBytes = conv_rows<Policy>() * 64;      // raw e4m3 bytes of one k-step of the converted operand
  uint8_t* smem_raw_ring = smem + kStages * kStageBytes;
  uint8_t* smem_c = smem_raw_ring + kStages * kRawBytes;
  uint8_t* smem_bm = smem_c + (Policy::kCTile ? Policy::kCBufs * kCTileBytes : 0);
  SharedTail& sh = *reinterpret_cast<SharedTail*>(smem_bm + (Policy::kBitmap ? kBitmapBytes : 0));
  constexpr uint32_t kCBufs = Policy::kCTile ? (uint32_t)Policy::kCBufs : 1u;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_tiles = Policy::num_tiles(p);
  // a pair is one worker: both CTAs walk the same tiles
  uint32_t rank = 0u;
  if constexpr (PAIR) rank = cluster_ctarank();
  const int worker = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int n_workers = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&sh.full[s]), 1);
      mbar_init(smem_u32(&sh.empty[s]), 1);
      mbar_init(smem_u32(&sh.raw_full[s]), 1);
      mbar_init(smem_u32(&sh.conv_full[s]), kConvWarps);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&sh.tmem_full[b]), 1);
      mbar_init(smem_u32(&sh.tmem_empty[b]), (PAIR ? 2 : 1) * Policy::kEpiWarps);    // one arrival per epilogue warp
      mbar_init(smem_u32(&sh.c_full[b]), 1);
      mbar_init(smem_u32(&sh.c_done[b]), Policy::kEpiWarps);
      mbar_init(smem_u32(&sh.c_empty[b]), 1);
    }
    sh.ctl.abort = 0;
    sh.ctl.limit = Policy::wait_limit(p);
    fence_barrier_init();
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
    if constexpr (Policy::kCTile) tma_prefetch_desc(&map_c);
  }
  if (warp == 1) {
    if constexpr (PAIR) {
      tmem_alloc_pair(smem_u32(&sh.tmem_base), kTmemCols);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(smem_u32(&sh.tmem_base), kTmemCols);
      tmem_relinquish();
    }
  }
  pdl_launch_dependents();                  // the next kernel may start its prologue as SMs free up
  tc_fence_before();
  if constexpr (PAIR) cluster_sync_all();   // both CTAs' barriers exist before anything remote happens
  else __syncthreads();
  // Nothing above touches global memory written by earlier kernels.  From here on a role waits for the
  // kernels before this one only if it has to (Policy::kWaitRoles): a producer whose operands no recent
  // kernel writes streams the first tiles in while the previous kernel drains, and the MMA issuer, which
  // touches shared and tensor memory only, goes with it; whoever reads or writes what the previous
  // kernels share waits.
  {
    const int role = warp == 0 ? kRoleProducer : warp == 1 ? kRoleMma : warp < 2 + Policy::kEpiWarps ? kRoleEpilogue : kRoleExtra;
    if (Policy::kWaitRoles & role) pdl_wait();
  }
  tc_fence_after();
  const uint32_t tmem_base = sh.tmem_base;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    {
      // Both issuing roles share their scheduler with busy epilogue warps, so every instruction here
      // waits its turn.  The whole warp runs the loop on warp-uniform values (uniform registers and
      // datapath: no per-operand moves from the vector registers) and one elected lane issues; stage
      // index and phase are running counters, addresses and descriptors advance by adds.
      uint32_t s = 0, ph = 0, t_local = 0;
      bool ok = true;
      const uint32_t full0 = smem_u32(&sh.full[0]), empty0 = smem_u32(&sh.empty[0]), stage0 = smem_u32(smem);
      uint32_t full_leader = full0;                       // where this CTA's operand bytes are counted
      if constexpr (PAIR) full_leader = mapa_shared(full0, 0);
      for (int tile = worker; ok && tile < n_tiles; tile += n_workers, ++t_local) {
        Job job;
        Policy::job(p, tile, job);
        int c_col = 0;
        if constexpr (Policy::kCTile) c_col = Policy::c_col(job);
        if constexpr (PAIR) {
          job.a0 += kTileM * (int)rank;
          job.b0 += (int)rank * (job.n_eff >> 1);        // this CTA's half of the B rows
        }
        // The epilogue's read-modify-write block of this tile is requested as soon as its slot has been
        // stored back (the epilogue of tile t - kCBufs); until then the operand loads go ahead, and the
        // slot is polled once per k-step without blocking.
        bool c_pending = Policy::kCTile;
        const uint32_t cb = t_local % kCBufs, cph = (t_local / kCBufs) & 1u;
        auto issue_c = [&]() {
          if constexpr (Policy::kCTile) {
            const uint32_t bar = smem_u32(&sh.c_full[cb]);
            const uint32_t dst = smem_u32(smem_c + cb * kCTileBytes);
            if (elect_one()) {
              mbar_arrive_expect_tx(bar, kCTileBytes);
              tma_load_2d(dst, &map_c, bar, c_col, job.a0);
              tma_load_2d(dst + kCHalfBytes, &map_c, bar, c_col + 128, job.a0);
            }
            __syncwarp();
          }
          c_pending = false;
        };
        int kk = job.k_begin * (Policy::kMnMajor ? 64 : Policy::kElemsPerRow);
        for (int k = 0; k < job.k_steps; ++k) {
          if constexpr (Policy::kCTile) {
            if (c_pending && __any_sync(0xffffffffu, mbar_test_wait(smem_u32(&sh.c_empty[cb]), cph ^ 1u))) issue_c();
          }
          if (!mbar_wait_warp(empty0 + 8u * s, ph ^ 1u, &sh.ctl, p.status, 100 + (int)s)) {
            ok = false;
            break;
          }
          const uint32_t bar = full0 + 8u * s;
          const uint32_t sa = stage0 + s * kStageBytes;
          const uint32_t sb = sa + kStageABytes;
          if constexpr (!Policy::kMnMajor) {
            if (!Policy::skip_load(p, tile, k) && elect_one()) {
              if constexpr (PAIR) {
                if (rank == 0) mbar_arrive_expect_tx(bar, 2 * kStageBytes);       // the bytes of both CTAs
                const uint32_t lbar = full_leader + 8u * s;
                tma_load_2d_pair(sa, &map_a, lbar, kk, job.a0);
                tma_load_2d_pair(sb, &map_b, lbar, kk, job.b0);
              } else if constexpr (Policy::kConv == 0) {
                mbar_arrive_expect_tx(bar, kStageBytes);
                tma_load_2d(sa, &map_a, bar, kk, job.a0);
                tma_load_2d(sb, &map_b, bar, kk, job.b0);
              } else {
                // the converted operand arrives raw (64 bytes per row = the 64 bf16 elements of this k-step)
                const uint32_t rbar = smem_u32(&sh.raw_full[s]);
                const uint32_t raw = smem_u32(smem_raw_ring + s * kRawBytes);
                mbar_arrive_expect_tx(rbar, kRawBytes);
                if constexpr (Policy::kConv == 1) {
                  tma_load_2d(raw, &map_a, rbar, kk, job.a0);
                  mbar_arrive_expect_tx(bar, kStageBBytes);
                  tma_load_2d(sb, &map_b, bar, kk, job.b0);
                } else {
                  tma_load_2d(raw, &map_b, rbar, kk, job.b0);
                  mbar_arrive_expect_tx(bar, kStageABytes);
                  tma_load_2d(sa, &map_a, bar, kk, job.a0);
                }
              }
            }
            kk += Policy::kElemsPerRow;
          } else {
            const int nb = (job.n_eff + 63) >> 6;
            if (elect_one()) {
              mbar_arrive_expect_tx(bar, (2 + nb) * kMnBoxBytes);
              for (int j = 0; j < 2; ++j)
                tma_load_2d(sa + j * kMnBoxBytes, &map_a, bar, job.a0 + 64 * j, kk);
              for (int j = 0; j < nb; ++j)
                tma_load_2d(sb + j * kMnBoxBytes, &map_b, bar, job.b0 + 64 * j, kk);
            }
            kk += 64;
          }
          __syncwarp();
          if (++s == (uint32_t)kStages) {
            s = 0;
            ph ^= 1u;
          }
        }
        if constexpr (Policy::kCTile) {
          if (ok && c_pending) {
            if (!mbar_wait_warp(smem_u32(&sh.c_empty[cb]), cph ^ 1u, &sh.ctl, p.status, 600 + (int)cb)) break;
            issue_c();
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (of a pair: the leader's) ------------------------------
    if (!PAIR || rank == 0) {
      uint32_t s = 0, ph = 0, t_local = 0;
      bool ok = true;
      const uint32_t full0 = smem_u32(&sh.full[0]), empty0 = smem_u32(&sh.empty[0]);
      // K-major, 128B swizzle: rows of 128 B, 8-row groups 1024 B apart; one UMMA eats 32 B of K.
      // MN-major, 128B swizzle: blocks of 64 MN-elements (128 B) x 64 k-rows; 8-k-row groups 1024 B apart
      // (stride offset), MN blocks 8192 B apart (leading offset); one UMMA eats 16 k-rows = 2048 B.
      constexpr uint32_t kLbo = Policy::kMnMajor ? (uint32_t)kMnBoxBytes : 16u;
      constexpr uint32_t kDescStep = Policy::kMnMajor ? 128u : 2u;      // descriptor address units (16 B) per UMMA
      constexpr uint32_t desc_hi = smem_desc_hi_sw128(1024);
      const uint32_t a_lo0 = smem_desc_lo(smem_u32(smem), kLbo);
      for (int tile = worker; ok && tile < n_tiles; tile += n_workers, ++t_local) {
        Job job;
        Policy::job(p, tile, job);
        const uint32_t buf = t_local & 1u, aph = (t_local >> 1) & 1u;
        if (!mbar_wait_warp(smem_u32(&sh.tmem_empty[buf]), aph ^ 1u, &sh.ctl, p.status, 200 + (int)buf)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * kTileN;
        const uint32_t idesc = make_idesc(PAIR ? 2 * kTileM : kTileM, (uint32_t)job.n_eff, Policy::kFmt, Policy::kFmt,
                                          Policy::kMnMajor ? 1u : 0u, Policy::kMnMajor ? 1u : 0u);
        uint32_t acc = 0u;
        for (int k = 0; k < job.k_steps; ++k) {
          if (!mbar_wait_warp(full0 + 8u * s, ph, &sh.ctl, p.status, 300 + (int)s)) {
            ok = false;
            break;
          }
          if constexpr (Policy::kConv != 0) {
            if (!mbar_wait_warp(smem_u32(&sh.conv_full[s]), ph, &sh.ctl, p.status, 310 + (int)s)) {
              ok = false;
              break;
            }
          }
          tc_fence_after();
          const uint32_t a_lo = a_lo0 + s * (uint32_t)(kStageBytes >> 4);
          const uint32_t b_lo = a_lo + (uint32_t)(kStageABytes >> 4);
          if (elect_one()) {
#pragma unroll
            for (uint32_t u = 0; u < 4; ++u) {
              const uint32_t au = a_lo + kDescStep * u, bu = b_lo + kDescStep * u, accu = u == 0 ? acc : 1u;
              if constexpr (PAIR) {
                if constexpr (Policy::kFp8) umma_f8_lohi_pair(d_tmem, au, bu, desc_hi, idesc, accu);
                else umma_f16_lohi_pair(d_tmem, au, bu, desc_hi, idesc, accu);
              } else {
                if constexpr (Policy::kFp8) umma_f8_lohi(d_tmem, au, bu, desc_hi, idesc, accu);
                else umma_f16_lohi(d_tmem, au, bu, desc_hi, idesc, accu);
              }
            }
            // slot is free once these MMAs have read it (of a pair: in both CTAs)
            if constexpr (PAIR) umma_commit_pair(empty0 + 8u * s);
            else umma_commit(empty0 + 8u * s);
          }
          __syncwarp();
          acc = 1u;
          if (++s == (uint32_t)kStages) {
            s = 0;
            ph ^= 1u;
          }
        }
        if (ok && elect_one()) {
          if constexpr (PAIR) umma_commit_pair(smem_u32(&sh.tmem_full[buf]));
          else umma_commit(smem_u32(&sh.tmem_full[buf]));
        }
        __syncwarp();
      }
    }
  } else if (Policy::kConv != 0 && warp >= 2 + Policy::kEpiWarps) {
    // ------------------------------ operand converters ------------------------------
    // 128 threads rewrite the stage's raw e4m3 rows as bf16 in the K-major 128-byte-swizzled operand
    // layout (row r at r * 128, 16-byte piece c at c ^ (r & 7)).  Thread t takes (row, quarter) pairs
    // t, t + 128, ...: reads are consecutive 16-byte pieces, the two pieces written per pair of adjacent
    // rows cover all eight positions, so neither side has bank conflicts.  The raw bytes land only after
    // the producer has seen the stage released, so nothing else has to be waited for.
    if constexpr (Policy::kConv != 0) {
      const int ct = threadIdx.x - 32 * (2 + Policy::kEpiWarps);
      uint32_t s = 0, ph = 0;
      bool ok = true;
      for (int tile = worker; ok && tile < n_tiles; tile += n_workers) {
        Job job;
        Policy::job(p, tile, job);
        for (int k = 0; k < job.k_steps; ++k) {
          if (!mbar_wait(smem_u32(&sh.raw_full[s]), ph, &sh.ctl, p.status, 700 + (int)s)) {
            ok = false;
            break;
          }
          const uint8_t* raw = smem_raw_ring + s * kRawBytes;
          uint8_t* dst = smem + s * kStageBytes + (Policy::kConv == 2 ? kStageABytes : 0);
#pragma unroll
          for (int it = 0; it < conv_rows<Policy>() * 4 / (32 * kConvWarps); ++it) {
            const int pr = ct + it * 32 * kConvWarps;
            const int row = pr >> 2, kc = pr & 3;
            const uint4 v = *reinterpret_cast<const uint4*>(raw + row * 64 + kc * 16);
            uint4 o0, o1;
            e4m3x4_to_bf16x4(v.x, o0.x, o0.y);
            e4m3x4_to_bf16x4(v.y, o0.z, o0.w);
            e4m3x4_to_bf16x4(v.z, o1.x, o1.y);
            e4m3x4_to_bf16x4(v.w, o1.z, o1.w);
            uint8_t* rowp = dst + row * 128;
            *reinterpret_cast<uint4*>(rowp + (((2 * kc) ^ (row & 7)) << 4)) = o0;
            *reinterpret_cast<uint4*>(rowp + (((2 * kc + 1) ^ (row & 7)) << 4)) = o1;
          }
          fence_proxy_async();                            // generic-proxy writes -> tensor-core reads
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&sh.conv_full[s]));
          if (++s == (uint32_t)kStages) {
            s = 0;
            ph ^= 1u;
          }
        }
      }
    }
  } else if (Policy::kCTile && warp == 2 + Policy::kEpiWarps) {
    // ------------------------------ weight-block store ------------------------------
    // Once every epilogue warp has rewritten its part of the tile's block, store it back (whole lines;
    // rows and columns outside the tensor are clipped) and, when the copy has read shared memory, hand
    // the slot back to the producer.  A warp of its own: the epilogue warps go straight on to the next
    // accumulator instead of one of them sitting out the copy.
    if constexpr (Policy::kCTile) {
      static_assert(Policy::kConv == 0, "one extra role per policy");
      uint32_t t_local = 0;
      for (int tile = worker; tile < n_tiles; tile += n_workers, ++t_local) {
        Job job;
        Policy::job(p, tile, job);
        const int c_col = Policy::c_col(job);
        if constexpr (PAIR) job.a0 += kTileM * (int)rank;
        const uint32_t cb = t_local % kCBufs, cph = (t_local / kCBufs) & 1u;
        if (!mbar_wait_warp(smem_u32(&sh.c_done[cb]), cph, &sh.ctl, p.status, 620 + (int)cb)) break;
        if (lane == 0) {
          const uint32_t src = smem_u32(smem_c + cb * kCTileBytes);
          if (Policy::c_store(p, job)) {
            tma_store_2d(&map_c, src, c_col, job.a0);
            tma_store_2d(&map_c, src + kCHalfBytes, c_col + 128, job.a0);
            bulk_commit_group();
            bulk_wait_read_all();
          }
          mbar_arrive(smem_u32(&sh.c_empty[cb]));
        }
        __syncwarp();
      }
      if (lane == 0) bulk_wait_all();                    // the stores have landed before the CTA retires
      __syncwarp();
    }
  } else {
    // ------------------------------ epilogue ------------------------------
    // No block-level barrier is used in here: a warp that unwinds after a time-out must never
    // leave the others stuck in an unbounded bar.sync.  Warps cooperate through __syncwarp only.
    EpiCtx ec;
    ec.q = warp & 3;                                // TMEM lane quarter this warp may access
    ec.lane = lane;
    ec.slot = warp - 2;
    ec.h = ec.slot >> 2;                            // which of the column-group phases this warp takes
    ec.nsplit = Policy::kEpiWarps / 4;
    ec.ctile = nullptr;
    ec.bitmap = Policy::kBitmap ? reinterpret_cast<uint32_t*>(smem_bm) : nullptr;
    const int q = ec.q;
    typename Policy::EpilogueState st;
    Policy::epilogue_begin(p, st);
    uint32_t tmem_empty_leader = smem_u32(&sh.tmem_empty[0]);
    if constexpr (PAIR) tmem_empty_leader = mapa_shared(tmem_empty_leader, 0);
    uint32_t t_local = 0;
    for (int tile = worker; tile < n_tiles; tile += n_workers, ++t_local) {
      Job job;
      Policy::job(p, tile, job);
      if constexpr (PAIR) job.a0 += kTileM * (int)rank;          // this CTA's 128 rows of the pair's tile
      const uint32_t buf = t_local & 1u, aph = (t_local >> 1) & 1u;
      Policy::epilogue_pre(p, job, sh, ec, st);          // overlaps the tile's main loop
      if (tile + n_workers < n_tiles) {                  // start the next tile's small global reads a tile ahead
        Job next;
        Policy::job(p, tile + n_workers, next);
        if constexpr (PAIR) next.a0 += kTileM * (int)rank;
        Policy::epilogue_prefetch(p, next, st);
      }
      if (!mbar_wait(smem_u32(&sh.tmem_full[buf]), aph, &sh.ctl, p.status, 400 + (int)buf)) break;
      const uint32_t cb = t_local % kCBufs, cph = (t_local / kCBufs) & 1u;
      if constexpr (Policy::kCTile) {
        if (!mbar_wait(smem_u32(&sh.c_full[cb]), cph, &sh.ctl, p.status, 610 + (int)cb)) break;
        ec.ctile = smem_c + cb * kCTileBytes;
      }
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * kTileN;
      Policy::epilogue(p, job, taddr, job.k_steps > 0, sh, ec, st);
      // Hand the accumulator back: the warp's TMEM loads are complete (wait::ld is warp-wide), one lane
      // arrives for the warp -- hundreds of arrivals per tile on one barrier word, half of them from the
      // other SM, would queue up in front of the MMA issuer.
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if constexpr (PAIR) mbar_arrive_remote(tmem_empty_leader + 8u * buf);
        else mbar_arrive(tmem_empty_leader + 8u * buf);
      }
      if constexpr (Policy::kCTile) {
        // this warp's part of the block is rewritten: tell the store warp
        fence_proxy_async();                             // generic-proxy writes -> async-proxy (TMA) reads
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&sh.c_done[cb]));
        __syncwarp();                                    // the warp-wide TMEM loads of the next tile need all lanes
      }
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
  if constexpr (PAIR) cluster_sync_all();   // the peer may still be reading this CTA's shared memory or arriving on its barriers
  else __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    if constexpr (PAIR) tmem_dealloc_pair(tmem_base, kTmemCols);
    else tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace xmc
