// grad_X partial sums: partial[split][b][c] (+)= sum over a slice of the chunk's label rows of
// G[l][b] * W[l][c]   (reference: matmul_kernel.py:204-239 large_k_matmul, C = G^T W, operands
// rounded to bf16, fp32 accumulation).
//
// One CTA owns a 256 (batch) x 256 (feature) output tile for one slice of label rows: two 128-lane
// TMEM accumulators of 256 columns.  Both operands are "MN-major" for the tensor core (the
// contraction index, the label row, is the slow index of G[l][b] and W[l][c]), so G tiles land by
// TMA exactly as stored.  e4m3 weights are brought in raw (half the L2 traffic of a bf16 copy and
// no staging pass over HBM) and turned into the bf16 128-byte-swizzled operand layout by the eight
// epilogue warps while the previous stage is being multiplied; after the last stage the same warps
// drain the accumulators.  Each (split, tile) owns its slot of `partial` and adds to it in chunk
// order: fixed summation order, no atomics.
//
// PAIR = true: a CTA pair (cluster of two, cta_group::2) owns a 512 (batch) x 256 (feature) tile: two
// M = 256 accumulators of 256 columns, CTA r holding batch rows [256 h + 128 r, +128) of accumulator h in
// its own TMEM.  Each CTA fetches its own 2 x 128 batch columns of G and only ITS 128 feature columns of
// W (raw, converted by its own warps), so a weight element is converted once per 512 batch rows and a
// k-step costs 64 KB of shared-memory traffic per SM for 512 tensor-core cycles instead of 96 KB; the
// smaller stages buy a deeper ring.  Barriers: a_full / b_full live in the leader (bytes and converter
// warps of both CTAs), mma_done and tmem_full exist in both CTAs and are signalled together by the
// leader's commits.  Needs d % 256 == 0 (every CTA's half of a feature tile is two whole 64-column blocks).
#pragma once
#include "gemm_engine.cuh"
#include "numerics.cuh"

namespace xmc {

constexpr int kGxRows = 32;                           // label rows per pipeline stage
constexpr int kGxBlockBytes = kGxRows * 128;          // one 64-element block of a stage: 4 KB
constexpr int kGxABytes = 4 * kGxBlockBytes;          // 4 blocks of 64 batch columns: 16 KB
constexpr int kGxWarps = 8;
constexpr int kGxThreads = 64 + 32 * kGxWarps;
// per CTA: bf16 feature blocks per stage (a CTA of a pair holds half of the tile's 256 features), ring depths
template <bool PAIR> constexpr int kGxBBlocks = PAIR ? 2 : 4;
template <bool PAIR> constexpr int kGxBBytes = kGxBBlocks<PAIR> * kGxBlockBytes;       // 8 / 16 KB
template <bool PAIR> constexpr int kGxRawBytes = kGxBBlocks<PAIR> * kGxRows * 64;      // raw e4m3 tile: 4 / 8 KB
template <bool PAIR> constexpr int kGxStages = PAIR ? 7 : 5;
template <bool PAIR> constexpr int kGxRawStages = PAIR ? 8 : 6;
constexpr int kGxMaxStages = 8;

struct GxParams {
  int bpad, d;
  int n_btiles, n_dtiles, n_splits;   // batch tiles of 256, feature tiles of 256
  int total_ksteps;                   // cdiv(label rows written by the forward kernel, 32)
  int accumulate;                     // 0: overwrite the slot (first chunk of a step)
  float* partial;                     // [n_splits][bpad][d]
  int* status;
};

struct GxShared {
  uint64_t a_full[kGxMaxStages];
  uint64_t b_full[kGxMaxStages];        // converted (or TMA-loaded) weight block ready
  uint64_t mma_done[kGxMaxStages];      // the MMAs reading stage s have completed
  uint64_t raw_full[kGxMaxStages];
  uint64_t raw_empty[kGxMaxStages];
  uint64_t tmem_full;
  uint32_t tmem_base;
  Ctl ctl;
};

template <bool PAIR>
constexpr int kGxSmemBytes = kGxStages<PAIR> * (kGxABytes + kGxBBytes<PAIR>) + kGxRawStages<PAIR> * kGxRawBytes<PAIR> +
                             (int)sizeof(GxShared) + 1024;
static_assert(kGxSmemBytes<false> <= 232448 && kGxSmemBytes<true> <= 232448, "exceeds the shared memory a CTA can get");

template <bool CONVERT, bool PAIR = false>
__global__ void __launch_bounds__(kGxThreads, 1)
gradx_kernel(const __grid_constant__ CUtensorMap map_g, const __grid_constant__ CUtensorMap map_w,
             const GxParams p) {
  constexpr int kStages = kGxStages<PAIR>, kRawStages = kGxRawStages<PAIR>;
  constexpr int kBBytes = kGxBBytes<PAIR>, kRawBytes = kGxRawBytes<PAIR>, kBBlocks = kGxBBlocks<PAIR>;
  static_assert(!PAIR || CONVERT, "the pair kernel is written for e4m3 weights");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* smem_a = smem;                                         // [stage][4 blocks][32 rows][128 B]
  uint8_t* smem_b = smem + kStages * kGxABytes;                   // [stage][2 or 4 blocks][32 rows][128 B], bf16 weights
  uint8_t* smem_r = smem_b + kStages * kBBytes;                   // [raw stage][blocks][32 rows][64 B] e4m3
  GxShared& sh = *reinterpret_cast<GxShared*>(smem_r + kRawStages * kRawBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  static_assert(kGxWarps == 8 && kGxRows == 32, "converter mapping assumes 8 warps x 32 rows");
  uint32_t rank = 0u;
  if constexpr (PAIR) rank = cluster_ctarank();

  // tile coordinates: n_btiles counts batch tiles of 256 (single CTA) or 512 (pair)
  const int worker = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int per = p.n_btiles * p.n_dtiles;
  const int split = worker / per;
  const int rem = worker - split * per;
  const int bt = rem / p.n_dtiles, dt = rem - bt * p.n_dtiles;
  const int b0 = bt * (PAIR ? 512 : 256), c0 = dt * 256;
  const int k_begin = (int)(((long long)split * p.total_ksteps) / p.n_splits);
  const int k_steps = (int)(((long long)(split + 1) * p.total_ksteps) / p.n_splits) - k_begin;
  const int n_eff = PAIR ? 256 : min(256, (p.d - c0 + 15) & ~15);
  // accumulators in use, and this CTA's 128 batch rows of accumulator h: [b_cta + h * b_half, +128)
  const int m_halves = PAIR ? ((b0 + 256 < p.bpad) ? 2 : 1) : ((b0 + 128 < p.bpad) ? 2 : 1);
  const int b_half = PAIR ? 256 : 128;
  const int b_cta = b0 + (PAIR ? 128 * (int)rank : 0);
  const int c_cta = c0 + (PAIR ? 128 * (int)rank : 0);           // first feature column this CTA stages

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&sh.a_full[s]), 1);
      mbar_init(smem_u32(&sh.b_full[s]), CONVERT ? (PAIR ? 2 : 1) * kGxWarps : 1);
      mbar_init(smem_u32(&sh.mma_done[s]), 1);
    }
    for (int s = 0; s < kRawStages; ++s) {
      mbar_init(smem_u32(&sh.raw_full[s]), 1);
      mbar_init(smem_u32(&sh.raw_empty[s]), kGxWarps);
    }
    mbar_init(smem_u32(&sh.tmem_full), 1);
    sh.ctl.abort = 0;
    sh.ctl.limit = kWaitLimitCycles;
    fence_barrier_init();
    tma_prefetch_desc(&map_g);
    tma_prefetch_desc(&map_w);
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
  // The raw weight tiles depend on nothing before this kernel (the weights were last written a step ago):
  // the producer sends for its first ring of them, then everybody waits for the kernel that writes G.
  if constexpr (CONVERT) {
    if (warp == 0) {
      const int krow0 = k_begin * kGxRows;
      for (int r = 0; r < kRawStages && r < k_steps; ++r) {
        if (elect_one()) {
          const uint32_t rb = smem_u32(&sh.raw_full[r]);
          mbar_arrive_expect_tx(rb, kRawBytes);
          tma_load_3d(smem_u32(smem_r + r * kRawBytes), &map_w, rb, 0, krow0 + r * kGxRows, c_cta >> 6);
        }
        __syncwarp();
      }
    }
  }
  pdl_wait();
  tc_fence_after();
  const uint32_t tmem_base = sh.tmem_base;
  // barriers the two CTAs of a pair share live in the leader
  uint32_t a_full0 = smem_u32(&sh.a_full[0]), b_full0 = smem_u32(&sh.b_full[0]);
  if constexpr (PAIR) {
    a_full0 = mapa_shared(a_full0, 0);
    b_full0 = mapa_shared(b_full0, 0);
  }

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    // The whole warp runs the loop on warp-uniform values (uniform registers: the TMA instructions take
    // their operands there) and one elected lane issues; ring indices are running counters.
    {
      uint32_t s = 0, ph = 0, rs = 0, rph = 0;
      int krow = k_begin * kGxRows;
      // the first ring of raw weight tiles is already on its way (see above)
      int raw_ahead = 0;
      if constexpr (CONVERT) {
        raw_ahead = min(kRawStages, k_steps);
        rph = raw_ahead == kRawStages ? 1u : 0u;
        rs = raw_ahead == kRawStages ? 0u : (uint32_t)raw_ahead;
      }
      for (int i = 0; i < k_steps; ++i, krow += kGxRows) {
        if constexpr (CONVERT) {
          if (i + raw_ahead < k_steps) {                          // the raw tile raw_ahead k-steps on
            if (!mbar_wait_warp(smem_u32(&sh.raw_empty[rs]), rph ^ 1u, &sh.ctl, p.status, 500 + (int)rs)) break;
            if (elect_one()) {
              const uint32_t rb = smem_u32(&sh.raw_full[rs]);
              mbar_arrive_expect_tx(rb, kRawBytes);
              // one box: [feature blocks][32 rows][64 B]
              tma_load_3d(smem_u32(smem_r + rs * kRawBytes), &map_w, rb, 0, krow + raw_ahead * kGxRows, c_cta >> 6);
            }
            __syncwarp();
            if (++rs == (uint32_t)kRawStages) { rs = 0; rph ^= 1u; }
          }
        }
        if (!mbar_wait_warp(smem_u32(&sh.mma_done[s]), ph ^ 1u, &sh.ctl, p.status, 510 + (int)s)) break;
        if (elect_one()) {
          const uint32_t sa = smem_u32(smem_a + s * kGxABytes);
          if constexpr (PAIR) {
            // this CTA's 128 batch columns of either accumulator: two boxes [2 blocks][32 rows][128 B];
            // the bytes of both CTAs are counted on the leader's barrier
            if (rank == 0) mbar_arrive_expect_tx(smem_u32(&sh.a_full[s]), 2 * kGxABytes);
            const uint32_t ab = a_full0 + 8u * s;
            tma_load_3d_pair(sa, &map_g, ab, 0, krow, b_cta >> 6);
            tma_load_3d_pair(sa + 2 * kGxBlockBytes, &map_g, ab, 0, krow, (b_cta + 256) >> 6);
          } else {
            const uint32_t ab = smem_u32(&sh.a_full[s]);
            mbar_arrive_expect_tx(ab, kGxABytes);
            // one box: [4 batch blocks][32 rows][128 B], blocks beyond the batch are zero-filled
            tma_load_3d(sa, &map_g, ab, 0, krow, b0 >> 6);
            if constexpr (!CONVERT) {
              const uint32_t bb = smem_u32(&sh.b_full[s]);
              mbar_arrive_expect_tx(bb, kBBytes);
              tma_load_3d(smem_u32(smem_b + s * kBBytes), &map_w, bb, 0, krow, c0 >> 6);
            }
          }
        }
        __syncwarp();
        if (++s == (uint32_t)kStages) { s = 0; ph ^= 1u; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (of a pair: the leader's) ------------------------------
    if (!PAIR || rank == 0) {
      const uint32_t idesc = make_idesc(PAIR ? 256 : 128, (uint32_t)n_eff, 1u, 1u, 1u, 1u);
      // MN-major, 128B swizzle: 64-element blocks kGxBlockBytes apart (leading offset), 8-row
      // groups 1024 B apart (stride offset); one UMMA consumes 16 label rows = 2048 B per block
      constexpr uint32_t desc_hi = smem_desc_hi_sw128(1024);
      const uint32_t a_lo0 = smem_desc_lo(smem_u32(smem_a), kGxBlockBytes);
      const uint32_t b_lo0 = smem_desc_lo(smem_u32(smem_b), kGxBlockBytes);
      bool ok = true;
      uint32_t s = 0, ph = 0, acc = 0u;
      for (int i = 0; i < k_steps; ++i) {
        if (!mbar_wait_warp(smem_u32(&sh.a_full[s]), ph, &sh.ctl, p.status, 520 + (int)s) ||
            !mbar_wait_warp(smem_u32(&sh.b_full[s]), ph, &sh.ctl, p.status, 530 + (int)s)) {
          ok = false;
          break;
        }
        tc_fence_after();
        if (elect_one()) {
          const uint32_t a_lo = a_lo0 + s * (uint32_t)(kGxABytes >> 4), b_lo = b_lo0 + s * (uint32_t)(kBBytes >> 4);
          for (int hm = 0; hm < m_halves; ++hm) {
#pragma unroll
            for (uint32_t u = 0; u < kGxRows / 16; ++u) {
              // accumulator hm reads this CTA's (of a pair: either CTA's) blocks 2 hm, 2 hm + 1 of the G stage
              const uint32_t au = a_lo + (uint32_t)hm * (2u * kGxBlockBytes >> 4) + 128u * u, bu = b_lo + 128u * u;
              if constexpr (PAIR) umma_f16_lohi_pair(tmem_base + hm * 256, au, bu, desc_hi, idesc, u == 0 ? acc : 1u);
              else umma_f16_lohi(tmem_base + hm * 256, au, bu, desc_hi, idesc, u == 0 ? acc : 1u);
            }
          }
          if constexpr (PAIR) umma_commit_pair(smem_u32(&sh.mma_done[s]));
          else umma_commit(smem_u32(&sh.mma_done[s]));
        }
        __syncwarp();
        acc = 1u;
        if (++s == (uint32_t)kStages) { s = 0; ph ^= 1u; }
      }
      if (ok && elect_one()) {
        if constexpr (PAIR) umma_commit_pair(smem_u32(&sh.tmem_full));
        else umma_commit(smem_u32(&sh.tmem_full));
      }
      __syncwarp();
    }
  } else {
    // -------------------- converters, then epilogue (warps 2..9) --------------------
    const int cw = warp - 2;                                      // 0..7
    bool ok = true;
    if constexpr (CONVERT) {
      uint32_t s = 0, ph = 0, rs = 0, rph = 0;
      for (int i = 0; i < k_steps && ok; ++i) {
        if (!mbar_wait(smem_u32(&sh.raw_full[rs]), rph, &sh.ctl, p.status, 540 + (int)rs) ||
            !mbar_wait(smem_u32(&sh.mma_done[s]), ph ^ 1u, &sh.ctl, p.status, 550 + (int)s)) {
          ok = false;
          break;
        }
        // A warp takes one 64-feature block and a band of rows; per pass 8 rows x 64 B of the block: the
        // reads are one contiguous 512 B run, the swizzled writes hit every bank equally often.
        // Single CTA: 4 blocks x 2 bands of 16 rows (2 passes); pair: 2 blocks x 4 bands of 8 rows (1 pass).
        constexpr int kBands = kGxWarps / kBBlocks, kPasses = kGxRows / (8 * kBands);
        const int blk = cw % kBBlocks, band = cw / kBBlocks;
        const uint8_t* raw = smem_r + rs * kRawBytes + blk * (kGxRows * 64);
        uint8_t* dst = smem_b + s * kBBytes + blk * kGxBlockBytes;
#pragma unroll
        for (int it = 0; it < kPasses; ++it) {
          const int row = 8 * (kPasses * band + it) + (lane >> 2), kc = lane & 3;
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
        fence_proxy_async();                                      // generic-proxy writes -> tensor-core reads
        __syncwarp();                                             // one arrival per warp: 256 arrivals on one
        if (lane == 0) {                                          // barrier word would serialise the stage
          if constexpr (PAIR) mbar_arrive_remote(b_full0 + 8u * s);    // the leader's barrier counts the warps of both CTAs
          else mbar_arrive(b_full0 + 8u * s);
          mbar_arrive(smem_u32(&sh.raw_empty[rs]));
        }
        if (++s == (uint32_t)kStages) { s = 0; ph ^= 1u; }
        if (++rs == (uint32_t)kRawStages) { rs = 0; rph ^= 1u; }
      }
    }
    if (ok && mbar_wait(smem_u32(&sh.tmem_full), 0u, &sh.ctl, p.status, 560)) {
      tc_fence_after();
      const int q = warp & 3;
      const int hm = cw >> 2;                                     // warps 2..5 -> accumulator 0, 6..9 -> 1
      const bool have_acc = k_steps > 0;
      if (have_acc || !p.accumulate) {
        // Drain through a per-warp 32 x 32 staging tile in the (now idle) operand stages so that the
        // global accesses run along rows: 8 lanes cover 128 contiguous bytes of one batch row instead
        // of 32 lanes touching 32 different rows with 16 bytes each.
        const int brow0 = b_cta + hm * b_half + q * 32;           // first batch row of this warp
        float* dst0 = p.partial + ((size_t)split * p.bpad + brow0) * p.d + c0;
        float4* stage = reinterpret_cast<float4*>(smem_a + cw * 4096);   // [32 rows][8 chunks of 16 B], XOR-swizzled
        const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + hm * 256;
        const int rr = lane >> 3, ch = lane & 7;                  // read side: row within a group of 4, 16-byte chunk
        for (int cg = 0; cg < n_eff; cg += 32) {
          uint32_t v[32];
          if (have_acc && hm < m_halves) {
            tmem_ld32(taddr + cg, v);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = 0u;
          }
          __syncwarp();                                           // the previous group's reads are done
#pragma unroll
          for (int i = 0; i < 8; ++i)
            stage[lane * 8 + (i ^ (lane & 7))] = make_float4(__uint_as_float(v[4 * i]), __uint_as_float(v[4 * i + 1]),
                                                             __uint_as_float(v[4 * i + 2]), __uint_as_float(v[4 * i + 3]));
          __syncwarp();
          const bool col_ok = c0 + cg + 4 * ch < p.d;             // d is a multiple of 4
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int r = 4 * j + rr;
            const float4 o = stage[r * 8 + (ch ^ (r & 7))];
            if (!col_ok || brow0 + r >= p.bpad || hm >= m_halves) continue;
            float4* ptr = reinterpret_cast<float4*>(dst0 + (size_t)r * p.d + cg + 4 * ch);
            if (p.accumulate) {
              // Fire-and-forget vector reduction at L2: no read latency in the kernel's tail.  Each
              // element has exactly one writer per launch and launches are stream-ordered, so the
              // order of additions is still fixed.
              asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(ptr), "f"(o.x), "f"(o.y),
                           "f"(o.z), "f"(o.w)
                           : "memory");
            } else {
              *ptr = o;
            }
          }
        }
      }
    }
  }

  __syncwarp();
  if (sh.ctl.abort) {
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
