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
#pragma once
#include "gemm_engine.cuh"
#include "numerics.cuh"

namespace xmc {

constexpr int kGxRows = 32;                           // label rows per pipeline stage
constexpr int kGxStages = 5;
constexpr int kGxRawStages = 6;
constexpr int kGxABytes = 4 * kGxRows * 128;          // 4 blocks of 64 batch columns: 16 KB
constexpr int kGxBBytes = 4 * kGxRows * 128;          // 4 blocks of 64 features, bf16: 16 KB
constexpr int kGxRawBytes = kGxRows * 256;            // raw e4m3 tile: 8 KB
constexpr int kGxBlockBytes = kGxRows * 128;          // one 64-element block of a stage: 4 KB
constexpr int kGxWarps = 8;
constexpr int kGxThreads = 64 + 32 * kGxWarps;

struct GxParams {
  int bpad, d;
  int n_btiles, n_dtiles, n_splits;   // batch tiles of 256, feature tiles of 256
  int total_ksteps;                   // cdiv(label rows written by the forward kernel, 32)
  int accumulate;                     // 0: overwrite the slot (first chunk of a step)
  float* partial;                     // [n_splits][bpad][d]
  int* status;
};

struct GxShared {
  uint64_t a_full[kGxStages];
  uint64_t b_full[kGxStages];         // converted (or TMA-loaded) weight block ready
  uint64_t mma_done[kGxStages];       // the MMAs reading stage s have completed
  uint64_t raw_full[kGxRawStages];
  uint64_t raw_empty[kGxRawStages];
  uint64_t tmem_full;
  uint32_t tmem_base;
  Ctl ctl;
};

constexpr int kGxSmemBytes = kGxStages * (kGxABytes + kGxBBytes) + kGxRawStages * kGxRawBytes +
                             (int)sizeof(GxShared) + 1024;

template <bool CONVERT>
__global__ void __launch_bounds__(kGxThreads, 1)
gradx_kernel(const __grid_constant__ CUtensorMap map_g, const __grid_constant__ CUtensorMap map_w,
             const GxParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* smem_a = smem;                                         // [stage][4 blocks][32 rows][128 B]
  uint8_t* smem_b = smem + kGxStages * kGxABytes;                 // same shape, bf16 weights
  uint8_t* smem_r = smem_b + kGxStages * kGxBBytes;               // [raw stage][32 rows][256 B] e4m3
  GxShared& sh = *reinterpret_cast<GxShared*>(smem_r + kGxRawStages * kGxRawBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  static_assert(kGxWarps == 8 && kGxRows == 32, "converter mapping assumes 8 warps x 32 rows");

  // tile coordinates
  const int per = p.n_btiles * p.n_dtiles;
  const int split = blockIdx.x / per;
  const int rem = blockIdx.x - split * per;
  const int bt = rem / p.n_dtiles, dt = rem - bt * p.n_dtiles;
  const int b0 = bt * 256, c0 = dt * 256;
  const int k_begin = (int)(((long long)split * p.total_ksteps) / p.n_splits);
  const int k_steps = (int)(((long long)(split + 1) * p.total_ksteps) / p.n_splits) - k_begin;
  const int n_eff = min(256, (p.d - c0 + 15) & ~15);
  const int m_halves = (b0 + 128 < p.bpad) ? 2 : 1;               // accumulators in use

  if (threadIdx.x == 0) {
    for (int s = 0; s < kGxStages; ++s) {
      mbar_init(smem_u32(&sh.a_full[s]), 1);
      mbar_init(smem_u32(&sh.b_full[s]), CONVERT ? kGxWarps : 1);
      mbar_init(smem_u32(&sh.mma_done[s]), 1);
    }
    for (int s = 0; s < kGxRawStages; ++s) {
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
    // The whole warp runs the loop on warp-uniform values (uniform registers: the TMA instructions take
    // their operands there) and one elected lane issues; ring indices are running counters.
    {
      uint32_t s = 0, ph = 0, rs = 0, rph = 0;
      int krow = k_begin * kGxRows;
      for (int i = 0; i < k_steps; ++i, krow += kGxRows) {
        if constexpr (CONVERT) {
          if (!mbar_wait_warp(smem_u32(&sh.raw_empty[rs]), rph ^ 1u, &sh.ctl, p.status, 500 + (int)rs)) break;
          if (elect_one()) {
            const uint32_t rb = smem_u32(&sh.raw_full[rs]);
            mbar_arrive_expect_tx(rb, kGxRawBytes);
            // one box: [4 feature blocks][32 rows][64 B]
            tma_load_3d(smem_u32(smem_r + rs * kGxRawBytes), &map_w, rb, 0, krow, c0 >> 6);
          }
          __syncwarp();
          if (++rs == (uint32_t)kGxRawStages) { rs = 0; rph ^= 1u; }
        }
        if (!mbar_wait_warp(smem_u32(&sh.mma_done[s]), ph ^ 1u, &sh.ctl, p.status, 510 + (int)s)) break;
        if (elect_one()) {
          const uint32_t ab = smem_u32(&sh.a_full[s]);
          mbar_arrive_expect_tx(ab, kGxABytes);
          // one box: [4 batch blocks][32 rows][128 B], blocks beyond the batch are zero-filled
          tma_load_3d(smem_u32(smem_a + s * kGxABytes), &map_g, ab, 0, krow, b0 >> 6);
          if constexpr (!CONVERT) {
            const uint32_t bb = smem_u32(&sh.b_full[s]);
            mbar_arrive_expect_tx(bb, kGxBBytes);
            tma_load_3d(smem_u32(smem_b + s * kGxBBytes), &map_w, bb, 0, krow, c0 >> 6);
          }
        }
        __syncwarp();
        if (++s == (uint32_t)kGxStages) { s = 0; ph ^= 1u; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    {
      const uint32_t idesc = make_idesc(128, (uint32_t)n_eff, 1u, 1u, 1u, 1u);
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
          const uint32_t a_lo = a_lo0 + s * (uint32_t)(kGxABytes >> 4), b_lo = b_lo0 + s * (uint32_t)(kGxBBytes >> 4);
          for (int hm = 0; hm < m_halves; ++hm) {
#pragma unroll
            for (uint32_t u = 0; u < kGxRows / 16; ++u)
              umma_f16_lohi(tmem_base + hm * 256, a_lo + (uint32_t)hm * (2u * kGxBlockBytes >> 4) + 128u * u, b_lo + 128u * u,
                            desc_hi, idesc, u == 0 ? acc : 1u);
          }
          umma_commit(smem_u32(&sh.mma_done[s]));
        }
        __syncwarp();
        acc = 1u;
        if (++s == (uint32_t)kGxStages) { s = 0; ph ^= 1u; }
      }
      if (ok && elect_one()) umma_commit(smem_u32(&sh.tmem_full));
      __syncwarp();
    }
  } else {
    // -------------------- converters, then epilogue (warps 2..9) --------------------
    const int cw = warp - 2;                                      // 0..7
    bool ok = true;
    if constexpr (CONVERT) {
      for (int i = 0; i < k_steps && ok; ++i) {
        const uint32_t s = i % kGxStages, ph = (i / kGxStages) & 1u;
        const uint32_t rs = i % kGxRawStages, rph = (i / kGxRawStages) & 1u;
        if (!mbar_wait(smem_u32(&sh.raw_full[rs]), rph, &sh.ctl, p.status, 540 + (int)rs) ||
            !mbar_wait(smem_u32(&sh.mma_done[s]), ph ^ 1u, &sh.ctl, p.status, 550 + (int)s)) {
          ok = false;
          break;
        }
        // warp (block = cw & 3, row half = cw >> 2); per pass 8 rows x 64 B of one block: the reads
        // are one contiguous 512 B run, the swizzled writes hit every bank equally often
        const uint8_t* raw = smem_r + rs * kGxRawBytes + (cw & 3) * (kGxRows * 64);
        uint8_t* dst = smem_b + s * kGxBBytes + (cw & 3) * kGxBlockBytes;
#pragma unroll
        for (int it = 0; it < 2; ++it) {
          const int row = 16 * (cw >> 2) + 8 * it + (lane >> 2), kc = lane & 3;
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
          mbar_arrive(smem_u32(&sh.b_full[s]));
          mbar_arrive(smem_u32(&sh.raw_empty[rs]));
        }
      }
    }
    if (ok && mbar_wait_relaxed(smem_u32(&sh.tmem_full), 0u, &sh.ctl, p.status, 560)) {
      tc_fence_after();
      const int q = warp & 3;
      const int hm = cw >> 2;                                     // warps 2..5 -> accumulator 0, 6..9 -> 1
      const bool have_acc = k_steps > 0;
      if (have_acc || !p.accumulate) {
        // Drain through a per-warp 32 x 32 staging tile in the (now idle) operand stages so that the
        // global accesses run along rows: 8 lanes cover 128 contiguous bytes of one batch row instead
        // of 32 lanes touching 32 different rows with 16 bytes each.
        const int brow0 = b0 + hm * 128 + q * 32;                 // first batch row of this warp
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
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace xmc
