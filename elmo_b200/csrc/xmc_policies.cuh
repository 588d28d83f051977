// GEMM policies (tile mapping + epilogue) of the chunked XMC step:
//   FwdPolicy    Z^T[labels x batch] = W X^T  ->  G = sigmoid(Z) - Y  (bf16, label-major), loss terms
//   UpdPolicy    acc[labels x d] = G X        ->  W <- round(W - lr*(acc + wd*W))   (dW never stored)
//   LogitsPolicy out[batch x labels] = bf16(X W^T)  (inference forward)
//   PlainPolicy  D = A B^T (engine self-test)
#pragma once
#include "gemm_engine.cuh"
#include "numerics.cuh"

namespace xmc {

__device__ __forceinline__ int round_up16(int v) { return (v + 15) & ~15; }

// x / d for 0 <= x < 2^32 / d by one multiply: the roles recompute their tile coordinates once per tile,
// and a real division (its reciprocal comes from the special-function pipe the forward epilogue
// saturates) put hundreds of cycles between two tiles.  mul = floor(2^32 / d) + 1, or 0 for d == 1.
struct FastDiv {
  uint32_t mul;
  int d;
};
__host__ __device__ inline FastDiv make_fastdiv(int d) {
  FastDiv f;
  f.d = d;
  f.mul = d <= 1 ? 0u : (uint32_t)(0x100000000ull / (unsigned long long)d) + 1u;
  return f;
}
__device__ __forceinline__ int fast_div(int x, const FastDiv& f) {
  return f.mul == 0u ? x : (int)__umulhi((uint32_t)x, f.mul);
}

struct NoState {};

// -------------------------------------------------------------------------------------------------
// Forward + loss-gradient epilogue.
// Reference arithmetic reproduced here: logits rounded to bf16 (output dtype of torch._scaled_mm /
// torch.matmul, chunked_fp8xmc_clf.py:98-102), sigmoid rounded to bf16 (:107), "-1" applied in bf16 at
// the positives with set semantics (:108).
// -------------------------------------------------------------------------------------------------
struct FwdParams {
  int m_rows;              // label rows per M tile (128)
  int rows_valid;          // label rows of this scheduling chunk
  int n_ltiles, n_btiles;  // label tiles (m_rows) x batch tiles (256)
  FastDiv div_btiles;      // make_fastdiv(n_btiles)
  int batch, bpad;         // valid batch rows, padded row length of G (multiple of 16)
  int k_steps;             // cdiv(d * elem_size, 128)
  float w_scale;
  __nv_bfloat16* G;        // [n_ltiles*128 x bpad]
  uint8_t* G8;             // WRITE_G8 variants: e4m3(G * 256), same shape (operand of the FP8 dW contraction)
  const int* bucket_off;   // positives bucketed by label tile: offsets ...
  const uint32_t* bucket_ent;  // ... entries: batch row | (label-in-tile << 16)
  int tile_base;           // bucket index of this chunk's label tile 0
  double* loss_partial;    // [gridDim.x * 4] or nullptr
  int* status;
};

constexpr float kG8Scale = 256.0f;      // |G| < 1: e4m3(G * 256) stays below 448

// CONV: bf16 arithmetic on e4m3-stored weights ("simulated FP8"): the weight operand (A) is converted in
// shared memory by the engine's converter warps.
template <bool FP8, bool LOSS, bool WRITE_G8 = false, bool CONV = false>
struct FwdPolicy {
  static_assert(!(FP8 && CONV), "the FP8 contraction takes the e4m3 weights as they are");
  using Params = FwdParams;
  static constexpr bool kMnMajor = false;
  static constexpr bool kFp8 = FP8;
  static constexpr uint32_t kFmt = FP8 ? 0u : 1u;            // e4m3 | bf16
  static constexpr int kElemsPerRow = FP8 ? 128 : 64;
  // sixteen epilogue warps (the converter variant keeps eight: its four converter warps already fill the
  // register file)
  static constexpr int kEpiWarps = CONV ? 8 : 16;
  static constexpr int kStages = CONV ? 3 : 4;
  static constexpr int kStagesPair = 6;
  static constexpr bool kCTile = false;
  static constexpr int kCBufs = 1;
  static constexpr int kConv = CONV ? 1 : 0;
  static constexpr bool kBitmap = true;
  // W of this chunk was last written a step ago and the quantised X by a kernel that ordinary (fully
  // serialising) launches separate from this one: the operand loads need not wait for the kernels before.
  // The epilogue overwrites G, which the previous chunk's kernels read: it waits.
  static constexpr int kWaitRoles = kRoleEpilogue | kRoleExtra;
  __device__ static long long wait_limit(const Params&) { return kWaitLimitCycles; }
  __device__ static bool skip_load(const Params&, int, int) { return false; }
  struct EpilogueState {
    float loss;
    int has_pos;
    int next_bkt, next_beg, next_end;   // bucket range of the CTA's next tile, read a tile ahead
  };

  __device__ static int num_tiles(const Params& p) { return p.n_ltiles * p.n_btiles; }
  __device__ static void job(const Params& p, int tile, Job& j) {
    j.t0 = fast_div(tile, p.div_btiles);   // label tile
    j.t1 = tile - j.t0 * p.n_btiles;   // batch tile
    j.a0 = j.t0 * p.m_rows;
    j.b0 = j.t1 * kTileN;
    j.k_begin = 0;
    j.k_steps = p.k_steps;
    j.n_eff = min(kTileN, round_up16(p.bpad - j.b0));
  }
  __device__ static void epilogue_begin(const Params&, EpilogueState& st) {
    st.loss = 0.f;
    st.has_pos = 0;
    st.next_bkt = -1;
    st.next_beg = st.next_end = 0;
  }
  // The bucket offsets are two dependent-free global reads whose latency would otherwise sit between two
  // epilogues (the epilogue warps are the busiest role of this kernel): issue them one tile ahead.
  __device__ static void epilogue_prefetch(const Params& p, const Job& jn, EpilogueState& st) {
    st.next_bkt = -1;
    if (jn.a0 >= p.rows_valid) return;
    st.next_bkt = p.tile_base + (jn.a0 >> 7);
    st.next_beg = p.bucket_off[st.next_bkt];
    st.next_end = p.bucket_off[st.next_bkt + 1];
  }
  // Build this warp's 32 rows of the positives bitmap (duplicates collapse: set semantics).
  // Each warp owns the bitmap words of its rows (quarter q) and of its column groups (phase h).
  __device__ static void epilogue_pre(const Params& p, const Job& j, SharedTail& sh, const EpiCtx& ec,
                                      EpilogueState& st) {
    st.has_pos = 0;
    if (j.a0 >= p.rows_valid) return;               // second CTA of a pair on an odd last tile: nothing to do
    const int bkt = p.tile_base + (j.a0 >> 7);      // buckets are per 128 label rows
    int beg, end;
    if (bkt == st.next_bkt) {
      beg = st.next_beg;
      end = st.next_end;
    } else {
      beg = p.bucket_off[bkt];
      end = p.bucket_off[bkt + 1];
    }
    st.has_pos = end > beg;
    if (!st.has_pos) return;
    constexpr int kWordsPerRow = kTileN / 32;
    __syncwarp();
    for (int w = ec.lane; w < 32 * kWordsPerRow; w += 32) {
      if ((w % kWordsPerRow) % ec.nsplit == ec.h) ec.bitmap[ec.q * 32 * kWordsPerRow + w] = 0u;
    }
    __syncwarp();
    for (int e = beg + ec.lane; e < end; e += 32) {
      const uint32_t ent = p.bucket_ent[e];
      const int lrow = (int)(ent >> 16), bl = (int)(ent & 0xFFFFu) - j.b0;
      if ((lrow >> 5) == ec.q && bl >= 0 && bl < kTileN && ((bl >> 5) % ec.nsplit) == ec.h)
        atomicOr(&ec.bitmap[lrow * kWordsPerRow + (bl >> 5)], 1u << (bl & 31));
    }
    __syncwarp();
  }
  __device__ static void epilogue(const Params& p, const Job& j, uint32_t taddr, bool have_acc,
                                  SharedTail& sh, const EpiCtx& ec, EpilogueState& st) {
    if (j.a0 >= p.rows_valid) return;               // whole CTA tile beyond the chunk (pairs only): G has no such rows
    const int row = ec.q * 32 + ec.lane;
    const int crow = j.a0 + row;
    const bool row_valid = crow < p.rows_valid;
    for (int c0 = 32 * ec.h; c0 < j.n_eff; c0 += 32 * ec.nsplit) {
      uint32_t v[32];
      if (have_acc) {
        tmem_ld32(taddr + c0, v);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = 0u;
      }
      const uint32_t bits = st.has_pos ? ec.bitmap[row * (kTileN / 32) + (c0 >> 5)] : 0u;
      uint32_t out[16];
      // Per pair: one packed cvt rounds the logits to bf16, ex2 + rcp give the sigmoid, one packed cvt
      // rounds and packs it.  The two special-function operations per logit are what bounds this epilogue.
      // (Keeping the next column group's accumulator load in flight in a second register buffer was
      // measured: 17 more registers, forward 5 % slower.)
#pragma unroll
      for (int i = 0; i < 32; i += 2) {
        const uint32_t zz = pack_bf16x2(__uint_as_float(v[i]) * p.w_scale, __uint_as_float(v[i + 1]) * p.w_scale);
        const float z0 = __uint_as_float(zz << 16), z1 = __uint_as_float(zz & 0xFFFF0000u);
        const float s0 = fast_sigmoid(z0), s1 = fast_sigmoid(z1);
        out[i >> 1] = pack_bf16x2(s0, s1);
        if (LOSS) {
          if (row_valid && j.b0 + c0 + i < p.batch) st.loss += bce_softplus(z0);
          if (row_valid && j.b0 + c0 + i + 1 < p.batch) st.loss += bce_softplus(z1);
        }
      }
      // positives: G = bf16(sigmoid) - 1 in bf16 arithmetic.  Rare (a few thousand pairs per step), so
      // only threads that own one take this path; indices stay compile-time to keep out[] in registers.
      if (bits != 0u) {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const uint32_t two = (bits >> (2 * i)) & 3u;
          if (two == 0u) continue;
          const uint32_t word = out[i];
          float lo = __uint_as_float(word << 16), hi = __uint_as_float(word & 0xFFFF0000u);
          if (two & 1u) lo = bf16_round(lo - 1.0f);
          if (two & 2u) hi = bf16_round(hi - 1.0f);
          out[i] = __byte_perm(__float_as_uint(lo), __float_as_uint(hi), 0x7632);
          if (LOSS && row_valid) {
            // loss term -y*z: z recomputed from the accumulator with the same rounding
            if ((two & 1u) && j.b0 + c0 + 2 * i < p.batch) st.loss -= bf16_round(__uint_as_float(v[2 * i]) * p.w_scale);
            if ((two & 2u) && j.b0 + c0 + 2 * i + 1 < p.batch) st.loss -= bf16_round(__uint_as_float(v[2 * i + 1]) * p.w_scale);
          }
        }
      }
      // rows beyond the chunk and batch columns beyond the batch carry G = 0
      if (!row_valid) {
#pragma unroll
        for (int i = 0; i < 16; ++i) out[i] = 0u;
      } else if (j.b0 + c0 + 32 > p.batch) {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const int b = j.b0 + c0 + 2 * i;
          if (b >= p.batch) out[i] = 0u;
          else if (b + 1 >= p.batch) out[i] &= 0x0000FFFFu;
        }
      }
      if constexpr (WRITE_G8) {
        // the same 32 values once more as e4m3(G * 256): one 32-byte sector
        if (j.b0 + c0 < p.bpad) {
          U32x8 g8;
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const uint32_t w0 = out[2 * k], w1 = out[2 * k + 1];
            const uint32_t lo = float2_to_e4m3x2(__uint_as_float(w0 << 16) * kG8Scale, __uint_as_float(w0 & 0xFFFF0000u) * kG8Scale);
            const uint32_t hi = float2_to_e4m3x2(__uint_as_float(w1 << 16) * kG8Scale, __uint_as_float(w1 & 0xFFFF0000u) * kG8Scale);
            g8.v[k] = lo | (hi << 16);
          }
          st_global_256(p.G8 + (size_t)crow * p.bpad + j.b0 + c0, g8);
        }
      }
      // two 256-bit stores: every thread writes whole 32-byte sectors of its row
      __nv_bfloat16* grow = p.G + (size_t)crow * p.bpad + j.b0 + c0;
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        if (j.b0 + c0 + 16 * i < p.bpad) {
          U32x8 o8;
#pragma unroll
          for (int k = 0; k < 8; ++k) o8.v[k] = out[8 * i + k];
          st_global_256(grow + 16 * i, o8);
        }
      }
    }
  }
  __device__ static void epilogue_end(const Params& p, SharedTail&, const EpiCtx& ec, EpilogueState& st) {
    if (!LOSS) return;
    float v = st.loss;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (ec.lane == 0 && p.loss_partial != nullptr) p.loss_partial[blockIdx.x * kMaxEpiWarps + ec.slot] = (double)v;
  }
};

// -------------------------------------------------------------------------------------------------
// Fused dW + SGD update (reference: fuse_kernel.py:63-131 naive_matmul_k / matmul_update; for bf16
// weights chunked.py:119 + stochastic_rounding_kernel.py:65-99).
// -------------------------------------------------------------------------------------------------
struct UpdParams {
  int m_rows;              // label rows per M tile: 128, or 256 on CTA pairs
  int rows_valid;
  int n_ltiles, n_dtiles;
  FastDiv div_dtiles;      // make_fastdiv(n_dtiles)
  int d;
  int k_steps;             // cdiv(bpad, 64)
  void* W;                 // first row of this scheduling chunk, row-major [rows x d]
  float lr_eff;            // lr / w_scale
  float wd;
  unsigned long long seed, step;
  uint32_t rkey[kSrRounds][2];   // Philox round keys (seed + round * Weyl constants), filled on the host: they sit in
                              // the constant bank, so a round costs two multiplies and two 3-input xors
  unsigned long long elem0;   // global flat element index of W[0][0] of this chunk (Philox counter origin)
  int round_dw_bf16;
  // Kahan-compensated head rows (reference: fuse_kernel.py:202-287, chunked_head_kahan_fp8xmc_clf.py:127-131)
  void* kahan;             // compensation rows of this chunk's row 0.., [kahan_rows x d] bf16 or e5m2; or nullptr
  int kahan_rows;          // rows [0, kahan_rows) of this chunk are compensated
  int kahan_e5m2;
  int* status;
};

// OPS8: the dW contraction takes e4m3 operands (G * 256 and X, both as the forward already quantises
// them) instead of bf16 ones; the caller folds the 1/256 into lr_eff.  Off in every reference-parity path.
template <bool W8, bool SR, bool ROUND_DW, bool HAS_WD, bool KAHAN = false, bool OPS8 = false>
struct UpdPolicy {
  using Params = UpdParams;
  static constexpr bool kMnMajor = false;
  static constexpr bool kFp8 = OPS8;
  static constexpr uint32_t kFmt = OPS8 ? 0u : 1u;
  static constexpr int kElemsPerRow = OPS8 ? 128 : 64;
  static constexpr int kEpiWarps = 16;
  // e4m3 weights: the tile's 128 x 256 weight bytes come in by TMA while the main loop runs and go back
  // by TMA (two 32 KB slots, paid for with one operand stage: with a single slot the refill has to wait
  // for the previous tile's store and the pipeline serialises -- measured 30 % slower); bf16 weights
  // (64 KB per tile) are read from and written to global memory by the epilogue threads
  static constexpr bool kCTile = W8;
  static constexpr int kCBufs = 2;
  static constexpr int kConv = 0;
  static constexpr bool kBitmap = false;
  static constexpr int kWaitRoles = kRoleAll;
  __device__ static long long wait_limit(const Params&) { return kWaitLimitCycles; }
  __device__ static bool skip_load(const Params&, int, int) { return false; }
  static constexpr int kStages = W8 ? 3 : 4;
  static constexpr int kStagesPair = W8 ? 5 : 6;
  // the weight block: columns [c_col, c_col + 256) of the CTA's 128 rows; not stored back when the CTA's
  // rows lie wholly beyond the chunk (second CTA of a pair on an odd last tile)
  __device__ static int c_col(const Job& j) { return j.b0; }
  __device__ static bool c_store(const Params& p, const Job& j) { return j.a0 < p.rows_valid; }
  static constexpr int kGroups = ((kTileN / 32) + (kEpiWarps / 4) - 1) / (kEpiWarps / 4);   // 32-column groups per thread and tile
  using EpilogueState = NoState;

  __device__ static int num_tiles(const Params& p) { return p.n_ltiles * p.n_dtiles; }
  __device__ static void job(const Params& p, int tile, Job& j) {
    j.t0 = fast_div(tile, p.div_dtiles);
    j.t1 = tile - j.t0 * p.n_dtiles;
    j.a0 = j.t0 * p.m_rows;   // rows of G
    j.b0 = j.t1 * kTileN;     // rows of X^T = feature index
    j.k_begin = 0;
    j.k_steps = p.k_steps;
    j.n_eff = min(kTileN, round_up16(p.d - j.b0));
  }
  __device__ static void epilogue_begin(const Params&, EpilogueState&) {}
  __device__ static void epilogue_end(const Params&, SharedTail&, const EpiCtx&, EpilogueState&) {}

  __device__ static void epilogue_pre(const Params&, const Job&, SharedTail&, const EpiCtx&, EpilogueState&) {}
  __device__ static void epilogue_prefetch(const Params&, const Job&, EpilogueState&) {}
  __device__ static void load_acc(uint32_t taddr, bool have_acc, uint32_t (&v)[32]) {
    if (have_acc) {
      tmem_ld32(taddr, v);
      tmem_ld_wait();
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = 0u;
    }
  }

  __device__ static float new_weight(const Params& p, float w, uint32_t acc_bits) {
    // no run-time branches in here: they would cut the per-element code into tiny basic blocks
    float a = __uint_as_float(acc_bits);
    if constexpr (ROUND_DW) a = bf16_round(a);
    if constexpr (HAS_WD) a = fmaf(p.wd, w, a);
    return fmaf(-p.lr_eff, a, w);
  }

  // ------------------------------------------------------------------------------------------------
  // e4m3 weights: eight consecutive elements of one row at a time -- one x8 accumulator load, 8 weight
  // bytes of the shared-memory block, ONE Philox call (8 x 16 bits).  The body is small on purpose: it
  // is looped, not unrolled, so that the epilogue's instruction stream stays resident in the instruction
  // cache next to the single-thread producer and MMA loops that run beside it.
  // ------------------------------------------------------------------------------------------------
  __device__ static uint4 random8(const Params& p, unsigned long long elem) {
    constexpr uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u;
    const unsigned long long q = elem >> 3;
    uint4 c = make_uint4((uint32_t)q, (uint32_t)(q >> 32), (uint32_t)p.step, (uint32_t)(p.step >> 32));
#pragma unroll
    for (int rd = 0; rd < kSrRounds; ++rd) {
      const unsigned long long p0 = (unsigned long long)M0 * c.x;
      const unsigned long long p1 = (unsigned long long)M1 * c.z;
      c = make_uint4((uint32_t)(p1 >> 32) ^ c.y ^ p.rkey[rd][0], (uint32_t)p1, (uint32_t)(p0 >> 32) ^ c.w ^ p.rkey[rd][1],
                     (uint32_t)p0);
    }
    return c;
  }

  // Fast path.  `bad` comes back true when stochastic rounding met a non-finite update (the bare
  // add-and-mask would mangle a NaN pattern); the caller then redoes the eight with update8_careful.
  // Detecting that costs one FMA-pipe add per element (a running sum of magnitudes) instead of a
  // compare and a select each.
  __device__ static uint2 update8(const Params& p, const uint32_t (&v)[8], uint2 wraw, uint4 r, bool& bad) {
    const uint32_t rw[2] = {wraw.x, wraw.y};
    const uint32_t rr[4] = {r.x, r.y, r.z, r.w};
    uint32_t ow[2];
    float mag = 0.f;
#pragma unroll
    for (int k = 0; k < 2; ++k) {            // 4 elements per 32-bit word
      float o[4];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const float2 f = e4m3x2_to_float2((uint16_t)(rw[k] >> (16 * i)));
        const int e = 4 * k + 2 * i;
        o[2 * i] = new_weight(p, f.x, v[e]);
        o[2 * i + 1] = new_weight(p, f.y, v[e + 1]);
        if (SR) {
          // both elements of a pair draw from the same Philox word: element j takes half (j & 1) of word j >> 1
          const uint32_t w32 = rr[e >> 1];
          const float x0 = o[2 * i] * kSrDown, x1 = o[2 * i + 1] * kSrDown;
          mag += fabsf(x0);
          mag += fabsf(x1);
          const uint32_t b0 = (__float_as_uint(x0) + ((w32 & 0xFFFFu) << 4)) & 0xFFF00000u;
          const uint32_t b1 = (__float_as_uint(x1) + ((w32 >> 16) << 4)) & 0xFFF00000u;
          o[2 * i] = __uint_as_float(b0) * kSrUp;
          o[2 * i + 1] = __uint_as_float(b1) * kSrUp;
        }
      }
      ow[k] = (uint32_t)float2_to_e4m3x2(o[0], o[1]) | ((uint32_t)float2_to_e4m3x2(o[2], o[3]) << 16);
    }
    bad = SR && !(mag < 1.0e30f);              // an Inf or NaN among the eight (finite updates sum to < 2^12 here)
    return make_uint2(ow[0], ow[1]);
  }

  // The same eight, element by element with the NaN-preserving rounding (rare).
  __device__ __noinline__ static uint2 update8_careful(const Params& p, uint32_t v0, uint32_t v1, uint32_t v2, uint32_t v3,
                                                       uint32_t v4, uint32_t v5, uint32_t v6, uint32_t v7, uint2 wraw, uint4 r) {
    const uint32_t v[8] = {v0, v1, v2, v3, v4, v5, v6, v7};
    const uint32_t rw[2] = {wraw.x, wraw.y};
    const uint32_t rr[4] = {r.x, r.y, r.z, r.w};
    uint32_t ow[2] = {0u, 0u};
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float w = e4m3x2_to_float2((uint16_t)(rw[e >> 2] >> (8 * (e & 3)))).x;
      const uint32_t r16 = (e & 1) ? (rr[e >> 1] >> 16) : (rr[e >> 1] & 0xFFFFu);
      const float o = sr_e4m3(new_weight(p, w, v[e]), r16);
      ow[e >> 2] |= ((uint32_t)float2_to_e4m3x2(o, 0.f) & 0xFFu) << (8 * (e & 3));
    }
    return make_uint2(ow[0], ow[1]);
  }

  // Kahan-compensated rows: w = W + D - lr*acc; W' = round(w); D' = cast(D + W - W' - lr*acc)
  // (fuse_kernel.py:253-273).  Not on the fast path: only the head rows of chunk 0 come here.
  // krow: the row's 8 compensation values (bf16: 16 bytes, e5m2: 8 bytes), updated in place.
  __device__ __noinline__ static uint2 update8_kahan(const Params& p, uint32_t v0, uint32_t v1, uint32_t v2, uint32_t v3,
                                                     uint32_t v4, uint32_t v5, uint32_t v6, uint32_t v7, uint2 wraw, uint4 r,
                                                     void* krow) {
    const uint32_t v[8] = {v0, v1, v2, v3, v4, v5, v6, v7};
    const uint32_t rw[2] = {wraw.x, wraw.y};
    const uint32_t rr[4] = {r.x, r.y, r.z, r.w};
    float dv[8];
    if (p.kahan_e5m2) {
      const uint2 raw = *reinterpret_cast<const uint2*>(krow);
      const uint32_t rk[2] = {raw.x, raw.y};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(rk[i >> 1] >> (16 * (i & 1))), __NV_E5M2);
        const float2 f = __half22float2(*reinterpret_cast<__half2*>(&hr));
        dv[2 * i] = f.x; dv[2 * i + 1] = f.y;
      }
    } else {
      const uint4 raw = *reinterpret_cast<const uint4*>(krow);
      const uint32_t rk[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        dv[2 * i] = bf16_bits_to_float(rk[i] & 0xFFFFu);
        dv[2 * i + 1] = bf16_bits_to_float(rk[i] >> 16);
      }
    }
    uint32_t ow[2] = {0u, 0u};
    float dn[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float wv = e4m3x2_to_float2((uint16_t)(rw[e >> 2] >> (8 * (e & 3)))).x;
      const float a = __uint_as_float(v[e]);
      float o = fmaf(-p.lr_eff, a, __fadd_rn(wv, dv[e]));
      if (SR) o = sr_e4m3(o, (e & 1) ? (rr[e >> 1] >> 16) : (rr[e >> 1] & 0xFFFFu));
      const uint32_t byte = (uint32_t)float2_to_e4m3x2(o, 0.f) & 0xFFu;
      o = e4m3x2_to_float2((uint16_t)byte).x;                       // the value W' holds
      ow[e >> 2] |= byte << (8 * (e & 3));
      dn[e] = __fsub_rn(__fsub_rn(__fadd_rn(dv[e], wv), o), __fmul_rn(p.lr_eff, a));
    }
    if (p.kahan_e5m2) {
      uint32_t ok[2];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint32_t pr = (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(dn[2 * i], dn[2 * i + 1]), __NV_NOSAT, __NV_E5M2);
        if (i & 1) ok[i >> 1] |= pr << 16; else ok[i >> 1] = pr;
      }
      *reinterpret_cast<uint2*>(krow) = make_uint2(ok[0], ok[1]);
    } else {
      *reinterpret_cast<uint4*>(krow) = make_uint4(pack_bf16x2(dn[0], dn[1]), pack_bf16x2(dn[2], dn[3]),
                                                   pack_bf16x2(dn[4], dn[5]), pack_bf16x2(dn[6], dn[7]));
    }
    return make_uint2(ow[0], ow[1]);
  }

  // the whole tile for e4m3 weights: 2 * kGroups sub-blocks of 16 columns per thread.  The two halves of
  // a sub-block (8 columns, one Philox call each) are independent chains in one basic block: a warp has
  // two of the long multiply-xor chains to interleave, which is what lets four warps per scheduler fill
  // its issue slots.
  __device__ static void epilogue_w8(const Params& p, const Job& j, uint32_t taddr, bool have_acc, const EpiCtx& ec) {
    const int row = ec.q * 32 + ec.lane;
    const int crow = j.a0 + row;
    const bool row_valid = crow < p.rows_valid;
    const unsigned long long erow = p.elem0 + (unsigned long long)crow * p.d + j.b0;
#pragma unroll 1
    for (int sb = 0; sb < 2 * kGroups; ++sb) {
      const int c0 = 32 * (ec.h + ec.nsplit * (sb >> 1)) + 16 * (sb & 1);
      if (c0 >= j.n_eff) break;                          // warp-uniform
      // tcgen05.ld / wait::ld are warp-wide (.sync.aligned): issued by all 32 lanes, outside every
      // lane-dependent branch; the loads are asynchronous, so the random bits are drawn while they fly
      uint32_t va[8], vb[8];
      if (have_acc) {
        tmem_ld8(taddr + c0, va);
        tmem_ld8(taddr + c0 + 8, vb);
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) va[i] = vb[i] = 0u;
      }
      // 16 weight bytes: one 16-byte piece of the swizzled block
      uint4* wslot = reinterpret_cast<uint4*>(ctile_ptr8(ec.ctile, row, c0));
      const uint4 wraw = *wslot;                         // rows / columns outside the tensor were zero-filled
      uint4 ra = make_uint4(0u, 0u, 0u, 0u), rb = ra;
      if (SR) {
        ra = random8(p, erow + c0);
        rb = random8(p, erow + c0 + 8);
      }
      if (have_acc) tmem_ld_wait_for(va, vb);
      const uint2 wa = make_uint2(wraw.x, wraw.y), wb = make_uint2(wraw.z, wraw.w);
      uint2 oa, ob;
      bool kahan_row = false;
      if constexpr (KAHAN) kahan_row = crow < p.kahan_rows;
      if (kahan_row) {
        oa = wa;
        ob = wb;
        if (row_valid) {
          uint8_t* krow = reinterpret_cast<uint8_t*>(p.kahan) + ((size_t)crow * p.d + j.b0 + c0) * (p.kahan_e5m2 ? 1 : 2);
          if (j.b0 + c0 < p.d) oa = update8_kahan(p, va[0], va[1], va[2], va[3], va[4], va[5], va[6], va[7], wa, ra, krow);
          if (j.b0 + c0 + 8 < p.d)
            ob = update8_kahan(p, vb[0], vb[1], vb[2], vb[3], vb[4], vb[5], vb[6], vb[7], wb, rb, krow + (p.kahan_e5m2 ? 8 : 16));
        }
      } else {
        bool bad_a = false, bad_b = false;
        oa = update8(p, va, wa, ra, bad_a);
        ob = update8(p, vb, wb, rb, bad_b);
        if (bad_a) oa = update8_careful(p, va[0], va[1], va[2], va[3], va[4], va[5], va[6], va[7], wa, ra);
        if (bad_b) ob = update8_careful(p, vb[0], vb[1], vb[2], vb[3], vb[4], vb[5], vb[6], vb[7], wb, rb);
      }
      if (row_valid) *wslot = make_uint4(oa.x, oa.y, ob.x, ob.y);   // in place; the engine stores the block back with TMA
    }
  }

  // 16 random bits for each of 32 consecutive elements starting at `elem` (bf16 weights): four Philox
  // calls, element e of the 32 takes half (e & 1) of word e >> 1
  __device__ static void random32(const Params& p, unsigned long long elem, uint32_t (&r)[16]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint4 c = random8(p, elem + 8 * i);
      r[4 * i] = c.x; r[4 * i + 1] = c.y; r[4 * i + 2] = c.z; r[4 * i + 3] = c.w;
    }
  }
  __device__ static uint32_t r16_of(const uint32_t (&r)[16], int e) {
    return (e & 1) ? (r[e >> 1] >> 16) : (r[e >> 1] & 0xFFFFu);
  }

  __device__ static void process_bf16(const Params& p, const uint32_t (&v)[32], unsigned long long elem,
                                      __nv_bfloat16* wp, int valid16) {
    uint32_t r[16];
    if (SR) random32(p, elem, r);
#pragma unroll
    for (int g16 = 0; g16 < 2; ++g16) {          // 16 bf16 = one 32-byte sector per access
      if (g16 >= valid16) break;
      const U32x8 raw = ld_global_256(wp + 16 * g16);
      U32x8 ow;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int e = 16 * g16 + 2 * i;
        const float o0 = new_weight(p, bf16_bits_to_float(raw.v[i] & 0xFFFFu), v[e]);
        const float o1 = new_weight(p, bf16_bits_to_float(raw.v[i] >> 16), v[e + 1]);
        if (SR) ow.v[i] = sr_bf16_bits(o0, r16_of(r, e)) | (sr_bf16_bits(o1, r16_of(r, e + 1)) << 16);
        else ow.v[i] = pack_bf16x2(o0, o1);
      }
      st_global_256(wp + 16 * g16, ow);
    }
  }

  __device__ static void epilogue(const Params& p, const Job& j, uint32_t taddr, bool have_acc,
                                  SharedTail&, const EpiCtx& ec, EpilogueState& st) {
    if (j.a0 >= p.rows_valid) return;               // whole CTA tile beyond the chunk (pairs only)
    if constexpr (W8) {
      epilogue_w8(p, j, taddr, have_acc, ec);
    } else {
      const int row = ec.q * 32 + ec.lane;
      const int crow = j.a0 + row;
      const bool row_valid = crow < p.rows_valid;
      const unsigned long long erow = p.elem0 + (unsigned long long)crow * p.d + j.b0;
      uint32_t v[32];
#pragma unroll 1
      for (int g = 0; g < kGroups; ++g) {
        const int c0 = 32 * (ec.h + ec.nsplit * g);
        if (c0 >= j.n_eff) break;
        const int col = j.b0 + c0;
        __nv_bfloat16* wp = reinterpret_cast<__nv_bfloat16*>(p.W) + (size_t)crow * p.d + col;
        load_acc(taddr + c0, have_acc, v);
        if (row_valid) process_bf16(p, v, erow + c0, wp, col + 16 < p.d ? 2 : (col < p.d ? 1 : 0));
      }
    }
  }
};

// -------------------------------------------------------------------------------------------------
// Inference logits (reference: chunked.py:48-53, chunked_fp8xmc_clf.py:45-60 xfc_forward):
// out[b][col0 + r] = bf16(w_scale * <x[b], W[r]>).  Batch rows sit on the TMEM lanes so that a thread
// stores runs of consecutive labels.
// -------------------------------------------------------------------------------------------------
struct LogitsParams {
  int m_rows;              // batch rows per M tile: 128, or 256 on CTA pairs
  int batch, rows;         // valid batch rows, label rows of this launch
  int n_mtiles, n_ntiles;  // batch tiles of m_rows, label tiles of 256
  int k_steps;
  float w_scale;
  __nv_bfloat16* out;      // [batch x ld_out]
  long long ld_out;
  long long col0;          // column of this launch's label row 0
  long long n_out;         // columns >= n_out are not written
  int* status;
};

template <bool FP8, bool CONV = false>
struct LogitsPolicy {
  static_assert(!(FP8 && CONV), "the FP8 contraction takes the e4m3 weights as they are");
  using Params = LogitsParams;
  static constexpr bool kMnMajor = false;
  static constexpr bool kFp8 = FP8;
  static constexpr uint32_t kFmt = FP8 ? 0u : 1u;
  static constexpr int kElemsPerRow = FP8 ? 128 : 64;
  static constexpr int kEpiWarps = 8;
  static constexpr int kStages = CONV ? 3 : 4;
  static constexpr int kStagesPair = 6;
  static constexpr bool kCTile = false;
  static constexpr int kCBufs = 1;
  static constexpr int kConv = CONV ? 2 : 0;      // the weights are the B operand here
  static constexpr bool kBitmap = false;
  static constexpr int kWaitRoles = kRoleAll;
  __device__ static long long wait_limit(const Params&) { return kWaitLimitCycles; }
  __device__ static bool skip_load(const Params&, int, int) { return false; }
  using EpilogueState = NoState;
  __device__ static int num_tiles(const Params& p) { return p.n_mtiles * p.n_ntiles; }
  __device__ static void job(const Params& p, int tile, Job& j) {
    j.t1 = tile / p.n_mtiles;            // label tile (adjacent CTAs share it)
    j.t0 = tile - j.t1 * p.n_mtiles;     // batch tile
    j.a0 = j.t0 * p.m_rows;
    j.b0 = j.t1 * kTileN;
    j.k_begin = 0;
    j.k_steps = p.k_steps;
    j.n_eff = min(kTileN, round_up16(p.rows - j.b0));
  }
  __device__ static void epilogue_begin(const Params&, EpilogueState&) {}
  __device__ static void epilogue_pre(const Params&, const Job&, SharedTail&, const EpiCtx&, EpilogueState&) {}
  __device__ static void epilogue_prefetch(const Params&, const Job&, EpilogueState&) {}
  __device__ static void epilogue_end(const Params&, SharedTail&, const EpiCtx&, EpilogueState&) {}
  __device__ static void epilogue(const Params& p, const Job& j, uint32_t taddr, bool have_acc,
                                  SharedTail&, const EpiCtx& ec, EpilogueState&) {
    const int b = j.a0 + ec.q * 32 + ec.lane;
    for (int c0 = 32 * ec.h; c0 < j.n_eff; c0 += 32 * ec.nsplit) {
      uint32_t v[32];
      if (have_acc) {
        tmem_ld32(taddr + c0, v);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = 0u;
      }
      if (b >= p.batch) continue;
      const long long col = p.col0 + j.b0 + c0;
      const int valid = (int)max(0ll, min(32ll, min((long long)(p.rows - j.b0 - c0), p.n_out - col)));
      __nv_bfloat16* dst = p.out + (size_t)b * p.ld_out + col;
      uint32_t o[16];
#pragma unroll
      for (int i = 0; i < 16; ++i)
        o[i] = pack_bf16x2(__uint_as_float(v[2 * i]) * p.w_scale, __uint_as_float(v[2 * i + 1]) * p.w_scale);
      if (valid == 32 && (((uintptr_t)dst) & 31u) == 0) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          U32x8 o8;
#pragma unroll
          for (int k = 0; k < 8; ++k) o8.v[k] = o[8 * i + k];
          st_global_256(dst + 16 * i, o8);
        }
      } else if (valid == 32 && (((uintptr_t)dst) & 15u) == 0) {
#pragma unroll
        for (int i = 0; i < 4; ++i)
          reinterpret_cast<uint4*>(dst)[i] = make_uint4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
      } else {
        const uint16_t* h16 = reinterpret_cast<const uint16_t*>(o);
        for (int i = 0; i < valid; ++i) reinterpret_cast<uint16_t*>(dst)[i] = h16[i];
      }
    }
  }
};

// -------------------------------------------------------------------------------------------------
// Fused logits + top-k (reference: evaluate.py:158-159 xfc_forward followed by torch.topk; the
// logits are never stored).  Same contraction as LogitsPolicy; every epilogue thread keeps the k
// best (bf16-rounded logit, label) pairs of ITS batch row over all label tiles its CTA visits, and
// writes them out once at the end; a merge kernel picks the final k per row.  A CTA's batch tile is
// fixed (the grid is a multiple of n_mtiles), so a thread's row never changes within a launch.
// -------------------------------------------------------------------------------------------------
struct TopkParams {
  int batch, rows;
  int n_mtiles, n_ntiles;
  int k_steps;
  int k, cap;              // wanted entries per row; capacity of one candidate list (> k)
  float w_scale;
  long long col0;          // index (within the handle) of this launch's label row 0
  long long n_out;         // rows >= n_out are ignored (padding)
  float* cand_val;         // [lists][cap + 32], list = (CTA * 8 + epilogue warp) * 32 + lane; lists live across launches
  int* cand_idx;
  int* list_cnt;           // [lists] entries in use
  float* list_thr;         // [lists] value a new candidate of this list must exceed
  float* list_max;         // [lists] largest value the list has ever held
  unsigned int* row_thr;   // [batch rows] ordered key of the best k-th value any list of the row has published
  int* status;
};

// monotone map float -> unsigned (larger float = larger key), and back
__device__ __forceinline__ unsigned int topk_key(float v) {
  const unsigned int b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float topk_unkey(unsigned int k) {
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7FFFFFFFu) : ~k);
}

// A thread owns one batch row of its CTA's batch tile and keeps an UNSORTED candidate list in global
// memory: a logit joins it when it beats the list's own threshold (strictly: later labels of a list
// have higher ids and lose ties) and reaches the row's published threshold (the best k-th value any
// list of that row has seen: nothing below it can be in the row's top-k).  A full list is cut back to
// its k best by a radix select, which raises both thresholds.  Appending is a few instructions, so the
// divergence of 32 lanes with 32 different rows stays cheap, and because all lists of a row share the
// published threshold the number of candidates per row stays near k ln(L/k) however many CTAs there are.
template <bool FP8, bool CONV = false>
struct TopkPolicy {
  static_assert(!(FP8 && CONV), "the FP8 contraction takes the e4m3 weights as they are");
  using Params = TopkParams;
  static constexpr bool kMnMajor = false;
  static constexpr bool kFp8 = FP8;
  static constexpr uint32_t kFmt = FP8 ? 0u : 1u;
  static constexpr int kElemsPerRow = FP8 ? 128 : 64;
  static constexpr int kEpiWarps = 8;
  static constexpr int kStages = CONV ? 3 : 4;
  static constexpr bool kCTile = false;
  static constexpr int kCBufs = 1;
  static constexpr int kConv = CONV ? 2 : 0;
  static constexpr bool kBitmap = false;
  static constexpr int kWaitRoles = kRoleAll;
  __device__ static long long wait_limit(const Params&) { return kWaitLimitCycles; }
  __device__ static bool skip_load(const Params&, int, int) { return false; }
  struct EpilogueState {
    float thr;             // own threshold
    float g;               // published threshold of the row (refreshed per tile)
    int cnt;
    int list;              // -1 until the first tile
    float mx;              // largest value appended so far
  };
  __device__ static int num_tiles(const Params& p) { return p.n_mtiles * p.n_ntiles; }
  __device__ static void job(const Params& p, int tile, Job& j) {
    j.t1 = tile / p.n_mtiles;
    j.t0 = tile - j.t1 * p.n_mtiles;
    j.a0 = j.t0 * kTileM;
    j.b0 = j.t1 * kTileN;
    j.k_begin = 0;
    j.k_steps = p.k_steps;
    j.n_eff = min(kTileN, round_up16(p.rows - j.b0));
  }
  __device__ static void epilogue_begin(const Params&, EpilogueState& st) { st.list = -1; }
  __device__ static void epilogue_prefetch(const Params&, const Job&, EpilogueState&) {}
  __device__ static void epilogue_pre(const Params& p, const Job& j, SharedTail&, const EpiCtx& ec, EpilogueState& st) {
    const int b = j.a0 + ec.q * 32 + ec.lane;
    if (st.list < 0) {
      st.list = ((int)blockIdx.x * kEpiWarps + ec.slot) * 32 + ec.lane;
      st.cnt = p.list_cnt[st.list];
      st.thr = p.list_thr[st.list];
      st.mx = p.list_max[st.list];
      // Once per launch and row (first CTA of the batch tile, first column phase): the k-th largest of
      // the best values of the row's lists is reached by k different labels, so nothing below it can be
      // among the row's k best.  This is far tighter than any single list's own k-th value.
      const int lists_row = ((int)gridDim.x / p.n_mtiles) * 2;
      if ((int)blockIdx.x < p.n_mtiles && ec.h == 0 && b < p.batch && p.k <= 8 && lists_row >= p.k) {
        float top[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) top[i] = -INFINITY;
        for (int r = 0; r < lists_row; ++r) {
          const int c = (r >> 1) * p.n_mtiles + (int)blockIdx.x;
          // the epilogue warp of column phase (r & 1) that owns this thread's TMEM quarter
          const int slot = 4 * (r & 1) + ((ec.q + 2) & 3);
          float x = __ldcg(&p.list_max[(c * kEpiWarps + slot) * 32 + ec.lane]);
#pragma unroll
          for (int i = 0; i < 8; ++i) {             // insertion into the descending array
            const float hi = fmaxf(top[i], x);
            x = fminf(top[i], x);
            top[i] = hi;
          }
        }
        float kth = top[0];
#pragma unroll
        for (int i = 1; i < 8; ++i) kth = (i < p.k) ? top[i] : kth;
        atomicMax(&p.row_thr[b], topk_key(kth));
      }
    }
    st.g = b < p.batch ? topk_unkey(__ldcg(&p.row_thr[b])) : INFINITY;
  }
  // The whole warp cuts one list of n entries back to its k best (ties: first come = lower id): a radix
  // select over the ordered keys with one warp-wide count per bit, then a stable compaction.  Returns
  // the new threshold (the k-th largest value) to every lane and publishes it for row b.
  __device__ __noinline__ static float prune_warp(const Params& p, int list, int n, int b, int lane) {
    float* val = p.cand_val + (size_t)list * kListStride(p);
    int* idx = p.cand_idx + (size_t)list * kListStride(p);
    const unsigned int lt = (1u << lane) - 1u;
    if (p.k <= 16 && n <= 128) {
      // few wanted, few held: k rounds of "largest remaining entry, earliest first", four entries per lane
      unsigned int key[4];
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) key[jj] = (lane + 32 * jj < n) ? topk_key(val[lane + 32 * jj]) : 0u;
      unsigned int taken = 0u, t_key = 0u;
      for (int r = 0; r < p.k; ++r) {
        unsigned int m = 0u;
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) m = ((taken >> jj) & 1u) ? m : max(m, key[jj]);
        m = __reduce_max_sync(0xffffffffu, m);
        int e_mine = 0x7fffffff;
#pragma unroll
        for (int jj = 3; jj >= 0; --jj)
          if (!((taken >> jj) & 1u) && key[jj] == m) e_mine = lane + 32 * jj;
        const int e_min = __reduce_min_sync(0xffffffffu, e_mine);
        if ((e_min & 31) == lane) taken |= 1u << (e_min >> 5);
        t_key = m;
      }
      int w = 0;
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        const int e = lane + 32 * jj;
        const bool keep = (taken >> jj) & 1u;
        const float v = keep ? val[e] : 0.f;
        const int id = keep ? idx[e] : 0;
        const unsigned int km = __ballot_sync(0xffffffffu, keep);
        __syncwarp();
        if (keep) {
          const int pos = w + __popc(km & lt);
          val[pos] = v;
          idx[pos] = id;
        }
        w += __popc(km);
        __syncwarp();
      }
      if (lane == 0) atomicMax(&p.row_thr[b], t_key);
      return topk_unkey(t_key);
    }
    unsigned int prefix = 0u, mask = 0u;
    int need = p.k;                                  // rank still wanted among the entries matching the prefix
    for (int bit = 31; bit >= 0; --bit) {
      const unsigned int bm = 1u << bit;
      int c = 0;
      for (int e = lane; e < n; e += 32) c += ((topk_key(val[e]) & (mask | bm)) == (prefix | bm)) ? 1 : 0;
      c = __reduce_add_sync(0xffffffffu, c);
      if (c >= need) prefix |= bm;
      else need -= c;
      mask |= bm;
    }
    const float t = topk_unkey(prefix);              // `need` entries equal to it survive
    int w = 0, eq = 0;
    for (int e0 = 0; e0 < n; e0 += 32) {
      const int e = e0 + lane;
      const float v = e < n ? val[e] : -INFINITY;
      const int id = e < n ? idx[e] : -1;
      const bool is_eq = e < n && v == t;
      const unsigned int eqm = __ballot_sync(0xffffffffu, is_eq);
      const bool keep = e < n && (v > t || (is_eq && eq + __popc(eqm & lt) < need));
      const unsigned int km = __ballot_sync(0xffffffffu, keep);
      __syncwarp();                                  // every lane holds its entry before any slot is rewritten
      if (keep) {
        const int pos = w + __popc(km & lt);
        val[pos] = v;
        idx[pos] = id;
      }
      w += __popc(km);
      eq += __popc(eqm);
      __syncwarp();
    }
    if (lane == 0) atomicMax(&p.row_thr[b], prefix);
    return t;
  }
  __device__ static int kListStride(const Params& p) { return p.cap + 32; }   // a group may overshoot cap by 31
  __device__ static void epilogue(const Params& p, const Job& j, uint32_t taddr, bool have_acc,
                                  SharedTail&, const EpiCtx& ec, EpilogueState& st) {
    const int b = j.a0 + ec.q * 32 + ec.lane;
    const bool active = b < p.batch;
    float* val = p.cand_val + (size_t)st.list * kListStride(p);
    int* idx = p.cand_idx + (size_t)st.list * kListStride(p);
    float thr = st.thr, g = st.g, mx = st.mx;
    int cnt = st.cnt;
    for (int c0 = 32 * ec.h; c0 < j.n_eff; c0 += 32 * ec.nsplit) {
      uint32_t v[32];
      if (have_acc) {
        tmem_ld32(taddr + c0, v);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = 0u;
      }
      const long long col = p.col0 + j.b0 + c0;
      const int valid = (int)max(0ll, min(32ll, min((long long)(p.rows - j.b0 - c0), p.n_out - col)));
      // pass 1, branch-free: which of the 32 logits reach the thresholds as they stand now
      const float lim = fmaxf(thr, g);
      uint32_t hit = 0u;
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const float z = bf16_round(__uint_as_float(v[i]) * p.w_scale);
        v[i] = __float_as_uint(z);
        hit |= (z >= lim ? 1u : 0u) << i;
      }
      hit &= valid >= 32 ? 0xFFFFFFFFu : ((1u << valid) - 1u);
      if (!active) hit = 0u;
      if (!__any_sync(0xffffffffu, hit != 0u)) continue;          // warp-uniform
      // pass 2, rare: append in label order (own threshold strict: later labels lose ties)
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        if (hit & (1u << i)) {
          const float z = __uint_as_float(v[i]);
          if (z > thr && z >= g) {
            val[cnt] = z;
            idx[cnt] = (int)(col + i);
            ++cnt;
            mx = fmaxf(mx, z);
          }
        }
      }
      __syncwarp();
      // full lists are cut back by the whole warp, one list at a time
      unsigned int full = __ballot_sync(0xffffffffu, cnt >= p.cap);
      while (full) {
        const int src = __ffs(full) - 1;
        full &= full - 1u;
        const int l_src = __shfl_sync(0xffffffffu, st.list, src);
        const int n_src = __shfl_sync(0xffffffffu, cnt, src);
        const int b_src = __shfl_sync(0xffffffffu, b, src);
        const float t = prune_warp(p, l_src, n_src, b_src, ec.lane);
        if (ec.lane == src) {
          thr = t;
          cnt = p.k;
          g = fmaxf(g, t);
        }
      }
    }
    st.thr = thr;
    st.g = g;
    st.cnt = cnt;
    st.mx = mx;
  }
  __device__ static void epilogue_end(const Params& p, SharedTail&, const EpiCtx&, EpilogueState& st) {
    if (st.list < 0) return;                          // this CTA had no tile
    p.list_cnt[st.list] = st.cnt;
    p.list_thr[st.list] = st.thr;
    p.list_max[st.list] = st.mx;
  }
};

// -------------------------------------------------------------------------------------------------
// Plain D = A B^T, fp32 out (engine self-test; also the logits kernel's skeleton)
// -------------------------------------------------------------------------------------------------
struct PlainParams {
  int m_rows;              // rows per M tile (128)
  int M, N;
  int n_mtiles, n_ntiles;
  int k_steps;
  float* D;                // [M x N]
  int checksum_only;       // 1: do not store D (times the main loop without the output traffic)
  long long test_wait_limit;   // > 0: every wait of the kernel gives up after this many cycles
  int test_skip_tile;      // the producer leaves out the second k-step of this tile (-1: none)
  int* status;
};

template <bool FP8, bool MN>
struct PlainPolicy {
  using Params = PlainParams;
  static constexpr bool kMnMajor = MN;
  static constexpr bool kFp8 = FP8;
  static constexpr uint32_t kFmt = FP8 ? 0u : 1u;
  static constexpr int kElemsPerRow = FP8 ? 128 : 64;
  static constexpr int kEpiWarps = 8;
  static constexpr int kStages = 4;
  static constexpr int kStagesPair = 6;
  static constexpr bool kCTile = false;
  static constexpr int kCBufs = 1;
  static constexpr int kConv = 0;
  static constexpr bool kBitmap = false;
  static constexpr int kWaitRoles = kRoleAll;
  // failure-injection of the self-test: a shortened wait limit and one operand load left out
  __device__ static long long wait_limit(const Params& p) { return p.test_wait_limit > 0 ? p.test_wait_limit : kWaitLimitCycles; }
  __device__ static bool skip_load(const Params& p, int tile, int k) { return tile == p.test_skip_tile && k == 1; }
  using EpilogueState = NoState;
  __device__ static int num_tiles(const Params& p) { return p.n_mtiles * p.n_ntiles; }
  __device__ static void job(const Params& p, int tile, Job& j) {
    j.t0 = tile / p.n_ntiles;
    j.t1 = tile - j.t0 * p.n_ntiles;
    j.a0 = j.t0 * p.m_rows;
    j.b0 = j.t1 * kTileN;
    j.k_begin = 0;
    j.k_steps = p.k_steps;
    j.n_eff = min(kTileN, round_up16(p.N - j.b0));
  }
  __device__ static void epilogue_begin(const Params&, EpilogueState&) {}
  __device__ static void epilogue_pre(const Params&, const Job&, SharedTail&, const EpiCtx&, EpilogueState&) {}
  __device__ static void epilogue_prefetch(const Params&, const Job&, EpilogueState&) {}
  __device__ static void epilogue_end(const Params&, SharedTail&, const EpiCtx&, EpilogueState&) {}
  __device__ static void epilogue(const Params& p, const Job& j, uint32_t taddr, bool have_acc,
                                  SharedTail&, const EpiCtx& ec, EpilogueState&) {
    const int m = j.a0 + ec.q * 32 + ec.lane;
    for (int c0 = 32 * ec.h; c0 < j.n_eff; c0 += 32 * ec.nsplit) {
      uint32_t v[32];
      if (have_acc) {
        tmem_ld32(taddr + c0, v);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = 0u;
      }
      if (m >= p.M) continue;
      if (p.checksum_only) {          // main-loop timing: fold the tile into one word per thread
        uint32_t x = 0;
#pragma unroll
        for (int i = 0; i < 32; ++i) x ^= v[i];
        if (x == 0x12345678u) p.D[0] = 1.f;
        continue;
      }
      float* drow = p.D + (size_t)m * p.N + j.b0 + c0;
      if ((p.N & 3) == 0 && j.b0 + c0 + 32 <= p.N) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
          reinterpret_cast<float4*>(drow)[i] = make_float4(__uint_as_float(v[4 * i]), __uint_as_float(v[4 * i + 1]),
                                                           __uint_as_float(v[4 * i + 2]), __uint_as_float(v[4 * i + 3]));
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (j.b0 + c0 + i < p.N) drow[i] = __uint_as_float(v[i]);
      }
    }
  }
};

}  // namespace xmc
