// GEMM policies (tile mapping + epilogue) of the chunked XMC step:
//   FwdPolicy    Z^T[labels x batch] = W X^T  ->  G = sigmoid(Z) - Y  (bf16, label-major), loss terms
//   UpdPolicy    acc[labels x d] = G X        ->  W <- round(W - lr*(acc + wd*W))   (dW never stored)
//   GradXPolicy  partial[batch x d] (+)= G^T W  over a slice of the chunk's label rows
//   PlainPolicy  D = A B^T (engine self-test)
#pragma once
#include "gemm_engine.cuh"
#include "numerics.cuh"

namespace xmc {

__device__ __forceinline__ int round_up16(int v) { return (v + 15) & ~15; }

struct NoState {};

// -------------------------------------------------------------------------------------------------
// Forward + loss-gradient epilogue.
// Reference arithmetic reproduced here: logits rounded to bf16 (output dtype of torch._scaled_mm /
// torch.matmul, chunked_fp8xmc_clf.py:98-102), sigmoid rounded to bf16 (:107), "-1" applied in bf16 at
// the positives with set semantics (:108).
// -------------------------------------------------------------------------------------------------
struct FwdParams {
  int rows_valid;          // label rows of this scheduling chunk
  int n_ltiles, n_btiles;  // label tiles (128) x batch tiles (256)
  int batch, bpad;         // valid batch rows, padded row length of G (multiple of 16)
  int k_steps;             // cdiv(d * elem_size, 128)
  float w_scale;
  __nv_bfloat16* G;        // [n_ltiles*128 x bpad]
  const int* bucket_off;   // positives bucketed by label tile: offsets ...
  const uint32_t* bucket_ent;  // ... entries: batch row | (label-in-tile << 16)
  int tile_base;           // bucket index of this chunk's label tile 0
  double* loss_partial;    // [gridDim.x * 4] or nullptr
  int* status;
};

template <bool FP8, bool LOSS>
struct FwdPolicy {
  using Params = FwdParams;
  static constexpr bool kMnMajor = false;
  static constexpr bool kFp8 = FP8;
  static constexpr uint32_t kFmt = FP8 ? 0u : 1u;            // e4m3 | bf16
  static constexpr int kElemsPerRow = FP8 ? 128 : 64;
  struct EpilogueState {
    float loss;
    int has_pos;
  };

  __device__ static int num_tiles(const Params& p) { return p.n_ltiles * p.n_btiles; }
  __device__ static void job(const Params& p, int tile, Job& j) {
    j.t0 = tile / p.n_btiles;          // label tile
    j.t1 = tile - j.t0 * p.n_btiles;   // batch tile
    j.a0 = j.t0 * kTileM;
    j.b0 = j.t1 * kTileN;
    j.k_begin = 0;
    j.k_steps = p.k_steps;
    j.n_eff = min(kTileN, round_up16(p.bpad - j.b0));
  }
  __device__ static void epilogue_begin(const Params&, EpilogueState& st) {
    st.loss = 0.f;
    st.has_pos = 0;
  }
  // Build this warp's 32 rows of the positives bitmap (duplicates collapse: set semantics).
  __device__ static void epilogue_pre(const Params& p, const Job& j, SharedTail& sh, int q, int lane,
                                      EpilogueState& st) {
    const int beg = p.bucket_off[p.tile_base + j.t0], end = p.bucket_off[p.tile_base + j.t0 + 1];
    st.has_pos = end > beg;
    if (!st.has_pos) return;
    uint32_t* bm = sh.bitmap + q * 32 * (kTileN / 32);
    __syncwarp();
    for (int w = lane; w < 32 * (kTileN / 32); w += 32) bm[w] = 0u;
    __syncwarp();
    for (int e = beg + lane; e < end; e += 32) {
      const uint32_t ent = p.bucket_ent[e];
      const int lrow = (int)(ent >> 16), bl = (int)(ent & 0xFFFFu) - j.b0;
      if ((lrow >> 5) == q && bl >= 0 && bl < kTileN)
        atomicOr(&sh.bitmap[lrow * (kTileN / 32) + (bl >> 5)], 1u << (bl & 31));
    }
    __syncwarp();
  }
  __device__ static void epilogue(const Params& p, const Job& j, uint32_t taddr, bool have_acc,
                                  SharedTail& sh, int q, int lane, EpilogueState& st) {
    const int row = q * 32 + lane;
    const int crow = j.a0 + row;
    const bool row_valid = crow < p.rows_valid;
    __nv_bfloat16* grow = p.G + (size_t)crow * p.bpad + j.b0;
    for (int c0 = 0; c0 < j.n_eff; c0 += 32) {
      uint32_t v[32];
      if (have_acc) {
        tmem_ld32(taddr + c0, v);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = 0u;
      }
      const uint32_t bits = st.has_pos ? sh.bitmap[row * (kTileN / 32) + (c0 >> 5)] : 0u;
      uint32_t out[16];
#pragma unroll
      for (int i = 0; i < 32; i += 2) {
        float g[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int b = j.b0 + c0 + i + h;
          const bool pos = (bits >> (i + h)) & 1u;
          const float z = bf16_round(__uint_as_float(v[i + h]) * p.w_scale);
          float s = sigmoid_bf16(z);
          if (pos) s = bf16_round(s - 1.0f);
          const bool ok = row_valid && b < p.batch;
          if (LOSS && ok) st.loss += bce_softplus(z) - (pos ? z : 0.f);
          g[h] = ok ? s : 0.f;
        }
        out[i >> 1] = pack_bf16x2(g[0], g[1]);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (j.b0 + c0 + 8 * i < p.bpad)
          *reinterpret_cast<uint4*>(grow + c0 + 8 * i) =
              make_uint4(out[4 * i], out[4 * i + 1], out[4 * i + 2], out[4 * i + 3]);
      }
    }
  }
  __device__ static void epilogue_end(const Params& p, SharedTail&, int q, int lane, EpilogueState& st) {
    if (!LOSS) return;
    float v = st.loss;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lane == 0 && p.loss_partial != nullptr) p.loss_partial[blockIdx.x * 4 + q] = (double)v;
  }
};

// -------------------------------------------------------------------------------------------------
// Fused dW + SGD update (reference: fuse_kernel.py:63-131 naive_matmul_k / matmul_update; for bf16
// weights chunked.py:119 + stochastic_rounding_kernel.py:65-99).
// -------------------------------------------------------------------------------------------------
struct UpdParams {
  int rows_valid;
  int n_ltiles, n_dtiles;
  int d;
  int k_steps;             // cdiv(bpad, 64)
  void* W;                 // first row of this scheduling chunk, row-major [rows x d]
  float lr_eff;            // lr / w_scale
  float wd;
  unsigned long long seed, step;
  unsigned long long elem0;   // global flat element index of W[0][0] of this chunk (Philox counter origin)
  int round_dw_bf16;
  int* status;
};

template <bool W8, bool SR>
struct UpdPolicy {
  using Params = UpdParams;
  static constexpr bool kMnMajor = false;
  static constexpr bool kFp8 = false;
  static constexpr uint32_t kFmt = 1u;
  static constexpr int kElemsPerRow = 64;
  using EpilogueState = NoState;

  __device__ static int num_tiles(const Params& p) { return p.n_ltiles * p.n_dtiles; }
  __device__ static void job(const Params& p, int tile, Job& j) {
    j.t0 = tile / p.n_dtiles;
    j.t1 = tile - j.t0 * p.n_dtiles;
    j.a0 = j.t0 * kTileM;     // rows of G
    j.b0 = j.t1 * kTileN;     // rows of X^T = feature index
    j.k_begin = 0;
    j.k_steps = p.k_steps;
    j.n_eff = min(kTileN, round_up16(p.d - j.b0));
  }
  __device__ static void epilogue_begin(const Params&, EpilogueState&) {}
  __device__ static void epilogue_pre(const Params&, const Job&, SharedTail&, int, int, EpilogueState&) {}
  __device__ static void epilogue_end(const Params&, SharedTail&, int, int, EpilogueState&) {}

  // new weights for 8 consecutive elements
  __device__ static void update8(const Params& p, const float (&w)[8], const uint32_t* acc,
                                 unsigned long long elem, float (&o)[8], uint32_t (&r16)[8]) {
    if (SR) {
      const unsigned long long qi = elem >> 3;
      const uint4 r = philox4x32_10(
          make_uint4((uint32_t)qi, (uint32_t)(qi >> 32), (uint32_t)p.step, (uint32_t)(p.step >> 32)),
          make_uint2((uint32_t)p.seed, (uint32_t)(p.seed >> 32)));
      r16[0] = r.x & 0xFFFFu; r16[1] = r.x >> 16; r16[2] = r.y & 0xFFFFu; r16[3] = r.y >> 16;
      r16[4] = r.z & 0xFFFFu; r16[5] = r.z >> 16; r16[6] = r.w & 0xFFFFu; r16[7] = r.w >> 16;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float a = __uint_as_float(acc[i]);
      if (p.round_dw_bf16) a = bf16_round(a);
      if (p.wd != 0.f) a = fmaf(p.wd, w[i], a);
      o[i] = fmaf(-p.lr_eff, a, w[i]);
    }
  }

  __device__ static void epilogue(const Params& p, const Job& j, uint32_t taddr, bool have_acc,
                                  SharedTail&, int q, int lane, EpilogueState&) {
    const int row = q * 32 + lane;
    const int crow = j.a0 + row;
    const bool row_valid = crow < p.rows_valid;
    for (int c0 = 0; c0 < j.n_eff; c0 += 32) {
      uint32_t v[32];
      if (have_acc) {
        tmem_ld32(taddr + c0, v);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = 0u;
      }
      if (!row_valid) continue;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int col = j.b0 + c0 + 16 * h;
        if (col >= p.d) continue;
        const unsigned long long e0 = p.elem0 + (unsigned long long)crow * p.d + col;
        if constexpr (W8) {
          uint8_t* wp = reinterpret_cast<uint8_t*>(p.W) + (size_t)crow * p.d + col;
          const uint4 raw = *reinterpret_cast<const uint4*>(wp);
          const uint32_t rw[4] = {raw.x, raw.y, raw.z, raw.w};
          uint32_t ow[4];
#pragma unroll
          for (int g8 = 0; g8 < 2; ++g8) {
            float w[8], o[8];
            uint32_t r16[8];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float2 f = e4m3x2_to_float2((uint16_t)(rw[2 * g8 + (i >> 1)] >> (16 * (i & 1))));
              w[2 * i] = f.x;
              w[2 * i + 1] = f.y;
            }
            update8(p, w, &v[16 * h + 8 * g8], e0 + 8 * g8, o, r16);
            if (SR) {
#pragma unroll
              for (int i = 0; i < 8; ++i) o[i] = sr_e4m3(o[i], r16[i]);
            }
#pragma unroll
            for (int i = 0; i < 2; ++i)
              ow[2 * g8 + i] = (uint32_t)float2_to_e4m3x2(o[4 * i], o[4 * i + 1]) |
                               ((uint32_t)float2_to_e4m3x2(o[4 * i + 2], o[4 * i + 3]) << 16);
          }
          *reinterpret_cast<uint4*>(wp) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
        } else {
          __nv_bfloat16* wp = reinterpret_cast<__nv_bfloat16*>(p.W) + (size_t)crow * p.d + col;
#pragma unroll
          for (int g8 = 0; g8 < 2; ++g8) {
            const uint4 raw = *reinterpret_cast<const uint4*>(wp + 8 * g8);
            const uint32_t rw[4] = {raw.x, raw.y, raw.z, raw.w};
            float w[8], o[8];
            uint32_t r16[8];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              w[2 * i] = bf16_bits_to_float(rw[i] & 0xFFFFu);
              w[2 * i + 1] = bf16_bits_to_float(rw[i] >> 16);
            }
            update8(p, w, &v[16 * h + 8 * g8], e0 + 8 * g8, o, r16);
            uint32_t ow[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              if (SR) ow[i] = sr_bf16_bits(o[2 * i], r16[2 * i]) | (sr_bf16_bits(o[2 * i + 1], r16[2 * i + 1]) << 16);
              else ow[i] = pack_bf16x2(o[2 * i], o[2 * i + 1]);
            }
            *reinterpret_cast<uint4*>(wp + 8 * g8) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
          }
        }
      }
    }
  }
};

// -------------------------------------------------------------------------------------------------
// grad_X partial sums (reference: matmul_kernel.py:204-239 large_k_matmul: C = G^T W, both operands
// bf16, fp32 accumulation).  Each (split, batch tile, d tile) owns one slot of `partial` and adds to
// it in chunk order, so the summation order is fixed (no atomics).
// -------------------------------------------------------------------------------------------------
struct GradXParams {
  int bpad, d;
  int n_btiles, n_dtiles, n_splits;
  int total_ksteps;        // cdiv(rows written by the forward kernel, 64)
  int accumulate;          // 0: overwrite the slot (first chunk of a step)
  float* partial;          // [n_splits][bpad][d]
  int* status;
};

struct GradXPolicy {
  using Params = GradXParams;
  static constexpr bool kMnMajor = true;
  static constexpr bool kFp8 = false;
  static constexpr uint32_t kFmt = 1u;
  static constexpr int kElemsPerRow = 64;
  using EpilogueState = NoState;

  __device__ static int num_tiles(const Params& p) { return p.n_btiles * p.n_dtiles * p.n_splits; }
  __device__ static void job(const Params& p, int tile, Job& j) {
    const int per = p.n_btiles * p.n_dtiles;
    j.t2 = tile / per;                      // split
    const int r = tile - j.t2 * per;
    j.t0 = r / p.n_dtiles;                  // batch tile
    j.t1 = r - j.t0 * p.n_dtiles;           // d tile
    j.a0 = j.t0 * kTileM;
    j.b0 = j.t1 * kTileN;
    j.k_begin = (int)(((long long)j.t2 * p.total_ksteps) / p.n_splits);
    j.k_steps = (int)(((long long)(j.t2 + 1) * p.total_ksteps) / p.n_splits) - j.k_begin;
    j.n_eff = min(kTileN, round_up16(p.d - j.b0));
  }
  __device__ static void epilogue_begin(const Params&, EpilogueState&) {}
  __device__ static void epilogue_pre(const Params&, const Job&, SharedTail&, int, int, EpilogueState&) {}
  __device__ static void epilogue_end(const Params&, SharedTail&, int, int, EpilogueState&) {}
  __device__ static void epilogue(const Params& p, const Job& j, uint32_t taddr, bool have_acc,
                                  SharedTail&, int q, int lane, EpilogueState&) {
    const int b = j.a0 + q * 32 + lane;
    const bool row_valid = b < p.bpad;
    if (!have_acc && p.accumulate) return;
    float* dst = p.partial + ((size_t)j.t2 * p.bpad + b) * p.d + j.b0;
    for (int c0 = 0; c0 < j.n_eff; c0 += 32) {
      uint32_t v[32];
      if (have_acc) {
        tmem_ld32(taddr + c0, v);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = 0u;
      }
      if (!row_valid) continue;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int col = j.b0 + c0 + 4 * i;
        if (col >= p.d) continue;
        float4 o = make_float4(__uint_as_float(v[4 * i]), __uint_as_float(v[4 * i + 1]),
                               __uint_as_float(v[4 * i + 2]), __uint_as_float(v[4 * i + 3]));
        float4* ptr = reinterpret_cast<float4*>(dst + c0 + 4 * i);
        if (p.accumulate) {
          const float4 old = *ptr;
          o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
        }
        *ptr = o;
      }
    }
  }
};

// -------------------------------------------------------------------------------------------------
// Plain D = A B^T, fp32 out (engine self-test; also the logits kernel's skeleton)
// -------------------------------------------------------------------------------------------------
struct PlainParams {
  int M, N;
  int n_mtiles, n_ntiles;
  int k_steps;
  float* D;                // [M x N]
  int* status;
};

template <bool FP8, bool MN>
struct PlainPolicy {
  using Params = PlainParams;
  static constexpr bool kMnMajor = MN;
  static constexpr bool kFp8 = FP8;
  static constexpr uint32_t kFmt = FP8 ? 0u : 1u;
  static constexpr int kElemsPerRow = FP8 ? 128 : 64;
  using EpilogueState = NoState;
  __device__ static int num_tiles(const Params& p) { return p.n_mtiles * p.n_ntiles; }
  __device__ static void job(const Params& p, int tile, Job& j) {
    j.t0 = tile / p.n_ntiles;
    j.t1 = tile - j.t0 * p.n_ntiles;
    j.a0 = j.t0 * kTileM;
    j.b0 = j.t1 * kTileN;
    j.k_begin = 0;
    j.k_steps = p.k_steps;
    j.n_eff = min(kTileN, round_up16(p.N - j.b0));
  }
  __device__ static void epilogue_begin(const Params&, EpilogueState&) {}
  __device__ static void epilogue_pre(const Params&, const Job&, SharedTail&, int, int, EpilogueState&) {}
  __device__ static void epilogue_end(const Params&, SharedTail&, int, int, EpilogueState&) {}
  __device__ static void epilogue(const Params& p, const Job& j, uint32_t taddr, bool have_acc,
                                  SharedTail&, int q, int lane, EpilogueState&) {
    const int m = j.a0 + q * 32 + lane;
    for (int c0 = 0; c0 < j.n_eff; c0 += 32) {
      uint32_t v[32];
      if (have_acc) {
        tmem_ld32(taddr + c0, v);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = 0u;
      }
      if (m >= p.M) continue;
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const int n = j.b0 + c0 + i;
        if (n < p.N) p.D[(size_t)m * p.N + n] = __uint_as_float(v[i]);
      }
    }
  }
};

}  // namespace xmc
