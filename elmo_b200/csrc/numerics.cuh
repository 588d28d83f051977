// Element arithmetic shared by the epilogues: bf16/e4m3 conversions with the reference's
// intermediate roundings, sigmoid / BCE terms, the Philox4x32 stream and rounding of the updated weight.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <stdint.h>

namespace xmc {

__device__ __forceinline__ float bf16_round(float x) {
  return __bfloat162float(__float2bfloat16_rn(x));
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float bf16_bits_to_float(uint32_t b16) { return __uint_as_float(b16 << 16); }

// two e4m3 bytes (low byte first) -> two floats, exact
__device__ __forceinline__ float2 e4m3x2_to_float2(uint16_t v) {
  __half2_raw h = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)v, __NV_E4M3);
  return __half22float2(*reinterpret_cast<__half2*>(&h));
}
// two floats -> two e4m3 bytes (x in the low byte), round-to-nearest-even, saturating at +-448
__device__ __forceinline__ uint16_t float2_to_e4m3x2(float x, float y) {
  return (uint16_t)__nv_cvt_float2_to_fp8x2(make_float2(x, y), __NV_SATFINITE, __NV_E4M3);
}

// sigmoid(z) = 1 / (1 + 2^(-z log2 e)) with the two approximate special-function ops (relative error
// ~2^-22, far below the bf16 rounding that follows).
__device__ __forceinline__ float fast_sigmoid(float z) {
  float e, r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(z * -1.4426950408889634f));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
  return r;
}
// max(z,0) + log(1 + exp(-|z|)): the label-independent part of BCE-with-logits (chunked.py:57-72)
__device__ __forceinline__ float bce_softplus(float z) {
  return fmaxf(z, 0.0f) + log1pf(__expf(-fabsf(z)));
}

// ---------------------------------------------------------------------------------------------
// Philox4x32 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3", SC'11) with kSrRounds = 7
// rounds: the round function and key schedule of Philox4x32-10, stopped after the seventh round -- the
// smallest round count its authors report as passing BigCrush (ten is their default margin; the rounds
// are a quarter of the update epilogue's instructions, and the bits only dither a rounding).  One call
// serves 8 consecutive weight elements with 16 bits each: counter = (q_lo, q_hi, step_lo, step_hi),
// q = global element index / 8, key = (seed_lo, seed_hi); element j takes half (j & 1) of output word
// (j >> 1).
// ---------------------------------------------------------------------------------------------
constexpr int kSrRounds = 7;
__device__ __forceinline__ uint4 philox4x32_sr(uint4 c, uint2 k) {
  constexpr uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
  for (int r = 0; r < kSrRounds; ++r) {
    const unsigned long long p0 = (unsigned long long)M0 * c.x;
    const unsigned long long p1 = (unsigned long long)M1 * c.z;
    c = make_uint4((uint32_t)(p1 >> 32) ^ c.y ^ k.x, (uint32_t)p1, (uint32_t)(p0 >> 32) ^ c.w ^ k.y, (uint32_t)p0);
    k.x += W0;
    k.y += W1;
  }
  return c;
}

// Exact stochastic rounding of fp32 w onto the e4m3 grid (subnormals included) with 16 random
// bits; returns a float that lies on the grid (or beyond +-448: the saturating e4m3 conversion
// that follows clamps it).  The sign is kept, also for a zero result; NaN propagates.
//
// The reference's bit trick (fuse_kernel.py:28-36) adds the random bits into the 20 mantissa bits
// an e4m3 normal discards and truncates; below 2^-6 the e4m3 grid is uniform (step 2^-9) and the
// trick no longer sees it.  Scaling by 2^-120 first maps e4m3's smallest normal onto fp32's
// (2^-126): e4m3 subnormals become fp32 subnormals, whose bit pattern is fixed point with bit 20
// worth exactly one e4m3 step, so ONE add-and-mask is exact stochastic rounding on the whole grid,
// carries from the subnormal into the normal range included.  Both scalings are exact (the first
// rounds only below 2^-149, i.e. 2^-29 before scaling).  Needs fp32 denormals (no -ftz).
constexpr float kSrDown = 7.52316384526264005e-37f;   // 2^-120
constexpr float kSrUp = 1.32922799578491587e+36f;     // 2^120
__device__ __forceinline__ float sr_e4m3_finite(float w, uint32_t r16) {
  const uint32_t b = (__float_as_uint(w * kSrDown) + (r16 << 4)) & 0xFFF00000u;
  return __uint_as_float(b) * kSrUp;
}
__device__ __forceinline__ float sr_e4m3(float w, uint32_t r16) {
  const float y = sr_e4m3_finite(w, r16);               // +-Inf stays +-Inf; a NaN pattern may wrap
  return w != w ? w : y;
}
// Stochastic rounding onto the bf16 grid: add 16 random bits below the kept mantissa, truncate
// (fuse_kernel.py:10-17).  Returns the bf16 bit pattern.
__device__ __forceinline__ uint32_t sr_bf16_bits(float w, uint32_t r16) {
  return (__float_as_uint(w) + r16) >> 16;
}

// four e4m3 bytes -> four bf16 (two packed words), exact, integer/FMA pipes only.
// (b & 0x7f) << 4 placed in a bf16 is the value times 2^-120, subnormals included; one packed
// multiply by 2^120 restores it.
__device__ __forceinline__ void e4m3x4_to_bf16x4(uint32_t w, uint32_t& lo, uint32_t& hi) {
  const uint32_t t0 = __byte_perm(w, 0u, 0x1404);     // b1 << 24 | b0 << 8
  const uint32_t t1 = __byte_perm(w, 0u, 0x3424);     // b3 << 24 | b2 << 8
  const uint32_t x0 = (t0 & 0x80008000u) | ((t0 >> 4) & 0x07F007F0u);
  const uint32_t x1 = (t1 & 0x80008000u) | ((t1 >> 4) & 0x07F007F0u);
  const uint32_t scale = 0x7B807B80u;                 // bf16x2 (2^120, 2^120)
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(lo) : "r"(x0), "r"(scale));
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(hi) : "r"(x1), "r"(scale));
}

}  // namespace xmc
