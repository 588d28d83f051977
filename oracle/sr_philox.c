/* TEST INFRASTRUCTURE ONLY -- C restatement of the stochastic-rounding definitions of
 * oracle/xmc_oracle.py (sr_e4m3_exact, sr_bf16) and oracle/philox.py (sr_bits16), so that the
 * CPU baseline is not dominated by numpy's Philox.  tests/test_oracle_philox.py checks that
 * this file and the numpy statements agree bit for bit.
 *
 * Philox4x32: Salmon et al., "Parallel random numbers: as easy as 1, 2, 3" (SC'11).
 * Build: gcc -O3 -fopenmp -shared -fPIC -o oracle/_build/liboracle_sr.so oracle/sr_philox.c
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

#define SR_ROUNDS 7   /* as oracle/philox.py: the library's stream stops Philox4x32 after seven rounds */
static inline void philox4x32_sr(uint32_t c[4], uint32_t k0, uint32_t k1) {
  for (int r = 0; r < SR_ROUNDS; ++r) {
    const uint64_t p0 = (uint64_t)0xD2511F53u * c[0];
    const uint64_t p1 = (uint64_t)0xCD9E8D57u * c[2];
    const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c[1] ^ k0;
    const uint32_t n2 = (uint32_t)(p0 >> 32) ^ c[3] ^ k1;
    c[1] = (uint32_t)p1;
    c[3] = (uint32_t)p0;
    c[0] = n0;
    c[2] = n2;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
}

static inline uint32_t bits16(uint64_t elem, uint64_t seed, uint64_t step) {
  const uint64_t q = elem >> 3;
  uint32_t c[4] = {(uint32_t)q, (uint32_t)(q >> 32), (uint32_t)step, (uint32_t)(step >> 32)};
  philox4x32_sr(c, (uint32_t)seed, (uint32_t)(seed >> 32));
  const int j = (int)(elem & 7);
  return (c[j >> 1] >> (16 * (j & 1))) & 0xFFFFu;
}

static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

/* out[i] = r16 of element first_elem + i */
void oracle_sr_bits16(uint64_t first_elem, uint64_t n, uint64_t seed, uint64_t step, uint32_t* out) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < (int64_t)n; ++i) out[i] = bits16(first_elem + (uint64_t)i, seed, step);
}

/* exact stochastic rounding onto the e4m3 grid (subnormals included), result as float */
void oracle_sr_e4m3(const float* w, uint64_t n, uint64_t first_elem, uint64_t seed, uint64_t step, float* out) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < (int64_t)n; ++i) {
    const float x = w[i];
    if (x != x) { out[i] = x; continue; }
    const uint32_t r = bits16(first_elem + (uint64_t)i, seed, step);
    float a = fminf(fabsf(x), 448.0f);
    const int small = a < 0.015625f;
    float y = small ? a + 0.015625f : a;
    y = u2f((f2u(y) + (r << 4)) & 0xFFF00000u);
    if (small) y -= 0.015625f;
    y = fminf(y, 448.0f);
    out[i] = copysignf(y, x);                         /* the sign is kept, also for a zero result */
  }
}

/* stochastic rounding onto the bf16 grid, result as float */
void oracle_sr_bf16(const float* w, uint64_t n, uint64_t first_elem, uint64_t seed, uint64_t step, float* out) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < (int64_t)n; ++i) {
    const uint32_t r = bits16(first_elem + (uint64_t)i, seed, step);
    out[i] = u2f((f2u(w[i]) + r) & 0xFFFF0000u);
  }
}
