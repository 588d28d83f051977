// Bandwidth-bound helper kernels around the GEMMs: embedding preparation, bucketing of the sparse
// positives by label tile, e4m3 -> bf16 weight staging, and the fixed-order final reductions.
#pragma once
#include "numerics.cuh"
#include "ptx.cuh"

namespace xmc {

// X [batch x d] (bf16 or e4m3) -> x8 [rows8 x d] e4m3, x16 [rows16 x d] bf16, xt [d x bpad] bf16.
// Rows/columns in [batch, bpad) are written as zero.  32x32 tiles through shared memory so that
// both the row-major and the transposed stores are coalesced.
template <bool IN_E4M3>
__global__ void prep_x_kernel(const void* __restrict__ x, int batch, int bpad, int d,
                              uint8_t* __restrict__ x8, __nv_bfloat16* __restrict__ x16,
                              __nv_bfloat16* __restrict__ xt, uint8_t* __restrict__ xt8) {
  __shared__ float tile[32][33];
  const int c0 = blockIdx.x * 32, b0 = blockIdx.y * 32;
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int b = b0 + i, c = c0 + threadIdx.x;
    float v = 0.f;
    if (b < batch && c < d) {
      if (IN_E4M3) {
        const uint8_t raw = reinterpret_cast<const uint8_t*>(x)[(size_t)b * d + c];
        v = e4m3x2_to_float2((uint16_t)raw).x;
      } else {
        v = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(x)[(size_t)b * d + c]);
      }
    }
    tile[i][threadIdx.x] = v;
    if (b < bpad && c < d) {
      if (x8 != nullptr) x8[(size_t)b * d + c] = (uint8_t)(float2_to_e4m3x2(v, 0.f) & 0xFFu);
      if (x16 != nullptr) x16[(size_t)b * d + c] = __float2bfloat16_rn(v);
    }
  }
  __syncthreads();
  if (xt != nullptr || xt8 != nullptr) {
    for (int i = threadIdx.y; i < 32; i += blockDim.y) {
      const int c = c0 + i, b = b0 + threadIdx.x;
      if (c < d && b < bpad) {
        if (xt != nullptr) xt[(size_t)c * bpad + b] = __float2bfloat16_rn(tile[threadIdx.x][i]);
        if (xt8 != nullptr) xt8[(size_t)c * bpad + b] = (uint8_t)(float2_to_e4m3x2(tile[threadIdx.x][i], 0.f) & 0xFFu);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Positives (row, global label id) -> buckets per 128-label tile, in launch order of the tiles.
// ---------------------------------------------------------------------------------------------
struct BucketGeom {
  long long label_offset;   // global id of the handle's row 0
  long long total_rows;
  long long rows_per_chunk; // rows of every bound weight chunk but the last
  int sched;                // labels per scheduling chunk (multiple of 128)
  int sched_per_chunk;      // cdiv(rows_per_chunk, sched)
  int n_buckets;
};

__device__ __forceinline__ bool bucket_of(const BucketGeom& g, int row, int col, int batch, int* status,
                                          int& bucket, int& lrow) {
  if (row < 0 || row >= batch || col < 0) {
    report(status, DEV_BAD_LABEL, row);
    return false;
  }
  const long long r = (long long)col - g.label_offset;
  if (r < 0 || r >= g.total_rows) return false;          // another shard's label
  const long long wc = r / g.rows_per_chunk;
  const int rr = (int)(r - wc * g.rows_per_chunk);
  const int sc = rr / g.sched;
  const int in = rr - sc * g.sched;
  bucket = ((int)wc * g.sched_per_chunk + sc) * (g.sched / 128) + (in >> 7);
  lrow = in & 127;
  return true;
}

__global__ void bucket_count_kernel(const int32_t* __restrict__ labels, long long nnz, int batch,
                                    BucketGeom g, int* __restrict__ count, int* status) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= nnz) return;
  int bucket, lrow;
  if (bucket_of(g, labels[2 * i], labels[2 * i + 1], batch, status, bucket, lrow))
    atomicAdd(&count[bucket], 1);
}

// exclusive scan of count[0..n) into off[0..n], single block
__global__ void bucket_scan_kernel(const int* __restrict__ count, int n, int* __restrict__ off) {
  __shared__ int warp_sum[32];
  __shared__ int carry;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int base = 0; base < n; base += blockDim.x) {
    const int i = base + threadIdx.x;
    const int v = i < n ? count[i] : 0;
    int s = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, s, o);
      if (lane >= o) s += t;
    }
    if (lane == 31) warp_sum[warp] = s;
    __syncthreads();
    if (warp == 0) {
      int w = lane < (int)(blockDim.x >> 5) ? warp_sum[lane] : 0;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, w, o);
        if (lane >= o) w += t;
      }
      warp_sum[lane] = w;
    }
    __syncthreads();
    const int before = carry + (warp > 0 ? warp_sum[warp - 1] : 0) + s - v;
    if (i < n) off[i] = before;
    __syncthreads();
    if (threadIdx.x == blockDim.x - 1) carry = before + v;
    __syncthreads();
  }
  if (threadIdx.x == 0) off[n] = carry;
}

__global__ void bucket_fill_kernel(const int32_t* __restrict__ labels, long long nnz, int batch,
                                   BucketGeom g, const int* __restrict__ off, int* __restrict__ cursor,
                                   uint32_t* __restrict__ entries) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= nnz) return;
  int bucket, lrow;
  const int row = labels[2 * i];
  if (bucket_of(g, row, labels[2 * i + 1], batch, nullptr, bucket, lrow)) {
    const int pos = atomicAdd(&cursor[bucket], 1);
    entries[off[bucket] + pos] = (uint32_t)row | ((uint32_t)lrow << 16);
  }
}

// Count, scan and fill in ONE launch of one 1024-thread block, for steps whose positives are few
// (the usual case: a few thousand pairs): three launches and a memset less per step.
// count[0..n) and cursor[0..n) need no prior clearing.
__global__ void __launch_bounds__(1024, 1)
bucket_all_kernel(const int32_t* __restrict__ labels, int nnz, int batch, BucketGeom g, int n,
                  int* count, int* cursor, int* off, uint32_t* __restrict__ entries, int* status) {
  __shared__ int warp_sum[32];
  __shared__ int carry;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    count[i] = 0;
    cursor[i] = 0;
  }
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < nnz; i += blockDim.x) {
    int bucket, lrow;
    if (bucket_of(g, labels[2 * i], labels[2 * i + 1], batch, status, bucket, lrow)) atomicAdd(&count[bucket], 1);
  }
  __syncthreads();
  // exclusive scan: every thread sums a contiguous run of buckets, one block-wide scan of the 1024
  // run totals, then each thread writes the offsets of its run
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int per = (n + (int)blockDim.x - 1) / (int)blockDim.x;
  const int beg = min(n, (int)threadIdx.x * per), end = min(n, beg + per);
  int run = 0;
  for (int i = beg; i < end; ++i) run += __ldcg(&count[i]);  // written by atomics: read at L2
  int s = run;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, s, o);
    if (lane >= o) s += t;
  }
  if (lane == 31) warp_sum[warp] = s;
  __syncthreads();
  if (warp == 0) {
    int w = warp_sum[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, w, o);
      if (lane >= o) w += t;
    }
    warp_sum[lane] = w;
  }
  __syncthreads();
  int before = (warp > 0 ? warp_sum[warp - 1] : 0) + s - run;
  for (int i = beg; i < end; ++i) {
    off[i] = before;
    before += __ldcg(&count[i]);
  }
  if (threadIdx.x == blockDim.x - 1) carry = before;        // the last thread's run ends at n (or is empty)
  __syncthreads();
  if (threadIdx.x == 0) off[n] = carry;
  __syncthreads();                                          // off[] written by this block is visible to it
  for (int i = threadIdx.x; i < nnz; i += blockDim.x) {
    int bucket, lrow;
    const int row = labels[2 * i];
    if (bucket_of(g, row, labels[2 * i + 1], batch, nullptr, bucket, lrow)) {
      const int pos = atomicAdd(&cursor[bucket], 1);
      entries[off[bucket] + pos] = (uint32_t)row | ((uint32_t)lrow << 16);
    }
  }
}

// Scale bookkeeping: one streaming pass over e4m3 weights (n16 groups of 16 bytes).
// counts[0] zeros, [1] sub-normal magnitudes (0 < |w| < 2^-6), [2] at +-448, [3] NaN; amax_bits = largest
// magnitude byte seen (e4m3 magnitudes order like their bytes).
__global__ void weight_stats_kernel(const uint4* __restrict__ w, long long n16, unsigned long long* counts,
                                    unsigned int* amax_bits) {
  unsigned int zeros = 0, sub = 0, sat = 0, nan = 0, amax = 0;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += stride) {
    const uint4 raw = w[i];
    const uint32_t ws[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const unsigned int m = (ws[k] >> (8 * b)) & 0x7Fu;
        zeros += m == 0u;
        sub += (m != 0u) & (m < 0x08u);
        sat += m == 0x7Eu;
        nan += m == 0x7Fu;
        amax = max(amax, m == 0x7Fu ? 0u : m);
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    zeros += __shfl_xor_sync(0xffffffffu, zeros, o);
    sub += __shfl_xor_sync(0xffffffffu, sub, o);
    sat += __shfl_xor_sync(0xffffffffu, sat, o);
    nan += __shfl_xor_sync(0xffffffffu, nan, o);
    amax = max(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  }
  if ((threadIdx.x & 31) == 0) {
    if (zeros) atomicAdd(&counts[0], (unsigned long long)zeros);
    if (sub) atomicAdd(&counts[1], (unsigned long long)sub);
    if (sat) atomicAdd(&counts[2], (unsigned long long)sat);
    if (nan) atomicAdd(&counts[3], (unsigned long long)nan);
    atomicMax(amax_bits, amax);
  }
}

// stored <- round(stored * factor) for a power-of-two factor (the per-tensor scale moves the other way).
// Growing is exact up to saturation at +-448; shrinking rounds what falls below the grid: to nearest, or
// stochastically with the step's Philox stream (counter = global element index / 8, as in the update).
__global__ void rescale_e4m3_kernel(uint2* __restrict__ w, long long n8, float factor, int stochastic,
                                    unsigned long long seed, unsigned long long step, unsigned long long elem0) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += stride) {
    const uint2 raw = w[i];
    const uint32_t rw[2] = {raw.x, raw.y};
    uint4 r = make_uint4(0u, 0u, 0u, 0u);
    if (stochastic) {
      const unsigned long long q = (elem0 >> 3) + (unsigned long long)i;
      r = philox4x32_sr(make_uint4((uint32_t)q, (uint32_t)(q >> 32), (uint32_t)step, (uint32_t)(step >> 32)),
                        make_uint2((uint32_t)seed, (uint32_t)(seed >> 32)));
    }
    const uint32_t rr[4] = {r.x, r.y, r.z, r.w};
    uint32_t ow[2] = {0u, 0u};
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      float v = e4m3x2_to_float2((uint16_t)(rw[e >> 2] >> (8 * (e & 3)))).x * factor;
      if (stochastic) v = sr_e4m3(v, (e & 1) ? (rr[e >> 1] >> 16) : (rr[e >> 1] & 0xFFFFu));
      ow[e >> 2] |= ((uint32_t)float2_to_e4m3x2(v, 0.f) & 0xFFu) << (8 * (e & 3));
    }
    w[i] = make_uint2(ow[0], ow[1]);
  }
}

// out[i] = bf16(sigmoid(in[i])) exactly as the forward epilogue computes it (test hook)
__global__ void sigmoid_probe_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = __float2bfloat16_rn(fast_sigmoid(__bfloat162float(in[i])));
}

// grad_X[b][c] = scale * sum_s partial[s][b][c], s ascending (fixed order)
__global__ void reduce_gradx_kernel(const float* __restrict__ partial, int n_splits, int batch, int bpad,
                                    int d, float scale, float* __restrict__ out32,
                                    __nv_bfloat16* __restrict__ out16) {
  const long long n = (long long)batch * d;
  const long long slot = (long long)bpad * d;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    float s = 0.f;
    for (int k = 0; k < n_splits; ++k) s += partial[k * slot + i];
    s *= scale;
    if (out32 != nullptr) out32[i] = s;
    if (out16 != nullptr) out16[i] = __float2bfloat16_rn(s);
  }
}

// State of the fused top-k before its first launch: empty lists, thresholds at -inf.
__global__ void topk_init_kernel(int* __restrict__ list_cnt, float* __restrict__ list_thr,
                                 float* __restrict__ list_max, int lists,
                                 unsigned int* __restrict__ row_thr, int rows) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < lists) {
    list_cnt[i] = 0;
    list_thr[i] = -INFINITY;
    list_max[i] = -INFINITY;
  }
  if (i < rows) row_thr[i] = 0x007FFFFFu;                // ordered key of -inf
}

// Selection over the candidate lists of one batch row.  One block per row.
// The row's lists are (CTA c with c % n_mtiles == row tile, the two epilogue warps of the row's TMEM
// quarter, lane).  A candidate becomes a 64-bit key: ordered value in the high word, ~label in the low
// word, so that a larger key means a larger value and, among equal values, the lower label; labels are
// unique, hence keys are.  The k-th largest key is found by a radix select, eight bits at a time (eight
// passes of a 256-bin histogram over the candidates that still match the digits chosen so far).
//   FINAL = false  mid-course pass between launches: publish the k-th best value seen so far as the row's
//                  threshold (nothing below it can end up among the k best), so that later launches
//                  append few candidates and rarely have to cut a list back;
//   FINAL = true   collect the k keys at or above the k-th, sort them, write (value desc, label asc).
// Candidates at or above the row's published threshold are first gathered into shared memory (key_cap
// keys); if they do not fit, every pass walks the lists in global memory instead.
__device__ __forceinline__ unsigned long long topk_key64(float v, int id) {
  const unsigned int bits = __float_as_uint(v);
  const unsigned int ord = (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
  return ((unsigned long long)ord << 32) | (unsigned long long)(0xFFFFFFFFu - (unsigned int)id);
}
template <bool FINAL>
__global__ void __launch_bounds__(256)
topk_select_kernel(const float* __restrict__ cand_val, const int* __restrict__ cand_idx, const int* __restrict__ list_cnt,
                   unsigned int* __restrict__ row_thr, int cap, int grid, int n_mtiles, int k, int batch,
                   long long label_offset, float* __restrict__ out_val, int* __restrict__ out_idx, int key_cap) {
  extern __shared__ unsigned long long sel_smem[];
  unsigned long long* keys = sel_smem;                   // [key_cap]
  unsigned long long* outk = sel_smem + key_cap;         // [128]
  __shared__ int hist[256];
  __shared__ int s_total, s_need, s_digit, s_nout;
  const int b = blockIdx.x;
  if (b >= batch) return;
  const int mt = b >> 7, q = (b >> 5) & 3, lane = b & 31;
  const int ctas = grid / n_mtiles;                     // CTAs that worked on this row's batch tile
  const int lists = ctas * 2;                           // two epilogue warps (column phases) per quarter
  const unsigned int tkey = row_thr[b];
  const float g = (tkey & 0x80000000u) ? __uint_as_float(tkey & 0x7FFFFFFFu) : __uint_as_float(~tkey);
  if (threadIdx.x == 0) { s_total = 0; s_nout = 0; }
  __syncthreads();
  auto list_of = [&](int r) {
    const int c = (r >> 1) * n_mtiles + mt, ph = r & 1;
    // epilogue warp slots 0..7 are warps 2..9; warp w owns quarter w & 3: slot -> quarter (slot + 2) & 3
    int slot = 4 * ph;
    for (int sl = 4 * ph; sl < 4 * ph + 4; ++sl)
      if (((sl + 2) & 3) == q) slot = sl;
    return (c * 8 + slot) * 32 + lane;
  };
  // visit every candidate at or above the published threshold, from the lists in global memory: a warp
  // per list, lanes along the list (coalesced)
  auto for_each_global = [&](auto&& f) {
    const int wid = threadIdx.x >> 5, ln = threadIdx.x & 31, nw = blockDim.x >> 5;
    for (int r = wid; r < lists; r += nw) {
      const int li = list_of(r);
      const size_t base = (size_t)li * (cap + 32);
      const int n = list_cnt[li];
      for (int e = ln; e < n; e += 32) {
        const float v = cand_val[base + e];
        if (v >= g) f(topk_key64(v, cand_idx[base + e]));
      }
    }
  };
  for_each_global([&](unsigned long long key) {
    const int at = atomicAdd(&s_total, 1);
    if (at < key_cap) keys[at] = key;
  });
  __syncthreads();
  const int total = s_total;
  const bool in_smem = total <= key_cap;
  auto for_each = [&](auto&& f) {
    if (in_smem) {
      for (int t = threadIdx.x; t < total; t += blockDim.x) f(keys[t]);
    } else {
      for_each_global(f);
    }
  };
  unsigned long long kth = 0ull;                         // every key is >= 0: with fewer than k candidates all are taken
  if (total > k) {
    unsigned long long prefix = 0ull, mask = 0ull;
    if (threadIdx.x == 0) s_need = k;
    for (int shift = 56; shift >= 0; shift -= 8) {
      hist[threadIdx.x] = 0;
      __syncthreads();
      for_each([&](unsigned long long key) {
        if ((key & mask) == prefix) atomicAdd(&hist[(int)((key >> shift) & 0xFFull)], 1);
      });
      __syncthreads();
      if (threadIdx.x == 0) {
        int need = s_need, d = 255;
        for (; d > 0; --d) {
          if (hist[d] >= need) break;
          need -= hist[d];
        }
        s_need = need;
        s_digit = d;
      }
      __syncthreads();
      prefix |= (unsigned long long)s_digit << shift;
      mask |= 0xFFull << shift;
    }
    kth = prefix;
  }
  if (!FINAL) {
    // the value part of the k-th best key is a valid lower bound of the row's final k-th value
    if (threadIdx.x == 0 && total >= k) atomicMax(&row_thr[b], (unsigned int)(kth >> 32));
    return;
  }
  for_each([&](unsigned long long key) {
    if (key >= kth) {
      const int at = atomicAdd(&s_nout, 1);
      if (at < 128) outk[at] = key;
    }
  });
  __syncthreads();
  const int n_out = min(s_nout, k);
  if (threadIdx.x < 128 && threadIdx.x >= n_out) outk[threadIdx.x] = 0ull;
  __syncthreads();
  // bitonic sort of 128 keys, descending
  for (int size = 2; size <= 128; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      if (threadIdx.x < 128) {
        const int i = threadIdx.x, j = i ^ stride;
        if (j > i) {
          const unsigned long long a = outk[i], c = outk[j];
          const bool desc = (i & size) == 0;
          if (desc ? a < c : a > c) { outk[i] = c; outk[j] = a; }
        }
      }
      __syncthreads();
    }
  }
  if (threadIdx.x < k) {
    const unsigned long long key = outk[threadIdx.x];
    if ((int)threadIdx.x < n_out) {
      const unsigned int ord = (unsigned int)(key >> 32);
      out_val[(size_t)b * k + threadIdx.x] = __uint_as_float((ord & 0x80000000u) ? (ord & 0x7FFFFFFFu) : ~ord);
      out_idx[(size_t)b * k + threadIdx.x] = (int)(label_offset + (long long)(0xFFFFFFFFu - (unsigned int)(key & 0xFFFFFFFFull)));
    } else {
      out_val[(size_t)b * k + threadIdx.x] = -INFINITY;
      out_idx[(size_t)b * k + threadIdx.x] = -1;
    }
  }
}

// loss = sum of n partials in index order, one thread (n is a few thousand at most)
__global__ void reduce_loss_kernel(const double* __restrict__ partial, int n, double* __restrict__ out) {
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    double s = 0.0;
    for (int i = 0; i < n; ++i) s += partial[i];
    *out = s;
  }
}

}  // namespace xmc
