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
                              __nv_bfloat16* __restrict__ xt) {
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
  if (xt != nullptr) {
    for (int i = threadIdx.y; i < 32; i += blockDim.y) {
      const int c = c0 + i, b = b0 + threadIdx.x;
      if (c < d && b < bpad) xt[(size_t)c * bpad + b] = __float2bfloat16_rn(tile[threadIdx.x][i]);
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

// e4m3 -> bf16 staging of one scheduling chunk of weights (exact); n16 = number of 16-byte groups
__global__ void e4m3_to_bf16_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, long long n16) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += stride) {
    const uint4 raw = src[i];
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
    uint32_t o[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float2 f = e4m3x2_to_float2((uint16_t)(w[k >> 1] >> (16 * (k & 1))));
      o[k] = pack_bf16x2(f.x, f.y);
    }
    dst[2 * i] = make_uint4(o[0], o[1], o[2], o[3]);
    dst[2 * i + 1] = make_uint4(o[4], o[5], o[6], o[7]);
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
      r = philox4x32_10(make_uint4((uint32_t)q, (uint32_t)(q >> 32), (uint32_t)step, (uint32_t)(step >> 32)),
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

// Final top-k of one batch row from the candidate lists of the top-k launches.  One block per row.
// The row's lists are (CTA c with c % n_mtiles == row tile, the two epilogue warps of the row's TMEM
// quarter, lane).  Candidates below the row's published threshold cannot be among the k best and are
// dropped while the rest is gathered into shared memory; then k rounds of "block-wide best remaining
// candidate" (value descending, id ascending).  If the gathered set does not fit, the rounds run over
// the lists in global memory instead.
constexpr int kTopkGather = 4096;
__global__ void __launch_bounds__(256)
topk_merge_kernel(const float* __restrict__ cand_val, int* __restrict__ cand_idx, const int* __restrict__ list_cnt,
                  const unsigned int* __restrict__ row_thr, int cap, int grid, int n_mtiles, int k, int batch,
                  long long label_offset, float* __restrict__ out_val, int* __restrict__ out_idx) {
  const int b = blockIdx.x;
  if (b >= batch) return;
  const int mt = b >> 7, q = (b >> 5) & 3, lane = b & 31;
  const int ctas = grid / n_mtiles;                     // CTAs that worked on this row's batch tile
  const int lists = ctas * 2;                           // two epilogue warps (column phases) per quarter
  __shared__ float g_val[kTopkGather];
  __shared__ int g_id[kTopkGather];
  __shared__ int g_n;
  __shared__ float s_val[8];
  __shared__ int s_pos[8];
  __shared__ int s_id[8];
  unsigned int key = row_thr[b];
  const float g = (key & 0x80000000u) ? __uint_as_float(key & 0x7FFFFFFFu) : __uint_as_float(~key);
  if (threadIdx.x == 0) g_n = 0;
  __syncthreads();
  auto list_of = [&](int r) {
    const int c = (r >> 1) * n_mtiles + mt, ph = r & 1;
    // epilogue warp slots 0..7 are warps 2..9; warp w owns quarter w & 3: slot -> quarter (slot + 2) & 3
    int slot = 4 * ph;
    for (int sl = 4 * ph; sl < 4 * ph + 4; ++sl)
      if (((sl + 2) & 3) == q) slot = sl;
    return (c * 8 + slot) * 32 + lane;
  };
  for (int r = threadIdx.x; r < lists; r += blockDim.x) {
    const int li = list_of(r);
    const int n = list_cnt[li];
    for (int e = 0; e < n; ++e) {
      const float v = cand_val[(size_t)li * (cap + 32) + e];
      if (v >= g) {
        const int at = atomicAdd(&g_n, 1);
        if (at < kTopkGather) {
          g_val[at] = v;
          g_id[at] = cand_idx[(size_t)li * (cap + 32) + e];
        }
      }
    }
  }
  __syncthreads();
  const int total = g_n;
  const bool in_smem = total <= kTopkGather;
  const int w = threadIdx.x >> 5, ln = threadIdx.x & 31;
  for (int round = 0; round < k; ++round) {
    float best = -INFINITY;
    int best_pos = -1, best_id = 0x7fffffff;
    if (in_smem) {
      for (int t = threadIdx.x; t < total; t += blockDim.x) {
        const float v = g_val[t];
        const int id = g_id[t];
        if (id >= 0 && (v > best || (v == best && id < best_id) || best_pos < 0)) { best = v; best_pos = t; best_id = id; }
      }
    } else {
      for (int r = threadIdx.x; r < lists; r += blockDim.x) {
        const int li = list_of(r);
        const int n = list_cnt[li];
        for (int e = 0; e < n; ++e) {
          const float v = cand_val[(size_t)li * (cap + 32) + e];
          const int id = cand_idx[(size_t)li * (cap + 32) + e];
          if (id >= 0 && (v > best || (v == best && id < best_id) || best_pos < 0)) { best = v; best_pos = li * (cap + 32) + e; best_id = id; }
        }
      }
    }
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int op = __shfl_xor_sync(0xffffffffu, best_pos, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_id, o);
      if (op >= 0 && (best_pos < 0 || ov > best || (ov == best && oi < best_id))) { best = ov; best_pos = op; best_id = oi; }
    }
    if (ln == 0) { s_val[w] = best; s_pos[w] = best_pos; s_id[w] = best_id; }
    __syncthreads();
    if (w == 0) {
      const int nw = blockDim.x >> 5;
      best = ln < nw ? s_val[ln] : -INFINITY;
      best_pos = ln < nw ? s_pos[ln] : -1;
      best_id = ln < nw ? s_id[ln] : 0x7fffffff;
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int op = __shfl_xor_sync(0xffffffffu, best_pos, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_id, o);
        if (op >= 0 && (best_pos < 0 || ov > best || (ov == best && oi < best_id))) { best = ov; best_pos = op; best_id = oi; }
      }
      if (ln == 0) {
        out_val[(size_t)b * k + round] = best_pos >= 0 ? best : -INFINITY;
        out_idx[(size_t)b * k + round] = best_pos >= 0 ? (int)(label_offset + best_id) : -1;
        if (best_pos >= 0) {                                              // consumed
          if (in_smem) g_id[best_pos] = -1;
          else cand_idx[best_pos] = -1;
        }
      }
    }
    __syncthreads();
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
