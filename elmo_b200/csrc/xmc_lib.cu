// C ABI of the chunked XMC classifier layer (see include/elmo_xmc.h): handle, workspaces, TMA
// descriptors and the per-step launch schedule.
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "../../include/elmo_xmc.h"
#include "aux_kernels.cuh"
#include "gemm_engine.cuh"
#include "gradx_kernel.cuh"
#include "xmc_policies.cuh"

namespace {

thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

#define CU_TRY(expr)                                                                         \
  do {                                                                                       \
    cudaError_t e_ = (expr);                                                                 \
    if (e_ != cudaSuccess)                                                                   \
      return fail(XMC_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e_), __FILE__, __LINE__); \
  } while (0)

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                              CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                              CUtensorMapFloatOOBfill);

int get_encode(EncodeFn* out) {
  static EncodeFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    CU_TRY(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q));
    if (p == nullptr || q != cudaDriverEntryPointSuccess)
      return fail(XMC_ERR_CUDA, "cuTensorMapEncodeTiled is not available in this driver");
    fn = reinterpret_cast<EncodeFn>(p);
  }
  *out = fn;
  return XMC_OK;
}

// Encoding a tensor map costs a few microseconds on the host and a step needs ~26 of them with
// arguments that repeat every step, so encoded maps are remembered (per thread, direct-mapped).
struct MapKey {
  uint64_t base, a, b, c;
  uint32_t kind, e4m3, box0, box1, swizzle, pad;
  bool operator==(const MapKey& o) const { return memcmp(this, &o, sizeof(MapKey)) == 0; }
};
struct MapSlot {
  MapKey key;
  CUtensorMap map;
  bool used = false;
};
constexpr int kMapSlots = 512;
inline MapSlot* map_slot(const MapKey& k) {
  static thread_local MapSlot slots[kMapSlots];
  uint64_t h = k.base * 0x9E3779B97F4A7C15ull ^ (k.a * 0xC2B2AE3D27D4EB4Full) ^ (k.b << 17) ^ (k.c << 3) ^
               ((uint64_t)k.kind << 60) ^ ((uint64_t)k.box1 << 40) ^ ((uint64_t)k.box0 << 50) ^ k.e4m3 ^ ((uint64_t)k.swizzle << 1);
  h ^= h >> 29;
  return &slots[h % kMapSlots];
}

// 2-D row-major tensor [outer x inner], box [box_outer x box_inner], 128-byte swizzle, zero fill.
int make_map(CUtensorMap* m, bool e4m3, const void* base, uint64_t inner, uint64_t outer,
             uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer, bool swizzle = true) {
  EncodeFn enc;
  if (int rc = get_encode(&enc)) return rc;
  if (((uintptr_t)base & 15u) != 0 || (row_stride_bytes & 15u) != 0)
    return fail(XMC_ERR_INVALID, "tensor base/stride must be 16-byte aligned (base %p, stride %llu)", base,
                (unsigned long long)row_stride_bytes);
  MapKey key;
  memset(&key, 0, sizeof(key));
  key.base = (uint64_t)(uintptr_t)base; key.a = inner; key.b = outer; key.c = row_stride_bytes;
  key.kind = 2; key.e4m3 = e4m3; key.box0 = box_inner; key.box1 = box_outer; key.swizzle = swizzle;
  MapSlot* slot = map_slot(key);
  if (slot->used && slot->key == key) {
    *m = slot->map;
    return XMC_OK;
  }
  const cuuint64_t dims[2] = {inner, outer};
  const cuuint64_t strides[1] = {row_stride_bytes};
  const cuuint32_t box[2] = {box_inner, box_outer};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(m, e4m3 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                         const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         swizzle ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(XMC_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d): inner %llu outer %llu stride %llu box %ux%u",
                (int)r, (unsigned long long)inner, (unsigned long long)outer,
                (unsigned long long)row_stride_bytes, box_inner, box_outer);
  slot->key = key;
  slot->map = *m;
  slot->used = true;
  return XMC_OK;
}
// [rows x cols] row-major matrix seen as [cols/64 blocks][rows][64 elements]: one box fetches
// `box_rows` rows of `box_blocks` consecutive 64-element blocks, laid out block after block in shared memory
// (each block = box_rows rows of 64 elements).  Blocks/rows outside the matrix read as zero.
int make_map_blocked(CUtensorMap* m, bool e4m3, const void* base, uint64_t cols, uint64_t rows,
                     uint64_t row_stride_elems, uint32_t box_rows, bool swizzle, uint32_t box_blocks = 4) {
  EncodeFn enc;
  if (int rc = get_encode(&enc)) return rc;
  const uint32_t es = e4m3 ? 1 : 2;
  if (cols % 64 != 0) return fail(XMC_ERR_INVALID, "blocked tensor map needs a multiple of 64 columns, got %llu", (unsigned long long)cols);
  if (((uintptr_t)base & 15u) != 0 || ((row_stride_elems * es) & 15u) != 0)
    return fail(XMC_ERR_INVALID, "tensor base/stride must be 16-byte aligned");
  MapKey key;
  memset(&key, 0, sizeof(key));
  key.base = (uint64_t)(uintptr_t)base; key.a = cols; key.b = rows; key.c = row_stride_elems;
  key.kind = 3; key.e4m3 = e4m3; key.box0 = 64; key.box1 = box_rows; key.swizzle = swizzle; key.pad = box_blocks;
  MapSlot* slot = map_slot(key);
  if (slot->used && slot->key == key) {
    *m = slot->map;
    return XMC_OK;
  }
  const cuuint64_t dims[3] = {64, rows, cols / 64};
  const cuuint64_t strides[2] = {row_stride_elems * es, 64ull * es};
  const cuuint32_t box[3] = {64, box_rows, box_blocks};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = enc(m, e4m3 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3,
                         const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         swizzle ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(XMC_ERR_CUDA, "cuTensorMapEncodeTiled (blocked) failed (%d): cols %llu rows %llu stride %llu",
                (int)r, (unsigned long long)cols, (unsigned long long)rows, (unsigned long long)row_stride_elems);
  slot->key = key;
  slot->map = *m;
  slot->used = true;
  return XMC_OK;
}
// operand whose K runs along the rows' contiguous direction
int make_map_kmajor(CUtensorMap* m, bool e4m3, const void* base, uint64_t k_elems, uint64_t rows,
                    uint64_t row_stride_elems, uint32_t box_rows) {
  const uint32_t es = e4m3 ? 1 : 2;
  return make_map(m, e4m3, base, k_elems, rows, row_stride_elems * es, 128 / es, box_rows);
}
// e4m3 rows [rows x k_bytes] fetched raw, 64 bytes (one bf16 k-step) of `box_rows` rows per box, for the
// in-kernel conversion to a bf16 operand
int make_map_raw8(CUtensorMap* m, const void* base, uint64_t k_bytes, uint64_t rows, uint64_t row_stride_bytes,
                  uint32_t box_rows) {
  return make_map(m, true, base, k_bytes, rows, row_stride_bytes, 64, box_rows, false);
}
// bf16 operand stored [k_rows x mn] (MN contiguous): boxes of box_rows k-rows x 64 elements
int make_map_mnmajor(CUtensorMap* m, const void* base, uint64_t mn, uint64_t k_rows,
                     uint64_t row_stride_elems, uint32_t box_rows = 64) {
  return make_map(m, false, base, mn, k_rows, row_stride_elems * 2, 64, box_rows);
}

// Launch with programmatic stream serialization: the kernel may be scheduled while its predecessor in
// the stream drains; it orders itself with griddepcontrol.wait before its first global access.
// cluster > 1 launches thread-block clusters of that many CTAs along x.
inline void launch_config(cudaLaunchConfig_t* cfg, cudaLaunchAttribute* at, int grid, int block, size_t smem,
                          cudaStream_t stream, int cluster) {
  memset(cfg, 0, sizeof(*cfg));
  cfg->gridDim = dim3((unsigned)grid);
  cfg->blockDim = dim3((unsigned)block);
  cfg->dynamicSmemBytes = smem;
  cfg->stream = stream;
  static const bool no_pdl = getenv("XMC_NO_PDL") != nullptr;
  int n = 0;
  if (!no_pdl) {
    at[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  if (cluster > 1) {
    at[n].id = cudaLaunchAttributeClusterDimension;
    at[n].val.clusterDim.x = (unsigned)cluster;
    at[n].val.clusterDim.y = 1;
    at[n].val.clusterDim.z = 1;
    ++n;
  }
  cfg->attrs = at;
  cfg->numAttrs = n;
}
template <class Kern, class... Args>
cudaError_t launch_pdl(Kern kern, int grid, int block, size_t smem, cudaStream_t stream, const Args&... args) {
  cudaLaunchConfig_t cfg;
  cudaLaunchAttribute at[2];
  launch_config(&cfg, at, grid, block, smem, stream, 1);
  return cudaLaunchKernelEx(&cfg, kern, args...);
}

// dynamic shared memory opt-in of the grad_X kernels, once per device; *max_pairs = CTA pairs of the pair
// kernel the device holds at once
int gradx_configure(int sm_count, int* max_pairs) {
  static std::atomic<uint64_t> configured{0};
  static std::atomic<int> pairs[64];
  int dev = 0;
  CU_TRY(cudaGetDevice(&dev));
  if (!((configured.load(std::memory_order_acquire) >> (dev & 63)) & 1ull)) {
    CU_TRY(cudaFuncSetAttribute(xmc::gradx_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, xmc::kGxSmemBytes<false>));
    CU_TRY(cudaFuncSetAttribute(xmc::gradx_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, xmc::kGxSmemBytes<false>));
    CU_TRY(cudaFuncSetAttribute(xmc::gradx_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, xmc::kGxSmemBytes<true>));
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute at[2];
    launch_config(&cfg, at, sm_count / 2 * 2, xmc::kGxThreads, xmc::kGxSmemBytes<true>, nullptr, 2);
    int n = 0;
    CU_TRY(cudaOccupancyMaxActiveClusters(&n, xmc::gradx_kernel<true, true>, &cfg));
    pairs[dev & 63].store(std::max(0, std::min(n, sm_count / 2)), std::memory_order_relaxed);
    configured.fetch_or(1ull << (dev & 63), std::memory_order_release);
  }
  *max_pairs = pairs[dev & 63].load(std::memory_order_relaxed);
  return XMC_OK;
}

// PAIR: the kernel runs on CTA pairs (clusters of two); n_tiles then counts the pairs' 256-row tiles and
// the grid is twice the number of pairs the device can hold at once (asked of the occupancy calculator:
// an SM that has no partner within its GPC cannot take part).
template <class Policy, bool PAIR = false>
int launch_gemm(const CUtensorMap& a, const CUtensorMap& b, const typename Policy::Params& p, int n_tiles,
                int sm_count, cudaStream_t stream, int grid_override = 0, const CUtensorMap* c = nullptr) {
  if (n_tiles <= 0) return XMC_OK;
  auto kern = xmc::gemm_kernel<Policy, PAIR>;
  constexpr int smem = xmc::smem_bytes<Policy, PAIR>();
  constexpr int block = xmc::block_threads<Policy>();
  // once per device and kernel (one process may drive several devices)
  static std::atomic<uint64_t> configured{0};
  static std::atomic<int> max_pairs[64];
  int dev = 0;
  CU_TRY(cudaGetDevice(&dev));
  if (!((configured.load(std::memory_order_acquire) >> (dev & 63)) & 1ull)) {
    CU_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    if (PAIR) {
      cudaLaunchConfig_t cfg;
      cudaLaunchAttribute at[2];
      launch_config(&cfg, at, sm_count / 2 * 2, block, smem, stream, 2);
      int n = 0;
      CU_TRY(cudaOccupancyMaxActiveClusters(&n, kern, &cfg));
      if (n <= 0) return fail(XMC_ERR_CUDA, "the device cannot hold a pair of CTAs of this kernel");
      max_pairs[dev & 63].store(std::min(n, sm_count / 2), std::memory_order_relaxed);
    }
    configured.fetch_or(1ull << (dev & 63), std::memory_order_release);
  }
  if (Policy::kCTile && c == nullptr) return fail(XMC_ERR_STATE, "this kernel needs its epilogue-input tensor map");
  cudaLaunchConfig_t cfg;
  cudaLaunchAttribute at[2];
  int grid;
  if (PAIR) grid = 2 * (grid_override > 0 ? grid_override : std::min(n_tiles, max_pairs[dev & 63].load(std::memory_order_relaxed)));
  else grid = grid_override > 0 ? grid_override : std::min(n_tiles, sm_count);
  launch_config(&cfg, at, grid, block, smem, stream, PAIR ? 2 : 1);
  CU_TRY(cudaLaunchKernelEx(&cfg, kern, a, b, c ? *c : a, p));
  return XMC_OK;
}

inline int cdiv(long long a, long long b) { return (int)((a + b - 1) / b); }
inline long long round_up(long long a, long long b) { return (a + b - 1) / b * b; }

}  // namespace

struct xmc_handle {
  xmc_config cfg{};
  int sm_count = 0;
  int bpad_max = 0;
  int sched = 0;                   // labels per scheduling chunk in use (set when the weights are bound)
  int sched_cfg = 0;               // the configured / automatic value
  int64_t g_rows = 0;              // rows of G currently allocated
  std::vector<void*> w_ptrs;
  std::vector<int64_t> w_rows;
  int64_t total_rows = 0;
  int64_t rows_per_chunk = 0;
  int n_buckets = 0;
  // workspaces
  uint8_t* x8 = nullptr;           // [max(bpad_max,256) x d] e4m3
  __nv_bfloat16* x16 = nullptr;    // [max(bpad_max,256) x d]
  __nv_bfloat16* xt = nullptr;     // [max(d,256) x bpad_max]
  __nv_bfloat16* G = nullptr;      // [sched x bpad_max]
  uint8_t* G8 = nullptr;           // [sched x bpad_max] e4m3(G * 256), allocated when the FP8 dW contraction is first asked for
  uint8_t* xt8 = nullptr;          // [max(d,256) x bpad_max] e4m3 X transposed, likewise
  int64_t g8_rows = 0;
  float* partial = nullptr;
  int64_t partial_floats = 0;
  int* bucket_cnt = nullptr;       // [2 * n_buckets] counts then cursors
  int* bucket_off = nullptr;       // [n_buckets + 1]
  uint32_t* entries = nullptr;
  int64_t ent_cap = 0;
  double* loss_partial = nullptr;
  int64_t loss_cap = 0;
  int* status = nullptr;           // 4 ints
  unsigned long long* stats = nullptr;   // weight statistics: 4 counters + the largest magnitude byte
  int64_t ws_bytes = 0;
  // bookkeeping for the bench: kernels launched so far, optional per-kernel-class event timing
  float* topk_val = nullptr;       // candidate lists of the fused top-k (grown on demand)
  int* topk_idx = nullptr;
  int64_t topk_cap = 0;            // entries
  int* topk_cnt = nullptr;         // per list: entries in use
  float* topk_thr = nullptr;       // per list: own threshold
  float* topk_max = nullptr;       // per list: largest value held so far
  unsigned int* topk_row = nullptr;  // per batch row: published threshold (ordered key)
  int topk_lists = 0;
  void* kahan = nullptr;           // borrowed compensation buffer for the first kahan_rows rows
  int64_t kahan_rows = 0;
  int kahan_e5m2 = 0;
  int64_t l2_persist_bytes = 0;    // size of the persisting-L2 carve-out this process asked for (0 = none)
  int64_t launches = 0;
  bool profile = false;
  std::vector<cudaEvent_t> ev_pool;
  std::vector<int> ev_kind;        // kind of the kernel that FOLLOWS event i
  size_t ev_used = 0;
};

namespace {

int dev_alloc(xmc_handle* h, void** p, size_t bytes, bool zero) {
  CU_TRY(cudaMalloc(p, bytes));
  if (zero) CU_TRY(cudaMemset(*p, 0, bytes));
  h->ws_bytes += (int64_t)bytes;
  return XMC_OK;
}

struct DeviceGuard {
  int prev = -1;
  explicit DeviceGuard(int dev) {
    cudaGetDevice(&prev);
    if (prev != dev) cudaSetDevice(dev);
  }
  ~DeviceGuard() {
    int cur = -1;
    cudaGetDevice(&cur);
    if (prev >= 0 && cur != prev) cudaSetDevice(prev);
  }
};

// Count a kernel launch; in profile mode also drop an event in front of it.
enum { K_PREP = 0, K_UNUSED = 1, K_FWD = 2, K_GRADX = 3, K_UPD = 4, K_REDUCE = 5, K_LOGITS = 6, K_END = 7 };
void mark(xmc_handle* h, int kind, cudaStream_t st) {
  if (kind != K_END) ++h->launches;
  if (!h->profile) return;
  if (h->ev_used == h->ev_pool.size()) {
    cudaEvent_t e;
    if (cudaEventCreate(&e) != cudaSuccess) return;
    h->ev_pool.push_back(e);
    h->ev_kind.push_back(kind);
  }
  h->ev_kind[h->ev_used] = kind;
  cudaEventRecord(h->ev_pool[h->ev_used], st);
  ++h->ev_used;
}

xmc::BucketGeom geom_of(const xmc_handle* h) {
  xmc::BucketGeom g;
  g.label_offset = h->cfg.label_offset;
  g.total_rows = h->total_rows;
  g.rows_per_chunk = h->rows_per_chunk;
  g.sched = h->sched;
  g.sched_per_chunk = cdiv(h->rows_per_chunk, h->sched);
  g.n_buckets = h->n_buckets;
  return g;
}

int prep_x(xmc_handle* h, const void* x, int x_dtype, int batch, int bpad, bool need_x8, bool need_x16,
           bool need_xt, cudaStream_t st, bool need_xt8 = false) {
  const int d = h->cfg.dim;
  dim3 grid(cdiv(d, 32), cdiv(bpad, 32)), block(32, 8);
  mark(h, K_PREP, st);
  if (x_dtype == XMC_DT_E4M3)
    xmc::prep_x_kernel<true><<<grid, block, 0, st>>>(x, batch, bpad, d, need_x8 ? h->x8 : nullptr,
                                                     need_x16 ? h->x16 : nullptr, need_xt ? h->xt : nullptr,
                                                     need_xt8 ? h->xt8 : nullptr);
  else
    xmc::prep_x_kernel<false><<<grid, block, 0, st>>>(x, batch, bpad, d, need_x8 ? h->x8 : nullptr,
                                                      need_x16 ? h->x16 : nullptr, need_xt ? h->xt : nullptr,
                                                      need_xt8 ? h->xt8 : nullptr);
  CU_TRY(cudaGetLastError());
  return XMC_OK;
}

}  // namespace

extern "C" {

const char* xmc_last_error(void) { return g_err; }
const char* xmc_version(void) { return "elmo_xmc sm_100a " __DATE__; }

int xmc_create(const xmc_config* cfg, xmc_handle** out) {
  if (cfg == nullptr || out == nullptr) return fail(XMC_ERR_INVALID, "null argument");
  *out = nullptr;
  if (cfg->dim <= 0 || cfg->dim % 64 != 0) return fail(XMC_ERR_INVALID, "dim must be a positive multiple of 64, got %d", cfg->dim);
  if (cfg->max_batch <= 0 || cfg->max_batch > 65535) return fail(XMC_ERR_INVALID, "max_batch must be in [1, 65535], got %d", cfg->max_batch);
  if (cfg->mode < XMC_MODE_BF16 || cfg->mode > XMC_MODE_SIMFP8) return fail(XMC_ERR_INVALID, "unknown mode %d", cfg->mode);
  if (!(cfg->w_scale > 0.f)) return fail(XMC_ERR_INVALID, "w_scale must be positive");
  if (cfg->sched_labels < 0 || cfg->sched_labels % 128 != 0) return fail(XMC_ERR_INVALID, "sched_labels must be a multiple of 128");
  int ndev = 0;
  CU_TRY(cudaGetDeviceCount(&ndev));
  if (cfg->device < 0 || cfg->device >= ndev) return fail(XMC_ERR_INVALID, "device %d out of range (%d devices)", cfg->device, ndev);
  DeviceGuard guard(cfg->device);
  cudaDeviceProp prop;
  CU_TRY(cudaGetDeviceProperties(&prop, cfg->device));
  if (prop.major != 10) return fail(XMC_ERR_CUDA, "device %d is sm_%d%d; this library holds sm_100a code only", cfg->device, prop.major, prop.minor);

  xmc_handle* h = new xmc_handle();
  h->cfg = *cfg;
  h->sm_count = prop.multiProcessorCount;
  h->bpad_max = (int)round_up(cfg->max_batch, 64);
  if (cfg->sched_labels > 0) {
    h->sched = (int)cfg->sched_labels;
  } else {
    // Labels per scheduling chunk: as many as the reference chunk allows (fewer, longer launches
    // amortise the per-launch ramp), bounded so that one chunk of G (sched x bpad bf16) stays <= 128 MB.
    long long s = (128ll << 20) / ((long long)h->bpad_max * 2);
    s = std::max(1024ll, std::min(s, 65536ll));
    h->sched = (int)(s / 128 * 128);
  }
  h->sched_cfg = h->sched;
  const int d = cfg->dim;
  int rc = XMC_OK;
  auto A = [&](void** p, size_t bytes, bool zero) { if (rc == XMC_OK) rc = dev_alloc(h, p, bytes, zero); };
  const size_t xrows = (size_t)std::max(h->bpad_max, 256);
  A((void**)&h->x8, xrows * d, true);
  A((void**)&h->x16, xrows * d * 2, true);
  A((void**)&h->xt, (size_t)std::max(d, 256) * h->bpad_max * 2, true);
  // G (and the bf16 staging copy of the simulated-FP8 forward) are sized when the weights are bound:
  // they never need more rows than the largest weight chunk.
  h->partial_floats = std::max<int64_t>((int64_t)h->sm_count * 256 * 256, (int64_t)h->bpad_max * round_up(d, 256));
  A((void**)&h->partial, (size_t)h->partial_floats * 4, true);
  A((void**)&h->status, 4 * sizeof(int), true);
  h->ent_cap = std::max<int64_t>(4096, (int64_t)cfg->max_batch * 64);
  A((void**)&h->entries, (size_t)h->ent_cap * 4, false);
  if (rc != XMC_OK) {
    xmc_destroy(h);
    return rc;
  }
  // L2 carve-out for the partial sums: cudaLimitPersistingL2CacheSize is a limit of the whole CUDA
  // context, so other kernels of the process see that much less L2 while it is set (documented in the
  // header; XMC_NO_L2_PERSIST=1 in the environment leaves the limit alone)
  if (getenv("XMC_NO_L2_PERSIST") == nullptr && prop.persistingL2CacheMaxSize > 0) {
    const size_t want = std::min<size_t>((size_t)h->partial_floats * 4, (size_t)prop.persistingL2CacheMaxSize);
    if (cudaDeviceSetLimit(cudaLimitPersistingL2CacheSize, want) == cudaSuccess) h->l2_persist_bytes = (int64_t)want;
    else cudaGetLastError();
  }
  *out = h;
  return XMC_OK;
}

int xmc_destroy(xmc_handle* h) {
  if (h == nullptr) return XMC_OK;
  DeviceGuard guard(h->cfg.device);
  if (h->l2_persist_bytes > 0) cudaCtxResetPersistingL2Cache();   // lines pinned for the partial sums become normal again
  void* ptrs[] = {h->x8, h->x16, h->xt, h->G, h->G8, h->xt8, h->partial, h->bucket_cnt, h->bucket_off,
                  h->entries, h->loss_partial, h->status, h->stats, h->topk_val, h->topk_idx, h->topk_cnt, h->topk_thr, h->topk_max, h->topk_row};
  for (void* p : ptrs)
    if (p != nullptr) cudaFree(p);
  for (cudaEvent_t e : h->ev_pool) cudaEventDestroy(e);
  delete h;
  return XMC_OK;
}

int64_t xmc_workspace_bytes(const xmc_handle* h) { return h ? h->ws_bytes : 0; }

int xmc_bind_weights(xmc_handle* h, int32_t n_chunks, void* const* ptrs, const int64_t* rows) {
  if (h == nullptr || ptrs == nullptr || rows == nullptr || n_chunks <= 0) return fail(XMC_ERR_INVALID, "null/empty argument");
  DeviceGuard guard(h->cfg.device);
  int64_t total = 0;
  for (int i = 0; i < n_chunks; ++i) {
    if (ptrs[i] == nullptr || ((uintptr_t)ptrs[i] & 31u)) return fail(XMC_ERR_INVALID, "weight chunk %d: null or not 32-byte aligned", i);
    if (rows[i] <= 0) return fail(XMC_ERR_INVALID, "weight chunk %d has %lld rows", i, (long long)rows[i]);
    if (i + 1 < n_chunks && rows[i] != rows[0]) return fail(XMC_ERR_INVALID, "all weight chunks but the last must have equal rows (chunk %d: %lld vs %lld)", i, (long long)rows[i], (long long)rows[0]);
    if (i + 1 == n_chunks && rows[i] > rows[0]) return fail(XMC_ERR_INVALID, "last weight chunk is larger than the others");
    total += rows[i];
  }
  if (total > (1ll << 31) - 256) return fail(XMC_ERR_INVALID, "too many label rows per handle (%lld)", (long long)total);
  h->w_ptrs.assign(ptrs, ptrs + n_chunks);
  h->w_rows.assign(rows, rows + n_chunks);
  h->total_rows = total;
  h->rows_per_chunk = rows[0];
  // A weight chunk slightly longer than the automatic scheduling chunk (the reference's padding rule
  // makes 65 552-row chunks out of 262 144 labels in 4 chunks) is taken in one piece instead of leaving a
  // launch of a few rows behind.
  h->sched = h->sched_cfg;
  if (h->cfg.sched_labels <= 0 && rows[0] > h->sched && rows[0] <= h->sched + h->sched / 16)
    h->sched = (int)round_up(rows[0], 128);
  const int64_t g_rows = std::min<int64_t>(h->sched, round_up(h->rows_per_chunk, 128));
  if (g_rows > h->g_rows) {
    if (h->G) { cudaFree(h->G); h->ws_bytes -= h->g_rows * h->bpad_max * 2; h->G = nullptr; }
    if (h->G8) { cudaFree(h->G8); h->ws_bytes -= h->g8_rows * h->bpad_max; h->G8 = nullptr; h->g8_rows = 0; }
    h->g_rows = 0;
    if (int rc = dev_alloc(h, (void**)&h->G, (size_t)g_rows * h->bpad_max * 2, true)) return rc;
    h->g_rows = g_rows;
  }
  const int spc = cdiv(h->rows_per_chunk, h->sched);
  const int nb = n_chunks * spc * (h->sched / 128);
  if (nb != h->n_buckets) {
    if (h->bucket_cnt) { cudaFree(h->bucket_cnt); h->ws_bytes -= (int64_t)h->n_buckets * 8; h->bucket_cnt = nullptr; }
    if (h->bucket_off) { cudaFree(h->bucket_off); h->ws_bytes -= (int64_t)(h->n_buckets + 1) * 4; h->bucket_off = nullptr; }
    if (h->loss_partial) { cudaFree(h->loss_partial); h->ws_bytes -= h->loss_cap * 8; h->loss_partial = nullptr; }
    h->n_buckets = nb;
    if (int rc = dev_alloc(h, (void**)&h->bucket_cnt, (size_t)nb * 8, true)) return rc;
    if (int rc = dev_alloc(h, (void**)&h->bucket_off, (size_t)(nb + 1) * 4, true)) return rc;
    h->loss_cap = (int64_t)n_chunks * spc * h->sm_count * xmc::kMaxEpiWarps;
    if (int rc = dev_alloc(h, (void**)&h->loss_partial, (size_t)h->loss_cap * 8, true)) return rc;
  }
  return XMC_OK;
}

int xmc_bind_kahan(xmc_handle* h, void* buf, int64_t rows, int32_t dtype) {
  if (h == nullptr) return fail(XMC_ERR_INVALID, "null handle");
  if (buf == nullptr || rows == 0) {
    h->kahan = nullptr;
    h->kahan_rows = 0;
    return XMC_OK;
  }
  if (h->cfg.mode != XMC_MODE_FP8) return fail(XMC_ERR_STATE, "the Kahan head is defined for the real-FP8 mode only");
  if (h->w_ptrs.empty()) return fail(XMC_ERR_STATE, "bind the weights first");
  if (dtype != XMC_DT_BF16 && dtype != XMC_DT_E5M2) return fail(XMC_ERR_INVALID, "compensation buffer must be bf16 or e5m2");
  if (rows < 0 || rows > h->w_rows[0]) return fail(XMC_ERR_INVALID, "head rows %lld exceed the first weight chunk (%lld rows)", (long long)rows, (long long)h->w_rows[0]);
  if ((uintptr_t)buf & 15u) return fail(XMC_ERR_INVALID, "compensation buffer not 16-byte aligned");
  h->kahan = buf;
  h->kahan_rows = rows;
  h->kahan_e5m2 = dtype == XMC_DT_E5M2 ? 1 : 0;
  return XMC_OK;
}

int xmc_weight_stats(xmc_handle* h, int64_t* counts, float* amax_stored, void* stream) {
  if (h == nullptr || counts == nullptr || amax_stored == nullptr) return fail(XMC_ERR_INVALID, "null argument");
  if (h->w_ptrs.empty()) return fail(XMC_ERR_STATE, "xmc_bind_weights has not been called");
  if (h->cfg.mode == XMC_MODE_BF16) return fail(XMC_ERR_STATE, "weight statistics are defined for e4m3 weights");
  DeviceGuard guard(h->cfg.device);
  cudaStream_t st = (cudaStream_t)stream;
  if (h->stats == nullptr) {
    if (int rc = dev_alloc(h, (void**)&h->stats, 8 * sizeof(unsigned long long), true)) return rc;
  }
  CU_TRY(cudaMemsetAsync(h->stats, 0, 8 * sizeof(unsigned long long), st));
  const int d = h->cfg.dim;
  for (size_t wc = 0; wc < h->w_ptrs.size(); ++wc) {
    const long long n16 = (long long)h->w_rows[wc] * d / 16;
    const int blocks = (int)std::min<long long>((n16 + 255) / 256, (long long)h->sm_count * 8);
    xmc::weight_stats_kernel<<<blocks, 256, 0, st>>>(reinterpret_cast<const uint4*>(h->w_ptrs[wc]), n16, h->stats,
                                                     reinterpret_cast<unsigned int*>(h->stats + 4));
    CU_TRY(cudaGetLastError());
  }
  unsigned long long host[8];
  CU_TRY(cudaMemcpyAsync(host, h->stats, sizeof(host), cudaMemcpyDeviceToHost, st));
  CU_TRY(cudaStreamSynchronize(st));
  for (int i = 0; i < 4; ++i) counts[i] = (int64_t)host[i];
  counts[4] = h->total_rows * d;
  // magnitude byte -> value: exponent field e, mantissa m: e ? 2^(e-7) (1 + m/8) : m 2^-9
  const unsigned int mb = (unsigned int)(host[4] & 0x7Fu);
  const int e = (int)(mb >> 3), m = (int)(mb & 7u);
  *amax_stored = e ? ldexpf(1.0f + (float)m / 8.0f, e - 7) : ldexpf((float)m, -9);
  return XMC_OK;
}

int xmc_rescale(xmc_handle* h, int32_t shift, int32_t stochastic, uint64_t seed, uint64_t step, void* stream) {
  if (h == nullptr) return fail(XMC_ERR_INVALID, "null handle");
  if (h->w_ptrs.empty()) return fail(XMC_ERR_STATE, "xmc_bind_weights has not been called");
  if (h->cfg.mode == XMC_MODE_BF16) return fail(XMC_ERR_STATE, "the per-tensor scale belongs to e4m3 weights");
  if (shift < -16 || shift > 16) return fail(XMC_ERR_INVALID, "shift %d outside [-16, 16]", shift);
  if (h->kahan != nullptr && shift != 0) return fail(XMC_ERR_STATE, "rescaling with a Kahan head bound is not defined");
  if (shift == 0) return XMC_OK;
  DeviceGuard guard(h->cfg.device);
  cudaStream_t st = (cudaStream_t)stream;
  const int d = h->cfg.dim;
  const float factor = ldexpf(1.0f, -shift);
  int64_t row_base = 0;
  for (size_t wc = 0; wc < h->w_ptrs.size(); ++wc) {
    const long long n8 = (long long)h->w_rows[wc] * d / 8;
    const int blocks = (int)std::min<long long>((n8 + 255) / 256, (long long)h->sm_count * 8);
    xmc::rescale_e4m3_kernel<<<blocks, 256, 0, st>>>(reinterpret_cast<uint2*>(h->w_ptrs[wc]), n8, factor, stochastic ? 1 : 0,
                                                     seed, step, (unsigned long long)(h->cfg.label_offset + row_base) * d);
    CU_TRY(cudaGetLastError());
    row_base += h->w_rows[wc];
  }
  h->cfg.w_scale = ldexpf(h->cfg.w_scale, shift);
  return XMC_OK;
}

float xmc_get_scale(const xmc_handle* h) { return h ? h->cfg.w_scale : 0.f; }

int xmc_set_scale(xmc_handle* h, float scale) {
  if (h == nullptr) return fail(XMC_ERR_INVALID, "null handle");
  if (!(scale > 0.f)) return fail(XMC_ERR_INVALID, "w_scale must be positive");
  h->cfg.w_scale = scale;
  return XMC_OK;
}

int xmc_check(xmc_handle* h, void* stream) {
  if (h == nullptr) return fail(XMC_ERR_INVALID, "null handle");
  DeviceGuard guard(h->cfg.device);
  cudaStream_t st = (cudaStream_t)stream;
  CU_TRY(cudaStreamSynchronize(st));
  int host[4] = {0, 0, 0, 0};
  CU_TRY(cudaMemcpy(host, h->status, sizeof(host), cudaMemcpyDeviceToHost));
  if (host[0] != xmc::DEV_OK) {
    CU_TRY(cudaMemset(h->status, 0, sizeof(host)));
    if (host[0] == xmc::DEV_WAIT_TIMEOUT)
      return fail(XMC_ERR_DEVICE_FLAG, "kernel wait timed out (block %d, site %d)", host[1], host[2]);
    if (host[0] == xmc::DEV_BAD_LABEL)
      return fail(XMC_ERR_DEVICE_FLAG, "label pair with batch row out of range or negative id (row %d)", host[2]);
    return fail(XMC_ERR_DEVICE_FLAG, "device status %d (block %d, info %d)", host[0], host[1], host[2]);
  }
  return XMC_OK;
}

int xmc_step(xmc_handle* h, const void* x, int32_t x_dtype, int32_t batch, const int32_t* labels,
             int64_t nnz, float lr, float wd, uint64_t seed, uint64_t step, uint32_t flags,
             float* grad_x_f32, void* grad_x_bf16, double* loss_out, void* stream) {
  if (h == nullptr || x == nullptr) return fail(XMC_ERR_INVALID, "null argument");
  if (h->w_ptrs.empty()) return fail(XMC_ERR_STATE, "xmc_bind_weights has not been called");
  if (x_dtype != XMC_DT_BF16) return fail(XMC_ERR_INVALID, "xmc_step takes bf16 embeddings");
  if (batch <= 0 || batch > h->cfg.max_batch) return fail(XMC_ERR_INVALID, "batch %d outside [1, %d]", batch, h->cfg.max_batch);
  if (nnz < 0 || (nnz > 0 && labels == nullptr)) return fail(XMC_ERR_INVALID, "labels missing");
  if ((flags & XMC_STEP_COMPUTE_LOSS) && loss_out == nullptr) return fail(XMC_ERR_INVALID, "loss_out missing");
  if (((uintptr_t)grad_x_f32 & 15u) || ((uintptr_t)grad_x_bf16 & 1u)) return fail(XMC_ERR_INVALID, "grad_x not aligned");
  DeviceGuard guard(h->cfg.device);
  cudaStream_t st = (cudaStream_t)stream;
  const int d = h->cfg.dim, mode = h->cfg.mode;
  const int bpad = (int)round_up(batch, 64);   // G rows are fetched in blocks of 64 batch columns
  const bool w8 = mode != XMC_MODE_BF16;
  const bool fwd_fp8 = mode == XMC_MODE_FP8;
  const bool want_loss = (flags & XMC_STEP_COMPUTE_LOSS) != 0;
  const bool sr = (flags & XMC_STEP_STOCHASTIC) != 0;
  const bool dw8 = (flags & XMC_STEP_FP8_DW) != 0;
  if (dw8) {
    if (!fwd_fp8) return fail(XMC_ERR_STATE, "the FP8 dW contraction belongs to the real-FP8 mode");
    if ((flags & XMC_STEP_ROUND_DW_BF16) || wd != 0.f || h->kahan != nullptr)
      return fail(XMC_ERR_STATE, "the FP8 dW contraction takes no weight decay, bf16 dW rounding or Kahan head");
    if (h->G8 == nullptr || h->g8_rows < h->g_rows) {
      CU_TRY(cudaStreamSynchronize(st));
      if (h->G8) { cudaFree(h->G8); h->ws_bytes -= h->g8_rows * h->bpad_max; h->G8 = nullptr; }
      if (int rc = dev_alloc(h, (void**)&h->G8, (size_t)h->g_rows * h->bpad_max, true)) return rc;
      h->g8_rows = h->g_rows;
    }
    if (h->xt8 == nullptr) {
      if (int rc = dev_alloc(h, (void**)&h->xt8, (size_t)std::max(h->cfg.dim, 256) * h->bpad_max, true)) return rc;
    }
  }

  // --- embeddings: e4m3 copy (forward), bf16 copy, bf16 transpose (update) ---
  if (int rc = prep_x(h, x, x_dtype, batch, bpad, fwd_fp8, !fwd_fp8, !dw8, st, dw8)) return rc;

  // --- bucket the positives by label tile ---
  if (nnz > h->ent_cap) {
    CU_TRY(cudaStreamSynchronize(st));
    CU_TRY(cudaFree(h->entries));
    h->ws_bytes -= h->ent_cap * 4;
    h->entries = nullptr;
    h->ent_cap = nnz + nnz / 2;
    if (int rc = dev_alloc(h, (void**)&h->entries, (size_t)h->ent_cap * 4, false)) return rc;
  }
  const xmc::BucketGeom geom = geom_of(h);
  if (nnz <= 131072) {
    // few positives: one single-block launch does the clearing, the count, the scan and the fill
    mark(h, K_PREP, st);
    xmc::bucket_all_kernel<<<1, 1024, 0, st>>>(labels, (int)nnz, batch, geom, h->n_buckets, h->bucket_cnt,
                                               h->bucket_cnt + h->n_buckets, h->bucket_off, h->entries, h->status);
    CU_TRY(cudaGetLastError());
  } else {
    CU_TRY(cudaMemsetAsync(h->bucket_cnt, 0, (size_t)h->n_buckets * 8, st));
    mark(h, K_PREP, st);
    xmc::bucket_count_kernel<<<cdiv(nnz, 256), 256, 0, st>>>(labels, nnz, batch, geom, h->bucket_cnt, h->status);
    CU_TRY(cudaGetLastError());
    mark(h, K_PREP, st);
    xmc::bucket_scan_kernel<<<1, 1024, 0, st>>>(h->bucket_cnt, h->n_buckets, h->bucket_off);
    CU_TRY(cudaGetLastError());
    mark(h, K_PREP, st);
    xmc::bucket_fill_kernel<<<cdiv(nnz, 256), 256, 0, st>>>(labels, nnz, batch, geom, h->bucket_off,
                                                            h->bucket_cnt + h->n_buckets, h->entries);
    CU_TRY(cudaGetLastError());
  }

  // --- grad_X partial geometry ---
  // On CTA pairs (512-row batch tiles) when the weights are e4m3, every feature tile is whole and both
  // CTAs of a pair have batch rows to work on; otherwise one CTA per 256 x 256 tile.
  static const bool no_pairs = getenv("XMC_NO_PAIRS") != nullptr;
  int gx_max_pairs = 0;
  if (int rc = gradx_configure(h->sm_count, &gx_max_pairs)) return rc;
  const bool pairs_ok = !no_pairs && gx_max_pairs >= 1;   // a device that cannot hold a pair runs everything on single CTAs
  const int n_dt = cdiv(d, 256);
  const bool pair_gx = pairs_ok && w8 && d % 256 == 0 && bpad >= 256;
  const int n_bt = cdiv(bpad, pair_gx ? 512 : 256);
  int n_splits = std::max(1, (pair_gx ? gx_max_pairs : h->sm_count) / (n_bt * n_dt));
  while (n_splits > 1 && (int64_t)n_splits * bpad * d > h->partial_floats) --n_splits;
  if ((int64_t)n_splits * bpad * d > h->partial_floats) return fail(XMC_ERR_STATE, "grad_X workspace too small");

  // Keep the grad_X partial sums resident in L2 across the chunk launches of this step: every
  // grad_X launch re-reads and re-writes them, and the weights/G streaming through L2 in between
  // would otherwise push them out to HBM each time.  The window covers only this private buffer.
  if (h->l2_persist_bytes > 0) {
    cudaStreamAttrValue attr;
    memset(&attr, 0, sizeof(attr));
    attr.accessPolicyWindow.base_ptr = h->partial;
    attr.accessPolicyWindow.num_bytes = std::min<size_t>((size_t)n_splits * bpad * d * 4, (size_t)h->l2_persist_bytes);
    attr.accessPolicyWindow.hitRatio = 1.0f;
    attr.accessPolicyWindow.hitProp = cudaAccessPropertyPersisting;
    attr.accessPolicyWindow.missProp = cudaAccessPropertyStreaming;
    CU_TRY(cudaStreamSetAttribute(st, cudaStreamAttributeAccessPolicyWindow, &attr));
  }

  // --- operand maps that do not change across chunks ---
  CUtensorMap map_x, map_xt, map_g_k, map_g_mn;
  const size_t xrows = (size_t)std::max(h->bpad_max, 256);
  // CTA pairs (256-row label tiles, each CTA staging half of the other operand's rows) for the kernels
  // that take their operands as stored: the FP8 and bf16 forward, every update
  const bool pair_fwd = pairs_ok && mode != XMC_MODE_SIMFP8;
  const bool pair_upd = pairs_ok;
  if (fwd_fp8) {
    if (int rc = make_map_kmajor(&map_x, true, h->x8, d, xrows, d, pair_fwd ? 128 : 256)) return rc;
  } else {
    if (int rc = make_map_kmajor(&map_x, false, h->x16, d, xrows, d, pair_fwd ? 128 : 256)) return rc;
  }
  if (dw8) {
    if (int rc = make_map_kmajor(&map_xt, true, h->xt8, bpad, std::max(d, 256), bpad, pair_upd ? 128 : 256)) return rc;
    if (int rc = make_map_kmajor(&map_g_k, true, h->G8, bpad, h->g8_rows, bpad, 128)) return rc;
  } else {
    if (int rc = make_map_kmajor(&map_xt, false, h->xt, bpad, std::max(d, 256), bpad, pair_upd ? 128 : 256)) return rc;
    if (int rc = make_map_kmajor(&map_g_k, false, h->G, bpad, h->g_rows, bpad, 128)) return rc;
  }
  if (int rc = make_map_blocked(&map_g_mn, false, h->G, bpad, h->g_rows, bpad, xmc::kGxRows, true, pair_gx ? 2 : 4)) return rc;

  const float lr_eff = lr / h->cfg.w_scale;
  const int tiles_per_sched = h->sched / 128;
  int launch_idx = 0;
  bool first = true;
  int64_t row_base = 0;
  for (size_t wc = 0; wc < h->w_ptrs.size(); ++wc) {
    const int64_t rows_wc = h->w_rows[wc];
    const int spc = cdiv(h->rows_per_chunk, h->sched);
    for (int sc = 0; sc < spc; ++sc) {
      const int64_t s0 = (int64_t)sc * h->sched;
      if (s0 >= rows_wc) break;
      const int rows_valid = (int)std::min<int64_t>(h->sched, rows_wc - s0);
      const int n_lt = cdiv(rows_valid, 128);
      const size_t esz = w8 ? 1 : 2;
      uint8_t* wbase = reinterpret_cast<uint8_t*>(h->w_ptrs[wc]) + (size_t)s0 * d * esz;

      // forward + loss gradient -> G
      CUtensorMap map_w;
      const bool sim = mode == XMC_MODE_SIMFP8;
      if (fwd_fp8) {
        if (int rc = make_map_kmajor(&map_w, true, wbase, d, rows_valid, d, 128)) return rc;
      } else if (sim) {
        // e4m3 storage, bf16 arithmetic: the kernel converts the weight operand in shared memory
        if (int rc = make_map_raw8(&map_w, wbase, d, rows_valid, d, 128)) return rc;
      } else {
        if (int rc = make_map_kmajor(&map_w, false, wbase, d, rows_valid, d, 128)) return rc;
      }
      xmc::FwdParams fp;
      fp.m_rows = pair_fwd ? 256 : 128;
      fp.rows_valid = rows_valid;
      fp.n_ltiles = cdiv(rows_valid, fp.m_rows);
      fp.n_btiles = cdiv(bpad, 256);
      fp.div_btiles = xmc::make_fastdiv(fp.n_btiles);
      fp.batch = batch;
      fp.bpad = bpad;
      fp.k_steps = cdiv((long long)d * (fwd_fp8 ? 1 : 2), 128);
      fp.w_scale = h->cfg.w_scale;
      fp.G = h->G;
      fp.G8 = h->G8;
      fp.bucket_off = h->bucket_off;
      fp.bucket_ent = h->entries;
      fp.tile_base = ((int)wc * spc + sc) * tiles_per_sched;
      fp.loss_partial = want_loss ? h->loss_partial + (size_t)launch_idx * h->sm_count * xmc::kMaxEpiWarps : nullptr;
      fp.status = h->status;
      const int f_tiles = fp.n_ltiles * fp.n_btiles;
      if (want_loss && (pair_fwd || f_tiles < h->sm_count)) {
        // slots of CTAs that are not launched must read as zero
        CU_TRY(cudaMemsetAsync(fp.loss_partial, 0, (size_t)h->sm_count * xmc::kMaxEpiWarps * sizeof(double), st));
      }
      int rc;
      mark(h, K_FWD, st);
#define XMC_FWD(PAIR_, FP8_, G8_, CONV_) \
  (want_loss ? launch_gemm<xmc::FwdPolicy<FP8_, true, G8_, CONV_>, PAIR_>(map_w, map_x, fp, f_tiles, h->sm_count, st) \
             : launch_gemm<xmc::FwdPolicy<FP8_, false, G8_, CONV_>, PAIR_>(map_w, map_x, fp, f_tiles, h->sm_count, st))
      if (sim) rc = XMC_FWD(false, false, false, true);
      else if (dw8) rc = pair_fwd ? XMC_FWD(true, true, true, false) : XMC_FWD(false, true, true, false);
      else if (fwd_fp8) rc = pair_fwd ? XMC_FWD(true, true, false, false) : XMC_FWD(false, true, false, false);
      else rc = pair_fwd ? XMC_FWD(true, false, false, false) : XMC_FWD(false, false, false, false);
#undef XMC_FWD
      if (rc) return rc;

      // grad_X partials: uses the pre-update weights (reference: chunked.py:116 precedes :119-127)
      CUtensorMap map_w_gx;
      if (w8) {
        // raw e4m3 rows, unswizzled boxes of 32 rows x 256 features; converted inside the kernel
        if (int rc2 = make_map_blocked(&map_w_gx, true, wbase, d, rows_valid, d, xmc::kGxRows, false, pair_gx ? 2 : 4)) return rc2;
      } else {
        if (int rc2 = make_map_blocked(&map_w_gx, false, wbase, d, rows_valid, d, xmc::kGxRows, true)) return rc2;
      }
      xmc::GxParams gp;
      gp.bpad = bpad;
      gp.d = d;
      gp.n_btiles = n_bt;
      gp.n_dtiles = n_dt;
      gp.n_splits = n_splits;
      gp.total_ksteps = cdiv(rows_valid, xmc::kGxRows);
      gp.accumulate = first ? 0 : 1;
      gp.partial = h->partial;
      gp.status = h->status;
      mark(h, K_GRADX, st);
      {
        const int grid = n_bt * n_dt * n_splits;
        if (pair_gx) {
          cudaLaunchConfig_t cfg;
          cudaLaunchAttribute at[2];
          launch_config(&cfg, at, 2 * grid, xmc::kGxThreads, xmc::kGxSmemBytes<true>, st, 2);
          CU_TRY(cudaLaunchKernelEx(&cfg, xmc::gradx_kernel<true, true>, map_g_mn, map_w_gx, gp));
        } else if (w8) {
          CU_TRY(launch_pdl(xmc::gradx_kernel<true, false>, grid, xmc::kGxThreads, xmc::kGxSmemBytes<false>, st, map_g_mn, map_w_gx, gp));
        } else {
          CU_TRY(launch_pdl(xmc::gradx_kernel<false, false>, grid, xmc::kGxThreads, xmc::kGxSmemBytes<false>, st, map_g_mn, map_w_gx, gp));
        }
        CU_TRY(cudaGetLastError());
      }

      // fused dW + SGD update of the chunk, in place
      xmc::UpdParams up;
      up.m_rows = pair_upd ? 256 : 128;
      up.rows_valid = rows_valid;
      up.n_ltiles = cdiv(rows_valid, up.m_rows);
      up.n_dtiles = n_dt;
      up.div_dtiles = xmc::make_fastdiv(n_dt);
      up.d = d;
      up.k_steps = cdiv(bpad, dw8 ? 128 : 64);
      up.W = wbase;
      up.lr_eff = dw8 ? lr_eff / xmc::kG8Scale : lr_eff;
      up.wd = wd;
      up.seed = seed;
      up.step = step;
      for (int rd = 0; rd < xmc::kSrRounds; ++rd) {
        up.rkey[rd][0] = (uint32_t)seed + (uint32_t)rd * 0x9E3779B9u;
        up.rkey[rd][1] = (uint32_t)(seed >> 32) + (uint32_t)rd * 0xBB67AE85u;
      }
      up.elem0 = (unsigned long long)(h->cfg.label_offset + row_base + s0) * (unsigned long long)d;
      up.round_dw_bf16 = (flags & XMC_STEP_ROUND_DW_BF16) ? 1 : 0;
      up.status = h->status;
      const int u_tiles = up.n_ltiles * n_dt;
      mark(h, K_UPD, st);
      // the reference pairs: e4m3 weights (no dW rounding), bf16 weights (dW materialised in bf16);
      // weight decay is off in both, so only those combinations get the branch-free fast kernels
      up.kahan = nullptr;
      up.kahan_rows = 0;
      up.kahan_e5m2 = h->kahan_e5m2;
      const bool kahan_here = h->kahan != nullptr && wc == 0 && s0 < h->kahan_rows;
      if (kahan_here) {
        if (!w8 || up.round_dw_bf16 || wd != 0.f) return fail(XMC_ERR_STATE, "the Kahan head needs e4m3 weights without weight decay");
        up.kahan = reinterpret_cast<uint8_t*>(h->kahan) + (size_t)s0 * d * (h->kahan_e5m2 ? 1 : 2);
        up.kahan_rows = (int)std::min<int64_t>(h->kahan_rows - s0, rows_valid);
      }
      const bool rdw = up.round_dw_bf16 != 0, has_wd = wd != 0.f;
      // the chunk's weights as the update epilogue's input: boxes of 128 rows x 128 bytes, 128-byte swizzle
      CUtensorMap map_wt;
      if (w8) {
        if (int rc2 = make_map(&map_wt, true, wbase, d, rows_valid, d, 128, 128)) return rc2;
      }
      const CUtensorMap* wt = w8 ? &map_wt : nullptr;
#define XMC_UPD(...) \
  (pair_upd ? launch_gemm<xmc::UpdPolicy<__VA_ARGS__>, true>(map_g_k, map_xt, up, u_tiles, h->sm_count, st, 0, wt) \
            : launch_gemm<xmc::UpdPolicy<__VA_ARGS__>, false>(map_g_k, map_xt, up, u_tiles, h->sm_count, st, 0, wt))
      if (dw8) {
        rc = sr ? XMC_UPD(true, true, false, false, false, true) : XMC_UPD(true, false, false, false, false, true);
      } else if (kahan_here) {
        rc = sr ? XMC_UPD(true, true, false, false, true) : XMC_UPD(true, false, false, false, true);
      } else if (w8) {
        if (!rdw && !has_wd) rc = sr ? XMC_UPD(true, true, false, false) : XMC_UPD(true, false, false, false);
        else if (!rdw) rc = sr ? XMC_UPD(true, true, false, true) : XMC_UPD(true, false, false, true);
        else rc = sr ? XMC_UPD(true, true, true, true) : XMC_UPD(true, false, true, true);
      } else {
        if (rdw && !has_wd) rc = sr ? XMC_UPD(false, true, true, false) : XMC_UPD(false, false, true, false);
        else if (rdw) rc = sr ? XMC_UPD(false, true, true, true) : XMC_UPD(false, false, true, true);
        else rc = sr ? XMC_UPD(false, true, false, true) : XMC_UPD(false, false, false, true);
      }
#undef XMC_UPD
      if (rc) return rc;
      first = false;
      ++launch_idx;
    }
    row_base += rows_wc;
  }

  if (grad_x_f32 != nullptr || grad_x_bf16 != nullptr) {
    const long long n = (long long)batch * d;
    const int blocks = (int)std::min<long long>((n + 255) / 256, (long long)h->sm_count * 8);
    mark(h, K_REDUCE, st);
    xmc::reduce_gradx_kernel<<<blocks, 256, 0, st>>>(h->partial, n_splits, batch, bpad, d, h->cfg.w_scale,
                                                     grad_x_f32, reinterpret_cast<__nv_bfloat16*>(grad_x_bf16));
    CU_TRY(cudaGetLastError());
  }
  if (want_loss) {
    mark(h, K_REDUCE, st);
    xmc::reduce_loss_kernel<<<1, 32, 0, st>>>(h->loss_partial, launch_idx * h->sm_count * xmc::kMaxEpiWarps, loss_out);
    CU_TRY(cudaGetLastError());
  }
  if (h->l2_persist_bytes > 0) {
    // the caller's stream leaves this call without the window (kernels launched after it are unaffected)
    cudaStreamAttrValue attr;
    memset(&attr, 0, sizeof(attr));
    CU_TRY(cudaStreamSetAttribute(st, cudaStreamAttributeAccessPolicyWindow, &attr));
  }
  mark(h, K_END, st);
  return XMC_OK;
}

int64_t xmc_launch_count(const xmc_handle* h) { return h ? h->launches : 0; }

int xmc_profile(xmc_handle* h, int32_t enable, double* ms_by_kind, int64_t* launches_by_kind) {
  if (h == nullptr) return fail(XMC_ERR_INVALID, "null handle");
  DeviceGuard guard(h->cfg.device);
  if (ms_by_kind != nullptr && launches_by_kind != nullptr) {
    for (int k = 0; k < 8; ++k) { ms_by_kind[k] = 0.0; launches_by_kind[k] = 0; }
    if (h->ev_used > 0) CU_TRY(cudaEventSynchronize(h->ev_pool[h->ev_used - 1]));
    for (size_t i = 0; i + 1 < h->ev_used; ++i) {
      const int kind = h->ev_kind[i];
      if (kind == K_END) continue;
      float ms = 0.f;
      CU_TRY(cudaEventElapsedTime(&ms, h->ev_pool[i], h->ev_pool[i + 1]));
      ms_by_kind[kind] += ms;
      launches_by_kind[kind] += 1;
    }
  }
  h->ev_used = 0;
  h->profile = enable != 0;
  return XMC_OK;
}

int xmc_forward_logits(xmc_handle* h, const void* x, int32_t x_dtype, int32_t batch, void* out_bf16,
                       int64_t ld_out, int64_t n_out, void* stream) {
  if (h == nullptr || x == nullptr || out_bf16 == nullptr) return fail(XMC_ERR_INVALID, "null argument");
  if (h->w_ptrs.empty()) return fail(XMC_ERR_STATE, "xmc_bind_weights has not been called");
  if (x_dtype != XMC_DT_BF16 && x_dtype != XMC_DT_E4M3) return fail(XMC_ERR_INVALID, "embeddings must be bf16 or e4m3");
  if (batch <= 0 || batch > h->cfg.max_batch) return fail(XMC_ERR_INVALID, "batch %d outside [1, %d]", batch, h->cfg.max_batch);
  if (n_out <= 0 || n_out > h->total_rows || ld_out < n_out || (ld_out & 7) || ((uintptr_t)out_bf16 & 15u))
    return fail(XMC_ERR_INVALID, "bad output geometry (n_out %lld, ld_out %lld, rows %lld)", (long long)n_out, (long long)ld_out, (long long)h->total_rows);
  DeviceGuard guard(h->cfg.device);
  cudaStream_t st = (cudaStream_t)stream;
  const int d = h->cfg.dim, mode = h->cfg.mode;
  const int bpad = (int)round_up(batch, 64);
  const bool fwd_fp8 = mode == XMC_MODE_FP8;
  if (int rc = prep_x(h, x, x_dtype, batch, bpad, fwd_fp8, !fwd_fp8, false, st)) return rc;
  // on CTA pairs (256 batch rows x 256 labels per pair, each CTA staging half of the tile's weight rows)
  // when the device holds pairs and the weights are multiplied as stored
  static const bool no_pairs = getenv("XMC_NO_PAIRS") != nullptr;
  int max_pairs = 0;
  if (int rc = gradx_configure(h->sm_count, &max_pairs)) return rc;
  const bool pair = !no_pairs && max_pairs >= 1 && mode != XMC_MODE_SIMFP8;
  CUtensorMap map_x;
  const size_t xrows = (size_t)std::max(h->bpad_max, 256);
  if (fwd_fp8) {
    if (int rc = make_map_kmajor(&map_x, true, h->x8, d, xrows, d, 128)) return rc;
  } else {
    if (int rc = make_map_kmajor(&map_x, false, h->x16, d, xrows, d, 128)) return rc;
  }
  int64_t row_base = 0;
  for (size_t wc = 0; wc < h->w_ptrs.size() && row_base < n_out; ++wc) {
    const int64_t rows_wc = h->w_rows[wc];
    for (int64_t s0 = 0; s0 < rows_wc && row_base + s0 < n_out; s0 += h->sched) {
      const int rows = (int)std::min<int64_t>(h->sched, rows_wc - s0);
      const size_t esz = mode == XMC_MODE_BF16 ? 2 : 1;
      const uint8_t* wbase = reinterpret_cast<const uint8_t*>(h->w_ptrs[wc]) + (size_t)s0 * d * esz;
      const bool sim = mode == XMC_MODE_SIMFP8;
      CUtensorMap map_w;
      if (sim) {
        if (int rc = make_map_raw8(&map_w, wbase, d, rows, d, 256)) return rc;
      } else {
        if (int rc = make_map_kmajor(&map_w, fwd_fp8, wbase, d, rows, d, pair ? 128 : 256)) return rc;
      }
      xmc::LogitsParams lp;
      lp.m_rows = pair ? 256 : 128;
      lp.batch = batch;
      lp.rows = rows;
      lp.n_mtiles = cdiv(batch, lp.m_rows);
      lp.n_ntiles = cdiv(rows, 256);
      lp.k_steps = cdiv((long long)d * (fwd_fp8 ? 1 : 2), 128);
      lp.w_scale = h->cfg.w_scale;
      lp.out = reinterpret_cast<__nv_bfloat16*>(out_bf16);
      lp.ld_out = ld_out;
      lp.col0 = row_base + s0;
      lp.n_out = n_out;
      lp.status = h->status;
      mark(h, K_LOGITS, st);
      const int tiles = lp.n_mtiles * lp.n_ntiles;
      int rc;
      if (sim) rc = launch_gemm<xmc::LogitsPolicy<false, true>>(map_x, map_w, lp, tiles, h->sm_count, st);
      else if (pair) rc = fwd_fp8 ? launch_gemm<xmc::LogitsPolicy<true>, true>(map_x, map_w, lp, tiles, h->sm_count, st)
                                  : launch_gemm<xmc::LogitsPolicy<false>, true>(map_x, map_w, lp, tiles, h->sm_count, st);
      else rc = fwd_fp8 ? launch_gemm<xmc::LogitsPolicy<true>>(map_x, map_w, lp, tiles, h->sm_count, st)
                        : launch_gemm<xmc::LogitsPolicy<false>>(map_x, map_w, lp, tiles, h->sm_count, st);
      if (rc) return rc;
    }
    row_base += rows_wc;
  }
  mark(h, K_END, st);
  return XMC_OK;
}
int xmc_forward_topk(xmc_handle* h, const void* x, int32_t x_dtype, int32_t batch, int32_t k, int64_t n_out,
                     float* vals, int32_t* idx, void* stream) {
  if (h == nullptr || x == nullptr || vals == nullptr || idx == nullptr) return fail(XMC_ERR_INVALID, "null argument");
  if (h->w_ptrs.empty()) return fail(XMC_ERR_STATE, "xmc_bind_weights has not been called");
  if (x_dtype != XMC_DT_BF16 && x_dtype != XMC_DT_E4M3) return fail(XMC_ERR_INVALID, "embeddings must be bf16 or e4m3");
  if (batch <= 0 || batch > h->cfg.max_batch) return fail(XMC_ERR_INVALID, "batch %d outside [1, %d]", batch, h->cfg.max_batch);
  if (k <= 0 || k > 128) return fail(XMC_ERR_INVALID, "k must be in [1, 128], got %d", k);
  if (n_out <= 0 || n_out > h->total_rows) return fail(XMC_ERR_INVALID, "n_out %lld outside [1, %lld]", (long long)n_out, (long long)h->total_rows);
  DeviceGuard guard(h->cfg.device);
  cudaStream_t st = (cudaStream_t)stream;
  const int d = h->cfg.dim, mode = h->cfg.mode;
  const int bpad = (int)round_up(batch, 64);
  const bool fwd_fp8 = mode == XMC_MODE_FP8;
  const int n_mt = cdiv(batch, 128);
  if (n_mt > h->sm_count) return fail(XMC_ERR_INVALID, "batch too large for the fused top-k");
  const int grid_max = h->sm_count / n_mt * n_mt;
  // candidate lists: one per (CTA, epilogue warp, lane), alive across the launches of this call
  const int lists = grid_max * 256;
  const int cap = k <= 16 ? 96 : (k <= 32 ? 128 : 256);
  const int64_t need = (int64_t)lists * (cap + 32);
  if (need > h->topk_cap || lists > h->topk_lists) {
    CU_TRY(cudaStreamSynchronize(st));
    if (h->topk_val) { cudaFree(h->topk_val); cudaFree(h->topk_idx); h->ws_bytes -= h->topk_cap * 8; h->topk_val = nullptr; h->topk_idx = nullptr; }
    if (h->topk_cnt) { cudaFree(h->topk_cnt); cudaFree(h->topk_thr); cudaFree(h->topk_max); h->ws_bytes -= (int64_t)h->topk_lists * 12; h->topk_cnt = nullptr; h->topk_thr = nullptr; h->topk_max = nullptr; }
    h->topk_cap = 0;
    h->topk_lists = 0;
    const int64_t cap_new = std::max<int64_t>(need, (int64_t)h->sm_count * 256 * (cap + 32));
    const int lists_new = h->sm_count * 256;
    if (int rc = dev_alloc(h, (void**)&h->topk_val, (size_t)cap_new * 4, false)) return rc;
    if (int rc = dev_alloc(h, (void**)&h->topk_idx, (size_t)cap_new * 4, false)) return rc;
    if (int rc = dev_alloc(h, (void**)&h->topk_cnt, (size_t)lists_new * 4, false)) return rc;
    if (int rc = dev_alloc(h, (void**)&h->topk_thr, (size_t)lists_new * 4, false)) return rc;
    if (int rc = dev_alloc(h, (void**)&h->topk_max, (size_t)lists_new * 4, false)) return rc;
    h->topk_cap = cap_new;
    h->topk_lists = lists_new;
  }
  if (h->topk_row == nullptr) {
    if (int rc = dev_alloc(h, (void**)&h->topk_row, (size_t)std::max(h->bpad_max, 128) * 4, false)) return rc;
  }
  xmc::topk_init_kernel<<<cdiv(std::max(lists, batch), 256), 256, 0, st>>>(h->topk_cnt, h->topk_thr, h->topk_max, lists, h->topk_row, batch);
  CU_TRY(cudaGetLastError());
  if (int rc = prep_x(h, x, x_dtype, batch, bpad, fwd_fp8, !fwd_fp8, false, st)) return rc;
  CUtensorMap map_x;
  const size_t xrows = (size_t)std::max(h->bpad_max, 256);
  if (fwd_fp8) {
    if (int rc = make_map_kmajor(&map_x, true, h->x8, d, xrows, d, 128)) return rc;
  } else {
    if (int rc = make_map_kmajor(&map_x, false, h->x16, d, xrows, d, 128)) return rc;
  }
  // selection kernels: up to 24 576 candidate keys of a row in shared memory (192 KB) + 128 output keys
  constexpr int kSelKeys = 24576;
  constexpr size_t sel_smem = (size_t)(kSelKeys + 128) * sizeof(unsigned long long);
  {
    static std::atomic<uint64_t> configured{0};
    if (!((configured.load(std::memory_order_relaxed) >> (h->cfg.device & 63)) & 1ull)) {
      CU_TRY(cudaFuncSetAttribute(xmc::topk_select_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sel_smem));
      CU_TRY(cudaFuncSetAttribute(xmc::topk_select_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sel_smem));
      configured.fetch_or(1ull << (h->cfg.device & 63));
    }
  }
  int launch = 0;
  int64_t row_base = 0;
  for (size_t wc = 0; wc < h->w_ptrs.size() && row_base < n_out; ++wc) {
    const int64_t rows_wc = h->w_rows[wc];
    int64_t s_next = 0;
    for (int64_t s0 = 0; s0 < rows_wc && row_base + s0 < n_out; s0 = s_next) {
      int rows = (int)std::min<int64_t>(h->sched, rows_wc - s0);
      // While nothing is known every logit is a candidate: for k > 8 the very first launch therefore covers
      // only 8192 label rows (few enough that no list fills up), and the threshold pass that follows it
      // gives the rest of the call a bound to prune against.
      if (k > 8 && launch == 0) rows = std::min(rows, 8192);
      s_next = s0 + rows;
      const size_t esz = mode == XMC_MODE_BF16 ? 2 : 1;
      const uint8_t* wbase = reinterpret_cast<const uint8_t*>(h->w_ptrs[wc]) + (size_t)s0 * d * esz;
      const bool sim = mode == XMC_MODE_SIMFP8;
      // Mid-course thresholds: for k > 8 (the in-kernel k-th-of-maxima bound covers smaller k) the exact
      // k-th best value of what the lists hold is published after launches 1, 2, 4, 8, ...; the first one
      // turns the flood of the first launch (every logit is a candidate while nothing is known) into a
      // threshold the rest of the call lives on.
      if (k > 8 && launch > 0 && (launch & (launch - 1)) == 0) {
        mark(h, K_LOGITS, st);
        xmc::topk_select_kernel<false><<<batch, 256, sel_smem, st>>>(h->topk_val, h->topk_idx, h->topk_cnt, h->topk_row, cap,
                                                                     grid_max, n_mt, k, batch, h->cfg.label_offset, nullptr,
                                                                     nullptr, kSelKeys);
        CU_TRY(cudaGetLastError());
      }
      CUtensorMap map_w;
      if (sim) {
        if (int rc = make_map_raw8(&map_w, wbase, d, rows, d, 256)) return rc;
      } else {
        if (int rc = make_map_kmajor(&map_w, fwd_fp8, wbase, d, rows, d, 256)) return rc;
      }
      xmc::TopkParams tp;
      tp.batch = batch;
      tp.rows = rows;
      tp.n_mtiles = n_mt;
      tp.n_ntiles = cdiv(rows, 256);
      tp.k_steps = cdiv((long long)d * (fwd_fp8 ? 1 : 2), 128);
      tp.k = k;
      tp.w_scale = h->cfg.w_scale;
      tp.col0 = row_base + s0;
      tp.n_out = n_out;
      tp.cap = cap;
      tp.cand_val = h->topk_val;
      tp.cand_idx = h->topk_idx;
      tp.list_cnt = h->topk_cnt;
      tp.list_thr = h->topk_thr;
      tp.list_max = h->topk_max;
      tp.row_thr = h->topk_row;
      tp.status = h->status;
      const int tiles = tp.n_mtiles * tp.n_ntiles;
      // every launch uses the same grid, so that a list keeps its (CTA, warp, lane) owner; CTAs beyond
      // the tile count find no work and leave their lists untouched
      const int grid = grid_max;
      mark(h, K_LOGITS, st);
      int rc;
      rc = fwd_fp8 ? launch_gemm<xmc::TopkPolicy<true>>(map_x, map_w, tp, tiles, h->sm_count, st, grid)
           : sim   ? launch_gemm<xmc::TopkPolicy<false, true>>(map_x, map_w, tp, tiles, h->sm_count, st, grid)
                   : launch_gemm<xmc::TopkPolicy<false>>(map_x, map_w, tp, tiles, h->sm_count, st, grid);
      if (rc) return rc;
      ++launch;
    }
    row_base += rows_wc;
  }
  mark(h, K_LOGITS, st);
  xmc::topk_select_kernel<true><<<batch, 256, sel_smem, st>>>(h->topk_val, h->topk_idx, h->topk_cnt, h->topk_row, cap, grid_max,
                                                              n_mt, k, batch, h->cfg.label_offset, vals, idx, kSelKeys);
  CU_TRY(cudaGetLastError());
  mark(h, K_END, st);
  return XMC_OK;
}

// ---------------------------------------------------------------------------------------------
// Allocation-free contraction  C[m x n] = A^T B  (A given as [k x m] bf16, B as [k x n] bf16 or e4m3):
// the grad_X kernel with its split-K partial sums kept in a fixed device array owned by the library.
// ---------------------------------------------------------------------------------------------
namespace {
constexpr size_t kNoAllocFloats = 2u << 20;              // 8 MiB of partial sums
constexpr int kNoAllocMaxDevices = 64;
// [0, kNoAllocFloats): partial sums; then 4 ints of kernel status.  Every GPU that loads the library
// carries one copy until the process exits.
static __device__ __align__(256) float g_noalloc_scratch[kNoAllocFloats + 64];
// Device addresses of the array, one per device, filled on the first call for that device.  In host
// code the symbol itself is only a stand-in; the address a kernel can use comes from
// cudaGetSymbolAddress with the device current.
static std::atomic<float*> g_noalloc_ptr[kNoAllocMaxDevices];
}  // namespace

int xmc_large_k_matmul_noalloc(int32_t device, const void* a_bf16, const void* b, int32_t b_dtype,
                               int32_t k, int32_t m, int32_t n, float* c_f32, void* stream) {
  if (a_bf16 == nullptr || b == nullptr || c_f32 == nullptr) return fail(XMC_ERR_INVALID, "null argument");
  if (b_dtype != XMC_DT_BF16 && b_dtype != XMC_DT_E4M3) return fail(XMC_ERR_INVALID, "b must be bf16 or e4m3");
  if (k <= 0 || m <= 0 || n <= 0 || (m % 64) != 0 || (n % 64) != 0)
    return fail(XMC_ERR_INVALID, "need k > 0 and m, n positive multiples of 64 (got k %d, m %d, n %d)", k, m, n);
  if ((size_t)m * (size_t)n > kNoAllocFloats)
    return fail(XMC_ERR_INVALID, "m*n = %lld exceeds the built-in scratch of %lld floats (8 MiB): use the handle-based API",
                (long long)m * n, (long long)kNoAllocFloats);
  if (((uintptr_t)c_f32 & 15u) != 0 || ((uintptr_t)a_bf16 & 15u) != 0 || ((uintptr_t)b & 15u) != 0)
    return fail(XMC_ERR_INVALID, "a, b and c must be 16-byte aligned");
  if (device < 0 || device >= kNoAllocMaxDevices) return fail(XMC_ERR_INVALID, "device %d out of range", device);
  DeviceGuard guard(device);
  if (g_noalloc_ptr[device].load(std::memory_order_acquire) == nullptr) {
    // set-up, once per device, with that device current (the guard above)
    int cc_major = 0;
    CU_TRY(cudaDeviceGetAttribute(&cc_major, cudaDevAttrComputeCapabilityMajor, device));
    if (cc_major != 10) return fail(XMC_ERR_CUDA, "device %d is not sm_100", device);
    float* ptr = nullptr;
    CU_TRY(cudaGetSymbolAddress((void**)&ptr, g_noalloc_scratch));
    CU_TRY(cudaFuncSetAttribute(xmc::gradx_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, xmc::kGxSmemBytes<false>));
    CU_TRY(cudaFuncSetAttribute(xmc::gradx_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, xmc::kGxSmemBytes<false>));
    // two threads racing through the set-up compute the same address; the publication itself is atomic
    g_noalloc_ptr[device].store(ptr, std::memory_order_release);
  }
  float* scratch = g_noalloc_ptr[device].load(std::memory_order_acquire);
  int* status = reinterpret_cast<int*>(scratch + kNoAllocFloats);
  int sm_count = 0;
  CU_TRY(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device));
  cudaStream_t st = (cudaStream_t)stream;
  const bool f8 = b_dtype == XMC_DT_E4M3;
  CUtensorMap map_a, map_b;
  if (int rc = make_map_blocked(&map_a, false, a_bf16, m, k, m, xmc::kGxRows, true)) return rc;
  if (int rc = make_map_blocked(&map_b, f8, b, n, k, n, xmc::kGxRows, !f8)) return rc;
  xmc::GxParams gp;
  gp.bpad = m;
  gp.d = n;
  gp.n_btiles = cdiv(m, 256);
  gp.n_dtiles = cdiv(n, 256);
  const int tiles = gp.n_btiles * gp.n_dtiles;
  int n_splits = std::max(1, sm_count / tiles);
  n_splits = (int)std::min<size_t>((size_t)n_splits, kNoAllocFloats / ((size_t)m * n));
  gp.total_ksteps = cdiv(k, xmc::kGxRows);
  n_splits = std::max(1, std::min(n_splits, gp.total_ksteps));
  gp.n_splits = n_splits;
  gp.accumulate = 0;            // every slot in use is fully overwritten: nothing has to start at zero
  gp.partial = scratch;
  gp.status = status;           // zero in the library image; set by a kernel that gave up a wait, read and
                                // cleared by xmc_noalloc_check
  if (f8) xmc::gradx_kernel<true, false><<<tiles * n_splits, xmc::kGxThreads, xmc::kGxSmemBytes<false>, st>>>(map_a, map_b, gp);
  else xmc::gradx_kernel<false, false><<<tiles * n_splits, xmc::kGxThreads, xmc::kGxSmemBytes<false>, st>>>(map_a, map_b, gp);
  CU_TRY(cudaGetLastError());
  const long long total = (long long)m * n;
  const int blocks = (int)std::min<long long>((total + 255) / 256, (long long)sm_count * 8);
  xmc::reduce_gradx_kernel<<<blocks, 256, 0, st>>>(scratch, n_splits, m, m, n, 1.0f, c_f32, nullptr);
  CU_TRY(cudaGetLastError());
  return XMC_OK;
}

int xmc_noalloc_check(int32_t device, void* stream) {
  if (device < 0 || device >= kNoAllocMaxDevices) return fail(XMC_ERR_INVALID, "device %d out of range", device);
  float* scratch = g_noalloc_ptr[device].load(std::memory_order_acquire);
  if (scratch == nullptr) return XMC_OK;                 // no allocation-free call has run on this device yet
  DeviceGuard guard(device);
  cudaStream_t st = (cudaStream_t)stream;
  CU_TRY(cudaStreamSynchronize(st));
  int host[4] = {0, 0, 0, 0};                            // a stack array: this call allocates nothing either
  int* status = reinterpret_cast<int*>(scratch + kNoAllocFloats);
  CU_TRY(cudaMemcpy(host, status, sizeof(host), cudaMemcpyDeviceToHost));
  if (host[0] != xmc::DEV_OK) {
    CU_TRY(cudaMemset(status, 0, sizeof(host)));
    return fail(XMC_ERR_DEVICE_FLAG, "allocation-free contraction: device status %d (block %d, site %d)", host[0], host[1], host[2]);
  }
  return XMC_OK;
}

int xmc_test_sigmoid(int32_t device, const void* in_bf16, void* out_bf16, int32_t n, void* stream) {
  if (in_bf16 == nullptr || out_bf16 == nullptr || n <= 0) return fail(XMC_ERR_INVALID, "bad argument");
  DeviceGuard guard(device);
  xmc::sigmoid_probe_kernel<<<cdiv(n, 256), 256, 0, (cudaStream_t)stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(in_bf16), reinterpret_cast<__nv_bfloat16*>(out_bf16), n);
  CU_TRY(cudaGetLastError());
  return XMC_OK;
}

int xmc_test_gemm(int32_t device, int32_t layout, int32_t dtype, int32_t M, int32_t N, int32_t K,
                  const void* A, const void* B, float* D, void* stream) {
  if (A == nullptr || B == nullptr || D == nullptr || M <= 0 || N <= 0 || K <= 0) return fail(XMC_ERR_INVALID, "bad argument");
  const bool inject = (layout & 8) != 0;
  const bool pair = (layout & 4) != 0;
  layout &= ~12;
  if (layout < 0 || layout > 3) return fail(XMC_ERR_INVALID, "layout must be 0..3 (| 4 | 8)");
  if (pair && (layout & 1) != 0) return fail(XMC_ERR_INVALID, "CTA pairs take K-major operands");
  if (inject && ((layout & 1) != 0 || K < 2 * (dtype == XMC_DT_E4M3 ? 128 : 64)))
    return fail(XMC_ERR_INVALID, "the wait-limit test takes K-major operands with at least two k-steps");
  if ((layout & 1) == 1 && dtype != XMC_DT_BF16) return fail(XMC_ERR_INVALID, "MN-major test takes bf16");
  if (dtype != XMC_DT_BF16 && dtype != XMC_DT_E4M3) return fail(XMC_ERR_INVALID, "dtype");
  DeviceGuard guard(device);
  int cc_major = 0, sm_count = 0;
  CU_TRY(cudaDeviceGetAttribute(&cc_major, cudaDevAttrComputeCapabilityMajor, device));
  CU_TRY(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device));
  if (cc_major != 10) return fail(XMC_ERR_CUDA, "device is not sm_100");
  int* status = nullptr;
  CU_TRY(cudaMalloc((void**)&status, 16));
  CU_TRY(cudaMemset(status, 0, 16));
  cudaStream_t st = (cudaStream_t)stream;
  const bool f8 = dtype == XMC_DT_E4M3;
  CUtensorMap ma, mb;
  xmc::PlainParams p;
  p.M = M; p.N = N;
  p.n_ntiles = cdiv(N, 256);
  p.D = D;
  p.checksum_only = (layout & 2) ? 1 : 0;
  p.test_wait_limit = inject ? 2000000ll : 0;      // ~1 ms
  p.test_skip_tile = inject ? 0 : -1;
  layout &= 1;
  p.m_rows = pair ? 256 : 128;
  p.n_mtiles = cdiv(M, p.m_rows);
  p.status = status;
  int rc = XMC_OK;
  if (layout == 0) {
    if ((rc = make_map_kmajor(&ma, f8, A, K, M, K, 128))) { cudaFree(status); return rc; }
    // a CTA of a pair stages only its half of the B rows
    if ((rc = make_map_kmajor(&mb, f8, B, K, N, K, pair ? 128 : 256))) { cudaFree(status); return rc; }
    p.k_steps = cdiv((long long)K * (f8 ? 1 : 2), 128);
    const int tiles = p.n_mtiles * p.n_ntiles;
    if (pair) rc = f8 ? launch_gemm<xmc::PlainPolicy<true, false>, true>(ma, mb, p, tiles, sm_count, st)
                      : launch_gemm<xmc::PlainPolicy<false, false>, true>(ma, mb, p, tiles, sm_count, st);
    else rc = f8 ? launch_gemm<xmc::PlainPolicy<true, false>>(ma, mb, p, tiles, sm_count, st)
                 : launch_gemm<xmc::PlainPolicy<false, false>>(ma, mb, p, tiles, sm_count, st);
  } else {
    if ((rc = make_map_mnmajor(&ma, A, M, K, M))) { cudaFree(status); return rc; }
    if ((rc = make_map_mnmajor(&mb, B, N, K, N))) { cudaFree(status); return rc; }
    p.k_steps = cdiv(K, 64);
    rc = launch_gemm<xmc::PlainPolicy<false, true>>(ma, mb, p, p.n_mtiles * p.n_ntiles, sm_count, st);
  }
  if (rc == XMC_OK) {
    cudaError_t e = cudaStreamSynchronize(st);
    int host[4] = {0, 0, 0, 0};
    if (e == cudaSuccess) e = cudaMemcpy(host, status, 16, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) rc = fail(XMC_ERR_CUDA, "test gemm: %s", cudaGetErrorString(e));
    else if (host[0] != 0) rc = fail(XMC_ERR_DEVICE_FLAG, "test gemm: device status %d (block %d, site %d)", host[0], host[1], host[2]);
  }
  cudaFree(status);
  return rc;
}

}  // extern "C"


