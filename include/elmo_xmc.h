/*
 * C ABI of the B200 (sm_100a) chunked XMC classifier layer.
 *
 * This is the boundary a binding of the reference (xmc-aalto/elmo, 100 % Python) would call
 * through ctypes/cffi in place of its torch + Triton code.  Every function returns an int
 * status (0 = XMC_OK); none throws, aborts or allocates through any framework.  All data
 * pointers are DEVICE pointers owned by the caller unless stated otherwise; `stream` is a
 * cudaStream_t passed as void* (NULL = legacy default stream).  Calls only enqueue work on
 * `stream`; results are valid after the stream is synchronised.
 *
 * Reference interfaces replaced (paths relative to the reference's root):
 *   xmc_create / xmc_bind_weights  src/xmc_classifiers/chunked.py:17-46,
 *                                  src/xmc_classifiers/chunked_fp8xmc_clf.py:15-43 (constructors)
 *   xmc_step                       chunked.py:75-133  xfc_forward_backward (bf16 weights)
 *                                  chunked_fp8xmc_clf.py:81-123 xfc_forward_backward (e4m3
 *                                  weights, real and simulated FP8), including its kernels
 *                                  src/triton_kernels/matmul_kernel.py:204-239,342-353
 *                                  (large_k_matmul), src/triton_kernels/fuse_kernel.py:63-131
 *                                  (matmul_update), :134-199 (fakefp8_matmul_update),
 *                                  src/triton_kernels/stochastic_rounding_kernel.py:65-99 (sgd_update)
 *   xmc_forward_logits             chunked.py:48-53, chunked_fp8xmc_clf.py:45-60 xfc_forward
 *   xmc_forward_topk               src/evaluate.py:158-159,235-236 (xfc_forward + torch.topk)
 */
#ifndef ELMO_XMC_H_
#define ELMO_XMC_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* status codes */
enum {
  XMC_OK = 0,
  XMC_ERR_INVALID = 1,     /* bad argument (shape, alignment, enum)               */
  XMC_ERR_CUDA = 2,        /* a CUDA runtime/driver call failed                   */
  XMC_ERR_STATE = 3,       /* call order (weights not bound, ...)                 */
  XMC_ERR_DEVICE_FLAG = 4  /* a kernel reported a bounded-wait time-out or a bad label */
};

/* element types */
enum { XMC_DT_BF16 = 0, XMC_DT_E4M3 = 1, XMC_DT_F32 = 2, XMC_DT_E5M2 = 3 };

/* arithmetic of the forward contraction */
enum {
  XMC_MODE_BF16 = 0,   /* bf16 weights, bf16 x bf16 contractions (reference 'chunked' in bfloat16)   */
  XMC_MODE_FP8 = 1,    /* e4m3 weights, forward e4m3 x e4m3 (X cast to e4m3), backward in bf16        */
  XMC_MODE_SIMFP8 = 2  /* e4m3 weights up-converted to bf16, all contractions bf16 ('simulated_fp8') */
};

/* flags of xmc_step */
enum {
  XMC_STEP_COMPUTE_LOSS = 1,      /* skip_loss == False: write the summed BCE loss             */
  XMC_STEP_STOCHASTIC = 2,        /* stochastic rounding of W (else round-to-nearest-even)     */
  XMC_STEP_ROUND_DW_BF16 = 4,     /* round the dW accumulator to bf16 before the update, as the
                                     reference's 'chunked' class does by materialising dW
                                     (chunked.py:119)                                            */
  XMC_STEP_FP8_DW = 8             /* NOT the reference's arithmetic (fuse_kernel.py:88-92 multiplies
                                     bf16 operands): the dW contraction takes e4m3 operands,
                                     e4m3(G * 256) and e4m3(X), at twice the tensor rate.  Real-FP8
                                     mode only; grad_X keeps its bf16 operands.  Off by default.   */
};

typedef struct xmc_handle xmc_handle;

typedef struct {
  int32_t device;          /* CUDA device ordinal                                              */
  int32_t dim;             /* d, features per label row; multiple of 64                        */
  int32_t max_batch;       /* largest B a step will see (<= 65535)                             */
  int32_t mode;            /* XMC_MODE_*                                                       */
  int64_t label_offset;    /* global id of this handle's first label row (label-range shards)  */
  int64_t sched_labels;    /* labels per scheduling chunk (multiple of 128); 0 = choose so that
                              the chunk's logit-gradient tile stays L2 resident                */
  float w_scale;           /* real weight = stored weight * w_scale (per-tensor, constant);
                              1.0 reproduces the reference                                      */
  int32_t reserved;
} xmc_config;

/*
 * Create a handle and its workspaces on cfg->device (cudaMalloc; freed by xmc_destroy).
 * Side effect on the CUDA context: unless XMC_NO_L2_PERSIST is set in the environment, the call raises
 * cudaLimitPersistingL2CacheSize to the size of the grad_X partial sums (<= 38 MB on a B200); that much
 * L2 is then reserved for persisting lines process-wide.  xmc_step installs an access-policy window over
 * that private buffer on the caller's stream for the duration of its launches and removes it before it
 * returns; xmc_destroy resets the persisting lines.
 * The step kernels and the logits kernel are launched as thread-block clusters of two CTAs (CTA pairs,
 * tcgen05 cta_group::2) with programmatic stream serialization; the library asks the occupancy calculator
 * how many pairs the device holds and falls back to single-CTA kernels where it holds none.  Switches read
 * from the environment once per process, for debugging: XMC_NO_PAIRS (single CTAs everywhere), XMC_NO_PDL
 * (ordinary launches).
 */
int xmc_create(const xmc_config* cfg, xmc_handle** out);
int xmc_destroy(xmc_handle* h);

/*
 * Bind the weight storage: n_chunks row-major [rows[i] x dim] device arrays (bf16 in
 * XMC_MODE_BF16, else e4m3), 32-byte aligned, borrowed -- never freed by the library.
 * All chunks but the last must have the same number of rows.  The label rows of the handle are
 * the concatenation of the chunks; row r of the concatenation has global id label_offset + r.
 */
int xmc_bind_weights(xmc_handle* h, int32_t n_chunks, void* const* ptrs, const int64_t* rows);

/*
 * Kahan-compensated head (reference: src/xmc_classifiers/chunked_head_kahan_fp8xmc_clf.py:41-48,127-131,
 * src/triton_kernels/fuse_kernel.py:202-287): the first `rows` label rows (<= rows of the first weight
 * chunk) carry a compensation buffer D [rows x dim] (bf16 or e5m2, borrowed, updated in place):
 *   w = W + D - lr*acc;  W' = round(w);  D' = cast(D + W - W' - lr*acc).
 * Real-FP8 mode only; buf == NULL or rows == 0 removes it.
 */
int xmc_bind_kahan(xmc_handle* h, void* buf, int64_t rows, int32_t dtype);

/*
 * One train step over all bound label rows:
 *   Z = W X^T (per mode), G = sigmoid(Z) - Y, grad_X = w_scale * G^T W, W <- round(W - lr/w_scale * (G X)).
 * x        [batch x dim], x_dtype XMC_DT_BF16, row-major, contiguous
 * labels   int32 [nnz x 2] (batch row, GLOBAL label id); pairs outside this handle's label
 *          range are ignored, duplicates count once; may be NULL when nnz == 0
 * seed/step  Philox key / counter word for stochastic rounding
 * grad_x_f32 fp32 [batch x dim] or NULL;  grad_x_bf16 bf16 [batch x dim] or NULL
 * loss_out   device double, written when XMC_STEP_COMPUTE_LOSS is set (may be NULL otherwise)
 */
int xmc_step(xmc_handle* h, const void* x, int32_t x_dtype, int32_t batch,
             const int32_t* labels, int64_t nnz, float lr, float wd,
             uint64_t seed, uint64_t step, uint32_t flags,
             float* grad_x_f32, void* grad_x_bf16, double* loss_out, void* stream);

/*
 * Logits of all bound rows: out[b, r] = bf16(w_scale * <W[r], x[b]>) for r < n_out
 * (rows beyond n_out, e.g. the FP8 classes' padding, are not written).
 * x_dtype XMC_DT_BF16 or XMC_DT_E4M3 (the reference's evaluator hands in e4m3-cast embeds).
 * out is bf16 [batch x ld_out], ld_out >= n_out and a multiple of 8.
 */
int xmc_forward_logits(xmc_handle* h, const void* x, int32_t x_dtype, int32_t batch,
                       void* out_bf16, int64_t ld_out, int64_t n_out, void* stream);

/*
 * Fused logits + per-row top-k over rows r < n_out, without materialising the logits:
 * vals fp32 [batch x k] descending, idx int32 [batch x k] GLOBAL label ids
 * (label_offset + r); ties go to the lower id.  k <= 128.
 */
int xmc_forward_topk(xmc_handle* h, const void* x, int32_t x_dtype, int32_t batch, int32_t k,
                     int64_t n_out, float* vals, int32_t* idx, void* stream);

/*
 * Per-tensor scale bookkeeping (e4m3 modes).  The reference has none -- its scale is the constant 1.0
 * (src/xmc_classifiers/chunked_fp8xmc_clf.py:101-102) and Xavier-initialised weights of a 670 K-label
 * layer land on three e4m3 values (:29-32) -- so these calls have no counterpart there.
 *
 * xmc_weight_stats: one pass over the bound weights; synchronises `stream`.  counts (HOST array of 5):
 *   [0] zeros, [1] sub-normal magnitudes (0 < |w| < 2^-6 stored), [2] values at +-448, [3] NaN, [4] all
 *   elements; amax_stored (HOST float): largest stored magnitude.
 * xmc_rescale: scale <- scale * 2^shift and stored <- round(stored * 2^-shift), so that real weights keep
 *   their values: shift > 0 makes room at the top (what falls below the grid is rounded, to nearest or
 *   stochastically with the (seed, step) Philox stream), shift < 0 lifts small values into the normal
 *   range (exact up to saturation at +-448).  Subsequent steps use the new scale.
 * xmc_get_scale / xmc_set_scale: the scale in use; setting it declares what the stored weights mean
 *   (checkpoint restore) and rewrites nothing.
 */
int xmc_weight_stats(xmc_handle* h, int64_t* counts, float* amax_stored, void* stream);
int xmc_rescale(xmc_handle* h, int32_t shift, int32_t stochastic, uint64_t seed, uint64_t step, void* stream);
float xmc_get_scale(const xmc_handle* h);
int xmc_set_scale(xmc_handle* h, float scale);

/*
 * Synchronise `stream`, then read and clear the device status word.  Returns XMC_OK, or
 * XMC_ERR_DEVICE_FLAG with details in xmc_last_error (bounded wait expired inside a kernel,
 * label row >= batch, ...).
 */
int xmc_check(xmc_handle* h, void* stream);

/* Bytes of device memory the handle allocated for itself (workspaces; not the weights). */
int64_t xmc_workspace_bytes(const xmc_handle* h);

/* Number of kernels this handle has launched since creation (bench bookkeeping). */
int64_t xmc_launch_count(const xmc_handle* h);

/*
 * Per-kernel-class device timing for the bench.  While enabled, every kernel launched by the
 * handle is preceded by a CUDA event on its stream.  A call with non-NULL outputs waits for the
 * recorded events and returns, per class, the summed milliseconds and launch counts since the
 * previous call (8 entries: 0 prep/bucketing, 1 unused, 2 forward, 3 grad_X,
 * 4 update, 5 final reductions, 6 logits/top-k), then sets the mode to `enable`.
 */
int xmc_profile(xmc_handle* h, int32_t enable, double* ms_by_kind, int64_t* launches_by_kind);

/* Message of the most recent failing call on this thread ("" if none). */
const char* xmc_last_error(void);

/* Library build tag, e.g. "elmo_xmc sm_100a <date>". */
const char* xmc_version(void);

/*
 * C[m x n] (fp32) = A^T B for A stored [k x m] bf16 and B stored [k x n] (bf16 or e4m3): the
 * contraction over a very long k that grad_X needs, as a stand-alone call that ALLOCATES NOTHING.
 * This entry point has no counterpart in the reference (its large_k_matmul allocates its output and
 * runs wherever torch's allocator lets it).  It exists for callers that may not call cudaMalloc
 * where they invoke the library: code running under a memory pool that owns the whole device, inside
 * a region where allocation is forbidden (e.g. latency-critical serving loops), or plug-ins whose
 * host hands them buffers and nothing else.  The split-k partial sums that the kernel normally keeps
 * in a cudaMalloc'd workspace live in an 8 MiB array built into the library image instead (every GPU
 * that loads the library holds it until the process exits).
 *   - limit: m * n <= 2 097 152 (8 MiB of fp32); larger shapes are rejected with XMC_ERR_INVALID --
 *     use the handle-based API for those.  m and n must be multiples of 64; a, b and c 16-byte aligned.
 *   - the first call on a device looks up the array's device address and sets kernel attributes, which
 *     also makes the driver load the library's code and the 8 MiB array onto that device: make that
 *     first call outside any stream capture and before a pool takes all of the device's memory.
 *   - all calls share the one array and it keeps the last call's contents: two calls whose kernels
 *     overlap on the GPU (different streams) race.  Serialise them on one stream.  The first call per
 *     device may be made from several host threads at once (they agree on the address).
 *   - asynchronous on `stream`; neither cudaMalloc/cudaFree nor any allocating routine is called.
 *   - a kernel that gives up a bounded wait leaves a status word in the array; the call itself has long
 *     returned XMC_OK by then.  xmc_noalloc_check reads it.
 */
int xmc_large_k_matmul_noalloc(int32_t device, const void* a_bf16, const void* b, int32_t b_dtype,
                               int32_t k, int32_t m, int32_t n, float* c_f32, void* stream);

/*
 * Companion of xmc_large_k_matmul_noalloc, equally allocation-free and without a counterpart in the
 * reference: synchronise `stream`, then read and clear the status word the allocation-free kernels
 * report to (XMC_OK, or XMC_ERR_DEVICE_FLAG with block and wait site in xmc_last_error).
 */
int xmc_noalloc_check(int32_t device, void* stream);

/*
 * Test hook (not used by the layer classes): D[M x N] fp32 = A * B^T on the library's GEMM
 * engine, to validate the tensor-core path in isolation.
 *   layout 0: A [M x K], B [N x K] both K-major (row-major as written), dtype XMC_DT_BF16 or XMC_DT_E4M3
 *   layout 1: A given as [K x M], B as [K x N] row-major (both "MN-major"), dtype XMC_DT_BF16
 *   layout | 2: same contraction, but D is not stored (times the main loop alone)
 *   layout | 4 (with layout 0): the same contraction on CTA pairs (clusters of two, 256-row tiles)
 *   layout | 8 (with layout 0): exercises the kernels' failure handling without faulting anything: the
 *               producer leaves out one operand load of tile 0 and every wait of the launch is limited to
 *               about a millisecond, so the wait for that load gives up, the CTA unwinds, and the call
 *               returns XMC_ERR_DEVICE_FLAG naming the wait; D is then undefined, the context stays usable
 * M, N, K arbitrary positive (rows 16-byte aligned: inner extents multiples of 8 (bf16) / 16 (e4m3)).
 */
int xmc_test_gemm(int32_t device, int32_t layout, int32_t dtype, int32_t M, int32_t N, int32_t K,
                  const void* A, const void* B, float* D, void* stream);

/*
 * Test hook: out[i] = bf16(sigmoid(in[i])) for n bf16 values, computed exactly as the forward kernel's
 * epilogue computes the logit gradient (reference: torch.sigmoid on the bf16 logits,
 * src/xmc_classifiers/chunked_fp8xmc_clf.py:107).  Lets a test sweep all 65 536 bf16 inputs.
 */
int xmc_test_sigmoid(int32_t device, const void* in_bf16, void* out_bf16, int32_t n, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* ELMO_XMC_H_ */
