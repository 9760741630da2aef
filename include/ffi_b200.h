/*
 * C ABI of the B200 (sm_100a) fixed-fan-in (FFI) sparse layer.
 *
 *   y[b,o]     = bias[o] + sum_k W[o,k] * x[b, idx[o,k]]
 *   grad_W[o,k] = sum_b g[b,o] * x[b, idx[o,k]]
 *   grad_x[b,i] = sum over (o,k) with idx[o,k]==i of W[o,k] * g[b,o]
 *   grad_b[o]   = sum_b g[b,o]
 *
 * Every pointer is a DEVICE pointer unless said otherwise; the caller owns all
 * tensors and every workspace.  All work is enqueued on `stream` (a cudaStream_t
 * passed as void*); no call synchronises the device except the plan functions,
 * which say so.  Every function returns an ffi_status; ffi_last_error() gives the
 * text of the calling thread's last failure.  Nothing here aborts the process.
 *
 * Layouts are the reference's (tfsparse/cc/kernels/kernel_data.cu.h:197-225), all
 * row-major: x is [B,N], or [N,B] when x_transposed != 0; idx and W are [L,K];
 * y and g are [B,L]; grad_x has the layout of x; grad_W the layout of W.
 * idx holds int32 or uint32 values in [0,N) (both index types the reference
 * registers, tfsparse/cc/kernels/register.cpp:79-109, share these entry points
 * because values are < 2^31 by the reference's contract, forward.cu:24-28).
 * Duplicate indices within a row are legal and add.
 */
#ifndef FFI_B200_H
#define FFI_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum ffi_status {
    FFI_OK = 0,
    FFI_ERR_INVALID_ARGUMENT = 1, /* null pointer, non-positive or oversize dimension */
    FFI_ERR_UNSUPPORTED = 2,      /* dtype / shape outside what the kernels cover */
    FFI_ERR_WORKSPACE = 3,        /* workspace missing or too small */
    FFI_ERR_CUDA = 4,             /* a CUDA runtime call or launch failed */
    FFI_ERR_STALE_PLAN = 5,       /* plan does not match (L,K,N) of the call */
    FFI_ERR_INDEX_RANGE = 6,      /* an index outside [0,N) was found while planning */
    FFI_ERR_ALLOC = 7             /* device allocation failed while planning */
} ffi_status;

/* Storage type of x and W.  Accumulation, bias, y, g and all gradients are fp32. */
typedef enum ffi_dtype { FFI_F32 = 0, FFI_BF16 = 1 } ffi_dtype;

typedef struct ffi_plan ffi_plan; /* opaque: transposed (CSR-by-input) index of one idx table */

/* Text of the calling thread's most recent error ("" if none). Host pointer. */
const char* ffi_last_error(void);

/* Library ABI version (major*100 + minor). */
int ffi_version(void);

/*
 * Debug bounds checking (off by default; also switched on by FFI_DEBUG_BOUNDS=1 in the environment).  When on,
 * ffi_forward, ffi_forward_loss and the backward entry points first check that every value of idx lies in
 * [0, N) and return FFI_ERR_INDEX_RANGE instead of launching their kernels: the counterpart of the device-side
 * index asserts of the reference's audit build (tfsparse/cc/kernels/kernel_data.cu.h:26-43,211), as a status
 * code instead of a trap.  Costs one pass over idx and a stream synchronisation per call.
 * Every entry point also opens an NVTX range of its own name, visible to a profiler that is attached.
 */
int ffi_set_debug_bounds(int on);

/* ---------------------------------------------------------------- forward ---- */

/* Bytes of scratch ffi_forward needs for this shape (0 when none is needed). */
size_t ffi_forward_workspace_bytes(int64_t B, int64_t N, int64_t L, int64_t K, int x_transposed,
                                   int dtype);

/*
 * y = FFI(x, idx, W) (+ bias when bias != NULL).
 * Replaces FixedFanInSparseMatmulKernel<GPUDevice,...>::operator()
 * (tfsparse/cc/kernels/forward.cu:35-74) as called from
 * FixedFanInSparseMatmulOp::Compute (tfsparse/cc/kernels/register.cpp:18-39):
 * x_transposed=0 is op "FanInSparseMatmul", x_transposed=1 is "FanInSparseMatmulTp".
 * The optional bias replaces the separate tf.nn.bias_add of sparse/layer.py:245-247.
 */
int ffi_forward(const void* x, const int32_t* idx, const void* W, const float* bias, float* y,
                int64_t B, int64_t N, int64_t L, int64_t K, int x_transposed, int dtype,
                void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------- plan ---- */

/*
 * Builds the transposed index of `idx` on the device: a stable sort of the flat
 * positions p = o*K+k by key idx[p] (ties by p), plus the chunked form the grad_x
 * kernel walks.  Allocates device memory owned by the plan, and synchronises
 * `stream` once (to report FFI_ERR_INDEX_RANGE).  Call again whenever idx changes
 * (the reference rewires idx in sparse/custom_layer.py:32-43).  No counterpart in
 * the reference, whose grad_x uses atomicAdd (tfsparse/cc/kernels/backward.cu.h:119-182).
 */
int ffi_plan_create(const int32_t* idx, int64_t L, int64_t K, int64_t N, void* stream,
                    ffi_plan** out_plan);

/*
 * Rebuilds `plan` in place from a table of the same (L, K, N) whose contents changed (after a rewiring
 * step): same result as destroying it and calling ffi_plan_create, without allocating or freeing the
 * index arrays.  The first rebuild of a plan allocates its sort scratch (about 17 bytes per connection)
 * and keeps it until ffi_plan_destroy; later rebuilds allocate nothing.  Synchronises `stream`.
 * FFI_ERR_INDEX_RANGE leaves the plan unusable until a rebuild succeeds.
 */
int ffi_plan_rebuild(ffi_plan* plan, const int32_t* idx, void* stream);

int ffi_plan_destroy(ffi_plan* plan);

/* Host-side description of a plan. Any out pointer may be NULL. */
int ffi_plan_info(const ffi_plan* plan, int64_t* L, int64_t* K, int64_t* N, int64_t* chunk_rows,
                  int64_t* n_chunks, int64_t* device_bytes);

/*
 * Copies the canonical transposed index into caller buffers: rowptr[N+1], perm[L*K]
 * (int32, device).  rowptr[i] = number of entries with key < i; perm lists positions
 * by (key, position) ascending.
 */
int ffi_plan_export(const ffi_plan* plan, int32_t* rowptr, int32_t* perm, void* stream);

/* Same, but re-derived from the chunked lists the grad_x kernel reads (a self-check). */
int ffi_plan_export_chunked(const ffi_plan* plan, int32_t* rowptr, int32_t* perm, void* stream);

/* --------------------------------------------------------------- backward ---- */

/* Bytes of scratch ffi_backward needs. `plan` may be NULL when want_grad_x == 0. */
size_t ffi_backward_workspace_bytes(const ffi_plan* plan, int64_t B, int64_t N, int64_t L, int64_t K,
                                    int x_transposed, int dtype, int want_grad_x, int want_grad_w);

/*
 * grad_x, grad_W and (optionally) grad_bias from the upstream gradient g[B,L].
 * Any of grad_x / grad_w / grad_bias may be NULL to skip it.  grad_x needs `plan`
 * (built from this idx); it is computed over the transposed index, without atomics,
 * in a summation order that depends only on (idx, shape), so it is bit-reproducible.
 * Replaces FixedFanInSparseMatmulGradKernel<GPUDevice,...>::operator()
 * (tfsparse/cc/kernels/backward.cu:87-133) as called from
 * FixedFanInSparseMatmulGradOp::Compute (tfsparse/cc/kernels/register.cpp:48-72):
 * x_transposed=0 is op "FanInSparseMatmulGrad", 1 is "FanInSparseMatmulGradTp".
 * grad_bias replaces TensorFlow's BiasAddGrad for sparse/layer.py:247.
 */
int ffi_backward(const void* x, const int32_t* idx, const void* W, const float* g,
                 const ffi_plan* plan, float* grad_x, float* grad_w, float* grad_bias, int64_t B,
                 int64_t N, int64_t L, int64_t K, int x_transposed, int dtype, void* workspace,
                 size_t workspace_bytes, void* stream);

/*
 * The upstream gradient transposed: g[B,L] -> gT[L][ldg] (batch contiguous, columns B..ldg-1
 * zero), ldg = ffi_transposed_gradient_stride(B); grad_bias (nullable, [L]) receives
 * sum_b g[b,o] from the same pass (TensorFlow's BiasAddGrad for sparse/layer.py:247).
 * ffi_backward does this internally; the function is public because ffi_grad_x_static takes gT
 * as an input, and because a loss kernel of the caller can produce gT directly and skip it.
 * No counterpart in the reference (its kernels read g[B,L] column-wise, backward.cu.h:62-185).
 */
int64_t ffi_transposed_gradient_stride(int64_t B);
int ffi_transpose_gradient(const float* g, float* gT, float* grad_bias, int64_t B, int64_t L,
                           void* stream);

/*
 * ffi_backward for a caller that already holds the transposed gradient gT[L][ldg] (from
 * ffi_forward_bce or ffi_transpose_gradient): no transposition pass.  grad_bias, when requested,
 * is the row sum of gT.  Every shape ffi_backward takes is covered.
 */
int ffi_backward_from_transposed(const void* x, const int32_t* idx, const void* W, const float* gT,
                                 int64_t ldg, const ffi_plan* plan, float* grad_x, float* grad_w,
                                 float* grad_bias, int64_t B, int64_t N, int64_t L, int64_t K,
                                 int x_transposed, int dtype, void* workspace, size_t workspace_bytes,
                                 void* stream);

/*
 * Forward pass with the sigmoid-BCE gradient fused into its epilogue: the B*L logits are never
 * written.  Output: gT[L][ldg] (ldg = ffi_transposed_gradient_stride(B)) with
 *   gT[o][b] = (sigmoid(z[b,o]) - t[b,o]) / (B * L_total),  z = FFI(x) + bias,
 * zero in the padded batch columns, ready for ffi_backward_from_transposed; *loss (device float,
 * may be NULL) receives the mean BCE over B*L_total.  Targets as in ffi_bce_grad (CSR, labels of
 * one row distinct; L_total / label_offset describe a label shard).  Replaces the chain
 * FanInSparseMatmulTp -> bias_add -> SparseBinaryCrossEntropyLoss -> its gradient
 * (sparse/custom_layer.py:45-50, sparse/layer.py:245-247, sparse/metrics.py:132-139,167-173).
 * Every shape ffi_forward takes is covered (wide inputs and K % 4 != 0 run the tiled forward kernel
 * with the same epilogue).  Workspace: 256-byte aligned, ffi_forward_bce_workspace_bytes bytes.
 */
size_t ffi_forward_bce_workspace_bytes(int64_t B, int64_t N, int64_t L, int64_t K, int x_transposed,
                                       int dtype);
int ffi_forward_bce(const void* x, const int32_t* idx, const void* W, const float* bias,
                    const int32_t* row_ptr, const int32_t* labels, float* gT, float* loss, int64_t B,
                    int64_t N, int64_t L, int64_t K, int64_t L_total, int64_t label_offset,
                    int x_transposed, int dtype, void* workspace, size_t workspace_bytes, void* stream);

/*
 * The same fused forward + loss-gradient pass for each sparse loss of the reference
 * (sparse/metrics.py:132-173): FFI_LOSS_BCE (as ffi_forward_bce), FFI_LOSS_SQUARED_HINGE (the
 * "squared_hinge" its task files select, SparseSquaredHingeLoss, metrics.py:157-164) and
 * FFI_LOSS_HINGE (SparseHingeLoss, metrics.py:146-154).  With m = (2t-1)*z and h = max(0, 1-m):
 *   squared hinge: loss = mean h^2,  gT[o][b] = -2*(2t-1)*h / (B*L_total)
 *   hinge:         loss = mean h,    gT[o][b] = -(2t-1)*[h > 0] / (B*L_total)
 * The exact zeros of these gradients are what the reference's backward kernels skip
 * (tfsparse/cc/kernels/backward.cu.h:73,94,131,151).
 */
typedef enum ffi_loss_kind { FFI_LOSS_BCE = 0, FFI_LOSS_SQUARED_HINGE = 1, FFI_LOSS_HINGE = 2 } ffi_loss_kind;
int ffi_forward_loss(int loss_kind, const void* x, const int32_t* idx, const void* W, const float* bias,
                     const int32_t* row_ptr, const int32_t* labels, float* gT, float* loss, int64_t B,
                     int64_t N, int64_t L, int64_t K, int64_t L_total, int64_t label_offset,
                     int x_transposed, int dtype, void* workspace, size_t workspace_bytes, void* stream);

/*
 * grad_x without any allocation and without a caller workspace.  This entry point has no
 * counterpart in the reference.
 *
 * Who it is for: callers that must not allocate device memory at the call site.  An op kernel
 * inside TensorFlow or PyTorch is supposed to get its scratch from the framework's allocator,
 * which normally owns nearly all GPU memory already, so a raw cudaMalloc there may fail or
 * stall every stream; a latency-bound serving loop cannot accept cudaMalloc's device-wide
 * synchronisation either.  Here the scratch of the narrow-input grad_x kernel (its per-range
 * partial sums) lives in a fixed __device__ array inside the library: 20 MiB
 * (ffi_grad_x_static_max_scratch_bytes()), held by every GPU that loads the library until the
 * process exits.  The call performs no cudaMalloc/cudaFree and calls no allocating routine.
 * The plan must have been built on the device that is current at the call (FFI_ERR_STALE_PLAN).
 *
 * Inputs: W[L,K]; gT, the upstream gradient ALREADY transposed to [L][ldg] (batch contiguous,
 * ldg a multiple of 32 and >= ffi_transposed_gradient_stride(B), columns B..ldg-1 zero, 16-byte
 * aligned) - the transposed copy
 * that ffi_backward builds inside its workspace is an input here; the plan of idx.
 * Output: grad_x in the layout of x ([N,B] when x_transposed, else [B,N]).
 *
 * Limits and rules:
 *  - shapes whose partial sums exceed the array (roughly (SMs/ceil(N/256)) * N * roundup(B) * 4
 *    bytes; the headline shape B=128, N=768 needs 18.4 MiB) are refused with FFI_ERR_WORKSPACE;
 *    use ffi_backward with a caller workspace for those;
 *  - the first call on each device looks up the array's device address
 *    (cudaGetSymbolAddress): make that first call before starting any stream capture.  With lazy
 *    module loading (the CUDA default) that lookup is also the moment the driver loads the module
 *    and sets the 20 MiB aside on that device, so the "no allocation" property holds for every call
 *    after the first one on a device, and the first one is the place to take that one-time cost;
 *  - all calls on a device share the one array, so two calls that may overlap on the GPU
 *    (different streams) race with each other: serialise them.  The array keeps the previous
 *    call's contents; nothing has to be cleared because every word a call reads it has
 *    written before in the same call.
 */
size_t ffi_grad_x_static_max_scratch_bytes(void);
int ffi_grad_x_static(const float* W, const float* gT, int64_t ldg, const ffi_plan* plan,
                      float* grad_x, int64_t B, int64_t N, int64_t L, int64_t K, int x_transposed,
                      void* stream);

/*
 * Forward whose epilogue keeps, per sample, the k (<= 8) highest logits of this table's rows instead
 * of writing y: top_val[B][k] and top_idx[B][k] (row + label_offset; -1 where L < k) in the order of
 * tf.nn.top_k (value descending, lower index first on ties).  It is what PrecisionAtK
 * (sparse/metrics.py:9-70: topk_as_matrix + the overlap with the true labels) needs from the
 * B x L logits, which here never reach HBM; with a sharded label dimension every shard returns
 * its own k candidates.  Every shape ffi_forward takes is covered, fp32 and bf16 storage: the
 * barrier-free kernel where the x tile is resident in shared memory and K % 4 == 0, the CTA-tile
 * kernel (wide inputs gathered from L2, any K, bf16 read directly) elsewhere.
 */
size_t ffi_forward_topk_workspace_bytes(int64_t B, int64_t N, int64_t L, int64_t K, int x_transposed,
                                        int dtype);
int ffi_forward_topk(const void* x, const int32_t* idx, const void* W, const float* bias,
                     float* top_val, int32_t* top_idx, int k, int64_t B, int64_t N, int64_t L,
                     int64_t K, int64_t label_offset, int x_transposed, int dtype, void* workspace,
                     size_t workspace_bytes, void* stream);

/*
 * Sum of the per-GPU grad_x partials of a label-sharded layer over peer memory, one launch per step
 * (the small-message alternative to an all-reduce; no counterpart in the single-GPU reference).
 * peer_bufs[r] / peer_flags[r] (host arrays of `world` device pointers) are rank r's buffer
 * [2][n] floats and flag array [2][world] words as mapped into THIS process (e.g. the peer pointers
 * of a symmetric allocation), flags zeroed once before the first step.  The caller has put its own
 * partial of this step into peer_bufs[rank] + (step & 1) * n on `stream`; `step` counts 1, 2, 3, ...
 * and is the same on all ranks.  out[n] receives the sum in rank order (identical bits on all ranks).
 * Waits on other ranks are bounded (see ffi_wait_timeouts).
 */
int ffi_peer_sum(const void* const* peer_bufs, void* const* peer_flags, int rank, int world,
                 int64_t n, uint32_t step, float* out, void* stream);

/*
 * The fused backward waits for its bulk copies, and ffi_peer_sum for the other GPUs, with a time
 * limit (about two seconds) instead of forever; a wait that runs out is counted and the kernel winds down.  *out receives the count since
 * the library was loaded: 0 in a healthy process, anything else voids the calls that ran since the
 * last check.  Synchronises the device.  No counterpart in the reference.
 */
int ffi_wait_timeouts(int* out);

/*
 * Test hook: sets how long the bounded waits above may last on the current device, in clock64 ticks
 * (about 0.5 ns each; the default, 4e9, is about two seconds; at least 1000).  A test of the give-up path
 * lowers it so that a wait nothing will ever satisfy ends after a millisecond.  No counterpart in the reference.
 */
int ffi_set_wait_limit_ticks(int64_t ticks);

/* ------------------------------------------------------------ loss / Adam ---- */

/*
 * Sigmoid binary cross-entropy against sparse multi-hot targets (CSR: row_ptr[B+1],
 * labels[nnz], device int32; labels of one row distinct).
 *   g[b,o]  = (sigmoid(z[b,o]) - t[b,o]) / (B * L_total)          (may alias z)
 *   *loss   = (1/(B*L_total)) * sum (max(z,0) - z*t + log1p(exp(-|z|)))   (device float, may be NULL)
 * L_total is the full label count the mean runs over; it differs from L when z is one
 * label shard [B,L] whose first label has global id label_offset (labels outside the
 * shard are ignored).  Replaces SparseBinaryCrossEntropyLoss (sparse/metrics.py:132-139,
 * 167-173 with sparse/utils.py:15-21) plus the Keras batch mean and its gradient.
 * loss_workspace: at least ffi_bce_workspace_bytes(B, L) bytes.
 */
size_t ffi_bce_workspace_bytes(int64_t B, int64_t L);
int ffi_bce_grad(const float* z, const int32_t* row_ptr, const int32_t* labels, float* g,
                 float* loss, int64_t B, int64_t L, int64_t L_total, int64_t label_offset,
                 void* workspace, size_t workspace_bytes, void* stream);

/*
 * One Adam step on n weights, fused into one pass: t = step (1-based),
 *   alpha = lr*sqrt(1-beta2^t)/(1-beta1^t); m += (g-m)(1-beta1); v += (g*g-v)(1-beta2);
 *   w -= alpha*m/(sqrt(v)+eps).
 * This is the update of keras.optimizers.Adam, which sparse/optimizer.py:9-12 derives
 * SparseAdam from (used at run.py:126).  w is fp32 or bf16 (dtype); m, v, grad are fp32.
 */
int ffi_adam_step(void* w, float* m, float* v, const float* grad, int64_t n, float lr, float beta1,
                  float beta2, float eps, int64_t step, int dtype, void* stream);

/* --------------------------------------------------------------- rewiring ---- */

/*
 * One rewiring step on the flat arrays of a layer (n = L*K connections), entirely on the device:
 *   threshold = the num_selected-th smallest |w|  (FixedFractionSelector.select, sparse/layer.py:62-86,
 *               where num_selected = round(fraction * n) is computed by the caller);
 *   every position p with |w[p]| < threshold (strictly, as tf.less) is rewired:
 *     idx[p] = a new source uniform in [0, n_in) (StratifiedRewireLayerV2._rewire,
 *              sparse/custom_layer.py:32-43; here splitmix64 of (seed, p), bits >> 1, mod n_in),
 *     m[p] = v[p] = 0 when the Adam moments are given (custom_layer.py:20-30, sparse/optimizer.py:14-23);
 *   w is not modified.
 * *threshold_out (device float) and *count_out (device int32, the number of rewired positions) may be
 * NULL.  num_selected = 0 rewires nothing.  idx changed: build a new plan before the next backward.
 * Workspace: ffi_rewire_workspace_bytes() bytes, 16-byte aligned.  No host synchronisation.
 */
size_t ffi_rewire_workspace_bytes(void);
int ffi_rewire(const float* w, int32_t* idx, float* m, float* v, int64_t n, int64_t n_in, int64_t num_selected,
               uint64_t seed, float* threshold_out, int32_t* count_out, void* workspace, size_t workspace_bytes,
               void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FFI_B200_H */
