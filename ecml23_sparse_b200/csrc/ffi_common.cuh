// Internal helpers shared by the kernels behind include/ffi_b200.h (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_pipeline.h>
#include <cuda_runtime.h>
#include <nvtx3/nvToolsExt.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "ffi_b200.h"

namespace ffi {

// ---- error reporting ------------------------------------------------------------
void set_error(const char* fmt, ...);
int fail(int status, const char* fmt, ...);

#define FFI_CUDA_CHECK(expr)                                                               \
    do {                                                                                   \
        cudaError_t _e = (expr);                                                           \
        if (_e != cudaSuccess)                                                             \
            return ::ffi::fail(FFI_ERR_CUDA, "%s failed: %s (%s:%d)", #expr,               \
                               cudaGetErrorString(_e), __FILE__, __LINE__);                \
    } while (0)

#define FFI_LAUNCH_CHECK(name)                                                             \
    do {                                                                                   \
        cudaError_t _e = cudaGetLastError();                                               \
        if (_e != cudaSuccess)                                                             \
            return ::ffi::fail(FFI_ERR_CUDA, "launch of %s failed: %s", name,              \
                               cudaGetErrorString(_e));                                    \
    } while (0)

// ---- tracing: an NVTX range around every entry point (a no-op unless a profiler is attached) --------
struct TraceRange {
    explicit TraceRange(const char* name) { nvtxRangePushA(name); }
    ~TraceRange() { nvtxRangePop(); }
    TraceRange(const TraceRange&) = delete;
    TraceRange& operator=(const TraceRange&) = delete;
};
#define FFI_TRACE(name) ::ffi::TraceRange ffi_trace_range_(name)

// ---- debug bounds: with ffi_set_debug_bounds(1) (or FFI_DEBUG_BOUNDS=1 in the environment) every entry
// point that reads an index table first checks that all its values lie in [0, N) and returns
// FFI_ERR_INDEX_RANGE otherwise (one extra pass over idx and a stream synchronisation per call) ------------
bool debug_bounds_enabled();
int check_index_range(const int32_t* idx, int64_t n, int64_t N, cudaStream_t stream);

// ---- device properties (cached per device) ---------------------------------------
struct DeviceInfo {
    int sm_count = 0;
    int max_smem_optin = 0;  // bytes of dynamic shared memory one CTA may opt in to
};
int get_device_info(DeviceInfo* info);

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }
inline int64_t round_up(int64_t a, int64_t b) { return ceil_div(a, b) * b; }

// ---- vector of BPL batch elements held by one lane --------------------------------
template <int BPL>
struct Vec;
template <>
struct Vec<1> {
    using type = float;
};
template <>
struct Vec<2> {
    using type = float2;
};
template <>
struct Vec<4> {
    using type = float4;
};
template <>
struct Vec<8> {
    using type = uint4;  // eight bf16 values, still packed (bf16 storage only)
};

__device__ __forceinline__ float vec_get(const float& v, int) { return v; }
__device__ __forceinline__ float vec_get(const float2& v, int j) { return j == 0 ? v.x : v.y; }
__device__ __forceinline__ float vec_get(const float4& v, int j) {
    return j == 0 ? v.x : (j == 1 ? v.y : (j == 2 ? v.z : v.w));
}

__device__ __forceinline__ float vec_get(const uint4& v, int j) {
    const unsigned word = j < 2 ? v.x : (j < 4 ? v.y : (j < 6 ? v.z : v.w));
    return (j & 1) ? __uint_as_float(word & 0xffff0000u) : __uint_as_float(word << 16);
}

// ---- storage types of x and W: fp32 or bf16 (a bf16 value widens to fp32 exactly) ----------------
__device__ __forceinline__ float widen(float v) { return v; }
__device__ __forceinline__ float widen(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float bf16_lo(unsigned word) { return __uint_as_float(word << 16); }
__device__ __forceinline__ float bf16_hi(unsigned word) { return __uint_as_float(word & 0xffff0000u); }

// The BPL consecutive batch elements a lane holds, loaded from `base` (element type T) at vector index `v`.
template <int BPL>
__device__ __forceinline__ typename Vec<BPL>::type load_lane_vec(const float* base, size_t v) {
    return __ldg(reinterpret_cast<const typename Vec<BPL>::type*>(base) + v);
}
template <int BPL>
__device__ __forceinline__ typename Vec<BPL>::type load_lane_vec(const __nv_bfloat16* base, size_t v) {
    if constexpr (BPL == 8) {
        return __ldg(reinterpret_cast<const uint4*>(base) + v);
    } else if constexpr (BPL == 4) {
        const uint2 r = __ldg(reinterpret_cast<const uint2*>(base) + v);
        return make_float4(bf16_lo(r.x), bf16_hi(r.x), bf16_lo(r.y), bf16_hi(r.y));
    } else if constexpr (BPL == 2) {
        const unsigned r = __ldg(reinterpret_cast<const unsigned*>(base) + v);
        return make_float2(bf16_lo(r), bf16_hi(r));
    } else {
        return __bfloat162float(base[v]);
    }
}

// BPL consecutive fp32 values at base + lane * BPL (16-byte aligned rows)
template <int BPL>
__device__ __forceinline__ void load_lane_f32(const float* base, int lane, float (&out)[BPL]) {
    if constexpr (BPL >= 4) {
#pragma unroll
        for (int c = 0; c < BPL / 4; ++c) {
            const float4 t = __ldg(reinterpret_cast<const float4*>(base) + lane * (BPL / 4) + c);
            out[4 * c] = t.x, out[4 * c + 1] = t.y, out[4 * c + 2] = t.z, out[4 * c + 3] = t.w;
        }
    } else if constexpr (BPL == 2) {
        const float2 t = __ldg(reinterpret_cast<const float2*>(base) + lane);
        out[0] = t.x, out[1] = t.y;
    } else {
        out[0] = __ldg(base + lane);
    }
}
template <int BPL>
__device__ __forceinline__ void store_lane_f32(float* base, int lane, const float (&v)[BPL]) {
    if constexpr (BPL >= 4) {
#pragma unroll
        for (int c = 0; c < BPL / 4; ++c)
            reinterpret_cast<float4*>(base)[lane * (BPL / 4) + c] = make_float4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
    } else if constexpr (BPL == 2) {
        reinterpret_cast<float2*>(base)[lane] = make_float2(v[0], v[1]);
    } else {
        base[lane] = v[0];
    }
}

// ---- launchers implemented in the .cu files ---------------------------------------
// xT is x in [N][ldx] layout (batch contiguous); xT and W are fp32, or bf16 when `bf16` is set (only the
// tiled kernels take bf16; the callers see to that).
// loss and d(loss)/dz of one logit whose target is 0 (ffi_loss_kind: BCE, squared hinge, hinge);
// shared by the loss epilogues of all forward kernels, so that they agree bit for bit
__device__ __forceinline__ void loss_for_negative(int kind, float z, float& value, float& grad) {
    if (kind == 0) {
        // one exponential serves both: s = exp(-|z|), softplus(z) = max(z,0) + log(1+s),
        // sigmoid(z) = 1/(1+s) or s/(1+s); hardware approximations (a few ulp) are well inside 1e-5
        const float s = __expf(-fabsf(z));
        const float r = __fdividef(1.f, 1.f + s);
        value = fmaxf(z, 0.f) + __logf(1.f + s);
        grad = z >= 0.f ? r : s * r;
    } else {
        const float h = fmaxf(1.f + z, 0.f);
        value = kind == 1 ? h * h : h;
        grad = kind == 1 ? 2.f * h : (h > 0.f ? 1.f : 0.f);
    }
}

// Top-k epilogues of the forward kernels (evaluation: P@1, P@3, P@5 need 5 candidates per sample).
constexpr int kTopK = 8;  // capacity of a top-k list

// Sorted (value descending, row ascending) insertion; `better` orders candidates the way
// tf.nn.top_k does: higher value first, lower index on ties.
__device__ __forceinline__ bool topk_better(float v, int i, float v2, int i2) { return v > v2 || (v == v2 && i < i2); }
__device__ __forceinline__ void topk_insert(float (&tv)[kTopK], int (&ti)[kTopK], float v, int i) {
    if (!topk_better(v, i, tv[kTopK - 1], ti[kTopK - 1])) return;
    tv[kTopK - 1] = v;
    ti[kTopK - 1] = i;
#pragma unroll
    for (int j = kTopK - 1; j >= 1; --j) {
        if (topk_better(tv[j], ti[j], tv[j - 1], ti[j - 1])) {
            const float fv = tv[j];
            const int fi = ti[j];
            tv[j] = tv[j - 1], ti[j] = ti[j - 1];
            tv[j - 1] = fv, ti[j - 1] = fi;
        }
    }
}

struct FwdArgs {
    const void* xT;
    int64_t ldx;
    const int32_t* idx;
    const void* W;
    bool bf16 = false;
    const float* bias;
    float* y;
    int B, N, L, K;
};
int launch_forward(const FwdArgs& a, cudaStream_t stream);

struct GradWArgs {
    const void* xT;  // fp32, or bf16 when `bf16` is set (tiled kernel only)
    bool bf16 = false;
    int64_t ldx;
    const int32_t* idx;
    const float* g;
    const float* gT;  // g transposed to [L][ldg] (batch contiguous, zero padded), or nullptr
    int64_t ldg;
    float* gW;
    float* gbias;
    int B, N, L, K;
};
int launch_grad_w(const GradWArgs& a, cudaStream_t stream);
// True when launch_grad_w will take the barrier-free kernel, which reads gT instead of g.
bool grad_w_stream_applicable(int B, int N, int K, const void* idx);

// Row stride of the transposed upstream gradient gT[L][ldg] for a batch of B.
int64_t transposed_g_stride(int64_t B);
// g [B][L] -> gT [L][ldg], zero padded in the batch dimension; gbias (nullable) receives the
// column sums grad_bias[o] = sum_b g[b,o].
int launch_transpose_g(const float* g, float* gT, float* gbias, int B, int64_t L, int64_t ldg,
                       cudaStream_t stream);
// gbias[o] = sum_b gT[o][b]
int launch_bias_grad_rows(const float* gT, int64_t ldg, int64_t L, float* gbias, cudaStream_t stream);

// x [B,N] -> xT [N][ldx] (zero padded to ldx), fp32.
int launch_transpose_pad(const float* src, float* dst, int rows, int cols, int64_t ld_dst,
                         cudaStream_t stream);

}  // namespace ffi

// The plan object (defined in plan.cu, used by backward.cu and api.cu).
struct ffi_plan {
    int64_t L = 0, K = 0, N = 0;
    int device = 0;
    int chunk_rows = 0;     // T: outputs per chunk of the chunked lists
    int64_t n_chunks = 0;   // ceil(L / T)
    bool has_chunks = false;
    // largest number of entries any (chunk, slice of w consecutive inputs) holds, for w = 128, 256, 512, 1024
    int max_slice_entries[4] = {0, 0, 0, 0};
    int32_t* rowptr = nullptr;  // [N+1]   canonical CSR-by-input
    int32_t* perm = nullptr;    // [L*K]   positions sorted by (idx[p], p)
    int32_t* cperm = nullptr;   // [L*K]   chunk-major: chunk c holds its T*K positions sorted by (idx[p], p)
    int32_t* cptr = nullptr;    // [n_chunks][N+1] offsets of each input's run inside its chunk
    void* build_scratch = nullptr;  // sort scratch kept by ffi_plan_rebuild (none after ffi_plan_create alone)
    size_t device_bytes = 0;
};

namespace ffi {

// FFI_ERR_STALE_PLAN unless `plan` was built on the current device.
int check_plan_device(const ffi_plan* plan);

struct GradXArgs {
    const int32_t* idx;
    const void* W;       // fp32, or bf16 when w_bf16 is set (the wide-input kernel and the group kernel take bf16)
    bool w_bf16 = false;
    const float* g;
    const float* gT;  // as in GradWArgs; required by the narrow-input kernel
    int64_t ldg;
    const ffi_plan* plan;
    float* gx;
    int x_transposed;  // layout of gx: [N,B] if set, else [B,N]
    int B, N, L, K;
    void* workspace;
    size_t workspace_bytes;
};
size_t grad_x_workspace_bytes(const ffi_plan* plan, int64_t B);
// True when launch_grad_x will take the register-accumulator kernel, which reads gT.
bool grad_x_narrow_applicable(const ffi_plan* plan, int64_t B);
int launch_grad_x(const GradXArgs& a, cudaStream_t stream);

// grad_x and grad_W in one pass over the transposed index (narrow inputs, batch <= 128).
bool backward_fused_applicable(const ffi_plan* plan, int64_t B);
size_t backward_fused_workspace_bytes(const ffi_plan* plan, int64_t B);
bool backward_fused_takes_bf16(const ffi_plan* plan, int64_t B);
// xT (x as [N][ldx]) has the element type of a.W: fp32, or bf16 when a.w_bf16 is set.
int launch_backward_fused(const GradXArgs& a, const void* xT, int64_t ldx, float* gW, float* gbias,
                          cudaStream_t stream);

}  // namespace ffi
