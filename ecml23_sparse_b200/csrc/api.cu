// extern "C" entry points of include/ffi_b200.h: argument checks, x layout handling,
// workspace carving and dispatch to the kernel launchers.
#include <cstring>
#include <mutex>

#include "ffi_common.cuh"

namespace ffi {

namespace {
thread_local char g_error[512] = "";
}

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

int fail(int status, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return status;
}

int get_device_info(DeviceInfo* info) {
    static std::mutex mu;
    static DeviceInfo cache[64];
    static bool known[64] = {};
    int dev = 0;
    FFI_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(FFI_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lock(mu);
    if (!known[dev]) {
        DeviceInfo d;
        int major = 0;
        FFI_CUDA_CHECK(cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev));
        FFI_CUDA_CHECK(cudaDeviceGetAttribute(&d.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
        FFI_CUDA_CHECK(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
        if (major != 10)
            return fail(FFI_ERR_UNSUPPORTED, "this library is built for sm_100a only (device is sm_%d*)", major * 10);
        cache[dev] = d;
        known[dev] = true;
    }
    *info = cache[dev];
    return FFI_OK;
}

// A plan's index arrays live on the GPU it was built on: a call made with another GPU current would
// hand its kernels pointers into that other GPU's memory.
int check_plan_device(const ffi_plan* plan) {
    int dev = -1;
    FFI_CUDA_CHECK(cudaGetDevice(&dev));
    if (plan && plan->device != dev)
        return fail(FFI_ERR_STALE_PLAN, "plan was built on device %d, the current device is %d", plan->device, dev);
    return FFI_OK;
}

struct Bf16LossEpilogue {
    float* gT;
    long long ldg;
    float scale;
    double* loss_partials;
    int loss_kind;
    int* ctas;
};
int launch_forward_bf16(const void* xT, int64_t ldx, const int32_t* idx, const void* W, const float* bias, float* y,
                        int64_t B, int64_t N, int64_t L, int64_t K, const Bf16LossEpilogue* loss, cudaStream_t stream,
                        bool* handled);
int forward_bf16_warps(int64_t B, int64_t N, int64_t K, bool loss_epilogue);
int launch_transpose_pad_bf16(const void* src, void* dst, int rows, int cols, int64_t ld_dst, cudaStream_t stream);

bool forward_uses_smem_x(int B, int N, int K, int* bpl_out);
int launch_widen_bf16(const void* src, float* dst, int64_t n, cudaStream_t stream);
bool grad_w_uses_smem_x(int B, int N, int K, int* bpl_out);

namespace {

constexpr size_t kAlign = 256;
size_t align_up(size_t v) { return (v + kAlign - 1) / kAlign * kAlign; }

int check_shape(int64_t B, int64_t N, int64_t L, int64_t K) {
    if (B <= 0 || N <= 0 || L <= 0 || K <= 0)
        return fail(FFI_ERR_INVALID_ARGUMENT, "B, N, L, K must be positive (got %lld, %lld, %lld, %lld)",
                    (long long)B, (long long)N, (long long)L, (long long)K);
    // Same bound as the reference (tfsparse/cc/kernels/forward.cu:24-28); L*K indexes int32 positions.
    const int64_t lim = (1LL << 31) - 1;
    if (B >= lim || N >= lim || L >= lim || K >= lim || L * K >= lim - 1024)
        return fail(FFI_ERR_UNSUPPORTED, "dimension too large for 32-bit indexing");
    return FFI_OK;
}

// How x reaches the kernels: either used in place ([N,B] input, shared-memory path) or
// copied into the workspace as xT[N][Bpad].
struct XPlan {
    bool copy = false;
    int64_t ld = 0;
    size_t bytes = 0;
};

XPlan plan_x(bool smem_path, int64_t B, int64_t N, int x_transposed) {
    XPlan xp;
    if (smem_path && x_transposed) {
        xp.copy = false;
        xp.ld = B;
        return xp;
    }
    xp.copy = true;
    xp.ld = round_up(B, 128);
    xp.bytes = align_up(static_cast<size_t>(N) * xp.ld * 4);
    return xp;
}

int stage_x(const XPlan& xp, const float* x, float* ws, int64_t B, int64_t N, int x_transposed,
            cudaStream_t stream, const float** xT) {
    if (!xp.copy) {
        *xT = x;
        return FFI_OK;
    }
    if (x_transposed) {
        if (xp.ld != B) FFI_CUDA_CHECK(cudaMemsetAsync(ws, 0, static_cast<size_t>(N) * xp.ld * 4, stream));
        FFI_CUDA_CHECK(cudaMemcpy2DAsync(ws, xp.ld * 4, x, B * 4, B * 4, N, cudaMemcpyDeviceToDevice, stream));
    } else {
        int rc = launch_transpose_pad(x, ws, static_cast<int>(B), static_cast<int>(N), xp.ld, stream);
        if (rc != FFI_OK) return rc;
    }
    *xT = ws;
    return FFI_OK;
}

// bf16 storage of x and W: both are widened to fp32 at the front of the workspace (exact), the
// fp32 kernels then run on the copies with the rest of the workspace.
size_t widen_bytes(int64_t B, int64_t N, int64_t L, int64_t K) {
    return align_up(static_cast<size_t>(B) * N * 4) + align_up(static_cast<size_t>(L) * K * 4);
}

int widen_inputs(const void* x, const void* W, int64_t B, int64_t N, int64_t L, int64_t K, void* workspace,
                 size_t workspace_bytes, cudaStream_t stream, const float** x32, const float** W32, void** rest,
                 size_t* rest_bytes) {
    const size_t need = widen_bytes(B, N, L, K);
    if (!workspace || workspace_bytes < need || reinterpret_cast<uintptr_t>(workspace) % kAlign != 0)
        return fail(FFI_ERR_WORKSPACE, "bf16 inputs need %zu bytes of %zu-byte aligned workspace for their fp32 copies",
                    need, kAlign);
    unsigned char* ws = static_cast<unsigned char*>(workspace);
    float* xd = reinterpret_cast<float*>(ws);
    float* wd = reinterpret_cast<float*>(ws + align_up(static_cast<size_t>(B) * N * 4));
    int rc = launch_widen_bf16(x, xd, B * N, stream);
    if (rc != FFI_OK) return rc;
    rc = launch_widen_bf16(W, wd, L * K, stream);
    if (rc != FFI_OK) return rc;
    *x32 = xd;
    *W32 = wd;
    *rest = ws + need;
    *rest_bytes = workspace_bytes - need;
    return FFI_OK;
}

// bf16 storage goes to the tiled forward kernel natively where the fp32 dispatch would take that kernel too
// (x too wide for shared memory, or K not a multiple of 4).
bool bf16_takes_tiled_forward(int64_t B, int64_t N, int64_t K) {
    return K % 4 != 0 || !forward_uses_smem_x(static_cast<int>(B), static_cast<int>(N), static_cast<int>(K), nullptr);
}

// stage_x for bf16 elements (esize 2): the same [N][ld] layouts, half the bytes.
int stage_x_any(const XPlan& xp, const void* x, void* ws, int64_t B, int64_t N, int x_transposed, size_t esize,
                cudaStream_t stream, const void** xT) {
    if (!xp.copy) {
        *xT = x;
        return FFI_OK;
    }
    if (x_transposed) {
        if (xp.ld != B) FFI_CUDA_CHECK(cudaMemsetAsync(ws, 0, static_cast<size_t>(N) * xp.ld * esize, stream));
        FFI_CUDA_CHECK(cudaMemcpy2DAsync(ws, xp.ld * esize, x, B * esize, B * esize, N, cudaMemcpyDeviceToDevice, stream));
    } else {
        const int rc = launch_transpose_pad_bf16(x, ws, static_cast<int>(B), static_cast<int>(N), xp.ld, stream);
        if (rc != FFI_OK) return rc;
    }
    *xT = ws;
    return FFI_OK;
}

// bf16 x as [N][ld]: used in place when it already is transposed, else transposed into the workspace.
int stage_x_bf16(const void* x, void* workspace, size_t workspace_bytes, int64_t B, int64_t N, int x_transposed,
                 cudaStream_t stream, const void** xT, int64_t* ldx) {
    if (x_transposed) {
        *xT = x;
        *ldx = B;
        return FFI_OK;
    }
    const int64_t ld = round_up(B, 128);
    const size_t need = static_cast<size_t>(N) * ld * 2;
    if (!workspace || workspace_bytes < need || reinterpret_cast<uintptr_t>(workspace) % 16 != 0)
        return fail(FFI_ERR_WORKSPACE, "bf16 x given as [B,N] needs %zu bytes of 16-byte aligned workspace", need);
    const int rc = launch_transpose_pad_bf16(x, workspace, static_cast<int>(B), static_cast<int>(N), ld, stream);
    if (rc != FFI_OK) return rc;
    *xT = workspace;
    *ldx = ld;
    return FFI_OK;
}

}  // namespace
}  // namespace ffi

using namespace ffi;

extern "C" const char* ffi_last_error(void) { return g_error; }

extern "C" int ffi_version(void) { return 100; }

extern "C" size_t ffi_forward_workspace_bytes(int64_t B, int64_t N, int64_t L, int64_t K, int x_transposed,
                                              int dtype) {
    if (check_shape(B, N, L, K) != FFI_OK || (dtype != FFI_F32 && dtype != FFI_BF16)) return 0;
    const bool smem = forward_uses_smem_x(static_cast<int>(B), static_cast<int>(N), static_cast<int>(K), nullptr);
    return plan_x(smem, B, N, x_transposed).bytes + (dtype == FFI_BF16 ? widen_bytes(B, N, L, K) : 0);
}

extern "C" int ffi_forward(const void* x, const int32_t* idx, const void* W, const float* bias, float* y,
                           int64_t B, int64_t N, int64_t L, int64_t K, int x_transposed, int dtype,
                           void* workspace, size_t workspace_bytes, void* stream_v) {
    FFI_TRACE("ffi_forward");
    if (!x || !idx || !W || !y) return fail(FFI_ERR_INVALID_ARGUMENT, "NULL tensor passed to ffi_forward");
    int rc = check_shape(B, N, L, K);
    if (rc != FFI_OK) return rc;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    if (debug_bounds_enabled()) {
        rc = check_index_range(idx, L * K, N, stream);
        if (rc != FFI_OK) return rc;
    }
    if (dtype == FFI_BF16) {
        // native bf16 kernel (x tile and W rows stay bf16 in shared memory) where the shape allows it
        if (forward_bf16_warps(B, N, K, false) >= 4) {
            const void* xT = nullptr;
            int64_t ldx = 0;
            rc = stage_x_bf16(x, workspace, workspace_bytes, B, N, x_transposed, stream, &xT, &ldx);
            if (rc != FFI_OK) return rc;
            bool handled = false;
            rc = launch_forward_bf16(xT, ldx, idx, W, bias, y, B, N, L, K, nullptr, stream, &handled);
            if (rc != FFI_OK || handled) return rc;
        }
        // wide inputs / odd fan-in: the tiled kernel reads bf16 x and W itself
        if (bf16_takes_tiled_forward(B, N, K)) {
            const XPlan xpb = plan_x(forward_uses_smem_x(static_cast<int>(B), static_cast<int>(N), static_cast<int>(K), nullptr),
                                     B, N, x_transposed);
            if (xpb.copy && (!workspace || workspace_bytes < xpb.bytes || reinterpret_cast<uintptr_t>(workspace) % 16 != 0))
                return fail(FFI_ERR_WORKSPACE, "ffi_forward needs %zu bytes of 16-byte aligned workspace, got %zu",
                            xpb.bytes, workspace_bytes);
            FwdArgs ab;
            rc = stage_x_any(xpb, x, workspace, B, N, x_transposed, 2, stream, &ab.xT);
            if (rc != FFI_OK) return rc;
            ab.ldx = xpb.ld;
            ab.idx = idx;
            ab.W = W;
            ab.bf16 = true;
            ab.bias = bias;
            ab.y = y;
            ab.B = static_cast<int>(B);
            ab.N = static_cast<int>(N);
            ab.L = static_cast<int>(L);
            ab.K = static_cast<int>(K);
            return launch_forward(ab, stream);
        }
        // otherwise both are widened (exactly) into the workspace and the fp32 kernels run
        const float *x32 = nullptr, *W32 = nullptr;
        void* rest = nullptr;
        size_t rest_bytes = 0;
        rc = widen_inputs(x, W, B, N, L, K, workspace, workspace_bytes, stream, &x32, &W32, &rest, &rest_bytes);
        if (rc != FFI_OK) return rc;
        return ffi_forward(x32, idx, W32, bias, y, B, N, L, K, x_transposed, FFI_F32, rest, rest_bytes, stream_v);
    }
    if (dtype != FFI_F32) return fail(FFI_ERR_UNSUPPORTED, "ffi_forward: dtype %d not supported", dtype);

    const bool smem = forward_uses_smem_x(static_cast<int>(B), static_cast<int>(N), static_cast<int>(K), nullptr);
    const XPlan xp = plan_x(smem, B, N, x_transposed);
    if (xp.copy && (!workspace || workspace_bytes < xp.bytes || reinterpret_cast<uintptr_t>(workspace) % 16 != 0))
        return fail(FFI_ERR_WORKSPACE, "ffi_forward needs %zu bytes of 16-byte aligned workspace, got %zu",
                    xp.bytes, workspace_bytes);
    const float* xT = nullptr;
    rc = stage_x(xp, static_cast<const float*>(x), static_cast<float*>(workspace), B, N, x_transposed, stream, &xT);
    if (rc != FFI_OK) return rc;

    FwdArgs a;
    a.xT = xT;
    a.ldx = xp.ld;
    a.idx = idx;
    a.W = static_cast<const float*>(W);
    a.bias = bias;
    a.y = y;
    a.B = static_cast<int>(B);
    a.N = static_cast<int>(N);
    a.L = static_cast<int>(L);
    a.K = static_cast<int>(K);
    return launch_forward(a, stream);
}

extern "C" int64_t ffi_transposed_gradient_stride(int64_t B) { return B > 0 ? transposed_g_stride(B) : 0; }

extern "C" int ffi_transpose_gradient(const float* g, float* gT, float* grad_bias, int64_t B, int64_t L,
                                      void* stream_v) {
    FFI_TRACE("ffi_transpose_gradient");
    if (!g || !gT) return fail(FFI_ERR_INVALID_ARGUMENT, "NULL tensor passed to ffi_transpose_gradient");
    if (B <= 0 || L <= 0 || B >= (1LL << 31) - 1 || L >= (1LL << 31) - 1)
        return fail(FFI_ERR_INVALID_ARGUMENT, "B and L must be positive and fit 32 bits");
    if (reinterpret_cast<uintptr_t>(gT) % 16 != 0) return fail(FFI_ERR_INVALID_ARGUMENT, "gT must be 16-byte aligned");
    return launch_transpose_g(g, gT, grad_bias, static_cast<int>(B), L, transposed_g_stride(B),
                              static_cast<cudaStream_t>(stream_v));
}

extern "C" size_t ffi_backward_workspace_bytes(const ffi_plan* plan, int64_t B, int64_t N, int64_t L, int64_t K,
                                               int x_transposed, int dtype, int want_grad_x, int want_grad_w) {
    if (check_shape(B, N, L, K) != FFI_OK || (dtype != FFI_F32 && dtype != FFI_BF16)) return 0;
    size_t total = dtype == FFI_BF16 ? widen_bytes(B, N, L, K) : 0;
    if (want_grad_w) {
        const bool smem = grad_w_uses_smem_x(static_cast<int>(B), static_cast<int>(N), static_cast<int>(K), nullptr);
        total += plan_x(smem, B, N, x_transposed).bytes;
    }
    if (want_grad_x && plan) {
        const size_t sep = grad_x_workspace_bytes(plan, B), fus = backward_fused_workspace_bytes(plan, B);
        total += align_up(sep > fus ? sep : fus);
        total += align_up(static_cast<size_t>(N) * round_up(B, 128) * 4);  // xT copy of the fused kernel
    }
    // the transposed upstream gradient gT[L][ldg], shared by grad_x and the barrier-free grad_W kernel
    if (want_grad_x || (want_grad_w && K % 4 == 0))
        total += align_up(static_cast<size_t>(L) * transposed_g_stride(B) * 4);
    return total;
}

// g is the upstream gradient [B,L]; alternatively gT_in (already transposed, stride ldg_in) is given.
static int backward_impl(const void* x, const int32_t* idx, const void* W, const float* g, const float* gT_in,
                         int64_t ldg_in, const ffi_plan* plan, float* grad_x, float* grad_w, float* grad_bias,
                         int64_t B, int64_t N, int64_t L, int64_t K, int x_transposed, int dtype, void* workspace,
                         size_t workspace_bytes, void* stream_v) {
    if (!x || !idx || !W || (!g && !gT_in)) return fail(FFI_ERR_INVALID_ARGUMENT, "NULL tensor passed to ffi_backward");
    int rc = check_shape(B, N, L, K);
    if (rc != FFI_OK) return rc;
    if (dtype != FFI_F32 && dtype != FFI_BF16) return fail(FFI_ERR_UNSUPPORTED, "ffi_backward: dtype %d not supported", dtype);
    if (debug_bounds_enabled()) {
        rc = check_index_range(idx, L * K, N, static_cast<cudaStream_t>(stream_v));
        if (rc != FFI_OK) return rc;
    }
    // bf16 storage: the group kernel (one pass, batch <= 128) and the kernels for wide inputs read bf16 x and W
    // themselves; for the other shapes both are widened (exactly) into the workspace and the fp32 kernels run.
    bool bf16 = false;
    if (dtype == FFI_BF16) {
        const bool one_pass = grad_x && grad_w && plan && backward_fused_takes_bf16(plan, B);
        const bool w_native = !(grad_w || grad_bias) ||
                              !grad_w_stream_applicable(static_cast<int>(B), static_cast<int>(N), static_cast<int>(K), idx);
        const bool x_native = !grad_x || (plan && !plan->has_chunks);
        bf16 = one_pass || (w_native && x_native && !(grad_x && grad_w && plan && backward_fused_applicable(plan, B)));
        if (!bf16) {
            const float *x32 = nullptr, *W32 = nullptr;
            void* rest = nullptr;
            size_t rest_bytes = 0;
            rc = widen_inputs(x, W, B, N, L, K, workspace, workspace_bytes, static_cast<cudaStream_t>(stream_v), &x32,
                              &W32, &rest, &rest_bytes);
            if (rc != FFI_OK) return rc;
            return backward_impl(x32, idx, W32, g, gT_in, ldg_in, plan, grad_x, grad_w, grad_bias, B, N, L, K,
                                 x_transposed, FFI_F32, rest, rest_bytes, stream_v);
        }
    }
    const size_t esize = bf16 ? 2 : 4;
    if (grad_x) {
        if (!plan) return fail(FFI_ERR_INVALID_ARGUMENT, "grad_x needs a plan (ffi_plan_create)");
        if (plan->L != L || plan->K != K || plan->N != N)
            return fail(FFI_ERR_STALE_PLAN, "plan was built for (L,K,N)=(%lld,%lld,%lld), call has (%lld,%lld,%lld)",
                        (long long)plan->L, (long long)plan->K, (long long)plan->N, (long long)L, (long long)K,
                        (long long)N);
        rc = check_plan_device(plan);
        if (rc != FFI_OK) return rc;
    }
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    unsigned char* ws = static_cast<unsigned char*>(workspace);
    size_t used = 0;
    if (workspace && reinterpret_cast<uintptr_t>(workspace) % kAlign != 0)
        return fail(FFI_ERR_WORKSPACE, "workspace must be %zu-byte aligned", kAlign);
    auto take = [&](size_t bytes, const char* what, void** out) -> int {
        bytes = align_up(bytes);
        if (!workspace || workspace_bytes < used + bytes)
            return fail(FFI_ERR_WORKSPACE, "ffi_backward needs %zu more bytes of workspace for %s", bytes, what);
        *out = ws + used;
        used += bytes;
        return FFI_OK;
    };
    const int Bi = static_cast<int>(B), Ni = static_cast<int>(N), Li = static_cast<int>(L), Ki = static_cast<int>(K);

    // One pass for grad_x and grad_W when the shape allows it, else one kernel each.
    const bool fused = grad_x && grad_w && backward_fused_applicable(plan, B);
    const bool sep_w = !fused && (grad_w || grad_bias);
    const bool gw_stream = sep_w && grad_w_stream_applicable(Bi, Ni, Ki, idx);

    // g transposed to [L][ldg] once, for the kernels that read whole batch rows of g; the same
    // pass produces grad_bias.
    const float* gT = gT_in;
    const int64_t ldg = gT_in ? ldg_in : transposed_g_stride(B);
    bool bias_done = false;
    if (gT_in) {
        if (ldg_in < B || ldg_in % 32 != 0 || reinterpret_cast<uintptr_t>(gT_in) % 16 != 0)
            return fail(FFI_ERR_INVALID_ARGUMENT, "gT needs a row stride that is a multiple of 32 and >= B, 16-byte aligned");
        if (grad_bias && !fused) {  // the fused backward sums grad_bias from the g tiles it loads
            rc = launch_bias_grad_rows(gT_in, ldg_in, L, grad_bias, stream);
            if (rc != FFI_OK) return rc;
            bias_done = true;
        }
    } else if (grad_x || gw_stream) {
        void* dst = nullptr;
        rc = take(static_cast<size_t>(L) * ldg * 4, "the transposed gradient", &dst);
        if (rc != FFI_OK) return rc;
        rc = launch_transpose_g(g, static_cast<float*>(dst), grad_bias, Bi, L, ldg, stream);
        if (rc != FFI_OK) return rc;
        gT = static_cast<const float*>(dst);
        bias_done = grad_bias != nullptr;
    }

    GradXArgs ax;
    ax.idx = idx;
    ax.W = W;
    ax.w_bf16 = bf16;
    ax.g = g;
    ax.gT = gT;
    ax.ldg = ldg;
    ax.plan = plan;
    ax.gx = grad_x;
    ax.x_transposed = x_transposed;
    ax.B = Bi;
    ax.N = Ni;
    ax.L = Li;
    ax.K = Ki;

    if (fused) {
        const void* xT = x;
        int64_t ldx = B;
        if (!x_transposed) {
            ldx = round_up(B, 128);
            void* dst = nullptr;
            rc = take(static_cast<size_t>(N) * ldx * esize, "the transposed x", &dst);
            if (rc != FFI_OK) return rc;
            rc = bf16 ? launch_transpose_pad_bf16(x, dst, Bi, Ni, ldx, stream)
                      : launch_transpose_pad(static_cast<const float*>(x), static_cast<float*>(dst), Bi, Ni, ldx, stream);
            if (rc != FFI_OK) return rc;
            xT = dst;
        }
        void* part = nullptr;
        rc = take(backward_fused_workspace_bytes(plan, B), "the grad_x partial sums", &part);
        if (rc != FFI_OK) return rc;
        ax.workspace = part;
        ax.workspace_bytes = workspace_bytes - (static_cast<unsigned char*>(part) - ws);
        return launch_backward_fused(ax, xT, ldx, grad_w, bias_done ? nullptr : grad_bias, stream);
    }

    if (grad_w || (grad_bias && !bias_done)) {
        const bool smem = grad_w_uses_smem_x(Bi, Ni, Ki, nullptr);
        const XPlan xp = plan_x(smem, B, N, x_transposed);
        void* xdst = nullptr;
        if (xp.copy) {
            rc = take(xp.bytes, "x", &xdst);
            if (rc != FFI_OK) return rc;
        }
        const void* xT = nullptr;
        if (bf16) {
            rc = stage_x_any(xp, x, xdst, B, N, x_transposed, 2, stream, &xT);
        } else {
            const float* xf = nullptr;
            rc = stage_x(xp, static_cast<const float*>(x), static_cast<float*>(xdst), B, N, x_transposed, stream, &xf);
            xT = xf;
        }
        if (rc != FFI_OK) return rc;
        GradWArgs a;
        a.xT = xT;
        a.bf16 = bf16;
        a.ldx = xp.ld;
        a.idx = idx;
        a.g = g;
        a.gT = gT;
        a.ldg = ldg;
        a.gW = grad_w;
        a.gbias = bias_done ? nullptr : grad_bias;
        a.B = Bi;
        a.N = Ni;
        a.L = Li;
        a.K = Ki;
        rc = launch_grad_w(a, stream);
        if (rc != FFI_OK) return rc;
    }
    if (grad_x) {
        ax.workspace = workspace ? ws + used : nullptr;
        ax.workspace_bytes = workspace_bytes > used ? workspace_bytes - used : 0;
        rc = launch_grad_x(ax, stream);
        if (rc != FFI_OK) return rc;
    }
    return FFI_OK;
}

extern "C" int ffi_backward(const void* x, const int32_t* idx, const void* W, const float* g,
                            const ffi_plan* plan, float* grad_x, float* grad_w, float* grad_bias, int64_t B,
                            int64_t N, int64_t L, int64_t K, int x_transposed, int dtype, void* workspace,
                            size_t workspace_bytes, void* stream_v) {
    FFI_TRACE("ffi_backward");
    if (!g) return fail(FFI_ERR_INVALID_ARGUMENT, "NULL tensor passed to ffi_backward");
    return backward_impl(x, idx, W, g, nullptr, 0, plan, grad_x, grad_w, grad_bias, B, N, L, K, x_transposed, dtype,
                         workspace, workspace_bytes, stream_v);
}

extern "C" int ffi_backward_from_transposed(const void* x, const int32_t* idx, const void* W, const float* gT,
                                            int64_t ldg, const ffi_plan* plan, float* grad_x, float* grad_w,
                                            float* grad_bias, int64_t B, int64_t N, int64_t L, int64_t K,
                                            int x_transposed, int dtype, void* workspace, size_t workspace_bytes,
                                            void* stream_v) {
    FFI_TRACE("ffi_backward_from_transposed");
    if (!gT) return fail(FFI_ERR_INVALID_ARGUMENT, "NULL tensor passed to ffi_backward_from_transposed");
    return backward_impl(x, idx, W, nullptr, gT, ldg, plan, grad_x, grad_w, grad_bias, B, N, L, K, x_transposed, dtype,
                         workspace, workspace_bytes, stream_v);
}

namespace ffi {
int launch_forward_bce_stream(const FwdArgs& a, float* gT, int64_t ldg, float scale, double* loss_partials, int* ctas,
                              int loss_kind, cudaStream_t stream, bool* handled);
int launch_forward_loss_tile(const FwdArgs& a, float* gT, int64_t ldg, float scale, double* loss_partials, int* ctas,
                             int loss_kind, cudaStream_t stream);
size_t forward_topk_workspace_bytes(int64_t B);
int launch_forward_topk_stream(const FwdArgs& a, void* scratch, float* top_val, int* top_idx, int kk, int label_offset,
                               cudaStream_t stream, bool* handled);
int launch_bce_positive_fix(const void* xT, int64_t ldx, const int* idx, const void* W, const float* bias,
                            const int* row_ptr, const int* labels, float* gT, int64_t ldg, float* loss,
                            const double* partials, int nPartials, double* pos_partials, float scale, int B,
                            int64_t L, int K, int64_t label_offset, int loss_kind, bool bf16, cudaStream_t stream);
constexpr size_t kBcePartialBytes = 1024 * sizeof(double);  // >= one partial per CTA of the forward kernel
}  // namespace ffi

extern "C" size_t ffi_forward_bce_workspace_bytes(int64_t B, int64_t N, int64_t L, int64_t K, int x_transposed,
                                                  int dtype) {
    return ffi_forward_workspace_bytes(B, N, L, K, x_transposed, dtype) + 2 * kAlign + kBcePartialBytes +
           static_cast<size_t>(B > 0 ? B : 0) * sizeof(double);
}

extern "C" int ffi_forward_loss(int loss_kind, const void* x, const int32_t* idx, const void* W, const float* bias,
                                const int32_t* row_ptr, const int32_t* labels, float* gT, float* loss, int64_t B,
                                int64_t N, int64_t L, int64_t K, int64_t L_total, int64_t label_offset,
                                int x_transposed, int dtype, void* workspace, size_t workspace_bytes, void* stream_v) {
    FFI_TRACE("ffi_forward_loss");
    if (!x || !idx || !W || !row_ptr || !labels || !gT)
        return fail(FFI_ERR_INVALID_ARGUMENT, "NULL tensor passed to ffi_forward_loss");
    if (loss_kind != FFI_LOSS_BCE && loss_kind != FFI_LOSS_SQUARED_HINGE && loss_kind != FFI_LOSS_HINGE)
        return fail(FFI_ERR_UNSUPPORTED, "unknown loss kind %d", loss_kind);
    int rc = check_shape(B, N, L, K);
    if (rc != FFI_OK) return rc;
    if (dtype != FFI_F32 && dtype != FFI_BF16)
        return fail(FFI_ERR_UNSUPPORTED, "ffi_forward_loss: dtype %d not supported", dtype);
    if (L_total < L) return fail(FFI_ERR_INVALID_ARGUMENT, "L_total must be >= L");
    if (reinterpret_cast<uintptr_t>(gT) % 16 != 0) return fail(FFI_ERR_INVALID_ARGUMENT, "gT must be 16-byte aligned");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    if (debug_bounds_enabled()) {
        rc = check_index_range(idx, L * K, N, stream);
        if (rc != FFI_OK) return rc;
    }
    if (!workspace || reinterpret_cast<uintptr_t>(workspace) % kAlign != 0 ||
        workspace_bytes < ffi_forward_bce_workspace_bytes(B, N, L, K, x_transposed, dtype))
        return fail(FFI_ERR_WORKSPACE, "ffi_forward_loss needs %zu bytes of %zu-byte aligned workspace",
                    ffi_forward_bce_workspace_bytes(B, N, L, K, x_transposed, dtype), kAlign);
    unsigned char* ws = static_cast<unsigned char*>(workspace);
    const bool bf16_tiled = dtype == FFI_BF16 && forward_bf16_warps(B, N, K, true) < 4 && bf16_takes_tiled_forward(B, N, K);
    if (dtype == FFI_BF16 && forward_bf16_warps(B, N, K, true) < 4 && !bf16_tiled) {
        // no native kernel for this shape: x and W are widened (exactly) at the front of the workspace
        const float *x32 = nullptr, *W32 = nullptr;
        void* rest = nullptr;
        size_t rest_bytes = 0;
        rc = widen_inputs(x, W, B, N, L, K, workspace, workspace_bytes, stream, &x32, &W32, &rest, &rest_bytes);
        if (rc != FFI_OK) return rc;
        return ffi_forward_loss(loss_kind, x32, idx, W32, bias, row_ptr, labels, gT, loss, B, N, L, K, L_total,
                                label_offset, x_transposed, FFI_F32, rest, rest_bytes, stream_v);
    }
    double* partials = reinterpret_cast<double*>(ws);
    double* pos_partials = reinterpret_cast<double*>(ws + align_up(kBcePartialBytes));
    float* xws = reinterpret_cast<float*>(ws + align_up(kBcePartialBytes) + align_up(static_cast<size_t>(B) * sizeof(double)));
    const float scale = static_cast<float>(1.0 / (static_cast<double>(B) * static_cast<double>(L_total)));
    const int64_t ldg = transposed_g_stride(B);
    if (bf16_tiled) {
        const XPlan xpb = plan_x(forward_uses_smem_x(static_cast<int>(B), static_cast<int>(N), static_cast<int>(K), nullptr),
                                 B, N, x_transposed);
        FwdArgs ab;
        rc = stage_x_any(xpb, x, xws, B, N, x_transposed, 2, stream, &ab.xT);
        if (rc != FFI_OK) return rc;
        ab.ldx = xpb.ld;
        ab.idx = idx;
        ab.W = W;
        ab.bf16 = true;
        ab.bias = bias;
        ab.y = nullptr;
        ab.B = static_cast<int>(B);
        ab.N = static_cast<int>(N);
        ab.L = static_cast<int>(L);
        ab.K = static_cast<int>(K);
        int ctas_t = 0;
        rc = launch_forward_loss_tile(ab, gT, ldg, scale, partials, &ctas_t, loss_kind, stream);
        if (rc != FFI_OK) return rc;
        return launch_bce_positive_fix(ab.xT, xpb.ld, idx, W, bias, row_ptr, labels, gT, ldg, loss, partials, ctas_t,
                                       pos_partials, scale, static_cast<int>(B), L, static_cast<int>(K), label_offset,
                                       loss_kind, true, stream);
    }
    if (dtype == FFI_BF16) {
        const size_t used = reinterpret_cast<unsigned char*>(xws) - ws;
        const void* xTb = nullptr;
        int64_t ldxb = 0;
        rc = stage_x_bf16(x, xws, workspace_bytes - used, B, N, x_transposed, stream, &xTb, &ldxb);
        if (rc != FFI_OK) return rc;
        int ctas_b = 0;
        bool handled_b = false;
        Bf16LossEpilogue e{gT, ldg, scale, partials, loss_kind, &ctas_b};
        rc = launch_forward_bf16(xTb, ldxb, idx, W, bias, nullptr, B, N, L, K, &e, stream, &handled_b);
        if (rc != FFI_OK) return rc;
        if (!handled_b) return fail(FFI_ERR_UNSUPPORTED, "ffi_forward_loss: unaligned bf16 W or idx");
        if (static_cast<size_t>(ctas_b) * sizeof(double) > kBcePartialBytes)
            return fail(FFI_ERR_UNSUPPORTED, "too many loss partials (%d)", ctas_b);
        return launch_bce_positive_fix(xTb, ldxb, idx, W, bias, row_ptr, labels, gT, ldg, loss, partials, ctas_b,
                                       pos_partials, scale, static_cast<int>(B), L, static_cast<int>(K), label_offset,
                                       loss_kind, true, stream);
    }

    const bool smem = forward_uses_smem_x(static_cast<int>(B), static_cast<int>(N), static_cast<int>(K), nullptr);
    const XPlan xp = plan_x(smem, B, N, x_transposed);
    const float* xT = nullptr;
    rc = stage_x(xp, static_cast<const float*>(x), xws, B, N, x_transposed, stream, &xT);
    if (rc != FFI_OK) return rc;
    FwdArgs a;
    a.xT = xT;
    a.ldx = xp.ld;
    a.idx = idx;
    a.W = static_cast<const float*>(W);
    a.bias = bias;
    a.y = nullptr;
    a.B = static_cast<int>(B);
    a.N = static_cast<int>(N);
    a.L = static_cast<int>(L);
    a.K = static_cast<int>(K);
    int ctas = 0;
    bool handled = false;
    rc = launch_forward_bce_stream(a, gT, ldg, scale, partials, &ctas, loss_kind, stream, &handled);
    if (rc != FFI_OK) return rc;
    if (!handled) {  // wide inputs or K % 4 != 0: the CTA-tile kernel with the same epilogue
        rc = launch_forward_loss_tile(a, gT, ldg, scale, partials, &ctas, loss_kind, stream);
        if (rc != FFI_OK) return rc;
    }
    if (static_cast<size_t>(ctas) * sizeof(double) > kBcePartialBytes)
        return fail(FFI_ERR_UNSUPPORTED, "too many loss partials (%d)", ctas);
    return launch_bce_positive_fix(xT, xp.ld, idx, a.W, bias, row_ptr, labels, gT, ldg, loss, partials, ctas,
                                   pos_partials, scale, static_cast<int>(B), L, static_cast<int>(K), label_offset, loss_kind,
                                   false, stream);
}

extern "C" size_t ffi_forward_topk_workspace_bytes(int64_t B, int64_t N, int64_t L, int64_t K, int x_transposed,
                                                   int dtype) {
    return ffi_forward_workspace_bytes(B, N, L, K, x_transposed, dtype) + kAlign + align_up(forward_topk_workspace_bytes(B));
}

extern "C" int ffi_forward_topk(const void* x, const int32_t* idx, const void* W, const float* bias, float* top_val,
                                int32_t* top_idx, int k, int64_t B, int64_t N, int64_t L, int64_t K,
                                int64_t label_offset, int x_transposed, int dtype, void* workspace,
                                size_t workspace_bytes, void* stream_v) {
    FFI_TRACE("ffi_forward_topk");
    if (!x || !idx || !W || !top_val || !top_idx)
        return fail(FFI_ERR_INVALID_ARGUMENT, "NULL tensor passed to ffi_forward_topk");
    int rc = check_shape(B, N, L, K);
    if (rc != FFI_OK) return rc;
    if (dtype != FFI_F32 && dtype != FFI_BF16)
        return fail(FFI_ERR_UNSUPPORTED, "ffi_forward_topk: dtype %d not supported", dtype);
    if (label_offset < 0 || label_offset + L >= (1LL << 31))
        return fail(FFI_ERR_INVALID_ARGUMENT, "label_offset + L must fit 31 bits");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    const size_t need = ffi_forward_topk_workspace_bytes(B, N, L, K, x_transposed, dtype);
    if (!workspace || reinterpret_cast<uintptr_t>(workspace) % kAlign != 0 || workspace_bytes < need)
        return fail(FFI_ERR_WORKSPACE, "ffi_forward_topk needs %zu bytes of %zu-byte aligned workspace", need, kAlign);
    const bool bf16 = dtype == FFI_BF16;
    if (bf16 && !bf16_takes_tiled_forward(B, N, K)) {
        // narrow inputs in bf16 storage: widened (exactly) into the workspace, then the fp32 kernels
        const float *x32 = nullptr, *W32 = nullptr;
        void* rest = nullptr;
        size_t rest_bytes = 0;
        rc = widen_inputs(x, W, B, N, L, K, workspace, workspace_bytes, stream, &x32, &W32, &rest, &rest_bytes);
        if (rc != FFI_OK) return rc;
        return ffi_forward_topk(x32, idx, W32, bias, top_val, top_idx, k, B, N, L, K, label_offset, x_transposed, FFI_F32,
                                rest, rest_bytes, stream_v);
    }
    unsigned char* ws = static_cast<unsigned char*>(workspace);
    void* lists = ws;
    void* xws = ws + align_up(forward_topk_workspace_bytes(B));

    const bool smem = forward_uses_smem_x(static_cast<int>(B), static_cast<int>(N), static_cast<int>(K), nullptr);
    const XPlan xp = plan_x(smem, B, N, x_transposed);
    FwdArgs a;
    if (bf16) {
        rc = stage_x_any(xp, x, xws, B, N, x_transposed, 2, stream, &a.xT);
    } else {
        const float* xT = nullptr;
        rc = stage_x(xp, static_cast<const float*>(x), static_cast<float*>(xws), B, N, x_transposed, stream, &xT);
        a.xT = xT;
    }
    if (rc != FFI_OK) return rc;
    a.ldx = xp.ld;
    a.idx = idx;
    a.W = W;
    a.bf16 = bf16;
    a.bias = bias;
    a.y = nullptr;
    a.B = static_cast<int>(B);
    a.N = static_cast<int>(N);
    a.L = static_cast<int>(L);
    a.K = static_cast<int>(K);
    bool handled = false;
    rc = launch_forward_topk_stream(a, lists, top_val, top_idx, k, static_cast<int>(label_offset), stream, &handled);
    if (rc != FFI_OK) return rc;
    if (!handled) return fail(FFI_ERR_UNSUPPORTED, "ffi_forward_topk: no kernel takes this shape");
    return FFI_OK;
}

extern "C" int ffi_forward_bce(const void* x, const int32_t* idx, const void* W, const float* bias,
                               const int32_t* row_ptr, const int32_t* labels, float* gT, float* loss, int64_t B,
                               int64_t N, int64_t L, int64_t K, int64_t L_total, int64_t label_offset, int x_transposed,
                               int dtype, void* workspace, size_t workspace_bytes, void* stream_v) {
    return ffi_forward_loss(FFI_LOSS_BCE, x, idx, W, bias, row_ptr, labels, gT, loss, B, N, L, K, L_total, label_offset,
                            x_transposed, dtype, workspace, workspace_bytes, stream_v);
}
