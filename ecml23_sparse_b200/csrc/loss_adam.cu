// Sigmoid-BCE gradient against sparse multi-hot targets, and the fused Adam step.
//
// ffi_bce_grad replaces the loss graph SparseBinaryCrossEntropyLoss builds
// (sparse/metrics.py:132-139,167-173; sparse/utils.py:15-21: a dense
// sigmoid_cross_entropy_with_logits over all B*L logits with zero targets, positives
// patched in by scatter, mean over labels, then the Keras mean over the batch) together
// with its gradient, in one dense pass plus a pass over the few positives.
// ffi_adam_step replaces the per-variable elementwise kernels of keras.optimizers.Adam
// (the base class of SparseAdam, sparse/optimizer.py:9-12).
// Both reductions run in a fixed order: results are bit-reproducible.
#include "ffi_common.cuh"

namespace ffi {
namespace {

constexpr int kBceBlocks = 1184;  // 8 per SM on a 148-SM part; fixed so the sum order is fixed
constexpr int kBceThreads = 256;

__device__ __forceinline__ float softplus_f(float z) { return fmaxf(z, 0.f) + log1pf(expf(-fabsf(z))); }
__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }

__device__ __forceinline__ double block_sum(double v, double* sh) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int off = 16; off >= 1; off /= 2) v += __shfl_xor_sync(0xffffffffu, v, off);
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    double t = 0.0;
    if (threadIdx.x == 0)
        for (int w = 0; w < (blockDim.x >> 5); ++w) t += sh[w];
    return t;  // valid in thread 0
}

// ws[0] = sum of z over the positives that fall in this shard.
__global__ void bce_positive_sum_kernel(const float* __restrict__ z, const int* __restrict__ row_ptr,
                                        const int* __restrict__ labels, int B, long long L,
                                        long long label_offset, double* __restrict__ ws) {
    __shared__ double sh[32];
    double s = 0.0;
    for (int b = 0; b < B; ++b) {
        const int lo = row_ptr[b], hi = row_ptr[b + 1];
        for (int e = lo + threadIdx.x; e < hi; e += blockDim.x) {
            const long long o = static_cast<long long>(labels[e]) - label_offset;
            if (o >= 0 && o < L) s += static_cast<double>(z[static_cast<size_t>(b) * L + o]);
        }
    }
    const double t = block_sum(s, sh);
    if (threadIdx.x == 0) ws[0] = t;
}

// g = scale * sigmoid(z) over the flat array; ws[1 + block] = sum softplus(z) of the block.
__global__ void __launch_bounds__(kBceThreads) bce_dense_kernel(const float* z, float* g, long long n,
                                                                float scale, double* __restrict__ ws,
                                                                int vec4) {
    __shared__ double sh[32];
    float local = 0.f;
    const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    if (vec4) {
        const long long n4 = n / 4;
        const float4* z4 = reinterpret_cast<const float4*>(z);
        float4* g4 = reinterpret_cast<float4*>(g);
        for (long long e = tid; e < n4; e += stride) {
            const float4 v = z4[e];
            local += (softplus_f(v.x) + softplus_f(v.y)) + (softplus_f(v.z) + softplus_f(v.w));
            g4[e] = make_float4(scale * sigmoid_f(v.x), scale * sigmoid_f(v.y), scale * sigmoid_f(v.z),
                                scale * sigmoid_f(v.w));
        }
        for (long long e = n4 * 4 + tid; e < n; e += stride) {
            const float v = z[e];
            local += softplus_f(v);
            g[e] = scale * sigmoid_f(v);
        }
    } else {
        for (long long e = tid; e < n; e += stride) {
            const float v = z[e];
            local += softplus_f(v);
            g[e] = scale * sigmoid_f(v);
        }
    }
    const double t = block_sum(static_cast<double>(local), sh);
    if (threadIdx.x == 0) ws[1 + blockIdx.x] = t;
}

// loss = scale * (sum of block partials - positive sum); g[b,label] -= scale at the positives.
__global__ void bce_finalize_kernel(const int* __restrict__ row_ptr, const int* __restrict__ labels,
                                    float* __restrict__ g, float* __restrict__ loss, int B, long long L,
                                    long long label_offset, float scale, const double* __restrict__ ws,
                                    int nPartials) {
    __shared__ double sh[32];
    for (int b = 0; b < B; ++b) {
        const int lo = row_ptr[b], hi = row_ptr[b + 1];
        for (int e = lo + threadIdx.x; e < hi; e += blockDim.x) {
            const long long o = static_cast<long long>(labels[e]) - label_offset;
            if (o >= 0 && o < L) g[static_cast<size_t>(b) * L + o] -= scale;
        }
    }
    if (loss) {
        double s = 0.0;
        for (int j = threadIdx.x; j < nPartials; j += blockDim.x) s += ws[1 + j];
        const double t = block_sum(s, sh);
        if (threadIdx.x == 0) *loss = static_cast<float>((t - ws[0]) * static_cast<double>(scale));
    }
}

// After the forward kernel with the fused loss epilogue, which took every target as 0: corrects gT at
// the positives (BCE: scale * (sigmoid(z) - 1); squared hinge: -2 * scale * max(0, 1 - z); hinge: -scale
// where z < 1), recomputing z of the few positive (b,o) pairs.  One block per sample; pos_partials[b] = the sample's sum of
// loss(z, target 1) - loss(z, target 0) over its positives (fixed order).
__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__global__ void __launch_bounds__(256) bce_positive_fix_kernel(
    const T* __restrict__ xT, long long ldx, const int* __restrict__ idx, const T* __restrict__ W,
    const float* __restrict__ bias, const int* __restrict__ row_ptr, const int* __restrict__ labels,
    float* __restrict__ gT, long long ldg, double* __restrict__ pos_partials, float scale, long long L, int K,
    long long label_offset, int loss_kind) {
    __shared__ double sh[32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int b = blockIdx.x;
    double possum = 0.0;  // kept by lane 0 of each warp
    const int lo = row_ptr[b], hi = row_ptr[b + 1];
    for (int e = lo + warp; e < hi; e += nwarps) {
        const long long o = static_cast<long long>(labels[e]) - label_offset;
        if (o < 0 || o >= L) continue;
        float z = 0.f;
        for (int k = lane; k < K; k += 32) {
            const int i = idx[o * K + k];
            z = fmaf(to_f32(W[o * K + k]), to_f32(xT[static_cast<size_t>(i) * ldx + b]), z);
        }
#pragma unroll
        for (int off = 16; off >= 1; off /= 2) z += __shfl_xor_sync(0xffffffffu, z, off);
        if (lane == 0) {
            z += bias ? bias[o] : 0.f;
            // possum collects loss(target 1) - loss(target 0) of this logit
            if (loss_kind == 0) {
                possum -= static_cast<double>(z);
                gT[static_cast<size_t>(o) * ldg + b] -= scale;
            } else {
                const float hp = fmaxf(1.f - z, 0.f), hn = fmaxf(1.f + z, 0.f);
                if (loss_kind == 1) {
                    possum += static_cast<double>(hp * hp) - static_cast<double>(hn * hn);
                    gT[static_cast<size_t>(o) * ldg + b] = -2.f * hp * scale;
                } else {
                    possum += static_cast<double>(hp) - static_cast<double>(hn);
                    gT[static_cast<size_t>(o) * ldg + b] = hp > 0.f ? -scale : 0.f;
                }
            }
        }
    }
    if (lane == 0) sh[warp] = possum;
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0.0;
        for (int w = 0; w < nwarps; ++w) t += sh[w];
        pos_partials[b] = t;
    }
}

// loss = scale * (sum of the forward kernel's CTA partials (all targets taken as 0) + the positives' corrections).
__global__ void __launch_bounds__(256) bce_loss_finalize_kernel(const double* __restrict__ partials, int nPartials,
                                                                const double* __restrict__ pos_partials, int B,
                                                                float scale, float* __restrict__ loss) {
    __shared__ double sh[32];
    double s = 0.0;
    for (int j = threadIdx.x; j < nPartials; j += blockDim.x) s += partials[j];
    for (int j = threadIdx.x; j < B; j += blockDim.x) s += pos_partials[j];
    const double t = block_sum(s, sh);
    if (threadIdx.x == 0) *loss = static_cast<float>(t * static_cast<double>(scale));
}

// grad_bias[o] = sum_b gT[o][b]: one warp per row of the transposed gradient, fixed lane tree.
__global__ void __launch_bounds__(256) bias_grad_rows_kernel(const float* __restrict__ gT, long long ldg,
                                                             long long L, float* __restrict__ gbias) {
    const int lane = threadIdx.x & 31;
    const long long o = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (o >= L) return;
    float s = 0.f;
    for (long long b = lane; b < ldg; b += 32) s += gT[static_cast<size_t>(o) * ldg + b];
#pragma unroll
    for (int off = 16; off >= 1; off /= 2) s += __shfl_xor_sync(0xffffffffu, s, off);
    if (lane == 0) gbias[o] = s;
}

template <bool BF16>
__global__ void __launch_bounds__(256) adam_kernel(void* __restrict__ w_v, float* __restrict__ m,
                                                   float* __restrict__ v, const float* __restrict__ grad,
                                                   long long n, float alpha, float omb1, float omb2,
                                                   float eps) {
    const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long e = tid; e < n; e += stride) {
        const float gj = grad[e];
        float mj = m[e], vj = v[e];
        mj += (gj - mj) * omb1;
        vj += (gj * gj - vj) * omb2;
        m[e] = mj;
        v[e] = vj;
        const float upd = alpha * mj / (sqrtf(vj) + eps);
        if (BF16) {
            __nv_bfloat16* w = static_cast<__nv_bfloat16*>(w_v);
            w[e] = __float2bfloat16_rn(__bfloat162float(w[e]) - upd);
        } else {
            float* w = static_cast<float*>(w_v);
            w[e] = w[e] - upd;
        }
    }
}

__global__ void __launch_bounds__(256) adam_kernel_f32x4(float4* __restrict__ w, float4* __restrict__ m,
                                                         float4* __restrict__ v,
                                                         const float4* __restrict__ grad, long long n4,
                                                         float alpha, float omb1, float omb2, float eps) {
    const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long e = tid; e < n4; e += stride) {
        const float4 gj = grad[e];
        float4 mj = m[e], vj = v[e], wj = w[e];
#define FFI_ADAM_LANE(c)                                     \
    mj.c += (gj.c - mj.c) * omb1;                            \
    vj.c += (gj.c * gj.c - vj.c) * omb2;                     \
    wj.c -= alpha * mj.c / (sqrtf(vj.c) + eps);
        FFI_ADAM_LANE(x) FFI_ADAM_LANE(y) FFI_ADAM_LANE(z) FFI_ADAM_LANE(w)
#undef FFI_ADAM_LANE
        m[e] = mj;
        v[e] = vj;
        w[e] = wj;
    }
}

// bf16 weights, four at a time: 8-byte accesses to w, 16-byte accesses to m, v and the gradient
__global__ void __launch_bounds__(256) adam_kernel_bf16x4(uint2* __restrict__ w, float4* __restrict__ m,
                                                          float4* __restrict__ v, const float4* __restrict__ grad,
                                                          long long n4, float alpha, float omb1, float omb2, float eps) {
    const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long e = tid; e < n4; e += stride) {
        const float4 gj = grad[e];
        float4 mj = m[e], vj = v[e];
        const uint2 wr = w[e];
        float4 wj = make_float4(bf16_lo(wr.x), bf16_hi(wr.x), bf16_lo(wr.y), bf16_hi(wr.y));
#define FFI_ADAM_LANE(c)                                     \
    mj.c += (gj.c - mj.c) * omb1;                            \
    vj.c += (gj.c * gj.c - vj.c) * omb2;                     \
    wj.c -= alpha * mj.c / (sqrtf(vj.c) + eps);
        FFI_ADAM_LANE(x) FFI_ADAM_LANE(y) FFI_ADAM_LANE(z) FFI_ADAM_LANE(w)
#undef FFI_ADAM_LANE
        m[e] = mj;
        v[e] = vj;
        const unsigned lo = __bfloat16_as_ushort(__float2bfloat16_rn(wj.x)) |
                            (static_cast<unsigned>(__bfloat16_as_ushort(__float2bfloat16_rn(wj.y))) << 16);
        const unsigned hi = __bfloat16_as_ushort(__float2bfloat16_rn(wj.z)) |
                            (static_cast<unsigned>(__bfloat16_as_ushort(__float2bfloat16_rn(wj.w))) << 16);
        w[e] = make_uint2(lo, hi);
    }
}

}  // namespace
}  // namespace ffi

namespace ffi {
namespace {
__global__ void __launch_bounds__(256) widen_bf16_kernel(const __nv_bfloat16* __restrict__ src, float* __restrict__ dst,
                                                         long long n) {
    const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long e = tid; e < n; e += stride) dst[e] = __bfloat162float(src[e]);
}
}  // namespace

// bf16 -> fp32 (exact).
int launch_widen_bf16(const void* src, float* dst, int64_t n, cudaStream_t stream) {
    const long long blocks = (n + 255) / 256;
    widen_bf16_kernel<<<static_cast<unsigned>(blocks < 1184 * 4 ? (blocks < 1 ? 1 : blocks) : 1184 * 4), 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(src), dst, n);
    FFI_LAUNCH_CHECK("widen_bf16_kernel");
    return FFI_OK;
}

// xT and W are fp32, or bf16 when `bf16` is set.
int launch_bce_positive_fix(const void* xT, int64_t ldx, const int* idx, const void* W, const float* bias,
                            const int* row_ptr, const int* labels, float* gT, int64_t ldg, float* loss,
                            const double* partials, int nPartials, double* pos_partials, float scale, int B,
                            int64_t L, int K, int64_t label_offset, int loss_kind, bool bf16, cudaStream_t stream) {
    if (bf16)
        bce_positive_fix_kernel<__nv_bfloat16><<<static_cast<unsigned>(B), 256, 0, stream>>>(
            static_cast<const __nv_bfloat16*>(xT), ldx, idx, static_cast<const __nv_bfloat16*>(W), bias, row_ptr, labels,
            gT, ldg, pos_partials, scale, L, K, label_offset, loss_kind);
    else
        bce_positive_fix_kernel<float><<<static_cast<unsigned>(B), 256, 0, stream>>>(
            static_cast<const float*>(xT), ldx, idx, static_cast<const float*>(W), bias, row_ptr, labels, gT, ldg,
            pos_partials, scale, L, K, label_offset, loss_kind);
    if (loss) bce_loss_finalize_kernel<<<1, 256, 0, stream>>>(partials, nPartials, pos_partials, B, scale, loss);
    FFI_LAUNCH_CHECK("bce_positive_fix_kernel");
    return FFI_OK;
}

int launch_bias_grad_rows(const float* gT, int64_t ldg, int64_t L, float* gbias, cudaStream_t stream) {
    bias_grad_rows_kernel<<<static_cast<unsigned>(ceil_div(L, 8)), 256, 0, stream>>>(gT, ldg, L, gbias);
    FFI_LAUNCH_CHECK("bias_grad_rows_kernel");
    return FFI_OK;
}
}  // namespace ffi

using namespace ffi;

extern "C" size_t ffi_bce_workspace_bytes(int64_t, int64_t) { return (1 + kBceBlocks) * sizeof(double); }

extern "C" int ffi_bce_grad(const float* z, const int32_t* row_ptr, const int32_t* labels, float* g,
                            float* loss, int64_t B, int64_t L, int64_t L_total, int64_t label_offset,
                            void* workspace, size_t workspace_bytes, void* stream_v) {
    FFI_TRACE("ffi_bce_grad");
    if (!z || !row_ptr || !labels || !g) return fail(FFI_ERR_INVALID_ARGUMENT, "NULL argument to ffi_bce_grad");
    if (B <= 0 || L <= 0 || L_total < L || B >= (1LL << 31))
        return fail(FFI_ERR_INVALID_ARGUMENT, "bad shape B=%lld L=%lld L_total=%lld", (long long)B,
                    (long long)L, (long long)L_total);
    if (!workspace || workspace_bytes < ffi_bce_workspace_bytes(B, L) ||
        reinterpret_cast<uintptr_t>(workspace) % 8 != 0)
        return fail(FFI_ERR_WORKSPACE, "ffi_bce_grad needs %zu bytes of 8-byte aligned workspace",
                    ffi_bce_workspace_bytes(B, L));
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    double* ws = static_cast<double*>(workspace);
    const float scale = static_cast<float>(1.0 / (static_cast<double>(B) * static_cast<double>(L_total)));
    const long long n = B * L;
    bce_positive_sum_kernel<<<1, 256, 0, stream>>>(z, row_ptr, labels, static_cast<int>(B), L, label_offset, ws);
    const int vec4 = reinterpret_cast<uintptr_t>(z) % 16 == 0 && reinterpret_cast<uintptr_t>(g) % 16 == 0;
    bce_dense_kernel<<<kBceBlocks, kBceThreads, 0, stream>>>(z, g, n, scale, ws, vec4);
    bce_finalize_kernel<<<1, 256, 0, stream>>>(row_ptr, labels, g, loss, static_cast<int>(B), L, label_offset,
                                               scale, ws, kBceBlocks);
    FFI_LAUNCH_CHECK("bce kernels");
    return FFI_OK;
}

extern "C" int ffi_adam_step(void* w, float* m, float* v, const float* grad, int64_t n, float lr, float beta1,
                             float beta2, float eps, int64_t step, int dtype, void* stream_v) {
    FFI_TRACE("ffi_adam_step");
    if (!w || !m || !v || !grad) return fail(FFI_ERR_INVALID_ARGUMENT, "NULL argument to ffi_adam_step");
    if (n <= 0 || step < 1) return fail(FFI_ERR_INVALID_ARGUMENT, "n must be positive and step >= 1");
    if (dtype != FFI_F32 && dtype != FFI_BF16) return fail(FFI_ERR_UNSUPPORTED, "unknown dtype %d", dtype);
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    const double t = static_cast<double>(step);
    const float alpha = static_cast<float>(static_cast<double>(lr) * sqrt(1.0 - pow(static_cast<double>(beta2), t)) /
                                           (1.0 - pow(static_cast<double>(beta1), t)));
    const float omb1 = 1.f - beta1, omb2 = 1.f - beta2;
    DeviceInfo dev;
    int rc = get_device_info(&dev);
    if (rc != FFI_OK) return rc;
    const unsigned blocks = static_cast<unsigned>(dev.sm_count * 8);
    if (dtype == FFI_BF16) {
        const bool aligned = reinterpret_cast<uintptr_t>(w) % 8 == 0 &&
                             ((reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v) |
                               reinterpret_cast<uintptr_t>(grad)) % 16) == 0;
        const long long n4 = aligned ? n / 4 : 0;
        if (n4 > 0)
            adam_kernel_bf16x4<<<blocks, 256, 0, stream>>>(static_cast<uint2*>(w), reinterpret_cast<float4*>(m),
                                                           reinterpret_cast<float4*>(v),
                                                           reinterpret_cast<const float4*>(grad), n4, alpha, omb1, omb2,
                                                           eps);
        const long long rest = n - n4 * 4;
        if (rest > 0)
            adam_kernel<true><<<aligned ? 1 : blocks, 256, 0, stream>>>(static_cast<__nv_bfloat16*>(w) + n4 * 4,
                                                                       m + n4 * 4, v + n4 * 4, grad + n4 * 4, rest, alpha,
                                                                       omb1, omb2, eps);
    } else {
        const bool aligned = ((reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(m) |
                               reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(grad)) % 16) == 0;
        const long long n4 = aligned ? n / 4 : 0;
        if (n4 > 0)
            adam_kernel_f32x4<<<blocks, 256, 0, stream>>>(static_cast<float4*>(w), reinterpret_cast<float4*>(m),
                                                          reinterpret_cast<float4*>(v),
                                                          reinterpret_cast<const float4*>(grad), n4, alpha, omb1,
                                                          omb2, eps);
        const long long rest = n - n4 * 4;
        if (rest > 0)
            adam_kernel<false><<<aligned ? 1 : blocks, 256, 0, stream>>>(
                static_cast<float*>(w) + n4 * 4, m + n4 * 4, v + n4 * 4, grad + n4 * 4, rest, alpha, omb1, omb2, eps);
    }
    FFI_LAUNCH_CHECK("adam kernels");
    return FFI_OK;
}
