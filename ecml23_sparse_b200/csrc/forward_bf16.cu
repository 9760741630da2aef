// Forward of the fixed-fan-in sparse layer for bf16 storage of x and W (fp32 accumulation, fp32 bias and
// output), narrow inputs: the native counterpart of ffi_fwd_pair_kernel (forward_stream.cu) for the
// benchmark configurations that keep x and W in bf16.  The reference has fp32 kernels only
// (tfsparse/cc/kernels/register.cpp:79-109); the arithmetic is the same sum as forward.cu.h:33-48 on
// the widened values (a bf16 value widens to fp32 exactly).
//
// What bf16 storage buys: the kernel is bound by the shared-memory pipe (one gathered operand per FMA), and
// a bf16 operand is half an fp32 one.  The whole batch tile of x, [N][128] bf16, fits shared memory (192 KB
// at N = 768), a HALF warp covers the 128 batch columns of a row with ONE 16-byte load per lane and entry
// (8 batch elements per lane), and the two halves of a warp work on the two rows of a row pair.  Per
// (row, k, 128 batch) that is 2 shared-memory wavefronts instead of the 4 (plus a second fetch of W and idx
// for the second batch tile) of the fp32 kernel.  Widening happens in the multiply: the two bf16 halves of a
// 32-bit word feed the mixed-precision FMA of sm_100 (`fma.rn.f32.bf16`: bf16 x bf16 + fp32, the product of
// two bf16 values being exact in fp32), which measured faster than shifting and masking the halves into
// fp32 registers for the two-wide fp32 FMA (0.29 vs 0.34 ms at B=128, N=768, L=670,091, K=32 with the loss
// epilogue).
//
// As in the fp32 kernel every warp is its own pipeline (private cp.async double buffer for the W / idx rows
// of the next row pair, private 4-row result tile); no CTA barrier in the steady state.
#include "ffi_common.cuh"

namespace ffi {
namespace {

constexpr int BT = 128;  // batch columns of the x tile
constexpr int S = BT + 8;  // result-tile row stride (floats)

struct FwdBf16Params {
    const __nv_bfloat16* xT;  // [N][ldx]
    long long ldx;
    const int* idx;
    const __nv_bfloat16* W;
    const float* bias;
    float* y;
    int B, N, L, K;
    // loss epilogue (MODE 1), as in forward_stream.cu
    float* gT;
    long long ldg;
    float scale;
    double* loss_partials;
    int loss_kind;
};

__device__ __forceinline__ void loss_negative_bf(int kind, float z, float& value, float& grad) {
    if (kind == 0) {
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

// Row record in a warp's buffer: K int32 indices, then K bf16 weights (6 K bytes; K % 8 == 0 keeps both parts
// 16-byte aligned).
template <int MODE>
__global__ void __launch_bounds__(512, 1) ffi_fwd_bf16_kernel(FwdBf16Params p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int nwarps = blockDim.x >> 5;
    const int h = lane >> 4;  // which row of a pair
    const int q = lane & 15;
    const int K = p.K, L = p.L;

    __nv_bfloat16* x_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);
    const int rowBytes = 6 * K;
    const int regionBytes = 4 * rowBytes + (MODE == 0 ? 4 * S * 4 : 0);
    unsigned char* region = smem_raw + static_cast<size_t>(p.N) * BT * 2 + static_cast<size_t>(warp) * regionBytes;
    unsigned char* wi = region;
    float* ys = reinterpret_cast<float*>(region + 4 * rowBytes);

    // x tile: x_s[i][b], zero for b >= B
    if (p.ldx % 8 == 0 && reinterpret_cast<uintptr_t>(p.xT) % 16 == 0) {
        const int vecPerRow = BT / 8;
        const int total = p.N * vecPerRow;
        for (int e = tid; e < total; e += blockDim.x) {
            const int i = e / vecPerRow;
            const int b = (e - i * vecPerRow) * 8;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (b + 8 <= p.B) {
                v = *reinterpret_cast<const uint4*>(p.xT + static_cast<size_t>(i) * p.ldx + b);
            } else if (b < p.B) {
                unsigned short t[8];
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    t[j] = b + j < p.B ? __bfloat16_as_ushort(p.xT[static_cast<size_t>(i) * p.ldx + b + j]) : 0;
                auto two = [](unsigned short lo, unsigned short hi) { return static_cast<unsigned>(lo) | (static_cast<unsigned>(hi) << 16); };
                v = make_uint4(two(t[0], t[1]), two(t[2], t[3]), two(t[4], t[5]), two(t[6], t[7]));
            }
            *reinterpret_cast<uint4*>(x_s + static_cast<size_t>(i) * BT + b) = v;
        }
    } else {
        const int total = p.N * BT;
        for (int e = tid; e < total; e += blockDim.x) {
            const int i = e / BT;
            const int b = e - i * BT;
            x_s[e] = b < p.B ? p.xT[static_cast<size_t>(i) * p.ldx + b] : __ushort_as_bfloat16(0);
        }
    }
    __syncthreads();

    const unsigned char* xs_lane = reinterpret_cast<const unsigned char*>(x_s) + q * 16;
    const long long numQuads = (static_cast<long long>(L) + 3) / 4;
    const long long gw = static_cast<long long>(blockIdx.x) * nwarps + warp;
    const long long GW = static_cast<long long>(gridDim.x) * nwarps;
    const int idxChunks = K / 4, wChunks = K / 8;
    const int chunksPerRow = idxChunks + wChunks;

    // W and idx rows of row pair `pr` (rows 2 pr, 2 pr + 1) -> buffer buf, 16 bytes per cp.async
    auto issue = [&](long long pr, int buf) {
        unsigned char* dstbuf = wi + buf * 2 * rowBytes;
        for (int c = lane; c < 2 * chunksPerRow; c += 32) {
            const int row = c / chunksPerRow;
            const int within = c - row * chunksPerRow;
            const long long o = 2 * pr + row;
            if (o < L) {
                if (within < idxChunks)
                    __pipeline_memcpy_async(dstbuf + row * rowBytes + 16 * within, p.idx + o * K + 4 * within, 16);
                else
                    __pipeline_memcpy_async(dstbuf + row * rowBytes + 4 * K + 16 * (within - idxChunks),
                                            p.W + o * K + 8 * (within - idxChunks), 16);
            }
        }
        __pipeline_commit();
    };

    long long qd = gw;
    if (qd < numQuads) issue(2 * qd, 0);
    int s = 0;
    float loss_local = 0.f;
    for (; qd < numQuads; qd += GW) {
#pragma unroll
        for (int half = 0; half < 2; ++half, ++s) {
            const int buf = s & 1;
            const long long pr = 2 * qd + half;
            const long long nextPr = half == 0 ? pr + 1 : 2 * (qd + GW);
            const bool haveNext = half == 0 ? (2 * nextPr < L) : (qd + GW < numQuads);
            if (haveNext) {
                issue(nextPr, buf ^ 1);
                __pipeline_wait_prior(1);
            } else {
                __pipeline_wait_prior(0);
            }
            __syncwarp();

            const long long oA = 2 * pr;
            if (oA < L) {
                const bool mine = oA + h < L;  // false only for the missing second row of an odd L
                const long long o = mine ? oA + h : oA;
                const unsigned char* row = wi + buf * 2 * rowBytes + (mine ? h : 0) * rowBytes;
                const int4* ir = reinterpret_cast<const int4*>(row);
                const uint4* wr = reinterpret_cast<const uint4*>(row + 4 * K);
                const float bias = p.bias ? __ldg(p.bias + o) : 0.f;
                float zz[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                for (int k8 = 0; k8 < K / 8; ++k8) {
                    const int4 ia = ir[2 * k8], ib = ir[2 * k8 + 1];
                    const uint4 w8 = wr[k8];
                    const int ii[8] = {ia.x, ia.y, ia.z, ia.w, ib.x, ib.y, ib.z, ib.w};
                    const unsigned ww[4] = {w8.x, w8.y, w8.z, w8.w};
                    uint4 xv[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u) xv[u] = *reinterpret_cast<const uint4*>(xs_lane + ii[u] * (BT * 2));
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        unsigned short wl, wh;
                        asm("mov.b32 {%0, %1}, %2;" : "=h"(wl), "=h"(wh) : "r"(ww[u >> 1]));
                        const unsigned short w16 = (u & 1) ? wh : wl;
                        const unsigned words[4] = {xv[u].x, xv[u].y, xv[u].z, xv[u].w};
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            unsigned short xl, xh;
                            asm("mov.b32 {%0, %1}, %2;" : "=h"(xl), "=h"(xh) : "r"(words[j]));
                            asm("fma.rn.f32.bf16 %0, %1, %2, %0;" : "+f"(zz[2 * j]) : "h"(xl), "h"(w16));
                            asm("fma.rn.f32.bf16 %0, %1, %2, %0;" : "+f"(zz[2 * j + 1]) : "h"(xh), "h"(w16));
                        }
                    }
                }
                float z[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) z[j] = zz[j];
                if constexpr (MODE == 1) {
                    float gv[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const bool live = 8 * q + j < p.B;
                        float v, g;
                        loss_negative_bf(p.loss_kind, z[j] + bias, v, g);
                        if (live && mine) loss_local += v;
                        gv[j] = live ? p.scale * g : 0.f;
                    }
                    if (mine && 8 * q < p.ldg) {
                        float* dst = p.gT + static_cast<size_t>(o) * p.ldg + 8 * q;
                        *reinterpret_cast<float4*>(dst) = make_float4(gv[0], gv[1], gv[2], gv[3]);
                        *reinterpret_cast<float4*>(dst + 4) = make_float4(gv[4], gv[5], gv[6], gv[7]);
                    }
                } else {
                    float* yrow = ys + (2 * half + h) * S + 8 * q;
                    *reinterpret_cast<float4*>(yrow) = make_float4(z[0] + bias, z[1] + bias, z[2] + bias, z[3] + bias);
                    *reinterpret_cast<float4*>(yrow + 4) = make_float4(z[4] + bias, z[5] + bias, z[6] + bias, z[7] + bias);
                }
            }
            __syncwarp();
        }
        if constexpr (MODE == 0) {
            const long long oq = 4 * qd;
#pragma unroll
            for (int it = 0; it < BT * 4 / 32; ++it) {
                const int id = it * 32 + lane;
                const int bl = id >> 2, oo = id & 3;
                if (bl < p.B && oq + oo < L) p.y[static_cast<size_t>(bl) * L + oq + oo] = ys[oo * S + bl];
            }
            __syncwarp();
        }
    }
    __pipeline_wait_prior(0);

    if constexpr (MODE == 1) {
        double v = static_cast<double>(loss_local);
#pragma unroll
        for (int off = 16; off >= 1; off /= 2) v += __shfl_xor_sync(0xffffffffu, v, off);
        __syncthreads();
        double* red = reinterpret_cast<double*>(smem_raw);
        if (lane == 0) red[warp] = v;
        __syncthreads();
        if (tid == 0) {
            double t = 0.0;
            for (int w = 0; w < nwarps; ++w) t += red[w];
            p.loss_partials[blockIdx.x] = t;
        }
    }
}

template <typename T>
__global__ void transpose_pad_any_kernel(const T* __restrict__ src, T* __restrict__ dst, int rows, int cols,
                                         long long ld_dst) {
    // src [rows][cols] -> dst [cols][ld_dst], dst[c][r] = src[r][c]; r in [rows, ld_dst) zero
    __shared__ T tile[32][33];
    const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
    for (int dy = threadIdx.y; dy < 32; dy += blockDim.y) {
        const int r = r0 + dy, c = c0 + threadIdx.x;
        tile[dy][threadIdx.x] = (r < rows && c < cols) ? src[static_cast<size_t>(r) * cols + c] : T(0.f);
    }
    __syncthreads();
    for (int dy = threadIdx.y; dy < 32; dy += blockDim.y) {
        const int c = c0 + dy, r = r0 + threadIdx.x;
        if (c < cols && r < ld_dst) dst[static_cast<size_t>(c) * ld_dst + r] = tile[threadIdx.x][dy];
    }
}

}  // namespace

// x [B,N] bf16 -> xT [N][ld_dst] bf16, zero padded
int launch_transpose_pad_bf16(const void* src, void* dst, int rows, int cols, int64_t ld_dst, cudaStream_t stream) {
    dim3 block(32, 8);
    dim3 grid(static_cast<unsigned>(ceil_div(cols, 32)), static_cast<unsigned>(ceil_div(ld_dst, 32)));
    transpose_pad_any_kernel<__nv_bfloat16><<<grid, block, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(src), static_cast<__nv_bfloat16*>(dst), rows, cols, ld_dst);
    FFI_LAUNCH_CHECK("transpose_pad_any_kernel");
    return FFI_OK;
}

// Warps per CTA the native bf16 forward can run with for this shape (0: not applicable).
int forward_bf16_warps(int64_t B, int64_t N, int64_t K, bool loss_epilogue) {
    DeviceInfo dev;
    if (get_device_info(&dev) != FFI_OK) return 0;
    if (B > BT || K % 8 != 0 || K <= 0) return 0;
    const size_t tile = static_cast<size_t>(N) * BT * 2;
    const size_t region = 4 * 6 * static_cast<size_t>(K) + (loss_epilogue ? 0 : 4 * S * 4);
    if (tile + 4 * region > static_cast<size_t>(dev.max_smem_optin)) return 0;
    size_t warps = (dev.max_smem_optin - tile) / region;
    if (warps > 16) warps = 16;
    return static_cast<int>(warps);
}

struct Bf16LossEpilogue {
    float* gT;
    long long ldg;
    float scale;
    double* loss_partials;
    int loss_kind;
    int* ctas;
};

// xT: bf16 [N][ldx]; W: bf16 [L][K].  *handled = false when the shape needs another path.
int launch_forward_bf16(const void* xT, int64_t ldx, const int32_t* idx, const void* W, const float* bias, float* y,
                        int64_t B, int64_t N, int64_t L, int64_t K, const Bf16LossEpilogue* loss, cudaStream_t stream,
                        bool* handled) {
    *handled = false;
    DeviceInfo dev;
    int rc = get_device_info(&dev);
    if (rc != FFI_OK) return rc;
    const int warps = forward_bf16_warps(B, N, K, loss != nullptr);
    if (warps < 4 || reinterpret_cast<uintptr_t>(W) % 16 != 0 || reinterpret_cast<uintptr_t>(idx) % 16 != 0) return FFI_OK;
    FwdBf16Params p;
    p.xT = static_cast<const __nv_bfloat16*>(xT);
    p.ldx = ldx;
    p.idx = idx;
    p.W = static_cast<const __nv_bfloat16*>(W);
    p.bias = bias;
    p.y = y;
    p.B = static_cast<int>(B);
    p.N = static_cast<int>(N);
    p.L = static_cast<int>(L);
    p.K = static_cast<int>(K);
    p.gT = loss ? loss->gT : nullptr;
    p.ldg = loss ? loss->ldg : 0;
    p.scale = loss ? loss->scale : 0.f;
    p.loss_partials = loss ? loss->loss_partials : nullptr;
    p.loss_kind = loss ? loss->loss_kind : 0;
    const size_t region = 4 * 6 * static_cast<size_t>(K) + (loss ? 0 : 4 * S * 4);
    const size_t smem = static_cast<size_t>(N) * BT * 2 + static_cast<size_t>(warps) * region;
    const long long numQuads = (L + 3) / 4;
    const long long want = (numQuads + warps - 1) / warps;
    const unsigned grid = static_cast<unsigned>(want < dev.sm_count ? want : dev.sm_count);
    *handled = true;
    if (loss) {
        auto kern = ffi_fwd_bf16_kernel<1>;
        FFI_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        *loss->ctas = static_cast<int>(grid);
        kern<<<grid, warps * 32, smem, stream>>>(p);
    } else {
        auto kern = ffi_fwd_bf16_kernel<0>;
        FFI_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        kern<<<grid, warps * 32, smem, stream>>>(p);
    }
    FFI_LAUNCH_CHECK("ffi_fwd_bf16_kernel");
    return FFI_OK;
}

}  // namespace ffi
