// grad_W / grad_bias, barrier-free variant for the common case (x tile resident in shared
// memory, K a multiple of 4, 16-byte aligned idx).
//
// Same arithmetic, lane/batch geometry and butterfly reduction as ffi_grad_w_kernel
// (grad_w.cu), but every warp is its own pipeline: it takes row quads round-robin over the
// grid, prefetches the idx rows of the next row pair into a private shared-memory double
// buffer with its own cp.async, and keeps the g values of the next quad in registers
// (lane = batch element, four consecutive outputs per lane: the four 4-byte loads of a
// lane share one 32-byte sector).  No CTA-wide barrier in the steady state.
#include "ffi_common.cuh"

namespace ffi {
namespace {

constexpr int kThreads = 512;
constexpr int kWarps = kThreads / 32;

struct GradWStreamParams {
    const float* xT;
    long long ldx;
    const int* idx;
    const float* gT;   // upstream gradient transposed to [L][ldg]
    long long ldg;
    float* gW;
    float* gbias;
    int B, N, L, K;
    int b0;
    int accumulate;
};

template <int G>
__device__ __forceinline__ void butterfly_reduce_g(float (&s)[G], int lane) {
#pragma unroll
    for (int half = G / 2, off = 16; half >= 1; half /= 2, off /= 2) {
        const bool upper = (lane & off) != 0;
#pragma unroll
        for (int i = 0; i < half; ++i) {
            const float send = upper ? s[i] : s[i + half];
            const float keep = upper ? s[i + half] : s[i];
            s[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
        }
    }
    constexpr int consumed = G == 32 ? 5 : (G == 16 ? 4 : (G == 8 ? 3 : 2));
#pragma unroll
    for (int off = 16 >> consumed; off >= 1; off /= 2) s[0] += __shfl_xor_sync(0xffffffffu, s[0], off);
}

template <int BPL, int G>
__global__ void __launch_bounds__(kThreads, 1) ffi_grad_w_stream_kernel(GradWStreamParams p) {
    constexpr int BT = 32 * BPL;
    constexpr int LOG2G = G == 32 ? 5 : (G == 16 ? 4 : (G == 8 ? 3 : 2));
    using V = typename Vec<BPL>::type;
    extern __shared__ __align__(16) unsigned char smem_raw[];

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int b0 = p.b0;
    const int K = p.K, L = p.L;

    float* x_s = reinterpret_cast<float*>(smem_raw);
    int* ib = reinterpret_cast<int*>(x_s + static_cast<size_t>(p.N) * BT) + static_cast<size_t>(warp) * 4 * K;

    {
        const int total = p.N * BT;
#pragma unroll 8
        for (int e = tid; e < total; e += kThreads) {
            int i = e / BT;
            int bl = e - i * BT;
            int b = b0 + bl;
            float v = b < p.B ? p.xT[static_cast<size_t>(i) * p.ldx + b] : 0.f;
            x_s[i * BT + (bl & 31) * BPL + (bl >> 5)] = v;
        }
    }
    __syncthreads();

    const V* xs_lane = reinterpret_cast<const V*>(x_s) + lane;
    const long long numQuads = (static_cast<long long>(L) + 3) / 4;
    const long long gw = static_cast<long long>(blockIdx.x) * kWarps + warp;
    const long long GW = static_cast<long long>(gridDim.x) * kWarps;
    const int chunksPerRow = K / 4;
    const int nChunks = 2 * chunksPerRow;

    auto issue = [&](long long pr, int buf) {
        int* dst = ib + buf * 2 * K;
        for (int c = lane; c < nChunks; c += 32) {
            const int row = c / chunksPerRow;
            const int kc = c - row * chunksPerRow;
            const long long o = 2 * pr + row;
            if (o < L) __pipeline_memcpy_async(dst + row * K + 4 * kc, p.idx + o * K + 4 * kc, 16);
        }
        __pipeline_commit();
    };

    // g of a quad: gq[r][j] = g[b0 + lane + 32 j][4q + r]
    // read from the transposed gradient gT[L][ldg]: one coalesced 128-byte load per (row, j)
    auto load_g = [&](long long q, float (&dst)[4][BPL]) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const long long o = 4 * q + r;
            const float* row = p.gT + static_cast<size_t>(o) * p.ldg + b0 + lane;
#pragma unroll
            for (int j = 0; j < BPL; ++j) dst[r][j] = o < L ? __ldg(row + 32 * j) : 0.f;
        }
    };

    float gn[4][BPL];
    long long q = gw;
    if (q < numQuads) {
        issue(2 * q, 0);
        load_g(q, gn);
    }
    int s = 0;
    for (; q < numQuads; q += GW) {
        float gq[4][BPL];
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
            for (int j = 0; j < BPL; ++j) gq[r][j] = gn[r][j];
        if (q + GW < numQuads) load_g(q + GW, gn);

#pragma unroll
        for (int half = 0; half < 2; ++half, ++s) {
            const int buf = s & 1;
            const long long pr = 2 * q + half;
            const long long nextPr = half == 0 ? pr + 1 : 2 * (q + GW);
            const bool haveNext = half == 0 ? (2 * nextPr < L) : (q + GW < numQuads);
            if (haveNext) {
                issue(nextPr, buf ^ 1);
                __pipeline_wait_prior(1);
            } else {
                __pipeline_wait_prior(0);
            }
            __syncwarp();

#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const long long o = 2 * pr + r;
                if (o < L) {
                    float gv[BPL];
                    float gsum = 0.f;
#pragma unroll
                    for (int j = 0; j < BPL; ++j) {
                        gv[j] = gq[2 * half + r][j];
                        gsum += gv[j];
                    }
                    if (p.gbias) {
#pragma unroll
                        for (int off = 16; off >= 1; off /= 2) gsum += __shfl_xor_sync(0xffffffffu, gsum, off);
                        if (lane == 0) {
                            if (p.accumulate) p.gbias[o] += gsum;
                            else p.gbias[o] = gsum;
                        }
                    }
                    const int* ir = ib + buf * 2 * K + r * K;
                    for (int kg = 0; kg < K; kg += G) {
                        float sacc[G];
#pragma unroll
                        for (int k4 = 0; k4 < G / 4; ++k4) {
                            const int4 ii = *reinterpret_cast<const int4*>(ir + kg + 4 * k4);
                            const V v0 = xs_lane[ii.x * 32], v1 = xs_lane[ii.y * 32], v2 = xs_lane[ii.z * 32],
                                    v3 = xs_lane[ii.w * 32];
                            float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
                            for (int j = 0; j < BPL; ++j) {
                                a0 = fmaf(gv[j], vec_get(v0, j), a0);
                                a1 = fmaf(gv[j], vec_get(v1, j), a1);
                                a2 = fmaf(gv[j], vec_get(v2, j), a2);
                                a3 = fmaf(gv[j], vec_get(v3, j), a3);
                            }
                            sacc[4 * k4 + 0] = a0;
                            sacc[4 * k4 + 1] = a1;
                            sacc[4 * k4 + 2] = a2;
                            sacc[4 * k4 + 3] = a3;
                        }
                        butterfly_reduce_g<G>(sacc, lane);
                        const int k = kg + (lane >> (5 - LOG2G));
                        if (p.gW && (lane & ((1 << (5 - LOG2G)) - 1)) == 0) {
                            float* dst = p.gW + static_cast<size_t>(o) * K + k;
                            if (p.accumulate) *dst += sacc[0];
                            else *dst = sacc[0];
                        }
                    }
                }
            }
            __syncwarp();  // buffer `buf` may be overwritten by the next issue
        }
    }
    __pipeline_wait_prior(0);
}

template <int BPL, int G>
int launch_gws_t(GradWStreamParams p, size_t smem, int nBT, const DeviceInfo& dev, cudaStream_t stream) {
    auto kern = ffi_grad_w_stream_kernel<BPL, G>;
    FFI_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    int occ = 0;
    FFI_CUDA_CHECK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, kThreads, smem));
    if (occ < 1) return fail(FFI_ERR_CUDA, "streaming grad_W kernel does not fit on an SM (smem %zu)", smem);
    const long long numQuads = (static_cast<long long>(p.L) + 3) / 4;
    const long long want = (numQuads + kWarps - 1) / kWarps;
    const long long cap = static_cast<long long>(dev.sm_count) * occ;
    const unsigned grid = static_cast<unsigned>(want < cap ? want : cap);
    // Batch tiles run as consecutive launches so that tile t adds to what tile t-1 wrote.
    for (int bt = 0; bt < nBT; ++bt) {
        p.b0 = bt * 32 * BPL;
        p.accumulate = bt > 0;
        kern<<<grid, kThreads, smem, stream>>>(p);
        FFI_LAUNCH_CHECK("ffi_grad_w_stream_kernel");
    }
    return FFI_OK;
}

template <int BPL>
int launch_gws_g(const GradWStreamParams& p, int G, size_t smem, int nBT, const DeviceInfo& dev,
                 cudaStream_t stream) {
    switch (G) {
        case 32: return launch_gws_t<BPL, 32>(p, smem, nBT, dev, stream);
        case 16: return launch_gws_t<BPL, 16>(p, smem, nBT, dev, stream);
        case 8: return launch_gws_t<BPL, 8>(p, smem, nBT, dev, stream);
        default: return launch_gws_t<BPL, 4>(p, smem, nBT, dev, stream);
    }
}

}  // namespace

// Batch elements per lane the barrier-free kernel would use, 0 when it does not apply.
static int stream_bpl(int B, int N, int K, const void* idx, size_t* smem_out) {
    DeviceInfo dev;
    if (get_device_info(&dev) != FFI_OK) return 0;
    if (K % 4 != 0 || reinterpret_cast<uintptr_t>(idx) % 16 != 0) return 0;
    int bpl = B <= 32 ? 1 : (B <= 64 ? 2 : 4);
    for (; bpl >= 1; bpl /= 2) {
        const size_t smem = static_cast<size_t>(N) * 32 * bpl * 4 + static_cast<size_t>(kWarps) * 4 * K * 4;
        if (smem <= static_cast<size_t>(dev.max_smem_optin)) {
            if (smem_out) *smem_out = smem;
            return bpl;
        }
    }
    return 0;
}

bool grad_w_stream_applicable(int B, int N, int K, const void* idx) { return stream_bpl(B, N, K, idx, nullptr) > 0; }

// Launches the barrier-free kernel when the shape allows it; *handled tells the caller.
int launch_grad_w_stream(const GradWArgs& a, cudaStream_t stream, bool* handled) {
    *handled = false;
    DeviceInfo dev;
    int rc = get_device_info(&dev);
    if (rc != FFI_OK) return rc;
    size_t smem = 0;
    const int bpl = stream_bpl(a.B, a.N, a.K, a.idx, &smem);
    if (bpl < 1 || !a.gT || a.bf16) return FFI_OK;  // (this kernel reads fp32 x only)
    int G = 32;
    while (a.K % G != 0) G /= 2;  // K % 4 == 0, so G >= 4
    GradWStreamParams p;
    p.xT = static_cast<const float*>(a.xT);
    p.ldx = a.ldx;
    p.idx = a.idx;
    p.gT = a.gT;
    p.ldg = a.ldg;
    p.gW = a.gW;
    p.gbias = a.gbias;
    p.B = a.B;
    p.N = a.N;
    p.L = a.L;
    p.K = a.K;
    p.b0 = 0;
    p.accumulate = 0;
    const int nBT = static_cast<int>(ceil_div(a.B, 32 * bpl));
    *handled = true;
    if (bpl == 4) return launch_gws_g<4>(p, G, smem, nBT, dev, stream);
    if (bpl == 2) return launch_gws_g<2>(p, G, smem, nBT, dev, stream);
    return launch_gws_g<1>(p, G, smem, nBT, dev, stream);
}

}  // namespace ffi
