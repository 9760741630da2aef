// Forward of the fixed-fan-in sparse layer, barrier-free variant for the common case
// (x tile resident in shared memory, K a multiple of 4, 16-byte aligned W and idx).
//
// Same arithmetic and the same lane/batch geometry as ffi_fwd_kernel (forward.cu), but
// every warp is its own pipeline: it owns a private double buffer for the W/idx rows of
// the next row pair (filled by the warp's own cp.async: 2 rows x (W + idx) of K=32 are
// exactly one 16-byte copy per lane) and a private 4-row result tile, so the steady state
// has no CTA-wide barrier at all and the shared-memory pipe never drains at tile edges.
// Warps take row quads round-robin over the whole grid.  Results leave through the
// private tile as 16-byte runs along o (4 consecutive outputs per batch row).
#include "ffi_common.cuh"

namespace ffi {
namespace {

constexpr int kThreads = 512;
constexpr int kWarps = kThreads / 32;

struct FwdStreamParams {
    const float* xT;
    long long ldx;
    const int* idx;
    const float* W;
    const float* bias;
    float* y;
    int B, N, L, K;
    // fused sigmoid-BCE epilogue (BCE variant): instead of y the kernel writes the loss gradient,
    // already transposed, gT[o][b] = scale * sigmoid(z[b,o]) (positives are corrected afterwards),
    // and one partial sum of softplus(z) per CTA
    float* gT;
    long long ldg;
    float scale;
    double* loss_partials;
    int loss_kind;  // ffi_loss_kind: BCE, squared hinge or hinge (for target 0; positives are corrected afterwards)
};

// loss and d(loss)/dz of one logit whose target is 0
__device__ __forceinline__ void loss_negative(int kind, float z, float& value, float& grad) {
    if (kind == 0) {
        value = fmaxf(z, 0.f) + log1pf(expf(-fabsf(z)));
        grad = 1.f / (1.f + expf(-z));
    } else {
        const float h = fmaxf(1.f + z, 0.f);
        value = kind == 1 ? h * h : h;
        grad = kind == 1 ? 2.f * h : (h > 0.f ? 1.f : 0.f);
    }
}

template <int BPL, bool BCE>
__global__ void __launch_bounds__(kThreads, 1) ffi_fwd_stream_kernel(FwdStreamParams p) {
    constexpr int BT = 32 * BPL;
    constexpr int S = BT + 8;  // result-tile row stride: conflict-free for both access patterns
    using V = typename Vec<BPL>::type;
    extern __shared__ __align__(16) unsigned char smem_raw[];

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int b0 = blockIdx.y * BT;
    const int K = p.K, L = p.L;

    float* x_s = reinterpret_cast<float*>(smem_raw);
    // per-warp region: wi[2 buffers][2 rows][W[K] | idx[K]] then ys[4][S]
    const int regionWords = 8 * K + 4 * S;
    float* region = x_s + static_cast<size_t>(p.N) * BT + static_cast<size_t>(warp) * regionWords;
    float* wi = region;
    float* ys = region + 8 * K;

    {
        // x_s[i][lane*BPL + j] holds batch element b0 + lane + 32*j.
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
    const int chunksPerRow = K / 2;     // 16-byte chunks of one row: K/4 of W then K/4 of idx
    const int nChunks = 2 * chunksPerRow;

    // Copies rows (2*pr, 2*pr+1) of W and idx into buffer `buf` of this warp.
    auto issue = [&](long long pr, int buf) {
        float* dstbuf = wi + buf * 4 * K;
        for (int c = lane; c < nChunks; c += 32) {
            const int row = c / chunksPerRow;
            const int within = c - row * chunksPerRow;
            const bool isIdx = within >= K / 4;
            const int kc = isIdx ? within - K / 4 : within;
            const long long o = 2 * pr + row;
            if (o < L) {
                const void* src = isIdx ? static_cast<const void*>(p.idx + o * K + 4 * kc)
                                        : static_cast<const void*>(p.W + o * K + 4 * kc);
                __pipeline_memcpy_async(dstbuf + row * 2 * K + (isIdx ? K : 0) + 4 * kc, src, 16);
            }
        }
        __pipeline_commit();
    };

    long long q = gw;
    if (q < numQuads) issue(2 * q, 0);
    int s = 0;
    float loss_local = 0.f;  // BCE: sum of softplus(z) over this lane's (b, o) pairs
    for (; q < numQuads; q += GW) {
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

            const long long oA = 2 * pr;
            if (oA < L) {
                const bool validB = oA + 1 < L;
                const float* rowA = wi + buf * 4 * K;
                const float* rowB = validB ? rowA + 2 * K : rowA;
                const float biasA = p.bias ? __ldg(p.bias + oA) : 0.f;
                const float biasB = (p.bias && validB) ? __ldg(p.bias + oA + 1) : 0.f;
                float accA[BPL], accB[BPL];
#pragma unroll
                for (int j = 0; j < BPL; ++j) accA[j] = accB[j] = 0.f;
                const float4* wrA = reinterpret_cast<const float4*>(rowA);
                const int4* irA = reinterpret_cast<const int4*>(rowA + K);
                const float4* wrB = reinterpret_cast<const float4*>(rowB);
                const int4* irB = reinterpret_cast<const int4*>(rowB + K);
#pragma unroll 2
                for (int k4 = 0; k4 < K / 4; ++k4) {
                    const int4 iA = irA[k4], iB = irB[k4];
                    const float4 wA = wrA[k4], wB = wrB[k4];
                    const V a0 = xs_lane[iA.x * 32], a1 = xs_lane[iA.y * 32], a2 = xs_lane[iA.z * 32],
                            a3 = xs_lane[iA.w * 32];
                    const V c0 = xs_lane[iB.x * 32], c1 = xs_lane[iB.y * 32], c2 = xs_lane[iB.z * 32],
                            c3 = xs_lane[iB.w * 32];
#pragma unroll
                    for (int j = 0; j < BPL; ++j) {
                        accA[j] = fmaf(wA.x, vec_get(a0, j), accA[j]);
                        accB[j] = fmaf(wB.x, vec_get(c0, j), accB[j]);
                        accA[j] = fmaf(wA.y, vec_get(a1, j), accA[j]);
                        accB[j] = fmaf(wB.y, vec_get(c1, j), accB[j]);
                        accA[j] = fmaf(wA.z, vec_get(a2, j), accA[j]);
                        accB[j] = fmaf(wB.z, vec_get(c2, j), accB[j]);
                        accA[j] = fmaf(wA.w, vec_get(a3, j), accA[j]);
                        accB[j] = fmaf(wB.w, vec_get(c3, j), accB[j]);
                    }
                }
                if constexpr (BCE) {
                    // lanes hold consecutive batch elements: each (row, j) is one coalesced 128-byte store
#pragma unroll
                    for (int j = 0; j < BPL; ++j) {
                        const int b = b0 + lane + 32 * j;
                        const bool live = b < p.B;
                        const float zA = accA[j] + biasA, zB = accB[j] + biasB;
                        float vA, gA, vB, gB;
                        loss_negative(p.loss_kind, zA, vA, gA);
                        loss_negative(p.loss_kind, zB, vB, gB);
                        if (live) loss_local += vA + (validB ? vB : 0.f);
                        if (b < p.ldg) {
                            p.gT[static_cast<size_t>(oA) * p.ldg + b] = live ? p.scale * gA : 0.f;
                            if (validB) p.gT[static_cast<size_t>(oA + 1) * p.ldg + b] = live ? p.scale * gB : 0.f;
                        }
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < BPL; ++j) {
                        ys[(2 * half) * S + lane + 32 * j] = accA[j] + biasA;
                        ys[(2 * half + 1) * S + lane + 32 * j] = accB[j] + biasB;
                    }
                }
            }
            __syncwarp();  // buffer `buf` may be overwritten by the next issue; ys rows are visible
        }
        if constexpr (!BCE) {
            // Write out rows 4q .. 4q+3: lane = (batch row, output) -> 16-byte runs along o.
            const long long oq = 4 * q;
#pragma unroll
            for (int it = 0; it < BT * 4 / 32; ++it) {
                const int id = it * 32 + lane;
                const int bl = id >> 2, oo = id & 3;
                if (b0 + bl < p.B && oq + oo < L)
                    p.y[static_cast<size_t>(b0 + bl) * L + oq + oo] = ys[oo * S + bl];
            }
            __syncwarp();  // ys is rewritten by the next quad
        }
    }
    __pipeline_wait_prior(0);

    if constexpr (BCE) {
        // CTA partial of the loss sum in a fixed order: lanes (tree), then warps (serial).
        double v = static_cast<double>(loss_local);
#pragma unroll
        for (int off = 16; off >= 1; off /= 2) v += __shfl_xor_sync(0xffffffffu, v, off);
        __syncthreads();  // every warp is done with its shared-memory region
        double* red = reinterpret_cast<double*>(smem_raw);
        if (lane == 0) red[warp] = v;
        __syncthreads();
        if (tid == 0) {
            double t = 0.0;
            for (int w = 0; w < kWarps; ++w) t += red[w];
            p.loss_partials[static_cast<size_t>(blockIdx.y) * gridDim.x + blockIdx.x] = t;
        }
    }
}

template <int BPL, bool BCE>
int launch_stream_t(const FwdStreamParams& p, size_t smem, int nBT, const DeviceInfo& dev, cudaStream_t stream,
                    int* ctas_out) {
    auto kern = ffi_fwd_stream_kernel<BPL, BCE>;
    FFI_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    int occ = 0;
    FFI_CUDA_CHECK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, kThreads, smem));
    if (occ < 1) return fail(FFI_ERR_CUDA, "streaming forward kernel does not fit on an SM (smem %zu)", smem);
    int per_bt = dev.sm_count * occ / nBT;
    if (per_bt < 1) per_bt = 1;
    const long long numQuads = (static_cast<long long>(p.L) + 3) / 4;
    const long long want = (numQuads + kWarps - 1) / kWarps;
    dim3 grid(static_cast<unsigned>(want < per_bt ? want : per_bt), static_cast<unsigned>(nBT));
    if (ctas_out) *ctas_out = static_cast<int>(grid.x * grid.y);
    kern<<<grid, kThreads, smem, stream>>>(p);
    FFI_LAUNCH_CHECK("ffi_fwd_stream_kernel");
    return FFI_OK;
}

}  // namespace

// Shared launcher: BCE epilogue when bce != nullptr.
struct BceEpilogue {
    float* gT;
    long long ldg;
    float scale;
    double* loss_partials;
    int* ctas;  // out: number of CTAs = number of loss partials written
    int loss_kind;
};

static int launch_forward_stream_impl(const FwdArgs& a, const BceEpilogue* bce, cudaStream_t stream, bool* handled) {
    *handled = false;
    DeviceInfo dev;
    int rc = get_device_info(&dev);
    if (rc != FFI_OK) return rc;
    if (a.K % 4 != 0 || reinterpret_cast<uintptr_t>(a.W) % 16 != 0 || reinterpret_cast<uintptr_t>(a.idx) % 16 != 0)
        return FFI_OK;
    int bpl = a.B <= 32 ? 1 : (a.B <= 64 ? 2 : 4);
    size_t smem = 0;
    for (; bpl >= 1; bpl /= 2) {
        const size_t BT = 32 * bpl;
        smem = static_cast<size_t>(a.N) * BT * 4 + static_cast<size_t>(kWarps) * (8 * a.K + 4 * (BT + 8)) * 4;
        if (smem <= static_cast<size_t>(dev.max_smem_optin)) break;
    }
    if (bpl < 1) return FFI_OK;
    FwdStreamParams p;
    p.xT = a.xT;
    p.ldx = a.ldx;
    p.idx = a.idx;
    p.W = a.W;
    p.bias = a.bias;
    p.y = a.y;
    p.B = a.B;
    p.N = a.N;
    p.L = a.L;
    p.K = a.K;
    p.gT = bce ? bce->gT : nullptr;
    p.ldg = bce ? bce->ldg : 0;
    p.scale = bce ? bce->scale : 0.f;
    p.loss_partials = bce ? bce->loss_partials : nullptr;
    p.loss_kind = bce ? bce->loss_kind : 0;
    const int nBT = static_cast<int>(ceil_div(a.B, 32 * bpl));
    *handled = true;
    if (bce) {
        if (bpl == 4) return launch_stream_t<4, true>(p, smem, nBT, dev, stream, bce->ctas);
        if (bpl == 2) return launch_stream_t<2, true>(p, smem, nBT, dev, stream, bce->ctas);
        return launch_stream_t<1, true>(p, smem, nBT, dev, stream, bce->ctas);
    }
    if (bpl == 4) return launch_stream_t<4, false>(p, smem, nBT, dev, stream, nullptr);
    if (bpl == 2) return launch_stream_t<2, false>(p, smem, nBT, dev, stream, nullptr);
    return launch_stream_t<1, false>(p, smem, nBT, dev, stream, nullptr);
}

// Launches the barrier-free kernel when the shape allows it; *handled tells the caller.
int launch_forward_stream(const FwdArgs& a, cudaStream_t stream, bool* handled) {
    return launch_forward_stream_impl(a, nullptr, stream, handled);
}

// Forward with the fused sigmoid-BCE epilogue: writes gT[o][b] = scale * sigmoid(z[b,o]) (zero in the
// padded batch columns) and one partial of sum softplus(z) per CTA; *ctas receives their number
// (at most 2 * SM count).  *handled is false when the shape needs the unfused path.
int launch_forward_bce_stream(const FwdArgs& a, float* gT, int64_t ldg, float scale, double* loss_partials, int* ctas,
                              int loss_kind, cudaStream_t stream, bool* handled) {
    BceEpilogue e{gT, ldg, scale, loss_partials, ctas, loss_kind};
    return launch_forward_stream_impl(a, &e, stream, handled);
}

}  // namespace ffi
