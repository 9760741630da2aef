// Forward of the fixed-fan-in sparse layer for wide inputs on sm_100a: x does not fit shared memory, every
// entry gathers its operand row x[:, idx[o,k]] from L2.
//   y[b,o] = bias[o] + sum_k W[o,k] * x[b, idx[o,k]]
//
// Replaces the reference's forward kernels (tfsparse/cc/kernels/forward.cu.h:231-264) for the output layers of
// the stacked configurations (hidden widths of 32,768 ... 100,000).
//
// As in the gather kernel for grad_W, what bounds this shape is the number of gathered bytes in flight per SM,
// so every warp is its own pipeline with few registers: a lane owns BPL batch elements, the warp's W and idx
// rows arrive by its own cp.async into a private double buffer, eight gathers are issued back to back, and the
// row's results either leave at once as the loss gradient (rows of gT are batch-contiguous: one vector store per
// lane) or wait in a private tile of eight rows and leave as runs of eight consecutive outputs per batch row.
// 64 registers per thread, 32 warps per SM, no CTA barrier in the steady state.
#include <type_traits>

#include "ffi_common.cuh"

namespace ffi {
namespace {

constexpr int kThreads = 512;
constexpr int kWarps = kThreads / 32;
// rows of results a warp collects before it writes y (fewer for the widest lanes, whose rows are twice as long)
template <int BPL>
struct ResultRows {
    static constexpr int value = BPL == 8 ? 4 : 8;
};

struct FwdGatherParams {
    const void* xT;  // [N][ldx], element type TX
    long long ldx;
    const int* idx;
    const void* W;   // element type TX
    const float* bias;
    float* y;
    int B, N, L, K;
    // loss epilogue (MODE 1), as in the tiled kernel: gT[o][b] = scale * dloss/dz for target 0, zero in the padded
    // batch columns up to ldg, and one partial sum of the loss values per CTA
    float* gT;
    long long ldg;
    float scale;
    double* loss_partials;
    int loss_kind;
};

template <int BPL, int MODE, typename TX>
__global__ void __launch_bounds__(kThreads, 2) ffi_fwd_gather_kernel(FwdGatherParams p) {
    constexpr int BT = 32 * BPL;
    constexpr int S = BT + 4;  // row stride of the result tile
    constexpr int kRows = ResultRows<BPL>::value;
    constexpr bool kBf16 = !std::is_same<TX, float>::value;
    constexpr int WPE = kBf16 ? 2 : 1;  // weights per 32-bit word of a staged W row
    using V = typename Vec<BPL>::type;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int K = p.K, L = p.L;
    const int b0 = blockIdx.y * BT;
    // per warp: two (W row, idx row) buffers, then the result tile (MODE 0)
    const int wWords = K / WPE;
    const int rowWords = wWords + K;
    const int warpWords = 2 * rowWords + (MODE == 0 ? kRows * S : 0);
    unsigned* wbuf = reinterpret_cast<unsigned*>(smem_raw) + static_cast<size_t>(warp) * warpWords;
    float* ys = reinterpret_cast<float*>(wbuf + 2 * rowWords);

    const TX* xg = static_cast<const TX*>(p.xT) + b0;
    const size_t ldv = static_cast<size_t>(p.ldx / BPL);
    const long long GW = static_cast<long long>(gridDim.x) * kWarps;
    // a warp takes blocks of kRows consecutive rows, so that its results leave as runs along o
    const long long numBlocks = (static_cast<long long>(L) + kRows - 1) / kRows;
    long long blk = static_cast<long long>(blockIdx.x) * kWarps + warp;

    auto issue = [&](long long row, int buf) {
        if (row < L) {
            unsigned* dst = wbuf + buf * rowWords;
            const unsigned* wsrc = reinterpret_cast<const unsigned*>(static_cast<const TX*>(p.W) + row * K);
            for (int c = lane; c < wWords / 4; c += 32) __pipeline_memcpy_async(dst + 4 * c, wsrc + 4 * c, 16);
            for (int c = lane; c < K / 4; c += 32)
                __pipeline_memcpy_async(dst + wWords + 4 * c, p.idx + row * K + 4 * c, 16);
        }
        __pipeline_commit();
    };
    auto weight = [&](const unsigned* wr, int k) -> float {
        if constexpr (kBf16) {
            const unsigned word = wr[k >> 1];
            return (k & 1) ? bf16_hi(word) : bf16_lo(word);
        } else {
            return __uint_as_float(wr[k]);
        }
    };

    float loss_local = 0.f;
    int s = 0;
    if (blk < numBlocks) issue(blk * kRows, 0);
    for (; blk < numBlocks; blk += GW) {
        const long long o0 = blk * kRows;
#pragma unroll 1
        for (int r = 0; r < kRows; ++r, s ^= 1) {
            const long long o = o0 + r;
            // the row after this one: the next of the block, or the first row of the warp's next block
            const long long next = r + 1 < kRows ? o + 1 : (blk + GW) * kRows;
            issue(next, s ^ 1);
            __pipeline_wait_prior(1);
            __syncwarp();
            if (o < L) {
                const unsigned* wr = wbuf + s * rowWords;
                const int* ir = reinterpret_cast<const int*>(wr + wWords);
                float acc[BPL];
#pragma unroll
                for (int j = 0; j < BPL; ++j) acc[j] = 0.f;
                int k = 0;
                for (; k + 8 <= K; k += 8) {
                    const int4 i0 = *reinterpret_cast<const int4*>(ir + k);
                    const int4 i1 = *reinterpret_cast<const int4*>(ir + k + 4);
                    const int ii[8] = {i0.x, i0.y, i0.z, i0.w, i1.x, i1.y, i1.z, i1.w};
                    V v[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u) v[u] = load_lane_vec<BPL>(xg, static_cast<size_t>(ii[u]) * ldv + lane);
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        const float w = weight(wr, k + u);
#pragma unroll
                        for (int j = 0; j < BPL; ++j) acc[j] = fmaf(w, vec_get(v[u], j), acc[j]);
                    }
                }
                if (k < K) {  // four entries left
                    const int4 i0 = *reinterpret_cast<const int4*>(ir + k);
                    const int ii[4] = {i0.x, i0.y, i0.z, i0.w};
                    V v[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) v[u] = load_lane_vec<BPL>(xg, static_cast<size_t>(ii[u]) * ldv + lane);
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const float w = weight(wr, k + u);
#pragma unroll
                        for (int j = 0; j < BPL; ++j) acc[j] = fmaf(w, vec_get(v[u], j), acc[j]);
                    }
                }
                const float bias = p.bias ? __ldg(p.bias + o) : 0.f;
                if constexpr (MODE == 1) {
                    float gv[BPL];
#pragma unroll
                    for (int j = 0; j < BPL; ++j) {
                        const int b = b0 + lane * BPL + j;
                        float v, g;
                        loss_for_negative(p.loss_kind, acc[j] + bias, v, g);
                        if (b < p.B) loss_local += v;
                        gv[j] = b < p.B ? p.scale * g : 0.f;
                    }
                    // the stored row is ldg wide (a multiple of BPL): the columns past B receive zeros
                    if (b0 + lane * BPL < p.ldg) store_lane_f32<BPL>(p.gT + static_cast<size_t>(o) * p.ldg + b0, lane, gv);
                } else {
                    float out[BPL];
#pragma unroll
                    for (int j = 0; j < BPL; ++j) out[j] = acc[j] + bias;
                    store_lane_f32<BPL>(ys + r * S, lane, out);
                }
            }
            __syncwarp();
        }
        if constexpr (MODE == 0) {
            // kRows consecutive lanes write the kRows outputs of one batch row: 32- or 16-byte runs along o
            const int rows = static_cast<int>(L - o0 < kRows ? L - o0 : kRows);
            const int oo = lane & (kRows - 1);
#pragma unroll 4
            for (int bl = lane / kRows; bl < BT; bl += 32 / kRows)
                if (b0 + bl < p.B && oo < rows) p.y[static_cast<size_t>(b0 + bl) * L + o0 + oo] = ys[oo * S + bl];
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
        if (threadIdx.x == 0) {
            double t = 0.0;
            for (int w = 0; w < kWarps; ++w) t += red[w];
            p.loss_partials[static_cast<size_t>(blockIdx.y) * gridDim.x + blockIdx.x] = t;
        }
    }
}

template <int BPL, int MODE, typename TX>
int launch_fwd_gather_t(const FwdGatherParams& p, int nBT, int max_partials, const DeviceInfo& dev, cudaStream_t stream,
                        int* ctas_out) {
    constexpr int BT = 32 * BPL;
    constexpr int kRows = ResultRows<BPL>::value;
    constexpr int WPE = std::is_same<TX, float>::value ? 1 : 2;
    auto kern = ffi_fwd_gather_kernel<BPL, MODE, TX>;
    const size_t warpWords = 2 * static_cast<size_t>(p.K / WPE + p.K) + (MODE == 0 ? kRows * (BT + 4) : 0);
    const size_t smem = kWarps * warpWords * 4;
    FFI_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    int occ = 0;
    FFI_CUDA_CHECK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, kThreads, smem));
    if (occ < 1) return fail(FFI_ERR_CUDA, "forward gather kernel does not fit on an SM (smem %zu)", smem);
    const long long want = ceil_div(ceil_div(p.L, kRows), kWarps);
    long long per_bt = static_cast<long long>(dev.sm_count) * occ / nBT;
    if (per_bt < 1) per_bt = 1;
    dim3 grid(static_cast<unsigned>(want < per_bt ? want : per_bt), static_cast<unsigned>(nBT));
    if (MODE == 1 && static_cast<long long>(grid.x) * grid.y > max_partials)
        return fail(FFI_ERR_UNSUPPORTED, "the fused loss keeps at most %d per-CTA partials; this batch needs %u",
                    max_partials, grid.x * grid.y);
    if (ctas_out) *ctas_out = static_cast<int>(grid.x * grid.y);
    kern<<<grid, kThreads, smem, stream>>>(p);
    FFI_LAUNCH_CHECK("ffi_fwd_gather_kernel");
    return FFI_OK;
}

template <int MODE, typename TX>
int launch_fwd_gather_b(const FwdGatherParams& p, int bpl, int nBT, int max_partials, const DeviceInfo& dev,
                        cudaStream_t stream, int* ctas_out) {
    if (bpl == 4) return launch_fwd_gather_t<4, MODE, TX>(p, nBT, max_partials, dev, stream, ctas_out);
    if (bpl == 2) return launch_fwd_gather_t<2, MODE, TX>(p, nBT, max_partials, dev, stream, ctas_out);
    return launch_fwd_gather_t<1, MODE, TX>(p, nBT, max_partials, dev, stream, ctas_out);
}

}  // namespace

// Takes the shapes the tiled kernel would gather from L2 for (x too wide for shared memory) when K is a multiple
// of 4 (8 for bf16 storage) and the rows are aligned; *handled tells the caller.  With gT set it writes the loss
// gradient and per-CTA loss partials (at most max_partials; *ctas receives their number) instead of y.
int launch_forward_gather(const FwdArgs& a, int bpl, float* gT, int64_t ldg, float scale, double* loss_partials,
                          int loss_kind, int max_partials, int* ctas, cudaStream_t stream, bool* handled) {
    *handled = false;
    DeviceInfo dev;
    int rc = get_device_info(&dev);
    if (rc != FFI_OK) return rc;
    // bf16 storage: eight batch elements per lane (one 16-byte gather covers 256 batch
    // columns per warp, W and idx are streamed once per 256 instead of once per 128) where the rows are padded to it
    if (a.bf16 && bpl == 4 && a.B > 128 && a.ldx % 256 == 0 && (!gT || ldg % 256 == 0)) bpl = 8;
    const int BT = 32 * bpl;
    const int nBT = static_cast<int>(ceil_div(a.B, BT));
    const int kq = a.bf16 ? 8 : 4;
    if (a.K % kq != 0 || reinterpret_cast<uintptr_t>(a.idx) % 16 != 0 || reinterpret_cast<uintptr_t>(a.W) % 16 != 0 ||
        a.ldx % BT != 0 || a.ldx < static_cast<int64_t>(nBT) * BT || reinterpret_cast<uintptr_t>(a.xT) % 16 != 0)
        return FFI_OK;
    if (gT && (ldg % bpl != 0 || ldg > static_cast<int64_t>(nBT) * BT || reinterpret_cast<uintptr_t>(gT) % 16 != 0 ||
               (ldg * 4) % 16 != 0))
        return FFI_OK;
    FwdGatherParams p;
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
    p.gT = gT;
    p.ldg = ldg;
    p.scale = scale;
    p.loss_partials = loss_partials;
    p.loss_kind = loss_kind;
    *handled = true;
    if (bpl == 8) {
        if (gT) return launch_fwd_gather_t<8, 1, __nv_bfloat16>(p, nBT, max_partials, dev, stream, ctas);
        return launch_fwd_gather_t<8, 0, __nv_bfloat16>(p, nBT, max_partials, dev, stream, ctas);
    }
    if (a.bf16) {
        if (gT) return launch_fwd_gather_b<1, __nv_bfloat16>(p, bpl, nBT, max_partials, dev, stream, ctas);
        return launch_fwd_gather_b<0, __nv_bfloat16>(p, bpl, nBT, max_partials, dev, stream, ctas);
    }
    if (gT) return launch_fwd_gather_b<1, float>(p, bpl, nBT, max_partials, dev, stream, ctas);
    return launch_fwd_gather_b<0, float>(p, bpl, nBT, max_partials, dev, stream, ctas);
}

}  // namespace ffi
