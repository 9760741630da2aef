// Forward of the fixed-fan-in sparse layer on sm_100a:
//   y[b,o] = bias[o] + sum_k W[o,k] * x[b, idx[o,k]]
//
// Replaces the reference's forward kernels (tfsparse/cc/kernels/forward.cu.h:231-264:
// forward_ob_scalar_tp for the transposed op, forward_ib_unrolled for the plain one),
// their output memset (forward.cu:63) and the separate bias_add (sparse/layer.py:247).
//
// Dataflow.  One lane owns BPL batch elements (a warp covers BT = 32*BPL of them) and a
// warp walks whole output rows, so (o,k) is warp-uniform:
//   * the batch tile of x sits in shared memory as x_s[N][BT] (batch contiguous), so the
//     gather x[:, idx[o,k]] is one conflict-free 4/8/16-byte LDS per lane;
//   * W and idx rows stream through a double-buffered shared-memory tile filled with
//     cp.async (no register staging) and are read back as 16-byte broadcasts;
//   * results go through a padded shared-memory tile so that the global stores of y run
//     along o (128 B per warp store) instead of striding by L.
// The kernel is persistent: gridDim.x CTAs per batch tile loop over the output tiles.
// When x_s does not fit (wide N), the same code gathers x from global memory (L2).
#include <type_traits>

#include "ffi_common.cuh"

namespace ffi {
namespace {

constexpr int kThreads = 512;
constexpr int kWarps = kThreads / 32;

struct FwdKernelParams {
    const void* xT;  // element type TX of the kernel: float or __nv_bfloat16
    long long ldx;
    const int* idx;
    const void* W;   // same element type
    const float* bias;
    float* y;
    int B, N, L, K;
    int Kp;        // K rounded up to a multiple of 4 (row stride of the staged tiles)
    int TO;        // outputs per tile
    int numTiles;  // ceil(L / TO)
    int vec16;     // tiles can be copied with 16-byte cp.async
    // loss epilogue (LOSS variant): instead of y the kernel writes the loss gradient for target 0, transposed,
    // gT[o][b] = scale * dloss/dz (zero in the padded batch columns up to ldg), and one partial sum of the
    // loss values per CTA; the few positives are corrected by a later kernel
    float* gT;
    long long ldg;
    float scale;
    double* loss_partials;
    int loss_kind;
    // top-k epilogue (MODE 2): thread (part, batch element) keeps the kTopK best logits of the rows
    // part, part + PARTS, ... of every tile of its CTA; lists [batch tile][cta][part][batch][kTopK] of (value, row)
    uint2* topk_lists;
};

// TX: storage type of x and W.  bf16 values are widened where they are loaded (the x tile and the staged W
// rows in shared memory are fp32; x gathered from global memory is widened in registers), so the
// arithmetic is that of the fp32 kernel on exactly the same values, at half the gather traffic.
// MODE 0 writes y, 1 the loss gradient (see FwdKernelParams), 2 the top-k lists.
template <int BPL, bool XSMEM, int MODE, typename TX>
__global__ void __launch_bounds__(kThreads, 1) ffi_fwd_kernel(FwdKernelParams p) {
    constexpr int BT = 32 * BPL;
    constexpr bool LOSS = MODE == 1;
    constexpr int PARTS = kThreads / BT;  // top-k: threads per batch element
    constexpr bool kBf16 = !std::is_same<TX, float>::value;
    const TX* xT = static_cast<const TX*>(p.xT);
    const TX* Wt = static_cast<const TX*>(p.W);
    using V = typename Vec<BPL>::type;
    extern __shared__ __align__(16) unsigned char smem_raw[];

    float* x_s = reinterpret_cast<float*>(smem_raw);
    float* w_s = x_s + (XSMEM ? static_cast<size_t>(p.N) * BT : 0);
    int* i_s = reinterpret_cast<int*>(w_s + 2 * p.TO * p.Kp);
    float* y_s = reinterpret_cast<float*>(i_s + 2 * p.TO * p.Kp);

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int b0 = blockIdx.y * BT;
    const int TO = p.TO, Kp = p.Kp, K = p.K, L = p.L;
    const int tileElems = TO * Kp;

    // Padding slots (k in [K,Kp)) and rows never copied must hold weight 0 / index 0.
    for (int e = tid; e < 2 * tileElems; e += kThreads) {
        w_s[e] = 0.f;
        i_s[e] = 0;
    }
    if (XSMEM) {
        // x_s[i][lane*BPL + j] holds batch element b0 + lane + 32*j.
        const int total = p.N * BT;
#pragma unroll 8
        for (int e = tid; e < total; e += kThreads) {
            int i = e / BT;
            int bl = e - i * BT;
            int b = b0 + bl;
            float v = b < p.B ? widen(xT[static_cast<size_t>(i) * p.ldx + b]) : 0.f;
            x_s[i * BT + (bl & 31) * BPL + (bl >> 5)] = v;
        }
    }
    __syncthreads();

    auto prefetch = [&](int t, int buf) {
        const long long o0 = static_cast<long long>(t) * TO;
        const int nrows = min(TO, static_cast<int>(L - o0));
        float* wd = w_s + buf * tileElems;
        int* id = i_s + buf * tileElems;
        const TX* wsrc = Wt + o0 * K;
        const int* isrc = p.idx + o0 * K;
        if (p.vec16) {
            const int nvec = nrows * K / 4;
            for (int v = tid; v < nvec; v += kThreads) {
                if constexpr (kBf16) {  // a widening copy: four bf16 weights -> four fp32 words
                    const uint2 r = __ldg(reinterpret_cast<const uint2*>(wsrc) + v);
                    *reinterpret_cast<float4*>(wd + 4 * v) = make_float4(bf16_lo(r.x), bf16_hi(r.x), bf16_lo(r.y), bf16_hi(r.y));
                } else {
                    __pipeline_memcpy_async(wd + 4 * v, wsrc + 4 * v, 16);
                }
                __pipeline_memcpy_async(id + 4 * v, isrc + 4 * v, 16);
            }
        } else {
            const int n = nrows * K;
            for (int e = tid; e < n; e += kThreads) {
                int r = e / K;
                int k = e - r * K;
                if constexpr (kBf16) wd[r * Kp + k] = widen(wsrc[e]);
                else __pipeline_memcpy_async(wd + r * Kp + k, wsrc + e, 4);
                __pipeline_memcpy_async(id + r * Kp + k, isrc + e, 4);
            }
        }
        __pipeline_commit();
    };

    const V* xs_lane = reinterpret_cast<const V*>(x_s) + lane;
    const TX* xg_base = xT + b0;
    const size_t ldv = static_cast<size_t>(p.ldx / BPL);

    // Coalesced write-out of a finished tile: one warp per batch row, lanes along o.
    float loss_local = 0.f;
    const int tk_bl = tid % BT, tk_part = tid / BT;
    float tv[kTopK];
    int ti[kTopK];
#pragma unroll
    for (int j = 0; j < kTopK; ++j) tv[j] = -INFINITY, ti[j] = 0x7fffffff;
    auto write_out = [&](long long o0, const float* ys) {
        if constexpr (MODE == 2) {
            const int rows = min(TO, static_cast<int>(L - o0));
            if (b0 + tk_bl < p.B)
                for (int c = tk_part; c < rows; c += PARTS)
                    topk_insert(tv, ti, ys[c * (BT + 1) + tk_bl], static_cast<int>(o0) + c);
        } else if constexpr (LOSS) {
            // one warp per output row, lanes along the batch: gT rows are batch-contiguous
            const bool last_bt = blockIdx.y + 1 == gridDim.y;
            const int cols = last_bt ? static_cast<int>(p.ldg) - b0 : BT;  // the last tile also clears the padding
            for (int c = warp; c < TO; c += kWarps) {
                if (o0 + c >= L) break;
                float* grow = p.gT + static_cast<size_t>(o0 + c) * p.ldg + b0;
                for (int bl = lane; bl < cols; bl += 32) {
                    float gv = 0.f;
                    if (bl < BT && b0 + bl < p.B) {
                        float v, g;
                        loss_for_negative(p.loss_kind, ys[c * (BT + 1) + bl], v, g);
                        loss_local += v;
                        gv = p.scale * g;
                    }
                    grow[bl] = gv;
                }
            }
        } else {
            for (int r = warp; r < BT; r += kWarps) {
                const int b = b0 + r;
                if (b >= p.B) break;
                float* yrow = p.y + static_cast<size_t>(b) * L + o0;
                for (int c = lane; c < TO; c += 32)
                    if (o0 + c < L) yrow[c] = ys[c * (BT + 1) + r];
            }
        }
    };

    auto gather = [&](int i) -> V {
        if (XSMEM) return xs_lane[i * 32];
        return load_lane_vec<BPL>(xg_base, static_cast<size_t>(i) * ldv + lane);
    };

    int t = blockIdx.x;
    int buf = 0;
    long long prev_o0 = -1;  // tile whose results wait in y_s[buf ^ 1]
    if (t < p.numTiles) prefetch(t, 0);
    for (; t < p.numTiles; t += gridDim.x, buf ^= 1) {
        __pipeline_wait_prior(0);
        // One barrier per tile: tile t has landed, every warp has finished computing tile t-1
        // (so y_s[buf^1] is complete and the other W/idx buffer is free) and writing out t-2.
        __syncthreads();
        const int tn = t + gridDim.x;
        if (tn < p.numTiles) prefetch(tn, buf ^ 1);
        if (prev_o0 >= 0) write_out(prev_o0, y_s + (buf ^ 1) * TO * (BT + 1));

        const long long o0 = static_cast<long long>(t) * TO;
        const float* wb = w_s + buf * tileElems;
        const int* ib = i_s + buf * tileElems;
        float* ys = y_s + buf * TO * (BT + 1);
        // Two rows per warp in flight: twice the independent loads and FMA chains per warp.
        for (int olA = warp; olA < TO; olA += 2 * kWarps) {
            if (o0 + olA >= L) break;
            const int olB = olA + kWarps;
            const bool validB = olB < TO && o0 + olB < L;
            const int olBc = validB ? olB : olA;
            const float biasA = p.bias ? __ldg(p.bias + o0 + olA) : 0.f;
            const float biasB = p.bias ? __ldg(p.bias + o0 + olBc) : 0.f;
            float accA[BPL], accB[BPL];
#pragma unroll
            for (int j = 0; j < BPL; ++j) accA[j] = accB[j] = 0.f;  // bias is added last
            const int4* irA = reinterpret_cast<const int4*>(ib + olA * Kp);
            const float4* wrA = reinterpret_cast<const float4*>(wb + olA * Kp);
            const int4* irB = reinterpret_cast<const int4*>(ib + olBc * Kp);
            const float4* wrB = reinterpret_cast<const float4*>(wb + olBc * Kp);
#pragma unroll 2
            for (int k4 = 0; k4 < Kp / 4; ++k4) {
                const int4 iA = irA[k4], iB = irB[k4];
                const float4 wA = wrA[k4], wB = wrB[k4];
                const V a0 = gather(iA.x), a1 = gather(iA.y), a2 = gather(iA.z), a3 = gather(iA.w);
                const V c0 = gather(iB.x), c1 = gather(iB.y), c2 = gather(iB.z), c3 = gather(iB.w);
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
#pragma unroll
            for (int j = 0; j < BPL; ++j) {
                const int bl = XSMEM ? lane + 32 * j : lane * BPL + j;
                ys[olA * (BT + 1) + bl] = accA[j] + biasA;
                if (validB) ys[olB * (BT + 1) + bl] = accB[j] + biasB;
            }
        }
        prev_o0 = o0;
    }
    __pipeline_wait_prior(0);
    __syncthreads();
    if (prev_o0 >= 0) write_out(prev_o0, y_s + (buf ^ 1) * TO * (BT + 1));
    if constexpr (MODE == 2) {
        if (b0 + tk_bl < p.B) {
            uint2* out = p.topk_lists +
                         ((static_cast<size_t>(blockIdx.y) * gridDim.x + blockIdx.x) * PARTS + tk_part) * (BT * kTopK) +
                         tk_bl * kTopK;
#pragma unroll
            for (int j = 0; j < kTopK; ++j) out[j] = make_uint2(__float_as_uint(tv[j]), static_cast<unsigned>(ti[j]));
        }
    }
    if constexpr (LOSS) {
        double v = static_cast<double>(loss_local);
#pragma unroll
        for (int off = 16; off >= 1; off /= 2) v += __shfl_xor_sync(0xffffffffu, v, off);
        __syncthreads();
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

__global__ void transpose_pad_kernel(const float* __restrict__ src, float* __restrict__ dst,
                                     int rows, int cols, long long ld_dst) {
    // src [rows][cols] -> dst [cols][ld_dst], dst[c][r] = src[r][c]; r in [rows, ld_dst) zero.
    __shared__ float tile[32][33];
    const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
    for (int dy = threadIdx.y; dy < 32; dy += blockDim.y) {
        int r = r0 + dy, c = c0 + threadIdx.x;
        tile[dy][threadIdx.x] = (r < rows && c < cols) ? src[static_cast<size_t>(r) * cols + c] : 0.f;
    }
    __syncthreads();
    for (int dy = threadIdx.y; dy < 32; dy += blockDim.y) {
        int c = c0 + dy, r = r0 + threadIdx.x;
        if (c < cols && r < ld_dst) dst[static_cast<size_t>(c) * ld_dst + r] = tile[threadIdx.x][dy];
    }
}

struct FwdConfig {
    int bpl;
    bool xsmem;
    int TO;
    size_t smem;
};

size_t fwd_smem_bytes(int N, int bpl, bool xsmem, int TO, int Kp) {
    const size_t BT = 32 * bpl;
    return (xsmem ? static_cast<size_t>(N) * BT * 4 : 0) + static_cast<size_t>(2) * TO * Kp * 8 +
           static_cast<size_t>(2) * TO * (BT + 1) * 4;
}

int pick_TO(size_t budget, int N, int bpl, bool xsmem, int Kp) {
    const size_t BT = 32 * bpl;
    const size_t fixed = xsmem ? static_cast<size_t>(N) * BT * 4 : 0;
    if (fixed >= budget) return 0;
    const size_t per_row = static_cast<size_t>(2) * Kp * 8 + 2 * (BT + 1) * 4;
    size_t to = (budget - fixed) / per_row;
    if (to > 128) to = 128;
    return static_cast<int>(to / 16 * 16);
}

constexpr int kMaxLossPartialsTile = 1024;  // doubles the caller's scratch holds for the per-CTA loss sums

template <int BPL, bool XSMEM, int MODE, typename TX>
int launch_fwd_t(const FwdKernelParams& p, size_t smem, int nBT, const DeviceInfo& dev,
                 cudaStream_t stream, int* ctas_out) {
    constexpr bool LOSS = MODE == 1;
    auto kern = ffi_fwd_kernel<BPL, XSMEM, MODE, TX>;
    FFI_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        static_cast<int>(smem)));
    int occ = 0;
    FFI_CUDA_CHECK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, kThreads, smem));
    if (occ < 1) return fail(FFI_ERR_CUDA, "forward kernel does not fit on an SM (smem %zu)", smem);
    if (MODE == 2) occ = 1;  // the scratch for the top-k lists is sized for one CTA per SM
    int per_bt = dev.sm_count * occ / nBT;
    if (per_bt < 1) per_bt = 1;
    dim3 grid(static_cast<unsigned>(min(p.numTiles, per_bt)), static_cast<unsigned>(nBT));
    if (LOSS && static_cast<long long>(grid.x) * grid.y > kMaxLossPartialsTile)
        return fail(FFI_ERR_UNSUPPORTED, "the fused loss keeps at most %d per-CTA partials; this batch needs %u",
                    kMaxLossPartialsTile, grid.x * grid.y);
    if (ctas_out) *ctas_out = static_cast<int>(grid.x * grid.y);
    kern<<<grid, kThreads, smem, stream>>>(p);
    FFI_LAUNCH_CHECK("ffi_fwd_kernel");
    return FFI_OK;
}

template <int LOSS, typename TX>
int launch_fwd_tile(const FwdKernelParams& p, size_t smem, int nBT, int bpl, bool xsmem, const DeviceInfo& dev,
                    cudaStream_t stream, int* ctas_out) {
    if (xsmem) {
        if (bpl == 4) return launch_fwd_t<4, true, LOSS, TX>(p, smem, nBT, dev, stream, ctas_out);
        if (bpl == 2) return launch_fwd_t<2, true, LOSS, TX>(p, smem, nBT, dev, stream, ctas_out);
        return launch_fwd_t<1, true, LOSS, TX>(p, smem, nBT, dev, stream, ctas_out);
    }
    if (bpl == 4) return launch_fwd_t<4, false, LOSS, TX>(p, smem, nBT, dev, stream, ctas_out);
    if (bpl == 2) return launch_fwd_t<2, false, LOSS, TX>(p, smem, nBT, dev, stream, ctas_out);
    return launch_fwd_t<1, false, LOSS, TX>(p, smem, nBT, dev, stream, ctas_out);
}

}  // namespace

// Chooses batch elements per lane and whether the x tile is shared-memory resident.
// Exposed so that the host wrapper can tell which x layout / padding the launch needs.
bool forward_uses_smem_x(int B, int N, int K, int* bpl_out) {
    DeviceInfo dev;
    if (get_device_info(&dev) != FFI_OK) return false;
    const int Kp = static_cast<int>(round_up(K, 4));
    int bpl = B <= 32 ? 1 : (B <= 64 ? 2 : 4);
    for (int c = bpl; c >= 1; c /= 2) {
        if (pick_TO(dev.max_smem_optin, N, c, true, Kp) >= 16) {
            if (bpl_out) *bpl_out = c;
            return true;
        }
    }
    if (bpl_out) *bpl_out = bpl;
    return false;
}

int launch_forward_stream(const FwdArgs& a, cudaStream_t stream, bool* handled);
int launch_forward_gather(const FwdArgs& a, int bpl, float* gT, int64_t ldg, float scale, double* loss_partials,
                          int loss_kind, int max_partials, int* ctas, cudaStream_t stream, bool* handled);

// The CTA-tile kernel (any K, unaligned rows, x gathered from L2 when its tile does not fit shared memory);
// with `loss` set it writes the loss gradient instead of y (see FwdKernelParams).
struct TileLossEpilogue {
    float* gT;
    long long ldg;
    float scale;
    double* loss_partials;
    int loss_kind;
    int* ctas;
};
struct TileTopkEpilogue {
    uint2* lists;
    int* lists_per_tile;  // out: CTAs per batch tile x threads per batch element
    int* bt;              // out: batch tile width
};

static int launch_forward_tile(const FwdArgs& a, const TileLossEpilogue* loss, const TileTopkEpilogue* topk,
                               cudaStream_t stream) {
    DeviceInfo dev;
    int rc = get_device_info(&dev);
    if (rc != FFI_OK) return rc;
    FwdKernelParams p;
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
    p.Kp = static_cast<int>(round_up(a.K, 4));
    p.vec16 = (a.K % 4 == 0) && (reinterpret_cast<uintptr_t>(a.W) % (a.bf16 ? 8 : 16) == 0) &&
              (reinterpret_cast<uintptr_t>(a.idx) % 16 == 0);
    p.gT = loss ? loss->gT : nullptr;
    p.ldg = loss ? loss->ldg : 0;
    p.scale = loss ? loss->scale : 0.f;
    p.loss_partials = loss ? loss->loss_partials : nullptr;
    p.loss_kind = loss ? loss->loss_kind : 0;
    p.topk_lists = topk ? topk->lists : nullptr;

    int bpl = 1;
    const bool xsmem = forward_uses_smem_x(a.B, a.N, a.K, &bpl);
    if (!xsmem && !topk) {
        // wide inputs: the per-warp gather kernel where fan-in and alignment allow it
        bool handled = false;
        rc = launch_forward_gather(a, bpl, loss ? loss->gT : nullptr, loss ? loss->ldg : 0, loss ? loss->scale : 0.f,
                                   loss ? loss->loss_partials : nullptr, loss ? loss->loss_kind : 0, kMaxLossPartialsTile,
                                   loss ? loss->ctas : nullptr, stream, &handled);
        if (rc != FFI_OK || handled) return rc;
    }
    p.TO = pick_TO(dev.max_smem_optin, a.N, bpl, xsmem, p.Kp);
    if (p.TO < 16) return fail(FFI_ERR_UNSUPPORTED, "fan-in K=%d too large for the staged tiles", a.K);
    p.numTiles = static_cast<int>(ceil_div(a.L, p.TO));
    const size_t smem = fwd_smem_bytes(a.N, bpl, xsmem, p.TO, p.Kp);
    const int nBT = static_cast<int>(ceil_div(a.B, 32 * bpl));
    if (!xsmem) {
        // The global-memory gather reads whole lane vectors: rows must be padded and aligned.
        if (a.ldx % (32 * bpl) != 0 || a.ldx < static_cast<int64_t>(nBT) * 32 * bpl ||
            reinterpret_cast<uintptr_t>(a.xT) % 16 != 0)
            return fail(FFI_ERR_INVALID_ARGUMENT, "wide-N forward needs a padded, aligned x copy");
    }
    if (topk) {
        int ctas = 0;
        rc = a.bf16 ? launch_fwd_tile<2, __nv_bfloat16>(p, smem, nBT, bpl, xsmem, dev, stream, &ctas)
                    : launch_fwd_tile<2, float>(p, smem, nBT, bpl, xsmem, dev, stream, &ctas);
        *topk->bt = 32 * bpl;
        *topk->lists_per_tile = ctas / nBT * (kThreads / (32 * bpl));
        return rc;
    }
    if (a.bf16) {
        if (loss) return launch_fwd_tile<1, __nv_bfloat16>(p, smem, nBT, bpl, xsmem, dev, stream, loss->ctas);
        return launch_fwd_tile<0, __nv_bfloat16>(p, smem, nBT, bpl, xsmem, dev, stream, nullptr);
    }
    if (loss) return launch_fwd_tile<1, float>(p, smem, nBT, bpl, xsmem, dev, stream, loss->ctas);
    return launch_fwd_tile<0, float>(p, smem, nBT, bpl, xsmem, dev, stream, nullptr);
}

int launch_forward(const FwdArgs& a, cudaStream_t stream) {
    if (!a.bf16) {
        // Preferred: the barrier-free kernel (x tile in shared memory, K % 4 == 0, aligned rows).
        bool handled = false;
        int rc = launch_forward_stream(a, stream, &handled);
        if (rc != FFI_OK || handled) return rc;
    }
    return launch_forward_tile(a, nullptr, nullptr, stream);
}

// Forward with the loss gradient in the epilogue for the shapes the barrier-free kernel does not take
// (wide inputs, K not a multiple of 4): same outputs as launch_forward_bce_stream.
int launch_forward_loss_tile(const FwdArgs& a, float* gT, int64_t ldg, float scale, double* loss_partials, int* ctas,
                             int loss_kind, cudaStream_t stream) {
    TileLossEpilogue e{gT, ldg, scale, loss_partials, loss_kind, ctas};
    return launch_forward_tile(a, &e, nullptr, stream);
}

// Forward with the top-k epilogue for those shapes (and for bf16 storage): fills `lists` as
// [batch tile][*lists_per_tile][*bt][kTopK] for the merge kernel of forward_stream.cu.
int launch_forward_topk_tile(const FwdArgs& a, void* lists, int* lists_per_tile, int* bt, cudaStream_t stream) {
    TileTopkEpilogue e{static_cast<uint2*>(lists), lists_per_tile, bt};
    return launch_forward_tile(a, nullptr, &e, stream);
}

int launch_transpose_pad(const float* src, float* dst, int rows, int cols, int64_t ld_dst,
                         cudaStream_t stream) {
    dim3 block(32, 8);
    dim3 grid(static_cast<unsigned>(ceil_div(cols, 32)), static_cast<unsigned>(ceil_div(ld_dst, 32)));
    transpose_pad_kernel<<<grid, block, 0, stream>>>(src, dst, rows, cols, ld_dst);
    FFI_LAUNCH_CHECK("transpose_pad_kernel");
    return FFI_OK;
}

}  // namespace ffi
