// Forward of the fixed-fan-in sparse layer, barrier-free variant for the common case
// (x tile resident in shared memory, K a multiple of 4, 16-byte aligned W and idx).
//
// Same arithmetic as ffi_fwd_kernel (forward.cu), but every warp is its own pipeline: it owns a private double buffer for the W/idx rows of
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
    // top-k epilogue: every warp keeps, per batch element of the tile, the kTopK best logits of the
    // rows it computed; lists [tile][cta][warp][batch][kTopK] of (value, row) go to `topk_lists`
    uint2* topk_lists;
};

constexpr size_t kMaxLossPartials = 1024;  // doubles the caller's scratch holds for the per-CTA loss sums

// A HALF warp covers the batch tile (16 lanes x VPL batch elements) and the two halves of a warp
// work on the two rows of a row pair at once.  The fetch of a row's W and idx values is then one
// shared-memory access for both rows (two addresses, one per half) instead of a warp-uniform access
// per row; against a whole warp per row this took a fifth off the traffic of the shared-memory pipe,
// the unit this kernel is bound by (0.56 -> 0.48 ms at B=128, N=768, L=670,091, K=32).
// x tile in natural order: x_s[i][b].
template <int VPL>
__device__ __forceinline__ int pair_column(int q, int j) {
    if constexpr (VPL == 8) return j < 4 ? 4 * q + j : 64 + 4 * q + (j - 4);
    else return VPL * q + j;
}

// (Keeping the indices as 16-bit values in the warp's buffer, four per 8-byte access, was measured:
// the repacking on the way in costs more than the narrower fetch saves, 0.50 vs 0.48 ms.)
template <int VPL, int MODE>
__global__ void __launch_bounds__(kThreads, 1) ffi_fwd_pair_kernel(FwdStreamParams p) {
    constexpr bool BCE = MODE == 1;  // 0: write y; 1: loss epilogue; 2: running top-k of the logits
    constexpr int BT = 16 * VPL;
    constexpr int S = BT + 8;  // result-tile row stride: 16-byte rows, conflict-free for both access patterns
    extern __shared__ __align__(16) unsigned char smem_raw[];

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int h = lane >> 4;  // which row of a pair
    const int q = lane & 15;
    const int b0 = blockIdx.y * BT;
    const int K = p.K, L = p.L;

    float* x_s = reinterpret_cast<float*>(smem_raw);
    const int regionWords = 8 * K + 4 * S;
    float* region = x_s + static_cast<size_t>(p.N) * BT + static_cast<size_t>(warp) * regionWords;
    float* wi = region;
    float* ys = region + 8 * K;

    const float* xs_lane = x_s + (VPL == 8 ? 4 : VPL) * q;
    const long long numQuads = (static_cast<long long>(L) + 3) / 4;
    const long long gw = static_cast<long long>(blockIdx.x) * kWarps + warp;
    const long long GW = static_cast<long long>(gridDim.x) * kWarps;
    const int chunksPerRow = K / 2;
    const int nChunks = 2 * chunksPerRow;

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

    // the warp's first W/idx rows are requested before the x tile is filled: both trips to memory overlap
    long long qd = gw;
    if (qd < numQuads) issue(2 * qd, 0);

    if (p.ldx % 4 == 0 && b0 + BT <= p.B && reinterpret_cast<uintptr_t>(p.xT) % 16 == 0) {
        // whole tile inside the batch, rows 16-byte aligned: 16-byte loads and stores
        constexpr int VR = BT / 4;
        const int total = p.N * VR;
#pragma unroll 12
        for (int e = tid; e < total; e += kThreads) {
            const int i = e / VR;
            const int v = e - i * VR;
            reinterpret_cast<float4*>(x_s)[e] =
                __ldg(reinterpret_cast<const float4*>(p.xT + static_cast<size_t>(i) * p.ldx + b0) + v);
        }
    } else {
        const int total = p.N * BT;
#pragma unroll 8
        for (int e = tid; e < total; e += kThreads) {
            const int i = e / BT;
            const int bl = e - i * BT;
            const int b = b0 + bl;
            x_s[e] = b < p.B ? p.xT[static_cast<size_t>(i) * p.ldx + b] : 0.f;
        }
    }
    __syncthreads();

    int s = 0;
    float loss_local = 0.f;
    // top-k mode: lane keeps the lists of batch columns lane, lane + 32, ... of the tile
    constexpr int TM = MODE == 2 ? (BT + 31) / 32 : 1;
    float tv[TM][kTopK];
    int ti[TM][kTopK];
#pragma unroll
    for (int m = 0; m < TM; ++m)
#pragma unroll
        for (int j = 0; j < kTopK; ++j) tv[m][j] = -INFINITY, ti[m][j] = 0x7fffffff;
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
                const bool mine = oA + h < L;       // false only for the missing second row of an odd L
                const long long o = mine ? oA + h : oA;
                const float* row = wi + buf * 4 * K + (mine ? h : 0) * 2 * K;
                const float4* wr = reinterpret_cast<const float4*>(row);
                const int4* ir = reinterpret_cast<const int4*>(row + K);
                const float bias = p.bias ? __ldg(p.bias + o) : 0.f;
                float acc[VPL];
#pragma unroll
                for (int j = 0; j < VPL; ++j) acc[j] = 0.f;
#pragma unroll 2
                for (int k4 = 0; k4 < K / 4; ++k4) {
                    const int4 i4 = ir[k4];
                    const float4 w4 = wr[k4];
                    const int ii[4] = {i4.x, i4.y, i4.z, i4.w};
                    const float ww[4] = {w4.x, w4.y, w4.z, w4.w};
                    float a[4][VPL];
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const float* src = xs_lane + ii[u] * BT;
                        if constexpr (VPL == 2) {
                            const float2 t = *reinterpret_cast<const float2*>(src);
                            a[u][0] = t.x, a[u][1] = t.y;
                        } else {
                            const float4 t = *reinterpret_cast<const float4*>(src);
                            a[u][0] = t.x, a[u][1] = t.y, a[u][2] = t.z, a[u][3] = t.w;
                            if constexpr (VPL == 8) {
                                const float4 t2 = *reinterpret_cast<const float4*>(src + 64);
                                a[u][4] = t2.x, a[u][5] = t2.y, a[u][6] = t2.z, a[u][7] = t2.w;
                            }
                        }
                    }
#pragma unroll
                    for (int u = 0; u < 4; ++u)
#pragma unroll
                        for (int j = 0; j < VPL; ++j) acc[j] = fmaf(ww[u], a[u][j], acc[j]);
                }
                if constexpr (BCE) {
                    // a lane holds runs of 4 (or 2) consecutive batch elements of its row: vector stores
#pragma unroll
                    for (int j0 = 0; j0 < VPL; j0 += (VPL == 2 ? 2 : 4)) {
                        constexpr int W4 = VPL == 2 ? 2 : 4;
                        const int b = b0 + pair_column<VPL>(q, j0);
                        float gv[W4];
#pragma unroll
                        for (int j = 0; j < W4; ++j) {
                            const bool live = b + j < p.B;
                            float v, g;
                            loss_for_negative(p.loss_kind, acc[j0 + j] + bias, v, g);
                            if (live && mine) loss_local += v;
                            gv[j] = live ? p.scale * g : 0.f;
                        }
                        if (mine && b < p.ldg) {
                            float* dst = p.gT + static_cast<size_t>(o) * p.ldg + b;
                            if constexpr (W4 == 4) *reinterpret_cast<float4*>(dst) = make_float4(gv[0], gv[1], gv[2], gv[3]);
                            else *reinterpret_cast<float2*>(dst) = make_float2(gv[0], gv[1]);
                        }
                    }
                } else {
                    float* yrow = ys + (2 * half + h) * S;
#pragma unroll
                    for (int j = 0; j < VPL; ++j) yrow[pair_column<VPL>(q, j)] = acc[j] + bias;
                }
            }
            __syncwarp();
        }
        if constexpr (MODE == 2) {
            const long long oq = 4 * qd;
#pragma unroll
            for (int m = 0; m < TM; ++m) {
                const int bl = lane + 32 * m;
                if (bl < BT && b0 + bl < p.B) {
#pragma unroll
                    for (int oo = 0; oo < 4; ++oo)
                        if (oq + oo < L) topk_insert(tv[m], ti[m], ys[oo * S + bl], static_cast<int>(oq + oo));
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
                if (b0 + bl < p.B && oq + oo < L)
                    p.y[static_cast<size_t>(b0 + bl) * L + oq + oo] = ys[oo * S + bl];
            }
            __syncwarp();
        }
    }
    __pipeline_wait_prior(0);

    if constexpr (MODE == 2) {
        uint2* out = p.topk_lists +
                     ((static_cast<size_t>(blockIdx.y) * gridDim.x + blockIdx.x) * kWarps + warp) * (BT * kTopK);
#pragma unroll
        for (int m = 0; m < TM; ++m) {
            const int bl = lane + 32 * m;
            if (bl < BT)
#pragma unroll
                for (int j = 0; j < kTopK; ++j)
                    out[bl * kTopK + j] = make_uint2(__float_as_uint(tv[m][j]), static_cast<unsigned>(ti[m][j]));
        }
    }

    if constexpr (BCE) {
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

template <int VPL, int MODE>
int launch_pair_t(const FwdStreamParams& p, size_t smem, int nBT, const DeviceInfo& dev, cudaStream_t stream,
                  int* ctas_out) {
    auto kern = ffi_fwd_pair_kernel<VPL, MODE>;
    FFI_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    int occ = 0;
    FFI_CUDA_CHECK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, kThreads, smem));
    if (occ < 1) return fail(FFI_ERR_CUDA, "streaming forward kernel does not fit on an SM (smem %zu)", smem);
    // The epilogue variants write one record per CTA (loss partial, top-k lists) into scratch that is
    // sized for one CTA per SM, whatever occupancy the kernel would allow.
    if (MODE != 0) occ = 1;
    int per_bt = dev.sm_count * occ / nBT;
    if (per_bt < 1) per_bt = 1;
    const long long numQuads = (static_cast<long long>(p.L) + 3) / 4;
    const long long want = (numQuads + kWarps - 1) / kWarps;
    dim3 grid(static_cast<unsigned>(want < per_bt ? want : per_bt), static_cast<unsigned>(nBT));
    if (MODE == 1 && static_cast<size_t>(grid.x) * grid.y > kMaxLossPartials)
        return fail(FFI_ERR_UNSUPPORTED, "the fused loss keeps at most %zu per-CTA partials; this batch needs %u",
                    kMaxLossPartials, grid.x * grid.y);
    if (ctas_out) *ctas_out = static_cast<int>(grid.x * grid.y);
    kern<<<grid, kThreads, smem, stream>>>(p);
    FFI_LAUNCH_CHECK("ffi_fwd_pair_kernel");
    return FFI_OK;
}

// One block per batch element: the best kk of all warp lists of its tile, in tf.nn.top_k order.
__global__ void __launch_bounds__(256) topk_merge_kernel(const uint2* __restrict__ lists, int listsPerTile, int BT,
                                                         int B, int kk, int label_offset,
                                                         float* __restrict__ out_val, int* __restrict__ out_idx) {
    __shared__ float sv[256][kTopK];
    __shared__ int si[256][kTopK];
    const int b = blockIdx.x;
    const int tile = b / BT, bl = b - tile * BT;
    float tv[kTopK];
    int ti[kTopK];
#pragma unroll
    for (int j = 0; j < kTopK; ++j) tv[j] = -INFINITY, ti[j] = 0x7fffffff;
    for (int l = threadIdx.x; l < listsPerTile; l += blockDim.x) {
        const uint2* src = lists + (static_cast<size_t>(tile) * listsPerTile + l) * (BT * kTopK) + bl * kTopK;
#pragma unroll
        for (int j = 0; j < kTopK; ++j) {
            const uint2 c = src[j];
            topk_insert(tv, ti, __uint_as_float(c.x), static_cast<int>(c.y));
        }
    }
    // tree over the threads: 256 -> 32 -> 1 lists
    for (int width = 256; width > 1; width /= 8) {
#pragma unroll
        for (int j = 0; j < kTopK; ++j) sv[threadIdx.x][j] = tv[j], si[threadIdx.x][j] = ti[j];
        __syncthreads();
        const int next = width / 8;
        if (static_cast<int>(threadIdx.x) < next) {
            for (int u = 1; u < 8; ++u) {
                const int src = threadIdx.x + u * next;
#pragma unroll
                for (int j = 0; j < kTopK; ++j) topk_insert(tv, ti, sv[src][j], si[src][j]);
            }
        }
        __syncthreads();
        if (next < 8 && next > 1) {  // 4 lists left: thread 0 finishes
#pragma unroll
            for (int j = 0; j < kTopK; ++j) sv[threadIdx.x][j] = tv[j], si[threadIdx.x][j] = ti[j];
            __syncthreads();
            if (threadIdx.x == 0)
                for (int u = 1; u < next; ++u)
#pragma unroll
                    for (int j = 0; j < kTopK; ++j) topk_insert(tv, ti, sv[u][j], si[u][j]);
            break;
        }
    }
    if (threadIdx.x == 0) {
        for (int j = 0; j < kk; ++j) {
            out_val[static_cast<size_t>(b) * kk + j] = tv[j];
            out_idx[static_cast<size_t>(b) * kk + j] = ti[j] == 0x7fffffff ? -1 : ti[j] + label_offset;
        }
    }
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
struct TopkEpilogue {
    uint2* lists;  // scratch from forward_topk_workspace_bytes
    int* ctas_x;   // out: CTAs per batch tile
    int* bt;       // out: batch tile width
};

static int launch_forward_stream_impl(const FwdArgs& a, const BceEpilogue* bce, const TopkEpilogue* topk,
                                      cudaStream_t stream, bool* handled) {
    *handled = false;
    DeviceInfo dev;
    int rc = get_device_info(&dev);
    if (rc != FFI_OK) return rc;
    if (a.bf16) return FFI_OK;  // this kernel reads fp32 only
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
    p.xT = static_cast<const float*>(a.xT);
    p.ldx = a.ldx;
    p.idx = a.idx;
    p.W = static_cast<const float*>(a.W);
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
    p.topk_lists = topk ? topk->lists : nullptr;
    const int nBT = static_cast<int>(ceil_div(a.B, 32 * bpl));
    *handled = true;
    // same tile sizes and shared-memory footprint: BT = 32 * bpl = 16 * VPL
    if (topk) {
        int ctas = 0;
        if (bpl == 4) rc = launch_pair_t<8, 2>(p, smem, nBT, dev, stream, &ctas);
        else if (bpl == 2) rc = launch_pair_t<4, 2>(p, smem, nBT, dev, stream, &ctas);
        else rc = launch_pair_t<2, 2>(p, smem, nBT, dev, stream, &ctas);
        *topk->ctas_x = ctas / nBT;
        *topk->bt = 32 * bpl;
        return rc;
    }
    if (bce) {
        if (bpl == 4) return launch_pair_t<8, 1>(p, smem, nBT, dev, stream, bce->ctas);
        if (bpl == 2) return launch_pair_t<4, 1>(p, smem, nBT, dev, stream, bce->ctas);
        return launch_pair_t<2, 1>(p, smem, nBT, dev, stream, bce->ctas);
    }
    if (bpl == 4) return launch_pair_t<8, 0>(p, smem, nBT, dev, stream, nullptr);
    if (bpl == 2) return launch_pair_t<4, 0>(p, smem, nBT, dev, stream, nullptr);
    return launch_pair_t<2, 0>(p, smem, nBT, dev, stream, nullptr);
}

// Launches the barrier-free kernel when the shape allows it; *handled tells the caller.
int launch_forward_stream(const FwdArgs& a, cudaStream_t stream, bool* handled) {
    return launch_forward_stream_impl(a, nullptr, nullptr, stream, handled);
}

// Forward with the fused sigmoid-BCE epilogue: writes gT[o][b] = scale * sigmoid(z[b,o]) (zero in the
// padded batch columns) and one partial of sum softplus(z) per CTA; *ctas receives their number
// (at most 2 * SM count).  *handled is false when the shape needs the unfused path.
int launch_forward_bce_stream(const FwdArgs& a, float* gT, int64_t ldg, float scale, double* loss_partials, int* ctas,
                              int loss_kind, cudaStream_t stream, bool* handled) {
    BceEpilogue e{gT, ldg, scale, loss_partials, ctas, loss_kind};
    return launch_forward_stream_impl(a, &e, nullptr, stream, handled);
}

int launch_forward_topk_tile(const FwdArgs& a, void* lists, int* lists_per_tile, int* bt, cudaStream_t stream);

// Scratch for the warp lists of forward_topk: an upper bound over the grids the launcher may choose.
size_t forward_topk_workspace_bytes(int64_t B) {
    DeviceInfo dev;
    if (get_device_info(&dev) != FFI_OK) return 0;
    // tiles * CTAs per tile <= SM count (one CTA per SM), BT <= 128
    const size_t lists = static_cast<size_t>(dev.sm_count + ceil_div(B, 32)) * kWarps;
    return lists * 128 * kTopK * sizeof(uint2);
}

// Forward whose epilogue keeps the best logits per batch element instead of writing y; top_val/top_idx
// [B][kk] receive them in tf.nn.top_k order (row + label_offset as the index).  *handled as above.
int launch_forward_topk_stream(const FwdArgs& a, void* scratch, float* top_val, int* top_idx, int kk, int label_offset,
                               cudaStream_t stream, bool* handled) {
    if (kk < 1 || kk > kTopK) return fail(FFI_ERR_UNSUPPORTED, "top-k supports 1 <= k <= %d", kTopK);
    int ctas_x = 0, bt = 0;
    TopkEpilogue e{static_cast<uint2*>(scratch), &ctas_x, &bt};
    int rc = launch_forward_stream_impl(a, nullptr, &e, stream, handled);
    if (rc != FFI_OK) return rc;
    int lists_per_tile = ctas_x * kWarps;
    if (!*handled) {  // wide inputs, K not a multiple of 4, bf16 storage: the CTA-tile kernel's top-k epilogue
        rc = launch_forward_topk_tile(a, scratch, &lists_per_tile, &bt, stream);
        if (rc != FFI_OK) return rc;
        *handled = true;
    }
    topk_merge_kernel<<<static_cast<unsigned>(a.B), 256, 0, stream>>>(static_cast<const uint2*>(scratch), lists_per_tile,
                                                                      bt, a.B, kk, label_offset, top_val, top_idx);
    FFI_LAUNCH_CHECK("topk_merge_kernel");
    return FFI_OK;
}

}  // namespace ffi
