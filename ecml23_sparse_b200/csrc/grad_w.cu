// grad_W and grad_bias of the fixed-fan-in sparse layer on sm_100a:
//   grad_W[o,k] = sum_b g[b,o] * x[b, idx[o,k]],   grad_bias[o] = sum_b g[b,o]
//
// Replaces the reference's backward_weights_vector / backward_weights_scalar kernels
// (tfsparse/cc/kernels/backward.cu.h:62-105,269-292) and TensorFlow's BiasAddGrad for
// the bias_add at sparse/layer.py:247.  (The reference's "skip g==0" test,
// backward.cu.h:73,94, only saves work; results are identical without it.)
//
// Dataflow.  Same geometry as the forward kernel: a lane owns BPL batch elements, a
// warp owns whole output rows, x_s[N][BT] is shared-memory resident and gathered with
// one conflict-free LDS per lane and entry.  Each lane multiplies the gathered x by its
// g[b,o] and the per-lane partial sums of a group of G entries are reduced across the
// warp with a transposing butterfly (G-1 + log2(32/G) shuffles per G entries), after
// which lane k holds grad_W[o,k]: the row is stored with one coalesced write.
// The batch is reduced in a fixed order (lane tree, then batch tiles in launch order),
// so results are bit-reproducible.
#include "ffi_common.cuh"

namespace ffi {
namespace {

constexpr int kThreads = 512;
constexpr int kWarps = kThreads / 32;
constexpr int kGRegs = 8;  // registers per thread that stage the next g tile

struct GradWKernelParams {
    const void* xT;    // element type TX of the kernel: float or __nv_bfloat16
    long long ldx;
    const int* idx;
    const float* g;    // upstream gradient [B][L], or nullptr when gT is given
    const float* gT;   // upstream gradient transposed to [L][ldg] (batch contiguous, zero padded)
    long long ldg;
    float* gW;
    float* gbias;
    int B, N, L, K;
    int Kp;        // K rounded up to a multiple of the group size G
    int TO;        // outputs per tile
    int numTiles;
    int vec16;
    int b0;         // first batch element of this launch's batch tile
    int accumulate; // add to gW / gbias instead of overwriting (batch tiles after the first)
};

// Sum s[0..G) over the 32 lanes. On return lane l holds in s[0] the total of entry
// (l >> (5 - log2 G)) ... see the caller for the mapping used.
template <int G>
__device__ __forceinline__ void butterfly_reduce(float (&s)[G], int lane) {
    // Halving steps: lanes whose bit `off` is set keep the upper half of the entries.
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
    // Remaining lane bits (below the ones consumed above) are plain all-reduce steps.
    constexpr int consumed = G == 32 ? 5 : (G == 16 ? 4 : (G == 8 ? 3 : (G == 4 ? 2 : (G == 2 ? 1 : 0))));
#pragma unroll
    for (int off = 16 >> consumed; off >= 1; off /= 2) s[0] += __shfl_xor_sync(0xffffffffu, s[0], off);
}

// TX: storage type of x; bf16 values are widened where they are loaded (exactly), so the arithmetic is
// that of the fp32 kernel on the same values.
template <int BPL, int G, bool XSMEM, typename TX>
__global__ void __launch_bounds__(kThreads, 1) ffi_grad_w_kernel(GradWKernelParams p) {
    constexpr int BT = 32 * BPL;
    const TX* xT = static_cast<const TX*>(p.xT);
    constexpr int LOG2G = G == 32 ? 5 : (G == 16 ? 4 : (G == 8 ? 3 : 2));
    using V = typename Vec<BPL>::type;
    extern __shared__ __align__(16) unsigned char smem_raw[];

    float* x_s = reinterpret_cast<float*>(smem_raw);
    int* i_s = reinterpret_cast<int*>(x_s + (XSMEM ? static_cast<size_t>(p.N) * BT : 0));
    float* g_s = reinterpret_cast<float*>(i_s + 2 * p.TO * p.Kp);

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int b0 = p.b0;
    const int TO = p.TO, Kp = p.Kp, K = p.K, L = p.L;
    const int tileElems = TO * Kp;

    for (int e = tid; e < 2 * tileElems; e += kThreads) i_s[e] = 0;
    if (XSMEM) {
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
        int* id = i_s + buf * tileElems;
        const int* isrc = p.idx + o0 * K;
        if (p.vec16) {
            const int nvec = nrows * K / 4;
            for (int v = tid; v < nvec; v += kThreads) __pipeline_memcpy_async(id + 4 * v, isrc + 4 * v, 16);
        } else {
            const int n = nrows * K;
            for (int e = tid; e < n; e += kThreads) {
                int r = e / K;
                int k = e - r * K;
                __pipeline_memcpy_async(id + r * Kp + k, isrc + e, 4);
            }
        }
        __pipeline_commit();
    };

    const V* xs_lane = reinterpret_cast<const V*>(x_s) + lane;
    const TX* xg_base = xT + b0;
    const size_t ldv = static_cast<size_t>(p.ldx / BPL);

    // The g tile of the next output tile is fetched into registers while the current tile is
    // being computed (kGRegs * 512 >= TO * BT by construction of TO).
    // Element e of the tile is (batch row r, output c): consecutive threads run along the contiguous
    // dimension of whichever layout the gradient comes in.
    const bool fromT = p.g == nullptr;
    auto tile_rc = [&](int e, int& r, int& c) {
        if (fromT) {
            c = e / BT;
            r = e - c * BT;
        } else {
            r = e / TO;
            c = e - r * TO;
        }
    };
    float gpre[kGRegs];
    auto load_g = [&](int t) {
        const long long o0 = static_cast<long long>(t) * TO;
#pragma unroll
        for (int u = 0; u < kGRegs; ++u) {
            int r, c;
            tile_rc(tid + u * kThreads, r, c);
            const int b = b0 + r;
            const bool live = r < BT && c < TO && b < p.B && o0 + c < L;
            const float* src = fromT ? p.gT + static_cast<size_t>(o0 + c) * p.ldg + b : p.g + static_cast<size_t>(b) * L + o0 + c;
            gpre[u] = live ? __ldg(src) : 0.f;
        }
    };

    int t = blockIdx.x;
    int buf = 0;
    if (t < p.numTiles) {
        prefetch(t, 0);
        load_g(t);
    }
    for (; t < p.numTiles; t += gridDim.x, buf ^= 1) {
        const long long o0 = static_cast<long long>(t) * TO;
        __syncthreads();  // everyone is done reading g_s of the previous tile
        // g tile, transposed into g_s[o][b] (row stride BT+1: conflict-free both ways).
#pragma unroll
        for (int u = 0; u < kGRegs; ++u) {
            int r, c;
            tile_rc(tid + u * kThreads, r, c);
            if (r < BT && c < TO) g_s[c * (BT + 1) + r] = gpre[u];
        }
        __pipeline_wait_prior(0);
        __syncthreads();  // idx tile t and g_s visible
        const int tn = t + gridDim.x;
        if (tn < p.numTiles) {
            prefetch(tn, buf ^ 1);
            load_g(tn);
        }

        const int* ib = i_s + buf * tileElems;
        for (int ol = warp; ol < TO; ol += kWarps) {
            const long long o = o0 + ol;
            if (o >= L) break;
            float gv[BPL];
            float gsum = 0.f;
#pragma unroll
            for (int j = 0; j < BPL; ++j) {
                const int bl = XSMEM ? lane + 32 * j : lane * BPL + j;
                gv[j] = g_s[ol * (BT + 1) + bl];
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
            const int* ir = ib + ol * Kp;
            for (int kg = 0; kg < Kp; kg += G) {
                float s[G];
#pragma unroll
                for (int k4 = 0; k4 < G / 4; ++k4) {
                    const int4 ii = *reinterpret_cast<const int4*>(ir + kg + 4 * k4);
                    V v0, v1, v2, v3;
                    if (XSMEM) {
                        v0 = xs_lane[ii.x * 32];
                        v1 = xs_lane[ii.y * 32];
                        v2 = xs_lane[ii.z * 32];
                        v3 = xs_lane[ii.w * 32];
                    } else {
                        v0 = load_lane_vec<BPL>(xg_base, static_cast<size_t>(ii.x) * ldv + lane);
                        v1 = load_lane_vec<BPL>(xg_base, static_cast<size_t>(ii.y) * ldv + lane);
                        v2 = load_lane_vec<BPL>(xg_base, static_cast<size_t>(ii.z) * ldv + lane);
                        v3 = load_lane_vec<BPL>(xg_base, static_cast<size_t>(ii.w) * ldv + lane);
                    }
                    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
                    for (int j = 0; j < BPL; ++j) {
                        a0 = fmaf(gv[j], vec_get(v0, j), a0);
                        a1 = fmaf(gv[j], vec_get(v1, j), a1);
                        a2 = fmaf(gv[j], vec_get(v2, j), a2);
                        a3 = fmaf(gv[j], vec_get(v3, j), a3);
                    }
                    s[4 * k4 + 0] = a0;
                    s[4 * k4 + 1] = a1;
                    s[4 * k4 + 2] = a2;
                    s[4 * k4 + 3] = a3;
                }
                butterfly_reduce<G>(s, lane);
                // After the halving steps the lane's top LOG2G bits select the entry.
                const int k = kg + (lane >> (5 - LOG2G));
                if (p.gW && (lane & ((1 << (5 - LOG2G)) - 1)) == 0 && k < K) {
                    float* dst = p.gW + static_cast<size_t>(o) * K + k;
                    if (p.accumulate) *dst += s[0];
                    else *dst = s[0];
                }
            }
        }
    }
    __pipeline_wait_prior(0);
}

size_t gw_smem_bytes(int N, int bpl, bool xsmem, int TO, int Kp) {
    const size_t BT = 32 * bpl;
    return (xsmem ? static_cast<size_t>(N) * BT * 4 : 0) + static_cast<size_t>(2) * TO * Kp * 4 +
           static_cast<size_t>(TO) * (BT + 1) * 4;
}

int gw_pick_TO(size_t budget, int N, int bpl, bool xsmem, int Kp) {
    const size_t BT = 32 * bpl;
    const size_t fixed = xsmem ? static_cast<size_t>(N) * BT * 4 : 0;
    if (fixed >= budget) return 0;
    const size_t per_row = static_cast<size_t>(2) * Kp * 4 + (BT + 1) * 4;
    size_t to = (budget - fixed) / per_row;
    if (to > 128) to = 128;
    if (to * BT > static_cast<size_t>(kGRegs) * kThreads) to = kGRegs * kThreads / BT;
    return static_cast<int>(to / 16 * 16);
}

template <int BPL, int G, bool XSMEM, typename TX>
int launch_gw_t(GradWKernelParams p, size_t smem, int nBT, const DeviceInfo& dev, cudaStream_t stream) {
    auto kern = ffi_grad_w_kernel<BPL, G, XSMEM, TX>;
    FFI_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        static_cast<int>(smem)));
    int occ = 0;
    FFI_CUDA_CHECK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, kThreads, smem));
    if (occ < 1) return fail(FFI_ERR_CUDA, "grad_W kernel does not fit on an SM (smem %zu)", smem);
    const unsigned grid = static_cast<unsigned>(min(p.numTiles, dev.sm_count * occ));
    // Batch tiles run as consecutive launches so that tile t adds to what tile t-1 wrote.
    for (int bt = 0; bt < nBT; ++bt) {
        p.b0 = bt * 32 * BPL;
        p.accumulate = bt > 0;
        kern<<<grid, kThreads, smem, stream>>>(p);
        FFI_LAUNCH_CHECK("ffi_grad_w_kernel");
    }
    return FFI_OK;
}

template <int BPL, bool XSMEM, typename TX>
int launch_gw_g(const GradWKernelParams& p, int G, size_t smem, int nBT, const DeviceInfo& dev,
                cudaStream_t stream) {
    switch (G) {
        case 4: return launch_gw_t<BPL, 4, XSMEM, TX>(p, smem, nBT, dev, stream);
        case 8: return launch_gw_t<BPL, 8, XSMEM, TX>(p, smem, nBT, dev, stream);
        case 16: return launch_gw_t<BPL, 16, XSMEM, TX>(p, smem, nBT, dev, stream);
        default: return launch_gw_t<BPL, 32, XSMEM, TX>(p, smem, nBT, dev, stream);
    }
}

template <typename TX>
int launch_gw_x(const GradWKernelParams& p, int G, size_t smem, int nBT, int bpl, bool xsmem, const DeviceInfo& dev,
                cudaStream_t stream) {
    if (xsmem) {
        if (bpl == 4) return launch_gw_g<4, true, TX>(p, G, smem, nBT, dev, stream);
        if (bpl == 2) return launch_gw_g<2, true, TX>(p, G, smem, nBT, dev, stream);
        return launch_gw_g<1, true, TX>(p, G, smem, nBT, dev, stream);
    }
    if (bpl == 4) return launch_gw_g<4, false, TX>(p, G, smem, nBT, dev, stream);
    if (bpl == 2) return launch_gw_g<2, false, TX>(p, G, smem, nBT, dev, stream);
    return launch_gw_g<1, false, TX>(p, G, smem, nBT, dev, stream);
}

int pick_group(int K) {
    // Fewest padded entries; larger groups win ties (fewer shuffles per entry).
    int best = 32;
    int64_t best_pad = round_up(K, 32);
    for (int G : {16, 8, 4}) {
        int64_t pad = round_up(K, G);
        if (pad < best_pad) {
            best = G;
            best_pad = pad;
        }
    }
    return best;
}

}  // namespace

bool grad_w_uses_smem_x(int B, int N, int K, int* bpl_out) {
    DeviceInfo dev;
    if (get_device_info(&dev) != FFI_OK) return false;
    const int G = pick_group(K);
    const int Kp = static_cast<int>(round_up(K, G));
    int bpl = B <= 32 ? 1 : (B <= 64 ? 2 : 4);
    for (int c = bpl; c >= 1; c /= 2) {
        if (gw_pick_TO(dev.max_smem_optin, N, c, true, Kp) >= 16) {
            if (bpl_out) *bpl_out = c;
            return true;
        }
    }
    if (bpl_out) *bpl_out = bpl;
    return false;
}

int launch_grad_w_stream(const GradWArgs& a, cudaStream_t stream, bool* handled);
int launch_grad_w_gather(const GradWArgs& a, int bpl, cudaStream_t stream, bool* handled);

int launch_grad_w(const GradWArgs& a, cudaStream_t stream) {
    DeviceInfo dev;
    int rc = get_device_info(&dev);
    if (rc != FFI_OK) return rc;
    {
        // Preferred: the barrier-free kernel (x tile in shared memory, K % 4 == 0, aligned idx).
        bool handled = false;
        rc = launch_grad_w_stream(a, stream, &handled);
        if (rc != FFI_OK || handled) return rc;
    }

    GradWKernelParams p;
    p.xT = a.xT;
    p.ldx = a.ldx;
    p.idx = a.idx;
    p.g = a.g;
    p.gT = a.gT;
    p.ldg = a.ldg;
    if (!a.g && !a.gT) return fail(FFI_ERR_INVALID_ARGUMENT, "grad_W needs the upstream gradient");
    p.gW = a.gW;
    p.gbias = a.gbias;
    p.B = a.B;
    p.N = a.N;
    p.L = a.L;
    p.K = a.K;
    const int G = pick_group(a.K);
    p.Kp = static_cast<int>(round_up(a.K, G));
    p.vec16 = (a.K % 4 == 0) && (p.Kp == a.K) && (reinterpret_cast<uintptr_t>(a.idx) % 16 == 0);
    p.b0 = 0;
    p.accumulate = 0;

    int bpl = 1;
    const bool xsmem = grad_w_uses_smem_x(a.B, a.N, a.K, &bpl);
    if (!xsmem) {
        // wide inputs: the per-warp gather kernel where the transposed gradient and aligned rows allow it
        bool handled = false;
        rc = launch_grad_w_gather(a, bpl, stream, &handled);
        if (rc != FFI_OK || handled) return rc;
    }
    p.TO = gw_pick_TO(dev.max_smem_optin, a.N, bpl, xsmem, p.Kp);
    if (p.TO < 16) return fail(FFI_ERR_UNSUPPORTED, "fan-in K=%d too large for the staged tiles", a.K);
    p.numTiles = static_cast<int>(ceil_div(a.L, p.TO));
    const size_t smem = gw_smem_bytes(a.N, bpl, xsmem, p.TO, p.Kp);
    const int nBT = static_cast<int>(ceil_div(a.B, 32 * bpl));
    if (!xsmem) {
        if (a.ldx % (32 * bpl) != 0 || a.ldx < static_cast<int64_t>(nBT) * 32 * bpl ||
            reinterpret_cast<uintptr_t>(a.xT) % 16 != 0)
            return fail(FFI_ERR_INVALID_ARGUMENT, "wide-N grad_W needs a padded, aligned x copy");
    }
    if (a.bf16) return launch_gw_x<__nv_bfloat16>(p, G, smem, nBT, bpl, xsmem, dev, stream);
    return launch_gw_x<float>(p, G, smem, nBT, bpl, xsmem, dev, stream);
}

}  // namespace ffi
