// grad_W (and grad_bias) for wide inputs on sm_100a: x does not fit shared memory, every entry gathers its
// operand row x[:, idx[o,k]] from L2.
//   grad_W[o,k] = sum_b g[b,o] * x[b, idx[o,k]],   grad_bias[o] = sum_b g[b,o]
//
// Replaces the reference's backward_weights_vector / backward_weights_scalar kernels
// (tfsparse/cc/kernels/backward.cu.h:62-105,269-292) for the output layers of the stacked configurations
// (hidden widths of 32,768 ... 100,000).
//
// What bounds this shape is the number of gathered bytes in flight per SM (B*L*K*e bytes cross the L2-to-SM
// fabric, every load takes about a microsecond), so the kernel is built to keep many loads in flight with few
// registers: every warp is its own pipeline (no CTA barrier), a lane owns BPL batch elements, its g values come
// straight from the transposed gradient (one vector load per row), eight gathers are issued back to back, each
// lane's partial product sum goes to a per-warp buffer in shared memory (32 entries x 32 lanes), and once a group
// of up to 32 entries is complete lane k adds the 32 partials of entry k in a fixed order and the row segment
// leaves as one coalesced store.  No shuffles, no accumulator array: 64 registers per thread, 32 warps per SM.
// Batch tiles run as consecutive launches (tile t adds to what tile t-1 wrote), so the batch is reduced in a
// fixed order and results are bit-reproducible.
#include <type_traits>

#include "ffi_common.cuh"

namespace ffi {
namespace {

constexpr int kThreads = 512;
constexpr int kWarps = kThreads / 32;
constexpr int kRow = 36;  // floats per buffered entry: 32 partials + padding (16-byte rows, conflict-free both ways)

struct GatherParams {
    const void* xT;  // [N][ldx], element type TX
    long long ldx;
    const int* idx;
    const float* gT;  // [L][ldg], batch contiguous, zero padded
    long long ldg;
    float* gW;
    float* gbias;
    int B, N, L, K;
    int b0;          // first batch element of this launch's batch tile
    int accumulate;  // add to gW / gbias instead of overwriting (batch tiles after the first)
};

template <int BPL, typename TX>
__global__ void __launch_bounds__(kThreads, 2) ffi_grad_w_gather_kernel(GatherParams p) {
    using V = typename Vec<BPL>::type;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int K = p.K, L = p.L;
    // per warp: 32 buffered entries, then two idx rows
    float* dbuf = reinterpret_cast<float*>(smem_raw) + static_cast<size_t>(warp) * (32 * kRow + 2 * K);
    int* ibuf = reinterpret_cast<int*>(dbuf + 32 * kRow);

    const TX* xg = static_cast<const TX*>(p.xT) + p.b0;
    const size_t ldv = static_cast<size_t>(p.ldx / BPL);
    const long long GW = static_cast<long long>(gridDim.x) * kWarps;
    long long o = static_cast<long long>(blockIdx.x) * kWarps + warp;

    auto issue = [&](long long row, int buf) {
        if (row < L)
            for (int c = lane; c < K / 4; c += 32)
                __pipeline_memcpy_async(ibuf + buf * K + 4 * c, p.idx + row * K + 4 * c, 16);
        __pipeline_commit();
    };

    issue(o, 0);
    const float4* drow = reinterpret_cast<const float4*>(dbuf + lane * kRow);
    for (int s = 0; o < L; o += GW, s ^= 1) {
        issue(o + GW, s ^ 1);
        // this lane's g values of the row
        float gv[BPL];
        load_lane_f32<BPL>(p.gT + static_cast<size_t>(o) * p.ldg + p.b0, lane, gv);
        if (p.gbias) {
            float gsum = 0.f;
#pragma unroll
            for (int j = 0; j < BPL; ++j) gsum += gv[j];
#pragma unroll
            for (int off = 16; off >= 1; off /= 2) gsum += __shfl_xor_sync(0xffffffffu, gsum, off);
            if (lane == 0) {
                if (p.accumulate) p.gbias[o] += gsum;
                else p.gbias[o] = gsum;
            }
        }
        __pipeline_wait_prior(1);
        __syncwarp();
        const int* ir = ibuf + s * K;
        for (int kg = 0; kg < K; kg += 32) {
            const int n = min(32, K - kg);  // a multiple of 4
            int k = 0;
            for (; k + 8 <= n; k += 8) {
                const int4 i0 = *reinterpret_cast<const int4*>(ir + kg + k);
                const int4 i1 = *reinterpret_cast<const int4*>(ir + kg + k + 4);
                const int ii[8] = {i0.x, i0.y, i0.z, i0.w, i1.x, i1.y, i1.z, i1.w};
                V v[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) v[u] = load_lane_vec<BPL>(xg, static_cast<size_t>(ii[u]) * ldv + lane);
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    float a = 0.f;
#pragma unroll
                    for (int j = 0; j < BPL; ++j) a = fmaf(gv[j], vec_get(v[u], j), a);
                    dbuf[(k + u) * kRow + lane] = a;
                }
            }
            if (k < n) {  // four entries left
                const int4 i0 = *reinterpret_cast<const int4*>(ir + kg + k);
                const int ii[4] = {i0.x, i0.y, i0.z, i0.w};
                V v[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) v[u] = load_lane_vec<BPL>(xg, static_cast<size_t>(ii[u]) * ldv + lane);
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    float a = 0.f;
#pragma unroll
                    for (int j = 0; j < BPL; ++j) a = fmaf(gv[j], vec_get(v[u], j), a);
                    dbuf[(k + u) * kRow + lane] = a;
                }
            }
            __syncwarp();
            if (lane < n) {
                // entry `lane` of the group: its 32 partials, added in a fixed order
                float t[8];
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const float4 q = drow[c];
                    t[c] = (q.x + q.y) + (q.z + q.w);
                }
                const float sum = ((t[0] + t[1]) + (t[2] + t[3])) + ((t[4] + t[5]) + (t[6] + t[7]));
                if (p.gW) {
                    float* dst = p.gW + static_cast<size_t>(o) * K + kg + lane;
                    if (p.accumulate) *dst += sum;
                    else *dst = sum;
                }
            }
            __syncwarp();
        }
    }
    __pipeline_wait_prior(0);
}

template <int BPL, typename TX>
int launch_gather_t(GatherParams p, int nBT, const DeviceInfo& dev, cudaStream_t stream) {
    auto kern = ffi_grad_w_gather_kernel<BPL, TX>;
    const size_t smem = static_cast<size_t>(kWarps) * (32 * kRow + 2 * p.K) * 4;
    FFI_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    int occ = 0;
    FFI_CUDA_CHECK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, kThreads, smem));
    if (occ < 1) return fail(FFI_ERR_CUDA, "grad_W gather kernel does not fit on an SM (smem %zu)", smem);
    const long long want = ceil_div(p.L, kWarps);
    const long long cap = static_cast<long long>(dev.sm_count) * occ;
    const unsigned grid = static_cast<unsigned>(want < cap ? want : cap);
    // Batch tiles run as consecutive launches so that tile t adds to what tile t-1 wrote.
    for (int bt = 0; bt < nBT; ++bt) {
        p.b0 = bt * 32 * BPL;
        p.accumulate = bt > 0;
        kern<<<grid, kThreads, smem, stream>>>(p);
        FFI_LAUNCH_CHECK("ffi_grad_w_gather_kernel");
    }
    return FFI_OK;
}

}  // namespace

// Takes the shapes the tiled kernel would gather from L2 for (x too wide for shared memory) when the transposed
// gradient is at hand, K is a multiple of 4 and the rows are aligned; *handled tells the caller.
int launch_grad_w_gather(const GradWArgs& a, int bpl, cudaStream_t stream, bool* handled) {
    *handled = false;
    DeviceInfo dev;
    int rc = get_device_info(&dev);
    if (rc != FFI_OK) return rc;
    // bf16 x: eight batch elements per lane (one 16-byte gather covers 256 batch columns per warp) where the
    // batch is that wide and the rows are padded to it
    if (a.bf16 && bpl == 4 && a.B > 128 && a.ldx % 256 == 0 && a.ldg % 256 == 0) bpl = 8;
    const int BT = 32 * bpl;
    const int nBT = static_cast<int>(ceil_div(a.B, BT));
    if (!a.gT || a.K % 4 != 0 || reinterpret_cast<uintptr_t>(a.idx) % 16 != 0 || a.ldg % 4 != 0 ||
        a.ldg < static_cast<int64_t>(nBT) * BT || reinterpret_cast<uintptr_t>(a.gT) % 16 != 0 || a.ldx % BT != 0 ||
        a.ldx < static_cast<int64_t>(nBT) * BT || reinterpret_cast<uintptr_t>(a.xT) % 16 != 0)
        return FFI_OK;
    const size_t smem = static_cast<size_t>(kWarps) * (32 * kRow + 2 * a.K) * 4;
    if (smem > static_cast<size_t>(dev.max_smem_optin)) return FFI_OK;
    GatherParams p;
    p.xT = a.xT;
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
    *handled = true;
    if (a.bf16) {
        if (bpl == 8) return launch_gather_t<8, __nv_bfloat16>(p, nBT, dev, stream);
        if (bpl == 4) return launch_gather_t<4, __nv_bfloat16>(p, nBT, dev, stream);
        if (bpl == 2) return launch_gather_t<2, __nv_bfloat16>(p, nBT, dev, stream);
        return launch_gather_t<1, __nv_bfloat16>(p, nBT, dev, stream);
    }
    if (bpl == 4) return launch_gather_t<4, float>(p, nBT, dev, stream);
    if (bpl == 2) return launch_gather_t<2, float>(p, nBT, dev, stream);
    return launch_gather_t<1, float>(p, nBT, dev, stream);
}

}  // namespace ffi
