// grad_x of the fixed-fan-in sparse layer on sm_100a, deterministic and atomic-free:
//   grad_x[b,i] = sum over (o,k) with idx[o,k]==i of W[o,k] * g[b,o]
//
// Replaces the reference's atomicAdd kernels backward_features_vector(_tp) / _scalar(_tp)
// and the memset before them (tfsparse/cc/kernels/backward.cu.h:107-185,
// backward.cu:96,121).  Both paths walk the transposed index of ffi_plan.
//
// Narrow inputs (N <= 2048): register-accumulator kernel.  The outputs are cut into the
// plan's chunks of T rows.  A CTA owns a contiguous range of chunks, a slice of 16*NI
// inputs and a tile of BT = 32*BPL batch elements; warp w owns NI inputs and keeps their
// NI x BPL partial sums in registers for the whole range.  Per chunk the CTA
//   1. copies g[b-tile, chunk] into shared memory transposed (g_s[o][b], 16-byte
//      granules XOR-swizzled by o so that both the 4-byte cp.async fill and the
//      per-entry vector gather are bank-conflict free),
//   2. stages its slice of the chunk's sorted entries as (W[p], row) pairs,
//   3. lets every warp walk the runs of its inputs: one broadcast LDS per two entries,
//      one gathered LDS.32/64/128 and BPL FMAs per entry.
// Range partials go to a workspace and a second kernel adds them in range order, so the
// summation order is a pure function of (idx, shape): results are bit-reproducible.
//
// Wide inputs: g is transposed once into gT[L][Bpad] (workspace) and one warp per
// (input, batch tile) walks the canonical row, gathering 128 contiguous batch values
// per entry.
#include <mutex>

#include "ffi_common.cuh"

namespace ffi {
namespace {

constexpr int kThreads = 512;
constexpr int kWarps = kThreads / 32;

template <int BPL>
__device__ __forceinline__ void store_vec(float* dst, const float (&v)[BPL]) {
    if constexpr (BPL == 4) *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
    else if constexpr (BPL == 2) *reinterpret_cast<float2*>(dst) = make_float2(v[0], v[1]);
    else *dst = v[0];
}

struct GxNarrowParams {
    const float* W;
    const float* gT;  // upstream gradient transposed to [L][ldg], zero padded batch
    long long ldg;
    const int* cperm;
    const int* cptr;
    float* partial;  // [R * S][N][Bpad]
    int B, N, L, K;
    int T;           // rows per chunk
    long long nChunks;
    int R;           // number of chunk ranges (gridDim.x)
    int Bpad;
    int entCap;      // capacity of the staged entry buffer (entries)
    int segChunks;   // chunks per flushed partial: the running fp32 sums restart after that many chunks
    int S;           // partial slots per range
};

template <int NI, int BPL>
__global__ void __launch_bounds__(kThreads, 1) ffi_grad_x_narrow_kernel(GxNarrowParams p) {
    constexpr int BT = 32 * BPL;
    constexpr int GR = BPL;  // floats per granule
    constexpr int SW = 32 / GR - 1;  // swizzle mask: rows copied by one warp get distinct granules
    using V = typename Vec<BPL>::type;
    extern __shared__ __align__(16) unsigned char smem_raw[];

    float* g_s = reinterpret_cast<float*>(smem_raw);                        // [T][BT], swizzled granules
    uint2* ent_s = reinterpret_cast<uint2*>(g_s + static_cast<size_t>(p.T) * BT);  // (W bits, row)
    int* cp_s = reinterpret_cast<int*>(ent_s + p.entCap);                   // [16*NI + 1]

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int r = blockIdx.x;
    const int i_lo = blockIdx.y * (kWarps * NI);
    const int i_hi = min(p.N, i_lo + kWarps * NI);
    const int b0 = blockIdx.z * BT;
    const int T = p.T, K = p.K, L = p.L, N = p.N;
    const long long c_begin = p.nChunks * r / p.R;
    const long long c_end = p.nChunks * (r + 1) / p.R;

    float acc[NI][BPL];
#pragma unroll
    for (int j = 0; j < NI; ++j)
#pragma unroll
        for (int q = 0; q < BPL; ++q) acc[j][q] = 0.f;

    for (long long c = c_begin; c < c_end; ++c) {
        const long long o0 = c * T;
        const int nrows = static_cast<int>(min(static_cast<long long>(T), static_cast<long long>(L) - o0));
        __syncthreads();  // the previous chunk's g_s / ent_s / cp_s are no longer read

        // (1) g tile.  Work item u = (row group of 8, granule, slot, row in group): a warp
        // covers 8 consecutive rows x BPL slots of one granule -> 32 distinct banks.
        // Item u = (granule gl, row ol): BPL coalesced 4-byte loads (lanes run along o), one
        // vector store of the granule.  Four items are in flight per thread.
        // The tile comes from the transposed gradient gT[L][ldg]: row ol is BT contiguous floats,
        // copied granule by granule (one 4/8/16-byte cp.async per lane, a warp covers one row).
        {
            const int totalItems = T * 32;
            for (int u = tid; u < totalItems; u += kThreads) {
                const int ol = u >> 5, gl = u & 31;
                float* dst = g_s + static_cast<size_t>(ol) * BT + ((gl ^ (ol & SW)) * GR);
                if (ol < nrows) {
                    __pipeline_memcpy_async(dst, p.gT + static_cast<size_t>(o0 + ol) * p.ldg + b0 + gl * GR, 4 * GR);
                } else {
                    const float zero[BPL] = {};
                    store_vec<BPL>(dst, zero);
                }
            }
            __pipeline_commit();
        }

        // (2) run offsets of my input slice and the staged entries.
        const int* cptr_c = p.cptr + c * (N + 1);
        const int e_lo = __ldg(cptr_c + i_lo);
        const int e_hi = __ldg(cptr_c + i_hi);
        for (int t = tid; t <= kWarps * NI; t += kThreads) {
            const int i = min(i_lo + t, i_hi);
            cp_s[t] = __ldg(cptr_c + i) - e_lo;
        }
        const int* cperm_c = p.cperm + c * static_cast<long long>(T) * K;
        for (int ebase = 0; ebase < e_hi - e_lo; ebase += p.entCap) {
            // The slice normally fits entCap at once; an adversarial idx (everything in
            // one slice) is handled in several rounds.
            const int cnt = min(p.entCap, e_hi - e_lo - ebase);
            if (ebase > 0) __syncthreads();
            for (int e = tid; e < cnt; e += kThreads) {
                const int pos = __ldg(cperm_c + e_lo + ebase + e);
                const int ol = pos / K - static_cast<int>(o0);
                ent_s[e] = make_uint2(__float_as_uint(__ldg(p.W + pos)), static_cast<unsigned>(ol));
            }
            __pipeline_wait_prior(0);
            __syncthreads();

            // (3) walk the runs.
            const V* gs_v = reinterpret_cast<const V*>(g_s);
#pragma unroll
            for (int j = 0; j < NI; ++j) {
                int s = cp_s[warp * NI + j] - ebase;
                int t = cp_s[warp * NI + j + 1] - ebase;
                s = max(s, 0);
                t = min(t, cnt);
                int e = s;
                if ((e & 1) && e < t) {
                    const uint2 en = ent_s[e];
                    const int ol = static_cast<int>(en.y);
                    const V v = gs_v[ol * 32 + (lane ^ (ol & SW))];
                    const float w = __uint_as_float(en.x);
#pragma unroll
                    for (int q = 0; q < BPL; ++q) acc[j][q] = fmaf(w, vec_get(v, q), acc[j][q]);
                    ++e;
                }
                for (; e + 2 <= t; e += 2) {
                    const uint4 en = *reinterpret_cast<const uint4*>(ent_s + e);
                    const int ol0 = static_cast<int>(en.y), ol1 = static_cast<int>(en.w);
                    const V v0 = gs_v[ol0 * 32 + (lane ^ (ol0 & SW))];
                    const V v1 = gs_v[ol1 * 32 + (lane ^ (ol1 & SW))];
                    const float w0 = __uint_as_float(en.x), w1 = __uint_as_float(en.z);
#pragma unroll
                    for (int q = 0; q < BPL; ++q) {
                        acc[j][q] = fmaf(w0, vec_get(v0, q), acc[j][q]);
                        acc[j][q] = fmaf(w1, vec_get(v1, q), acc[j][q]);
                    }
                }
                if (e < t) {
                    const uint2 en = ent_s[e];
                    const int ol = static_cast<int>(en.y);
                    const V v = gs_v[ol * 32 + (lane ^ (ol & SW))];
                    const float w = __uint_as_float(en.x);
#pragma unroll
                    for (int q = 0; q < BPL; ++q) acc[j][q] = fmaf(w, vec_get(v, q), acc[j][q]);
                }
            }
        }
        if (e_hi == e_lo) {
            __pipeline_wait_prior(0);
        }
        // Every segChunks chunks the running sums go out as one partial (partial[r*S + seg][i][b]) and
        // restart from zero, so that no fp32 sum runs over more than a few hundred products; the
        // partials are added in fp64 afterwards.
        const long long done = c - c_begin + 1;
        if (done % p.segChunks == 0 || c + 1 == c_end) {
            const int seg = static_cast<int>((done - 1) / p.segChunks);
#pragma unroll
            for (int j = 0; j < NI; ++j) {
                const int i = i_lo + warp * NI + j;
                if (i < N) {
                    float* dst = p.partial + ((static_cast<size_t>(r) * p.S + seg) * N + i) * p.Bpad + b0 + lane * BPL;
#pragma unroll
                    for (int q = 0; q < BPL; ++q) {
                        dst[q] = acc[j][q];
                        acc[j][q] = 0.f;
                    }
                }
            }
        }
    }
    __pipeline_wait_prior(0);

    // Segments a range never reached hold zeros (ranges differ by at most one chunk).
    for (int seg = static_cast<int>((c_end - c_begin + p.segChunks - 1) / p.segChunks); seg < p.S; ++seg) {
#pragma unroll
        for (int j = 0; j < NI; ++j) {
            const int i = i_lo + warp * NI + j;
            if (i < N) {
                float* dst = p.partial + ((static_cast<size_t>(r) * p.S + seg) * N + i) * p.Bpad + b0 + lane * BPL;
#pragma unroll
                for (int q = 0; q < BPL; ++q) dst[q] = 0.f;
            }
        }
    }
}

// gx = sum over ranges of partial[r][i][b], in range order; writes [B,N] or [N,B].
__global__ void reduce_partials_kernel(const float* __restrict__ partial, float* __restrict__ gx,
                                       int R, int N, int B, int Bpad, int x_transposed) {
    const long long id = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (id >= static_cast<long long>(N) * Bpad) return;
    const int i = static_cast<int>(id / Bpad);
    const int b = static_cast<int>(id - static_cast<long long>(i) * Bpad);
    if (b >= B) return;
    double acc = 0.0;  // the range partials are large next to a small total: add them in fp64
    for (int r = 0; r < R; ++r) acc += static_cast<double>(partial[(static_cast<size_t>(r) * N + i) * Bpad + b]);
    const float s = static_cast<float>(acc);
    if (x_transposed) gx[static_cast<size_t>(i) * B + b] = s;
    else gx[static_cast<size_t>(b) * N + i] = s;
}

// ---- wide inputs -------------------------------------------------------------------

// One warp per (input i, batch tile of 32*VEC): walks row i of the canonical index and gathers
// one row of the transposed gradient gT[L][ldg] per entry.
template <int VEC, typename TW>
__global__ void __launch_bounds__(256) ffi_grad_x_wide_kernel(const TW* __restrict__ W,
                                                              const float* __restrict__ gT,
                                                              const int* __restrict__ rowptr,
                                                              const int* __restrict__ perm,
                                                              float* __restrict__ gx, int B, int N,
                                                              int K, long long ldg, int x_transposed) {
    using V = typename Vec<VEC>::type;
    constexpr int BTW = 32 * VEC;
    const int lane = threadIdx.x & 31;
    const long long wid = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int nBT = static_cast<int>(ldg / BTW);
    if (wid >= static_cast<long long>(N) * nBT) return;
    const int i = static_cast<int>(wid / nBT);
    const int bt = static_cast<int>(wid - static_cast<long long>(i) * nBT);
    const V* gTv = reinterpret_cast<const V*>(gT + bt * BTW) + lane;
    const size_t ldv = static_cast<size_t>(ldg / VEC);
    float acc[VEC];
#pragma unroll
    for (int q = 0; q < VEC; ++q) acc[q] = 0.f;
    const int s = rowptr[i], t = rowptr[i + 1];
    for (int base = s; base < t; base += 32) {
        const int e = base + lane;
        int o = 0;
        float w = 0.f;
        if (e < t) {
            const int pos = __ldg(perm + e);
            o = pos / K;
            w = widen(W[pos]);
        }
        const int cnt = min(32, t - base);
        for (int u = 0; u < cnt; ++u) {
            const int ou = __shfl_sync(0xffffffffu, o, u);
            const float wu = __shfl_sync(0xffffffffu, w, u);
            const V v = __ldg(gTv + static_cast<size_t>(ou) * ldv);
#pragma unroll
            for (int q = 0; q < VEC; ++q) acc[q] = fmaf(wu, vec_get(v, q), acc[q]);
        }
    }
    const int b = bt * BTW + lane * VEC;
#pragma unroll
    for (int q = 0; q < VEC; ++q) {
        if (b + q < B) {
            if (x_transposed) gx[static_cast<size_t>(i) * B + b + q] = acc[q];
            else gx[static_cast<size_t>(b + q) * N + i] = acc[q];
        }
    }
}

template <int NI, int BPL>
int launch_narrow_t(const GxNarrowParams& p, size_t smem, int iparts, int nBT, cudaStream_t stream) {
    auto kern = ffi_grad_x_narrow_kernel<NI, BPL>;
    FFI_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        static_cast<int>(smem)));
    dim3 grid(static_cast<unsigned>(p.R), static_cast<unsigned>(iparts), static_cast<unsigned>(nBT));
    kern<<<grid, kThreads, smem, stream>>>(p);
    FFI_LAUNCH_CHECK("ffi_grad_x_narrow_kernel");
    return FFI_OK;
}

struct NarrowConfig {
    int bpl, ni, iparts, nBT, Bpad, R, entCap, segChunks, S;
    size_t smem;
};

// max_partial_bytes bounds the scratch for the range partials (R * S slots of N * Bpad floats): the segments
// get longer when the scratch is small (S = 1: one partial per range).
bool narrow_config(const ffi_plan* plan, int64_t B, const DeviceInfo& dev, NarrowConfig* c,
                   size_t max_partial_bytes = static_cast<size_t>(256) << 20) {
    if (!plan->has_chunks) return false;
    c->bpl = B <= 32 ? 1 : (B <= 64 ? 2 : 4);
    c->ni = 64 / c->bpl;  // 64 accumulator registers per lane
    const int BT = 32 * c->bpl;
    c->iparts = static_cast<int>(ceil_div(plan->N, kWarps * c->ni));
    c->nBT = static_cast<int>(ceil_div(B, BT));
    c->Bpad = c->nBT * BT;
    int R = dev.sm_count / (c->iparts * c->nBT);
    if (R < 1) R = 1;
    if (R > plan->n_chunks) R = static_cast<int>(plan->n_chunks);
    c->R = R;
    const size_t gbytes = static_cast<size_t>(plan->chunk_rows) * BT * 4;
    const size_t cpbytes = (kWarps * c->ni + 1) * 4 + 16;
    if (gbytes + cpbytes + 1024 > static_cast<size_t>(dev.max_smem_optin)) return false;
    size_t cap = (dev.max_smem_optin - gbytes - cpbytes) / 8;
    const size_t full = static_cast<size_t>(plan->chunk_rows) * plan->K;
    if (cap > full) cap = full;
    cap = cap / 2 * 2;
    if (cap < 64) return false;
    c->entCap = static_cast<int>(cap);
    c->smem = gbytes + cap * 8 + cpbytes;
    // flush after about 256 summands per (input, batch) pair, as far as the scratch allows
    const double per_chunk = static_cast<double>(plan->chunk_rows) * plan->K / static_cast<double>(plan->N);
    long long seg = static_cast<long long>(256.0 / (per_chunk > 1.0 ? per_chunk : 1.0));
    if (seg < 1) seg = 1;
    const long long perRange = ceil_div(plan->n_chunks, R);
    const size_t slot = static_cast<size_t>(plan->N) * c->Bpad * 4;
    long long maxS = static_cast<long long>(max_partial_bytes / (slot * R));
    if (maxS < 1) maxS = 1;
    long long S = ceil_div(perRange, seg);
    if (S > maxS) {
        S = maxS;
        seg = ceil_div(perRange, S);
        S = ceil_div(perRange, seg);
    }
    c->segChunks = static_cast<int>(seg);
    c->S = static_cast<int>(S);
    return true;
}

// g [B][L] -> gT [L][ldg] (zero padded batch), optionally with grad_bias[o] = sum_b g[b,o].
// One block owns `tro` <= 64 outputs and walks the whole batch in slabs of 128, so the column sums are
// complete inside the block and are added in a fixed order.  Rows of g start at arbitrary 4-byte
// offsets (L is odd in practice), so a 256-byte row segment costs one extra 32-byte sector.
// The launcher picks `tro` so that the blocks fill a whole number of waves over the GPU: with 64 outputs
// per block a short L (a shard of the label dimension) leaves the last wave nearly empty.
constexpr int kTrO = 64;        // most outputs per block
constexpr int kTrResident = 4;  // blocks per SM (launch bound)
__global__ void __launch_bounds__(256, kTrResident) transpose_g_kernel(const float* __restrict__ g, float* __restrict__ gT,
                                                                    float* __restrict__ gbias, int B, long long L,
                                                                    long long ldg, int tro) {
    __shared__ float tile[128][kTrO + 1];
    const int tid = threadIdx.x;
    const int tx = tid & (kTrO - 1), ty = tid / kTrO;  // load: tx = output, ty = batch row within a group of 4
    const int bx = tid & 127, oy0 = tid >> 7;           // store: bx = batch column, oy0 = first output row
    const long long o0 = static_cast<long long>(blockIdx.x) * tro;
    const int nrows = static_cast<int>(L - o0 < tro ? L - o0 : tro);  // outputs of this block
    const bool ocol = tx < nrows;
    float colsum = 0.f;
    for (long long bb = 0; bb < ldg; bb += 128) {
        const float* src = g + static_cast<size_t>(bb + ty) * L + o0 + tx;
#pragma unroll 16
        for (int u = 0; u < 32; ++u) {
            const long long b = bb + ty + 4 * u;
            const float v = (ocol && b < B) ? __ldcs(src + static_cast<size_t>(4 * u) * L) : 0.f;
            tile[ty + 4 * u][tx] = v;
            colsum += v;
        }
        __syncthreads();
        if (bb + bx < ldg) {
            float* dst = gT + static_cast<size_t>(o0) * ldg + bb + bx;
#pragma unroll 8
            for (int oy = oy0; oy < nrows; oy += 2) dst[static_cast<size_t>(oy) * ldg] = tile[bx][oy];
        }
        __syncthreads();
    }
    if (gbias) {
        tile[ty][tx] = colsum;
        __syncthreads();
        if (ty == 0 && ocol) {
            float s = 0.f;
#pragma unroll
            for (int y = 0; y < 256 / kTrO; ++y) s += tile[y][tx];
            gbias[o0 + tx] = s;
        }
    }
}

}  // namespace

int64_t transposed_g_stride(int64_t B) { return B <= 32 ? 32 : (B <= 64 ? 64 : round_up(B, 128)); }

int launch_transpose_g(const float* g, float* gT, float* gbias, int B, int64_t L, int64_t ldg, cudaStream_t stream) {
    DeviceInfo dev;
    const int rc = get_device_info(&dev);
    if (rc != FFI_OK) return rc;
    // the fewest waves that blocks of kTrO outputs need, then the narrowest blocks that still fit those waves
    const long long slots = static_cast<long long>(dev.sm_count) * kTrResident;
    const long long waves = ceil_div(ceil_div(L, kTrO), slots);
    long long tro = ceil_div(L, slots * waves);
    tro = tro < 8 ? 8 : (tro > kTrO ? kTrO : tro);
    const long long blocks_o = ceil_div(L, tro);
    if (blocks_o > 2147483647LL) return fail(FFI_ERR_UNSUPPORTED, "L too large");
    transpose_g_kernel<<<static_cast<unsigned>(blocks_o), 256, 0, stream>>>(g, gT, gbias, B, L, ldg, static_cast<int>(tro));
    FFI_LAUNCH_CHECK("transpose_g_kernel");
    return FFI_OK;
}

bool grad_x_narrow_applicable(const ffi_plan* plan, int64_t B) {
    DeviceInfo dev;
    if (!plan || get_device_info(&dev) != FFI_OK) return false;
    NarrowConfig c;
    return narrow_config(plan, B, dev, &c);
}

// Scratch beyond gT: the range partials of the narrow kernel (the wide kernel needs none).
size_t grad_x_workspace_bytes(const ffi_plan* plan, int64_t B) {
    DeviceInfo dev;
    if (get_device_info(&dev) != FFI_OK) return 0;
    NarrowConfig c;
    if (narrow_config(plan, B, dev, &c)) return static_cast<size_t>(c.R) * c.S * plan->N * c.Bpad * 4;
    return 0;
}

// The least scratch the narrow kernel can run with: one partial per range.
size_t grad_x_min_workspace_bytes(const ffi_plan* plan, int64_t B) {
    DeviceInfo dev;
    if (get_device_info(&dev) != FFI_OK) return 0;
    NarrowConfig c;
    if (narrow_config(plan, B, dev, &c, 1)) return static_cast<size_t>(c.R) * plan->N * c.Bpad * 4;
    return 0;
}

int launch_grad_x(const GradXArgs& a, cudaStream_t stream) {
    DeviceInfo dev;
    int rc = get_device_info(&dev);
    if (rc != FFI_OK) return rc;
    const ffi_plan* plan = a.plan;
    if (!a.gT || a.ldg < a.B || a.ldg % 32 != 0)
        return fail(FFI_ERR_INVALID_ARGUMENT, "grad_x needs the transposed upstream gradient");

    NarrowConfig c;
    if (a.w_bf16 && plan->has_chunks)
        return fail(FFI_ERR_UNSUPPORTED, "the narrow-input grad_x kernel reads fp32 weights");
    // a caller with little scratch (the allocation-free entry point) gets longer segments
    if (narrow_config(plan, a.B, dev, &c, a.workspace_bytes < (static_cast<size_t>(256) << 20) ? a.workspace_bytes
                                                                                                : (static_cast<size_t>(256) << 20))) {
        const size_t need = static_cast<size_t>(c.R) * c.S * plan->N * c.Bpad * 4;
        if (!a.workspace || a.workspace_bytes < need)
            return fail(FFI_ERR_WORKSPACE, "grad_x needs %zu bytes of workspace, got %zu", need, a.workspace_bytes);
        if (reinterpret_cast<uintptr_t>(a.workspace) % 16 != 0)
            return fail(FFI_ERR_WORKSPACE, "workspace must be 16-byte aligned");
        if (a.ldg < c.Bpad) return fail(FFI_ERR_INVALID_ARGUMENT, "transposed gradient stride too small");
        GxNarrowParams p;
        p.W = static_cast<const float*>(a.W);
        p.gT = a.gT;
        p.ldg = a.ldg;
        p.cperm = plan->cperm;
        p.cptr = plan->cptr;
        p.partial = static_cast<float*>(a.workspace);
        p.B = a.B;
        p.N = a.N;
        p.L = a.L;
        p.K = a.K;
        p.T = plan->chunk_rows;
        p.nChunks = plan->n_chunks;
        p.R = c.R;
        p.Bpad = c.Bpad;
        p.entCap = c.entCap;
        p.segChunks = c.segChunks;
        p.S = c.S;
        if (c.bpl == 4) rc = launch_narrow_t<16, 4>(p, c.smem, c.iparts, c.nBT, stream);
        else if (c.bpl == 2) rc = launch_narrow_t<32, 2>(p, c.smem, c.iparts, c.nBT, stream);
        else rc = launch_narrow_t<64, 1>(p, c.smem, c.iparts, c.nBT, stream);
        if (rc != FFI_OK) return rc;
        const long long total = static_cast<long long>(a.N) * c.Bpad;
        reduce_partials_kernel<<<static_cast<unsigned>(ceil_div(total, 256)), 256, 0, stream>>>(
            p.partial, a.gx, c.R * c.S, a.N, a.B, c.Bpad, a.x_transposed);
        FFI_LAUNCH_CHECK("reduce_partials_kernel");
        return FFI_OK;
    }

    // Wide inputs: one warp per (input, batch tile) over the canonical index.
    const int vec = a.ldg % 128 == 0 ? 4 : (a.ldg % 64 == 0 ? 2 : 1);
    const long long warps = static_cast<long long>(a.N) * (a.ldg / (32 * vec));
    const unsigned blocks = static_cast<unsigned>(ceil_div(warps, 8));
    auto launch_wide = [&](auto w_typed) {
        if (vec == 4)
            ffi_grad_x_wide_kernel<4><<<blocks, 256, 0, stream>>>(w_typed, a.gT, plan->rowptr, plan->perm, a.gx, a.B, a.N,
                                                                  a.K, a.ldg, a.x_transposed);
        else if (vec == 2)
            ffi_grad_x_wide_kernel<2><<<blocks, 256, 0, stream>>>(w_typed, a.gT, plan->rowptr, plan->perm, a.gx, a.B, a.N,
                                                                  a.K, a.ldg, a.x_transposed);
        else
            ffi_grad_x_wide_kernel<1><<<blocks, 256, 0, stream>>>(w_typed, a.gT, plan->rowptr, plan->perm, a.gx, a.B, a.N,
                                                                  a.K, a.ldg, a.x_transposed);
    };
    if (a.w_bf16) launch_wide(static_cast<const __nv_bfloat16*>(a.W));
    else launch_wide(static_cast<const float*>(a.W));
    FFI_LAUNCH_CHECK("ffi_grad_x_wide_kernel");
    return FFI_OK;
}

}  // namespace ffi

// ---- allocation-free entry point ------------------------------------------------------
//
// Some hosts of this library may not allocate device memory at the point where they call
// it: a TensorFlow or PyTorch op kernel is expected to take scratch from the framework's own
// allocator (which has usually reserved almost all of the GPU, so a raw cudaMalloc can fail
// or force a device-wide synchronisation), and a serving loop that has already started
// steady-state execution cannot afford cudaMalloc's implicit synchronisation either.  For
// those callers ffi_grad_x_static runs the narrow-input grad_x kernel with its range partials
// in a fixed array that lives in the library image instead of in a caller workspace.
namespace ffi {
namespace {

constexpr size_t kStaticScratchBytes = static_cast<size_t>(20) << 20;  // 20 MiB per GPU that loads the library
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// In host code `g_static_scratch` is only a handle of the symbol, not a device address: the
// address each device gave the array is looked up once per device, with that device current.
int static_scratch_address(void** out) {
    static std::mutex mu;
    static void* addr[64] = {};
    int dev = 0;
    FFI_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(FFI_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lock(mu);
    if (!addr[dev]) {
        void* ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
        if (e != cudaSuccess || !ptr)
            return fail(FFI_ERR_CUDA, "cudaGetSymbolAddress(static scratch) failed: %s", cudaGetErrorString(e));
        addr[dev] = ptr;
    }
    *out = addr[dev];
    return FFI_OK;
}

}  // namespace
}  // namespace ffi

extern "C" size_t ffi_grad_x_static_max_scratch_bytes(void) { return ffi::kStaticScratchBytes; }

extern "C" int ffi_grad_x_static(const float* W, const float* gT, int64_t ldg, const ffi_plan* plan, float* grad_x,
                                 int64_t B, int64_t N, int64_t L, int64_t K, int x_transposed, void* stream_v) {
    FFI_TRACE("ffi_grad_x_static");
    using namespace ffi;
    if (!W || !gT || !plan || !grad_x) return fail(FFI_ERR_INVALID_ARGUMENT, "NULL argument to ffi_grad_x_static");
    if (B <= 0 || N <= 0 || L <= 0 || K <= 0 || B >= (1LL << 31))
        return fail(FFI_ERR_INVALID_ARGUMENT, "B, N, L, K must be positive");
    if (plan->L != L || plan->K != K || plan->N != N)
        return fail(FFI_ERR_STALE_PLAN, "plan was built for (L,K,N)=(%lld,%lld,%lld), call has (%lld,%lld,%lld)",
                    (long long)plan->L, (long long)plan->K, (long long)plan->N, (long long)L, (long long)K,
                    (long long)N);
    int rc = check_plan_device(plan);
    if (rc != FFI_OK) return rc;
    if (ldg < transposed_g_stride(B) || ldg % 32 != 0 || reinterpret_cast<uintptr_t>(gT) % 16 != 0)
        return fail(FFI_ERR_INVALID_ARGUMENT,
                    "gT must be 16-byte aligned with a row stride that is a multiple of 32 and >= "
                    "ffi_transposed_gradient_stride(B) = %lld", (long long)transposed_g_stride(B));
    const size_t need = grad_x_min_workspace_bytes(plan, B);
    if (need > kStaticScratchBytes)
        return fail(FFI_ERR_WORKSPACE,
                    "ffi_grad_x_static: this shape needs %zu bytes of scratch, the built-in array holds %zu; "
                    "use ffi_backward with a caller workspace",
                    need, kStaticScratchBytes);
    void* scratch = nullptr;
    rc = static_scratch_address(&scratch);
    if (rc != FFI_OK) return rc;
    GradXArgs a;
    a.idx = nullptr;
    a.W = W;
    a.w_bf16 = false;
    a.g = nullptr;
    a.gT = gT;
    a.ldg = ldg;
    a.plan = plan;
    a.gx = grad_x;
    a.x_transposed = x_transposed;
    a.B = static_cast<int>(B);
    a.N = static_cast<int>(N);
    a.L = static_cast<int>(L);
    a.K = static_cast<int>(K);
    a.workspace = scratch;
    a.workspace_bytes = kStaticScratchBytes;
    return launch_grad_x(a, static_cast<cudaStream_t>(stream_v));
}

namespace ffi {
// Shared with the fused backward kernel: grad_x = sum over ranges of partial[r][i][b], range order.
int reduce_range_partials(const float* partial, float* gx, int R, int N, int B, int Bpad, int x_transposed,
                          cudaStream_t stream) {
    const long long total = static_cast<long long>(N) * Bpad;
    reduce_partials_kernel<<<static_cast<unsigned>(ceil_div(total, 256)), 256, 0, stream>>>(partial, gx, R, N, B, Bpad,
                                                                                           x_transposed);
    FFI_LAUNCH_CHECK("reduce_partials_kernel");
    return FFI_OK;
}
}  // namespace ffi
