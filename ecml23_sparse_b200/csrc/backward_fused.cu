// grad_x and grad_W of the fixed-fan-in sparse layer in ONE pass over the transposed index
// (narrow inputs, batch <= 128):
//   grad_x[b,i] = sum over entries (o,k) with idx[o,k]==i of W[o,k] * g[b,o]
//   grad_W[o,k] = sum_b g[b,o] * x[b, idx[o,k]]
//
// Replaces, for that case, both halves of the reference's grad functor
// (tfsparse/cc/kernels/backward.cu:112-133: feature_grad_launch_vector_tp + the
// weight_grad launch).  Walking the entries grouped by input i means x[:, i] is the same for a
// whole run of entries, so it sits in registers and grad_W needs NO gather of its own: the
// g[:, o] vector gathered for grad_x is multiplied by x[:, i] and reduced over the lanes.  This
// removes the B*L*K shared-memory gathers of a separate grad_W pass.
//
// Structure (per CTA = range of chunks x slice of 16*NI inputs; warp = NI inputs):
//   * grad_x accumulators and x[:, i] of the warp's inputs live in registers (NI x BPL each);
//     the loop over inputs is not unrolled, a switch moves the current run's registers in/out;
//   * per chunk: the g tile comes from gT by cp.async into XOR-swizzled granules while the NEXT
//     chunk's entries are staged as (W, row | k << 16) pairs (double buffer) together with a
//     per-row bit mask of the (row, k) positions this slice owns;
//   * per entry: one broadcast LDS.64 (entry), one gathered LDS.128 (g), 2*BPL FMA, one STS of the
//     lane's partial grad_W dot into a per-warp 16 x 32 buffer; every 16 entries two lanes per
//     entry add the buffer rows (fixed order) and drop the sums into a shared image of the chunk's
//     grad_W window;
//   * after the chunk the CTA stores its positions of the window with coalesced masked row stores.
// grad_x partials are flushed every few chunks and added in fp64 in a fixed order.
// No atomics on floating-point data: results are bit-reproducible.
#include "ffi_common.cuh"

namespace ffi {
namespace {

constexpr int kThreads = 512;
constexpr int kWarps = kThreads / 32;
constexpr int kSlots = 16;            // entries buffered per warp before the lane reduction
constexpr int kDRow = 33;             // row stride of the per-warp dot buffer (conflict-free)
constexpr int kStageUnroll = 4;       // staged entries per thread kept in flight

template <int BPL>
__device__ __forceinline__ void store_zero_vec(float* dst) {
    if constexpr (BPL == 4) *reinterpret_cast<float4*>(dst) = make_float4(0.f, 0.f, 0.f, 0.f);
    else if constexpr (BPL == 2) *reinterpret_cast<float2*>(dst) = make_float2(0.f, 0.f);
    else *dst = 0.f;
}

struct BwdFusedParams {
    const float* W;
    const float* gT;
    long long ldg;
    const float* xT;
    long long ldx;
    const int* cperm;
    const int* cptr;
    float* partial;  // [R*S][N][Bpad]
    float* gW;
    int B, N, L, K;
    int T;
    long long nChunks;
    int R;
    int Bpad;
    int entCap;
    int segChunks;  // chunks per flushed partial
    int S;          // partial slots per range
};

template <int NI, int BPL>
__global__ void __launch_bounds__(kThreads, 1) ffi_bwd_fused_kernel(BwdFusedParams p) {
    constexpr int BT = 32 * BPL;
    constexpr int GR = BPL;
    constexpr int SW = 32 / GR - 1;
    constexpr int CPN = kWarps * NI + 1;
    using V = typename Vec<BPL>::type;
    extern __shared__ __align__(16) unsigned char smem_raw[];

    const int T = p.T, K = p.K, L = p.L, N = p.N;
    float* g_s = reinterpret_cast<float*>(smem_raw);                                    // [T][BT] swizzled
    uint2* ent_s = reinterpret_cast<uint2*>(g_s + static_cast<size_t>(T) * BT);         // [2][entCap]
    float* dbuf_s = reinterpret_cast<float*>(ent_s + 2 * p.entCap);                     // [warps][kSlots][kDRow]
    int* cp_s = reinterpret_cast<int*>(dbuf_s + kWarps * kSlots * kDRow);               // [2][CPN]

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int r = blockIdx.x;
    const int i_lo = blockIdx.y * (kWarps * NI);
    const int i_hi = min(N, i_lo + kWarps * NI);
    const long long c_begin = p.nChunks * r / p.R;
    const long long c_end = p.nChunks * (r + 1) / p.R;

    float acc[NI][BPL];
    float xr[NI][BPL];
#pragma unroll
    for (int j = 0; j < NI; ++j) {
        const int i = i_lo + warp * NI + j;
#pragma unroll
        for (int q = 0; q < BPL; ++q) {
            const int b = lane * BPL + q;
            acc[j][q] = 0.f;
            xr[j][q] = (i < N && b < p.B) ? __ldg(p.xT + static_cast<size_t>(i) * p.ldx + b) : 0.f;
        }
    }

    // First entry and entry count of the slice in a chunk (two words of the plan's offset table);
    // fetched one chunk ahead of the staging that needs them.
    auto slice_bounds = [&](long long c, int& e_lo, int& cnt) {
        const int* cptr_c = p.cptr + c * (N + 1);
        e_lo = __ldg(cptr_c + i_lo);
        cnt = __ldg(cptr_c + i_hi) - e_lo;
    };

    // Entries (W, row | k << 16) and run offsets of the slice in chunk c -> buffer buf.
    // (The plan guarantees that a slice never holds more than entCap entries.)
    auto stage = [&](long long c, int buf, int e_lo, int cnt) {
        const int* cptr_c = p.cptr + c * (N + 1);
        for (int t = tid; t < CPN; t += kThreads) cp_s[buf * CPN + t] = __ldg(cptr_c + min(i_lo + t, i_hi)) - e_lo;
        const int* cperm_c = p.cperm + c * static_cast<long long>(T) * K + e_lo;
        const int o0 = static_cast<int>(c * T);
        uint2* dst = ent_s + buf * p.entCap;
        for (int e0 = tid; e0 < cnt; e0 += kThreads * kStageUnroll) {
            int pos[kStageUnroll];
            float w[kStageUnroll];
#pragma unroll
            for (int u = 0; u < kStageUnroll; ++u) {
                const int e = e0 + u * kThreads;
                pos[u] = e < cnt ? __ldg(cperm_c + e) : -1;
            }
#pragma unroll
            for (int u = 0; u < kStageUnroll; ++u) w[u] = pos[u] >= 0 ? __ldg(p.W + pos[u]) : 0.f;
#pragma unroll
            for (int u = 0; u < kStageUnroll; ++u) {
                if (pos[u] >= 0) {
                    const int o = pos[u] / K;
                    const int k = pos[u] - o * K;
                    dst[e0 + u * kThreads] =
                        make_uint2(__float_as_uint(w[u]), static_cast<unsigned>((o - o0) | (k << 16)));
                }
            }
        }
    };

    int nb_lo = 0, nb_cnt = 0;  // bounds of the chunk to be staged next
    if (c_begin < c_end) {
        slice_bounds(c_begin, nb_lo, nb_cnt);
        stage(c_begin, 0, nb_lo, nb_cnt);
        if (c_begin + 1 < c_end) slice_bounds(c_begin + 1, nb_lo, nb_cnt);
    }
    float* dbuf = dbuf_s + warp * (kSlots * kDRow);
    const V* gs_v = reinterpret_cast<const V*>(g_s);

    for (long long c = c_begin; c < c_end; ++c) {
        const int buf = static_cast<int>(c - c_begin) & 1;
        const long long o0 = c * T;
        const int nrows = static_cast<int>(min(static_cast<long long>(T), static_cast<long long>(L) - o0));
        __syncthreads();  // previous chunk's walk is done; buffer `buf` is staged

        for (int u = tid; u < T * 32; u += kThreads) {
            const int ol = u >> 5, gl = u & 31;
            float* dst = g_s + static_cast<size_t>(ol) * BT + ((gl ^ (ol & SW)) * GR);
            if (ol < nrows) __pipeline_memcpy_async(dst, p.gT + static_cast<size_t>(o0 + ol) * p.ldg + gl * GR, 4 * GR);
            else store_zero_vec<BPL>(dst);
        }
        __pipeline_commit();
        if (c + 1 < c_end) {  // overlaps with the tile copy
            stage(c + 1, buf ^ 1, nb_lo, nb_cnt);
            if (c + 2 < c_end) slice_bounds(c + 2, nb_lo, nb_cnt);
        }
        __pipeline_wait_prior(0);
        __syncthreads();

        // ---- walk the runs of this warp's inputs -------------------------------------------
        const uint2* ent = ent_s + buf * p.entCap;
        const int* cp = cp_s + buf * CPN + warp * NI;
        int slot = 0;
        int eblk = cp[0];  // entry held by slot 0 of the dot buffer

        // Adds the buffered per-lane dots of `n` entries (two lanes per entry, fixed order) and stores
        // grad_W[o,k] of those entries.
        auto reduce_slots = [&](int n) {
            __syncwarp();
            const int sl = lane >> 1, h = lane & 1;
            const float* row = dbuf + sl * kDRow + h * 16;
            float sum = 0.f;
#pragma unroll
            for (int m = 0; m < 16; ++m) sum += row[m];
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            if (h == 0 && sl < n && p.gW) {
                const unsigned code = ent[eblk + sl].y;
                p.gW[(static_cast<size_t>(o0) + (code & 0xffffu)) * K + (code >> 16)] = sum;
            }
            __syncwarp();
        };

#pragma unroll
        for (int j = 0; j < NI; ++j) {
            const int t = cp[j + 1];
            int e = cp[j];
            // groups of four entries: all loads of a group are issued before its stores (the
            // compiler cannot move loads across the shared-memory stores by itself)
            for (; e + 4 <= t; e += 4) {
                if (slot + 4 > kSlots) {
                    reduce_slots(slot);
                    eblk = e;
                    slot = 0;
                }
                uint2 en[4];
                V v[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) en[u] = ent[e + u];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int ol = static_cast<int>(en[u].y & 0xffffu);
                    v[u] = gs_v[ol * 32 + (lane ^ (ol & SW))];
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const float w = __uint_as_float(en[u].x);
                    float d = 0.f;
#pragma unroll
                    for (int q = 0; q < BPL; ++q) {
                        acc[j][q] = fmaf(w, vec_get(v[u], q), acc[j][q]);
                        d = fmaf(vec_get(v[u], q), xr[j][q], d);
                    }
                    dbuf[(slot + u) * kDRow + lane] = d;
                }
                slot += 4;
            }
            for (; e < t; ++e) {
                if (slot == kSlots) {
                    reduce_slots(slot);
                    eblk = e;
                    slot = 0;
                }
                const uint2 en = ent[e];
                const int ol = static_cast<int>(en.y & 0xffffu);
                const V v = gs_v[ol * 32 + (lane ^ (ol & SW))];
                const float w = __uint_as_float(en.x);
                float d = 0.f;
#pragma unroll
                for (int q = 0; q < BPL; ++q) {
                    acc[j][q] = fmaf(w, vec_get(v, q), acc[j][q]);
                    d = fmaf(vec_get(v, q), xr[j][q], d);
                }
                dbuf[slot * kDRow + lane] = d;
                ++slot;
            }
        }
        if (slot > 0) reduce_slots(slot);

        // Every segChunks chunks the running grad_x sums go out as one partial and restart from zero.
        const long long done = c - c_begin + 1;
        if (done % p.segChunks == 0 || c + 1 == c_end) {
            const int seg = static_cast<int>((done - 1) / p.segChunks);
#pragma unroll
            for (int j = 0; j < NI; ++j) {
                const int i = i_lo + warp * NI + j;
                if (i < N) {
                    float* dst = p.partial + ((static_cast<size_t>(r) * p.S + seg) * N + i) * p.Bpad + lane * BPL;
#pragma unroll
                    for (int q = 0; q < BPL; ++q) {
                        dst[q] = acc[j][q];
                        acc[j][q] = 0.f;
                    }
                }
            }
        }
    }

    // Segments a range never reached hold zeros (ranges differ by at most one chunk).
    for (int seg = static_cast<int>((c_end - c_begin + p.segChunks - 1) / p.segChunks); seg < p.S; ++seg) {
#pragma unroll
        for (int j = 0; j < NI; ++j) {
            const int i = i_lo + warp * NI + j;
            if (i < N) {
                float* dst = p.partial + ((static_cast<size_t>(r) * p.S + seg) * N + i) * p.Bpad + lane * BPL;
#pragma unroll
                for (int q = 0; q < BPL; ++q) dst[q] = 0.f;
            }
        }
    }
}

struct FusedConfig {
    int bpl, ni, iparts, Bpad, R, entCap, segChunks, S;
    size_t smem;
};

bool fused_config(const ffi_plan* plan, int64_t B, const DeviceInfo& dev, FusedConfig* c) {
    if (!plan || !plan->has_chunks || B > 128) return false;
    if (static_cast<long long>(plan->chunk_rows) > 65535 || plan->K > 65535) return false;
    c->bpl = B <= 32 ? 1 : (B <= 64 ? 2 : 4);
    c->ni = 32 / c->bpl;  // 32 accumulator + 32 x registers per lane
    const int BT = 32 * c->bpl;
    const int width = kWarps * c->ni;  // inputs per slice: 128, 256 or 512
    c->iparts = static_cast<int>(ceil_div(plan->N, width));
    c->Bpad = BT;
    int R = dev.sm_count / c->iparts;
    if (R < 1) R = 1;
    if (R > plan->n_chunks) R = static_cast<int>(plan->n_chunks);
    c->R = R;
    // flush after about 256 summands per (input, batch) pair
    const double per_chunk = static_cast<double>(plan->chunk_rows) * plan->K / static_cast<double>(plan->N);
    int seg = static_cast<int>(256.0 / (per_chunk > 1.0 ? per_chunk : 1.0));
    if (seg < 1) seg = 1;
    c->segChunks = seg;
    c->S = static_cast<int>(ceil_div(ceil_div(plan->n_chunks, R), seg));
    const int stat = width == 128 ? 0 : (width == 256 ? 1 : 2);
    const size_t cap = static_cast<size_t>((plan->max_slice_entries[stat] + 7) / 8 * 8 + 8);
    const size_t T = static_cast<size_t>(plan->chunk_rows);
    const size_t total = T * BT * 4 + 2 * cap * 8 + static_cast<size_t>(kWarps) * kSlots * kDRow * 4 +
                         2 * (kWarps * c->ni + 1) * 4 + 16;
    if (total > static_cast<size_t>(dev.max_smem_optin)) return false;  // unusually dense slice or large K: separate kernels
    c->entCap = static_cast<int>(cap);
    c->smem = total;
    return true;
}

template <int NI, int BPL>
int launch_fused_t(const BwdFusedParams& p, const FusedConfig& c, cudaStream_t stream) {
    auto kern = ffi_bwd_fused_kernel<NI, BPL>;
    FFI_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(c.smem)));
    dim3 grid(static_cast<unsigned>(c.R), static_cast<unsigned>(c.iparts), 1);
    kern<<<grid, kThreads, c.smem, stream>>>(p);
    FFI_LAUNCH_CHECK("ffi_bwd_fused_kernel");
    return FFI_OK;
}

}  // namespace

bool backward_fused_applicable(const ffi_plan* plan, int64_t B) {
    DeviceInfo dev;
    if (get_device_info(&dev) != FFI_OK) return false;
    FusedConfig c;
    return fused_config(plan, B, dev, &c);
}

size_t backward_fused_workspace_bytes(const ffi_plan* plan, int64_t B) {
    DeviceInfo dev;
    if (get_device_info(&dev) != FFI_OK) return 0;
    FusedConfig c;
    if (!fused_config(plan, B, dev, &c)) return 0;
    return static_cast<size_t>(c.R) * c.S * plan->N * c.Bpad * 4;
}

int reduce_range_partials(const float* partial, float* gx, int R, int N, int B, int Bpad, int x_transposed,
                          cudaStream_t stream);

// grad_x (always) and grad_W (when gW != nullptr) in one kernel.  xT is x as [N][ldx].
int launch_backward_fused(const GradXArgs& a, const float* xT, int64_t ldx, float* gW, cudaStream_t stream) {
    DeviceInfo dev;
    int rc = get_device_info(&dev);
    if (rc != FFI_OK) return rc;
    FusedConfig c;
    if (!fused_config(a.plan, a.B, dev, &c)) return fail(FFI_ERR_UNSUPPORTED, "fused backward does not cover this shape");
    const size_t need = static_cast<size_t>(c.R) * c.S * a.N * c.Bpad * 4;
    if (!a.workspace || a.workspace_bytes < need || reinterpret_cast<uintptr_t>(a.workspace) % 16 != 0)
        return fail(FFI_ERR_WORKSPACE, "fused backward needs %zu bytes of 16-byte aligned workspace", need);
    if (!a.gT || a.ldg < c.Bpad || a.ldg % 32 != 0 || !xT)
        return fail(FFI_ERR_INVALID_ARGUMENT, "fused backward needs gT and xT");
    BwdFusedParams p;
    p.W = a.W;
    p.gT = a.gT;
    p.ldg = a.ldg;
    p.xT = xT;
    p.ldx = ldx;
    p.cperm = a.plan->cperm;
    p.cptr = a.plan->cptr;
    p.partial = static_cast<float*>(a.workspace);
    p.gW = gW;
    p.B = a.B;
    p.N = a.N;
    p.L = a.L;
    p.K = a.K;
    p.T = a.plan->chunk_rows;
    p.nChunks = a.plan->n_chunks;
    p.R = c.R;
    p.Bpad = c.Bpad;
    p.entCap = c.entCap;
    p.segChunks = c.segChunks;
    p.S = c.S;
    if (c.bpl == 4) rc = launch_fused_t<8, 4>(p, c, stream);
    else if (c.bpl == 2) rc = launch_fused_t<16, 2>(p, c, stream);
    else rc = launch_fused_t<32, 1>(p, c, stream);
    if (rc != FFI_OK) return rc;
    return reduce_range_partials(p.partial, a.gx, c.R * c.S, a.N, a.B, c.Bpad, a.x_transposed, stream);
}

}  // namespace ffi
