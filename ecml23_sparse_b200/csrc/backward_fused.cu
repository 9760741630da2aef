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
//   * grad_x accumulators and x[:, i] of the warp's inputs live in registers (NI x BPL each, as
//     packed fp32 pairs: the axpy and the dot use the two-wide fp32 FMA of sm_100);
//   * per chunk: the g tile comes from gT by cp.async into XOR-swizzled granules; the NEXT chunk's
//     entries are staged meanwhile (double buffer) as (W, code) pairs, code = byte offset of the
//     entry's g row with its swizzle key | k << 18, the weights gathered by 4-byte cp.async that
//     complete behind the walk;
//   * per entry: one broadcast LDS.64 (entry), one XOR for the lane's address, one gathered LDS.128
//     (g), the FMAs, one STS of the lane's partial grad_W dot into a per-warp 16 x 32 buffer; every
//     16 entries two lanes per entry add the buffer rows (fixed order) and store grad_W[o,k].
// grad_x partials are flushed every few chunks and added in fp64 in a fixed order.
// No atomics on floating-point data: results are bit-reproducible.
#include "ffi_common.cuh"

namespace ffi {
namespace {

constexpr int kThreads = 512;
constexpr int kWarps = kThreads / 32;
constexpr int kSlots = 16;            // entries buffered per warp before the lane reduction
constexpr int kDRow = 36;             // row stride of the per-warp dot buffer: 16-byte rows, conflict-free
constexpr int kStageUnroll = 4;       // staged entries per thread kept in flight
constexpr int kKShift = 18;           // entry code = byte offset of the g row (with its swizzle key) | k << 18

// ---- packed fp32 pairs: sm_100 issues two IEEE fp32 operations per lane and instruction -----------
using u64 = unsigned long long;
__device__ __forceinline__ u64 pack2(float lo, float hi) {
    u64 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(u64 v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ u64 fma2(u64 a, u64 b, u64 c) {
    u64 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ u64 mul2(u64 a, u64 b) {
    u64 d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

// The BPL batch elements one lane holds of a vector over the batch (a g row, x[:, i], a grad_x sum).
template <int BPL>
struct LaneVec;
template <>
struct LaneVec<4> {
    u64 a, b;
    __device__ __forceinline__ void zero() { a = b = 0ull; }
    __device__ __forceinline__ void set(const float* v) { a = pack2(v[0], v[1]), b = pack2(v[2], v[3]); }
    __device__ __forceinline__ void get(float* v) const { unpack2(a, v[0], v[1]), unpack2(b, v[2], v[3]); }
    __device__ __forceinline__ void load_shared(const unsigned char* ptr) {
        const ulonglong2 t = *reinterpret_cast<const ulonglong2*>(ptr);
        a = t.x, b = t.y;
    }
    // this += w * g
    __device__ __forceinline__ void axpy(float w, const LaneVec& g) {
        const u64 ww = pack2(w, w);
        a = fma2(ww, g.a, a), b = fma2(ww, g.b, b);
    }
    __device__ __forceinline__ float dot(const LaneVec& g) const {
        float lo, hi;
        unpack2(fma2(g.b, b, mul2(g.a, a)), lo, hi);
        return lo + hi;
    }
};
template <>
struct LaneVec<2> {
    u64 a;
    __device__ __forceinline__ void zero() { a = 0ull; }
    __device__ __forceinline__ void set(const float* v) { a = pack2(v[0], v[1]); }
    __device__ __forceinline__ void get(float* v) const { unpack2(a, v[0], v[1]); }
    __device__ __forceinline__ void load_shared(const unsigned char* ptr) { a = *reinterpret_cast<const u64*>(ptr); }
    __device__ __forceinline__ void axpy(float w, const LaneVec& g) { a = fma2(pack2(w, w), g.a, a); }
    __device__ __forceinline__ float dot(const LaneVec& g) const {
        float lo, hi;
        unpack2(mul2(g.a, a), lo, hi);
        return lo + hi;
    }
};
template <>
struct LaneVec<1> {
    float a;
    __device__ __forceinline__ void zero() { a = 0.f; }
    __device__ __forceinline__ void set(const float* v) { a = v[0]; }
    __device__ __forceinline__ void get(float* v) const { v[0] = a; }
    __device__ __forceinline__ void load_shared(const unsigned char* ptr) { a = *reinterpret_cast<const float*>(ptr); }
    __device__ __forceinline__ void axpy(float w, const LaneVec& g) { a = fmaf(w, g.a, a); }
    __device__ __forceinline__ float dot(const LaneVec& g) const { return g.a * a; }
};

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
    int kShift;  // log2(K) when K is a power of two, else -1
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
    constexpr unsigned kRowMask = (1u << kKShift) - 1u;
    using LV = LaneVec<BPL>;
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

    LV acc[NI], xr[NI];
#pragma unroll
    for (int j = 0; j < NI; ++j) {
        const int i = i_lo + warp * NI + j;
        float xv[BPL];
#pragma unroll
        for (int q = 0; q < BPL; ++q) {
            const int b = lane * BPL + q;
            xv[q] = (i < N && b < p.B) ? __ldg(p.xT + static_cast<size_t>(i) * p.ldx + b) : 0.f;
        }
        acc[j].zero();
        xr[j].set(xv);
    }

    // First entry and entry count of the slice in a chunk (two words of the plan's offset table);
    // fetched one chunk ahead of the staging that needs them.
    auto slice_bounds = [&](long long c, int& e_lo, int& cnt) {
        const int* cptr_c = p.cptr + c * (N + 1);
        e_lo = __ldg(cptr_c + i_lo);
        cnt = __ldg(cptr_c + i_hi) - e_lo;
    };

    // Entries (W, code) and run offsets of the slice in chunk c -> buffer buf.  The codes are stored
    // at once; the weights are gathered by 4-byte cp.async straight into the entries, so that their
    // latency runs behind whatever the caller does next (the caller commits and waits).
    // (The plan guarantees that a slice never holds more than entCap entries.)
    auto stage = [&](long long c, int buf, int e_lo, int cnt) {
        const int* cptr_c = p.cptr + c * (N + 1);
        for (int t = tid; t < CPN; t += kThreads) cp_s[buf * CPN + t] = __ldg(cptr_c + min(i_lo + t, i_hi)) - e_lo;
        const int* cperm_c = p.cperm + c * static_cast<long long>(T) * K + e_lo;
        const int pos0 = static_cast<int>(c * T) * K;  // flat position of the chunk's first row
        uint2* dst = ent_s + buf * p.entCap;
        for (int e0 = tid; e0 < cnt; e0 += kThreads * kStageUnroll) {
            int pos[kStageUnroll];
#pragma unroll
            for (int u = 0; u < kStageUnroll; ++u) {
                const int e = e0 + u * kThreads;
                pos[u] = e < cnt ? __ldg(cperm_c + e) : -1;
            }
#pragma unroll
            for (int u = 0; u < kStageUnroll; ++u) {
                if (pos[u] >= 0) {
                    uint2* d = dst + e0 + u * kThreads;
                    __pipeline_memcpy_async(&d->x, p.W + pos[u], 4);
                    const int rel = pos[u] - pos0;
                    const int ol = p.kShift >= 0 ? (rel >> p.kShift) : rel / K;
                    const int k = rel - ol * K;
                    d->y = static_cast<unsigned>(ol * (BT * 4) + (ol & SW) * (GR * 4)) |
                           (static_cast<unsigned>(k) << kKShift);
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
    __pipeline_commit();
    __pipeline_wait_prior(0);
    float* dbuf = dbuf_s + warp * (kSlots * kDRow);
    // address of this lane's granule of row `code & kRowMask`: one XOR with the lane's byte offset
    const unsigned char* gs_bytes = reinterpret_cast<const unsigned char*>(g_s);
    const unsigned laneOff = static_cast<unsigned>(lane) * (GR * 4);

    for (long long c = c_begin; c < c_end; ++c) {
        const int buf = static_cast<int>(c - c_begin) & 1;
        const long long o0 = c * T;
        const int nrows = static_cast<int>(min(static_cast<long long>(T), static_cast<long long>(L) - o0));
        __syncthreads();  // previous chunk's walk is done; buffer `buf` is staged

        {
            // thread = (granule gl of a row, rows warp, warp + 16, ...)
            const int gl = lane;
            const float* src = p.gT + static_cast<size_t>(o0 + warp) * p.ldg + gl * GR;
            const size_t srcStep = static_cast<size_t>(kWarps) * p.ldg;
#pragma unroll 4
            for (int ol = warp; ol < T; ol += kWarps, src += srcStep) {
                float* dst = g_s + ol * BT + ((gl ^ (ol & SW)) * GR);
                if (ol < nrows) __pipeline_memcpy_async(dst, src, 4 * GR);
                else store_zero_vec<BPL>(dst);
            }
        }
        __pipeline_commit();
        if (c + 1 < c_end) {  // its index loads overlap the tile copy, its weight gathers the walk
            stage(c + 1, buf ^ 1, nb_lo, nb_cnt);
            if (c + 2 < c_end) slice_bounds(c + 2, nb_lo, nb_cnt);
        }
        __pipeline_commit();
        __pipeline_wait_prior(1);  // the tile has landed; the staged weights may still be in flight
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
            const float4* row = reinterpret_cast<const float4*>(dbuf + sl * kDRow + h * 16);
            const float4 q0 = row[0], q1 = row[1], q2 = row[2], q3 = row[3];
            float sum = (((q0.x + q0.y) + (q0.z + q0.w)) + ((q1.x + q1.y) + (q1.z + q1.w))) +
                        (((q2.x + q2.y) + (q2.z + q2.w)) + ((q3.x + q3.y) + (q3.z + q3.w)));
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            if (h == 0 && sl < n && p.gW) {
                const unsigned code = ent[eblk + sl].y;
                const unsigned ol = (code & kRowMask) / (BT * 4);
                p.gW[(static_cast<size_t>(o0) + ol) * K + (code >> kKShift)] = sum;
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
                uint2 en[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) en[u] = ent[e + u];
                if (slot + 4 > kSlots) {
                    reduce_slots(slot);
                    eblk = e;
                    slot = 0;
                }
                LV v[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) v[u].load_shared(gs_bytes + ((en[u].y & kRowMask) ^ laneOff));
                float* drow = dbuf + slot * kDRow + lane;
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    acc[j].axpy(__uint_as_float(en[u].x), v[u]);
                    drow[u * kDRow] = xr[j].dot(v[u]);
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
                LV v;
                v.load_shared(gs_bytes + ((en.y & kRowMask) ^ laneOff));
                acc[j].axpy(__uint_as_float(en.x), v);
                dbuf[slot * kDRow + lane] = xr[j].dot(v);
                ++slot;
            }
        }
        if (slot > 0) reduce_slots(slot);

        __pipeline_wait_prior(0);  // this thread's staged weights of the next chunk are in place

        // Every segChunks chunks the running grad_x sums go out as one partial and restart from zero.
        const long long done = c - c_begin + 1;
        if (done % p.segChunks == 0 || c + 1 == c_end) {
            const int seg = static_cast<int>((done - 1) / p.segChunks);
#pragma unroll
            for (int j = 0; j < NI; ++j) {
                const int i = i_lo + warp * NI + j;
                if (i < N) {
                    float* dst = p.partial + ((static_cast<size_t>(r) * p.S + seg) * N + i) * p.Bpad + lane * BPL;
                    float out[BPL];
                    acc[j].get(out);
#pragma unroll
                    for (int q = 0; q < BPL; ++q) dst[q] = out[q];
                    acc[j].zero();
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
    if (plan->K >= (1 << (32 - kKShift))) return false;  // k shares the entry's code word with the row offset
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
    const int stat = width <= 128 ? 0 : (width <= 256 ? 1 : 2);
    const size_t cap = static_cast<size_t>((plan->max_slice_entries[stat] + 7) / 8 * 8 + 8);
    const size_t T = static_cast<size_t>(plan->chunk_rows);
    if (T * BT * 4 > (size_t{1} << kKShift)) return false;
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
    p.kShift = -1;
    for (int sh = 0; sh < 31; ++sh)
        if ((1 << sh) == a.K) p.kShift = sh;
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
