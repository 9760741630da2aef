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
#include <cuda.h>

#include <type_traits>

#include "ffi_common.cuh"

namespace ffi {
int peer_wait_timeouts(int* out);  // peer_reduce.cu
int set_peer_wait_limit(long long ticks);
namespace {
__device__ int g_wait_timeouts = 0;  // bounded waits of this file's kernels that gave up
__device__ long long g_wait_limit = 4000000000ll;  // clock64 ticks a wait may last (about two seconds)

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
    const void* W;   // fp32; the group kernel also takes bf16 (its TX)
    const float* gT;
    long long ldg;
    const void* xT;  // same element type as W
    long long ldx;
    const int* cperm;
    const int* cptr;
    float* partial;  // [R*S][N][Bpad]
    float* gW;
    float* gbias;  // pair kernel only: grad_bias[o] = sum_b gT[o][b], from the g tiles it holds anyway
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
    extern __shared__ __align__(1024) unsigned char smem_raw[];

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
            xv[q] = (i < N && b < p.B) ? __ldg(static_cast<const float*>(p.xT) + static_cast<size_t>(i) * p.ldx + b) : 0.f;
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
                    __pipeline_memcpy_async(&d->x, static_cast<const float*>(p.W) + pos[u], 4);
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

// =====================================================================================
// Batch 65..128: two entries per warp step, accumulators and x parked in tensor memory.
//
// A half warp covers the 128 batch columns of one entry (lane q of a half holds columns 4q..4q+3
// and 64+4q..64+4q+3: two LDS.128, conflict-free without any swizzle), so the two halves of a
// warp work on two consecutive entries of the same run at once.  Against one entry per warp step
// this halves the entry fetches, the address arithmetic, the stores of the per-lane grad_W dots
// and the rows the lane reduction reads.  Both halves accumulate grad_x of the same input; they
// are added when a partial is flushed.
//
// A lane then needs 8 accumulators and 8 values of x[:, i] per input, too many registers for 8
// inputs per warp.  Both live in tensor memory (TMEM, otherwise unused here): TMEM lane = thread
// lane of the warp's quarter, 16 columns per input (8 sums | 8 x).  A run starts with one
// tcgen05.ld of the 16 columns and ends with one tcgen05.st of the sums, so the loop over the
// warp's inputs needs no unrolling and few registers.
// =====================================================================================
constexpr int kTmemCols = 512;            // per lane quarter: 4 warps x 8 inputs x 16 columns
constexpr unsigned kPadCode = 0xffffffffu;  // code of the missing second entry of an odd run's last step

__device__ __forceinline__ void tmem_alloc(void* smem_dst, unsigned ncols) {
    const unsigned a = static_cast<unsigned>(__cvta_generic_to_shared(smem_dst));
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(a), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(unsigned taddr, unsigned ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_fence_before_sync() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_fence_after_sync() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// 8 consecutive 32-bit columns of this thread's TMEM lane
__device__ __forceinline__ void tmem_store8(unsigned taddr, const unsigned (&r)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr),
                 "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}
__device__ __forceinline__ void tmem_wait_store() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_load8(unsigned taddr, unsigned (&r)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
}
// Completes the loads; naming the registers keeps their first use behind the wait.
__device__ __forceinline__ void tmem_wait_load(unsigned (&r)[8], unsigned (&s)[8]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                   "+r"(s[0]), "+r"(s[1]), "+r"(s[2]), "+r"(s[3]), "+r"(s[4]), "+r"(s[5]), "+r"(s[6]), "+r"(s[7])
                 :
                 : "memory");
}

// ---- mbarrier + TMA (one tiled bulk copy per g tile, no multicast) ------------------------------

__device__ __forceinline__ unsigned smem_u32(const void* ptr) {
    return static_cast<unsigned>(__cvta_generic_to_shared(ptr));
}
__device__ __forceinline__ void mbar_init(unsigned long long* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
// Orders this thread's earlier generic-proxy accesses to shared memory before later async-proxy ones.
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Box of the 2-D tensor `map` with first element (x, y) -> dst; completion is signalled on `bar`.
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, unsigned long long* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
            smem_u32(dst)),
        "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned long long* bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Waits for the phase with the given parity, at most about two seconds; false if it gave up.
__device__ __forceinline__ bool mbar_wait_bounded(unsigned long long* bar, unsigned parity) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long start = clock64();
    const long long limit = g_wait_limit;
    while (!mbar_try_wait(bar, parity))
        if (clock64() - start > limit) return false;
    return true;
}

// The 8 batch elements one lane of a half warp holds of a vector over the batch.
struct Lane8 {
    u64 a, b, c, d;
    __device__ __forceinline__ void zero() { a = b = c = d = 0ull; }
    // columns 4q..4q+3 at ptr, columns BT/2+4q..BT/2+4q+3 HALF bytes further (HALF = 2*BT: half a tile row)
    template <int HALF>
    __device__ __forceinline__ void load_shared(const unsigned char* ptr) {
        const ulonglong2 t0 = *reinterpret_cast<const ulonglong2*>(ptr);
        const ulonglong2 t1 = *reinterpret_cast<const ulonglong2*>(ptr + HALF);
        a = t0.x, b = t0.y, c = t1.x, d = t1.y;
    }
    __device__ __forceinline__ void axpy(float w, const Lane8& g) {
        const u64 ww = pack2(w, w);
        a = fma2(ww, g.a, a), b = fma2(ww, g.b, b), c = fma2(ww, g.c, c), d = fma2(ww, g.d, d);
    }
    __device__ __forceinline__ float dot(const Lane8& g) const {
        float lo, hi;
        unpack2(fma2(g.d, d, fma2(g.c, c, fma2(g.b, b, mul2(g.a, a)))), lo, hi);
        return lo + hi;
    }
    __device__ __forceinline__ float sum() const {
        float f[8];
        unpack2(a, f[0], f[1]), unpack2(b, f[2], f[3]), unpack2(c, f[4], f[5]), unpack2(d, f[6], f[7]);
        return ((f[0] + f[1]) + (f[2] + f[3])) + ((f[4] + f[5]) + (f[6] + f[7]));
    }
};

// 16 columns of this thread's TMEM lane -> (sums, x) of one input, complete on return.  The 32-bit
// halves are paired inside the asm block so that the loaded registers ARE the pairs.
__device__ __forceinline__ void tmem_load_input(unsigned taddr, Lane8& sums, Lane8& x) {
    asm volatile(
        "{\n"
        ".reg .b32 t<16>;\n"
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {t0, t1, t2, t3, t4, t5, t6, t7, t8, t9, t10, t11, t12, t13, t14, t15}, [%8];\n"
        "tcgen05.wait::ld.sync.aligned;\n"
        "mov.b64 %0, {t0, t1};\n mov.b64 %1, {t2, t3};\n mov.b64 %2, {t4, t5};\n mov.b64 %3, {t6, t7};\n"
        "mov.b64 %4, {t8, t9};\n mov.b64 %5, {t10, t11};\n mov.b64 %6, {t12, t13};\n mov.b64 %7, {t14, t15};\n"
        "}"
        : "=l"(sums.a), "=l"(sums.b), "=l"(sums.c), "=l"(sums.d), "=l"(x.a), "=l"(x.b), "=l"(x.c), "=l"(x.d)
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_store_sums(unsigned taddr, const Lane8& sums) {
    asm volatile(
        "{\n"
        ".reg .b32 t<8>;\n"
        "mov.b64 {t0, t1}, %1;\n mov.b64 {t2, t3}, %2;\n mov.b64 {t4, t5}, %3;\n mov.b64 {t6, t7}, %4;\n"
        "tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {t0, t1, t2, t3, t4, t5, t6, t7};\n"
        "}" ::"r"(taddr),
        "l"(sums.a), "l"(sums.b), "l"(sums.c), "l"(sums.d)
        : "memory");
}

// The 4 batch elements one lane holds when a group of 8 lanes covers a batch of at most 32.
struct Lane4 {
    u64 a, b;
    __device__ __forceinline__ void zero() { a = b = 0ull; }
    // columns 4q..4q+3 at ptr: one 16-byte piece
    template <int HALF>
    __device__ __forceinline__ void load_shared(const unsigned char* ptr) {
        const ulonglong2 t0 = *reinterpret_cast<const ulonglong2*>(ptr);
        a = t0.x, b = t0.y;
    }
    __device__ __forceinline__ void axpy(float w, const Lane4& g) {
        const u64 ww = pack2(w, w);
        a = fma2(ww, g.a, a), b = fma2(ww, g.b, b);
    }
    __device__ __forceinline__ float dot(const Lane4& g) const {
        float lo, hi;
        unpack2(fma2(g.b, b, mul2(g.a, a)), lo, hi);
        return lo + hi;
    }
    __device__ __forceinline__ float sum() const {
        float f[4];
        unpack2(a, f[0], f[1]), unpack2(b, f[2], f[3]);
        return (f[0] + f[1]) + (f[2] + f[3]);
    }
};
// 8 columns of this thread's TMEM lane -> (sums, x) of one input, complete on return
__device__ __forceinline__ void tmem_load_input(unsigned taddr, Lane4& sums, Lane4& x) {
    asm volatile(
        "{\n"
        ".reg .b32 t<8>;\n"
        "tcgen05.ld.sync.aligned.32x32b.x8.b32 {t0, t1, t2, t3, t4, t5, t6, t7}, [%4];\n"
        "tcgen05.wait::ld.sync.aligned;\n"
        "mov.b64 %0, {t0, t1};\n mov.b64 %1, {t2, t3};\n mov.b64 %2, {t4, t5};\n mov.b64 %3, {t6, t7};\n"
        "}"
        : "=l"(sums.a), "=l"(sums.b), "=l"(x.a), "=l"(x.b)
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_store_sums(unsigned taddr, const Lane4& sums) {
    asm volatile(
        "{\n"
        ".reg .b32 t<4>;\n"
        "mov.b64 {t0, t1}, %1;\n mov.b64 {t2, t3}, %2;\n"
        "tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {t0, t1, t2, t3};\n"
        "}" ::"r"(taddr),
        "l"(sums.a), "l"(sums.b)
        : "memory");
}
// VPL consecutive 32-bit columns of this thread's TMEM lane
template <int VPL>
__device__ __forceinline__ void tmem_store_cols(unsigned taddr, const unsigned (&r)[VPL]) {
    if constexpr (VPL == 8) {
        tmem_store8(taddr, r);
    } else {
        asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};" ::"r"(taddr), "r"(r[0]), "r"(r[1]),
                     "r"(r[2]), "r"(r[3])
                     : "memory");
    }
}
// ... loaded and complete on return
template <int VPL>
__device__ __forceinline__ void tmem_load_cols(unsigned taddr, unsigned (&r)[VPL]) {
    if constexpr (VPL == 8) {
        unsigned dummy[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
        tmem_load8(taddr, r);
        tmem_wait_load(r, dummy);
    } else {
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];\n"
            "tcgen05.wait::ld.sync.aligned;"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
            : "r"(taddr)
            : "memory");
    }
}
template <int VPL>
struct LaneOf {
    using type = Lane8;
};
template <>
struct LaneOf<4> {
    using type = Lane4;
};

// G lane groups per warp and VPL batch elements per lane: a group of 32/G lanes covers the BT = VPL*32/G batch
// columns of one entry, so a warp step works on G consecutive entries of a run.
//   batch 65..128: G = 2, VPL = 8 (the case described above; two 16-byte pieces of a tile row per lane);
//   batch 33..64:  G = 2, VPL = 4 (one 16-byte piece per lane, the tile is [T][64]);
//   batch <= 32:   G = 4, VPL = 4 (a quarter warp per entry, the tile is [T][32]).
// With VPL = 4 an input's state is 8 TMEM columns instead of 16, so a warp owns 16 inputs, a CTA 256, and three
// slices per range instead of six fetch each g tile.
//
// TX is the storage type of x and W.  bf16 x is widened (exactly) on its way into tensor memory.  A bf16
// weight is fetched as the aligned 4-byte word that holds it (cp.async copies at least 4 bytes) and turned
// into its fp32 bit pattern by the thread that fetched it once the copy has landed (the entry's code tells
// which half: the chunk's first position is even, so the parity of the position within the chunk is the
// parity of the flat position).
//
template <int NI, int THREADS, int SLOTS, int G, typename TX, int VPL = 8>
__global__ void __launch_bounds__(THREADS, 1)
    ffi_bwd_pairs_kernel(BwdFusedParams p, const __grid_constant__ CUtensorMap g_map) {
    constexpr bool kBf16 = !std::is_same<TX, float>::value;
    using LaneT = typename LaneOf<VPL>::type;
    const TX* xTt = static_cast<const TX*>(p.xT);
    constexpr int LG = 32 / G;    // lanes per group
    constexpr int BT = VPL * LG;  // batch columns of the tile
    constexpr int HALF = 2 * BT;  // bytes between a lane's two 16-byte pieces of a tile row (VPL = 8)
    constexpr int COLS = 2 * VPL; // TMEM columns of one input: its sums and its x values
    constexpr int kThreads = THREADS, kWarps = THREADS / 32, kSlots = SLOTS;  // shadow the file-wide values
    constexpr int CPN = kWarps * NI + 1;
    constexpr unsigned kRowMask = (1u << kKShift) - 1u;
    static_assert((THREADS / 128) * NI * COLS <= kTmemCols, "the warps of a lane quarter share the TMEM columns");
    static_assert(SLOTS * G == 32, "the lane reduction maps the 32 lanes to (buffered step, group)");
    static_assert(32 + G <= kDRow, "a dot-buffer row holds 32 dots and G entry codes");
    extern __shared__ __align__(1024) unsigned char smem_raw[];

    const int T = p.T, K = p.K, N = p.N;
    float* g_s = reinterpret_cast<float*>(smem_raw);                                    // [T][BT], row-major
    uint2* ent_s = reinterpret_cast<uint2*>(g_s + static_cast<size_t>(T) * BT);         // [2][entCap]
    float* dbuf_s = reinterpret_cast<float*>(ent_s + 2 * p.entCap);                     // [warps][kSlots][kDRow]
    int* cp_s = reinterpret_cast<int*>(dbuf_s + kWarps * kSlots * kDRow);               // [2][CPN]
    unsigned long long* g_bar = reinterpret_cast<unsigned long long*>(cp_s + 2 * CPN);  // tile arrival (2*CPN ints keep 8-byte alignment)
    unsigned* tmem_base_p = reinterpret_cast<unsigned*>(g_bar + 1);

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int grp = lane / LG;  // which entry of a step this lane works on
    const int q = lane % LG;
    const int r = blockIdx.x;
    const int i_lo = blockIdx.y * (kWarps * NI);
    const int i_hi = min(N, i_lo + kWarps * NI);
    const long long c_begin = p.nChunks * r / p.R;
    const long long c_end = p.nChunks * (r + 1) / p.R;

    if (warp == 0) tmem_alloc(tmem_base_p, kTmemCols);
    if (tid == 32) mbar_init(g_bar, 1);
    tmem_fence_before_sync();
    __syncthreads();
    tmem_fence_after_sync();
    const unsigned tmem_base = *tmem_base_p;
    // lanes 32*(warp % 4) .. +31 are the ones this warp may touch; its inputs take NI*COLS columns
    const unsigned taddr0 = tmem_base + ((static_cast<unsigned>(warp & 3) * 32u) << 16) +
                            static_cast<unsigned>(warp >> 2) * (NI * COLS);

    if constexpr (VPL == 8) {
        for (int j = 0; j < NI; ++j) {
            const int i = i_lo + warp * NI + j;
            unsigned xv[8], zero[8];
    #pragma unroll
            for (int m = 0; m < 8; ++m) {
                const int b = (m < 4 ? 0 : BT / 2) + 4 * q + (m & 3);
                xv[m] = __float_as_uint((i < N && b < p.B) ? widen(xTt[static_cast<size_t>(i) * p.ldx + b]) : 0.f);
                zero[m] = 0u;
            }
            tmem_store8(taddr0 + j * 16, zero);
            tmem_store8(taddr0 + j * 16 + 8, xv);
        }
    } else {
        for (int j = 0; j < NI; ++j) {
            const int i = i_lo + warp * NI + j;
            unsigned xv[VPL], zero[VPL];
    #pragma unroll
            for (int m = 0; m < VPL; ++m) {
                const int b = (m < 4 ? 0 : BT / 2) + 4 * q + (m & 3);
                xv[m] = __float_as_uint((i < N && b < p.B) ? widen(xTt[static_cast<size_t>(i) * p.ldx + b]) : 0.f);
                zero[m] = 0u;
            }
            tmem_store_cols<VPL>(taddr0 + j * COLS, zero);
            tmem_store_cols<VPL>(taddr0 + j * COLS + VPL, xv);
        }
    }
    tmem_wait_store();

    auto slice_bounds = [&](long long c, int& e_lo, int& cnt) {
        const int* cptr_c = p.cptr + c * (N + 1);
        e_lo = __ldg(cptr_c + i_lo);
        cnt = __ldg(cptr_c + i_hi) - e_lo;
    };

    // Staging of a chunk's entries runs two chunks ahead of its walk: the flat positions (and the run
    // offsets) are loaded into registers during the prologue two chunks earlier, and turned into
    // entries (W by 4-byte cp.async, code = byte offset of the entry's g row | position in the chunk
    // << 18) one chunk earlier, so that no prologue waits for a dependent global load.
    // (The plan guarantees that a slice never holds more than entCap entries.)
    int pos[kStageUnroll];
    int cpv = 0;
    auto load_pos = [&](long long c, int e_lo, int cnt) {
        const int* cperm_c = p.cperm + c * static_cast<long long>(T) * K + e_lo;
#pragma unroll
        for (int u = 0; u < kStageUnroll; ++u) {
            const int e = tid + u * kThreads;
            pos[u] = e < cnt ? __ldg(cperm_c + e) : -1;
        }
        if (tid < CPN) cpv = __ldg(p.cptr + c * (N + 1) + min(i_lo + tid, i_hi)) - e_lo;
    };
    auto emit_one = [&](uint2* d, int ps, int pos0) {
        if constexpr (kBf16) __pipeline_memcpy_async(&d->x, static_cast<const unsigned*>(p.W) + (ps >> 1), 4);
        else __pipeline_memcpy_async(&d->x, static_cast<const float*>(p.W) + ps, 4);
        const int rel = ps - pos0;
        const int ol = p.kShift >= 0 ? (rel >> p.kShift) : rel / K;
        d->y = static_cast<unsigned>(ol * (BT * 4)) | (static_cast<unsigned>(rel) << kKShift);
    };
    // bf16 weights: the words this thread fetched for buffer `buf` (cnt entries) become fp32 bit patterns
    auto widen_staged = [&](int buf, int cnt) {
        if constexpr (kBf16) {
            uint2* dst = ent_s + buf * p.entCap;
            for (int e = tid; e < cnt; e += kThreads) {
                const uint2 en = dst[e];
                dst[e].x = ((en.y >> kKShift) & 1u) ? (en.x & 0xffff0000u) : (en.x << 16);
            }
        }
    };
    auto emit = [&](long long c, int buf, int e_lo, int cnt) {
        const int pos0 = static_cast<int>(c * T) * K;
        uint2* dst = ent_s + buf * p.entCap;
        if (tid < CPN) cp_s[buf * CPN + tid] = cpv;
#pragma unroll
        for (int u = 0; u < kStageUnroll; ++u)
            if (pos[u] >= 0) emit_one(dst + tid + u * kThreads, pos[u], pos0);
        // a slice with more entries than the registers cover: the rest is fetched here
        const int* cperm_c = p.cperm + c * static_cast<long long>(T) * K + e_lo;
        for (int e = tid + kStageUnroll * kThreads; e < cnt; e += kThreads) emit_one(dst + e, __ldg(cperm_c + e), pos0);
    };

    int pl_lo = 0, pl_cnt = 0;  // bounds of the chunk whose positions the registers hold
    int nb_lo = 0, nb_cnt = 0;  // bounds of the chunk after that
    int first_cnt = 0;
    if (c_begin < c_end) {
        slice_bounds(c_begin, pl_lo, pl_cnt);
        load_pos(c_begin, pl_lo, pl_cnt);
        emit(c_begin, 0, pl_lo, pl_cnt);
        first_cnt = pl_cnt;
        if (c_begin + 1 < c_end) {
            slice_bounds(c_begin + 1, pl_lo, pl_cnt);
            load_pos(c_begin + 1, pl_lo, pl_cnt);
        }
        if (c_begin + 2 < c_end) slice_bounds(c_begin + 2, nb_lo, nb_cnt);
    }
    __pipeline_commit();
    __pipeline_wait_prior(0);
    widen_staged(0, first_cnt);
    float* dbuf = dbuf_s + warp * (kSlots * kDRow);
    float* dlane = dbuf + lane;                                   // this lane's column of the dot buffer
    const int dcode_delta = 32 + grp - lane;                      // from a lane's dot to its entry's code
    const float* dlast1 = dlane + (kSlots - 1) * kDRow;           // last row a single step may fill
    const float* dlast2 = dlane + (kSlots - 2) * kDRow;           // last row a double step may start at
    const int myrow = lane / G, myent = lane % G;                 // the (buffered step, entry) this lane reduces
    const float4* drow = reinterpret_cast<const float4*>(dbuf + myrow * kDRow + myent * LG);
    const unsigned* dmine = reinterpret_cast<const unsigned*>(dbuf) + myrow * kDRow + 32 + myent;
    const unsigned char* gs_lane = reinterpret_cast<const unsigned char*>(g_s) + q * 16;
    const unsigned tileBytes = static_cast<unsigned>(T) * (BT * 4);
    bool gave_up = false;
    long long pending = -1;  // chunk whose tile copy has been issued and not yet seen complete

    long long c = c_begin;
    for (; c < c_end; ++c) {
        const int buf = static_cast<int>(c - c_begin) & 1;
        const long long o0 = c * T;
        // previous chunk's walk is done; buffer `buf` is staged; nobody has given up on a wait
        if (__syncthreads_or(gave_up)) {
            gave_up = true;
            break;
        }

        // The g tile of the chunk: one TMA box [T rows][BT columns] of gT (rows past L and columns past the
        // stored row arrive as zeros).
        // (A second tile buffer filled one chunk ahead was measured: it needs T <= 168 to fit, and the
        // shorter runs cost more than the hidden copy saves.)
        if (tid == 0) {
            fence_proxy_async();
            mbar_expect_tx(g_bar, tileBytes);
            tma_load_2d(g_s, &g_map, 0, static_cast<int>(o0), g_bar);
        }
        pending = c;
        const int staged_cnt = c + 1 < c_end ? pl_cnt : 0;  // entries of chunk c + 1 going into the other buffer
        if (c + 1 < c_end) emit(c + 1, buf ^ 1, pl_lo, pl_cnt);
        __pipeline_commit();
        if (c + 2 < c_end) {
            pl_lo = nb_lo, pl_cnt = nb_cnt;
            load_pos(c + 2, pl_lo, pl_cnt);
        }
        if (c + 3 < c_end) slice_bounds(c + 3, nb_lo, nb_cnt);
        // Each thread waits for the tile itself; one that gives up says so at the next barrier (the
        // walk of this chunk then reads a stale tile, which is harmless: the result is void anyway).
        if (mbar_wait_bounded(g_bar, static_cast<unsigned>(c - c_begin) & 1u)) {
            pending = -1;
        } else {
            atomicAdd(&g_wait_timeouts, 1);
            gave_up = true;
        }

        // grad_bias of the chunk's rows: the slices of a range take turns, each row is one group's sum
        if (p.gbias && static_cast<int>(c % gridDim.y) == static_cast<int>(blockIdx.y)) {
            for (int rr = G * warp + grp; rr < T; rr += G * kWarps) {
                LaneT v;
                v.template load_shared<HALF>(gs_lane + rr * (BT * 4));
                float sum = v.sum();
#pragma unroll
                for (int off = LG / 2; off >= 1; off /= 2) sum += __shfl_xor_sync(0xffffffffu, sum, off);
                if (q == 0 && o0 + rr < p.L) p.gbias[o0 + rr] = sum;
            }
        }

        // ---- walk the runs of this warp's inputs, G entries per step ---------------------------
        const uint2* ent = ent_s + buf * p.entCap + grp;  // this group's entry of a step
        const int* cp = cp_s + buf * CPN + warp * NI;
        float* gWc = p.gW ? p.gW + static_cast<size_t>(o0) * K : nullptr;
        // Row of the dot buffer the next step fills: 32 per-lane dots, then the codes of its G entries.
        // dptr points at this lane's column of that row; the code of the lane's entry goes to
        // dptr + dcode_delta (written by every lane of the group: same address, same value).
        float* dptr = dlane;

        // Lane row*G + h adds the 32/G dots of entry h of buffered step `row` (fixed order) and stores
        // grad_W of that entry.
        auto reduce_slots = [&]() {
            __syncwarp();
            const int rows = static_cast<int>(dptr - dlane) / kDRow;
            float sum;
            if constexpr (LG == 16) {
                const float4 q0 = drow[0], q1 = drow[1], q2 = drow[2], q3 = drow[3];
                sum = (((q0.x + q0.y) + (q0.z + q0.w)) + ((q1.x + q1.y) + (q1.z + q1.w))) +
                      (((q2.x + q2.y) + (q2.z + q2.w)) + ((q3.x + q3.y) + (q3.z + q3.w)));
            } else {
                const float4 q0 = drow[0], q1 = drow[1];
                sum = ((q0.x + q0.y) + (q0.z + q0.w)) + ((q1.x + q1.y) + (q1.z + q1.w));
            }
            const unsigned code = *dmine;
            if (myrow < rows && code != kPadCode && gWc) gWc[code >> kKShift] = sum;
            __syncwarp();
            dptr = dlane;
        };

        int e = cp[0];
#pragma unroll 1
        for (int j = 0; j < NI; ++j) {
            const int t = cp[j + 1];
            if (e >= t) continue;
            LaneT acc, xr;
            tmem_load_input(taddr0 + j * COLS, acc, xr);
            // two steps (2 G entries) per iteration: all loads are issued before the stores
            for (; e + 2 * G <= t; e += 2 * G) {
                const uint2 en0 = ent[e], en1 = ent[e + G];
                LaneT g0, g1;
                g0.template load_shared<HALF>(gs_lane + (en0.y & kRowMask));
                g1.template load_shared<HALF>(gs_lane + (en1.y & kRowMask));
                if (dptr > dlast2) reduce_slots();
                acc.axpy(__uint_as_float(en0.x), g0);
                acc.axpy(__uint_as_float(en1.x), g1);
                dptr[0] = xr.dot(g0);
                dptr[kDRow] = xr.dot(g1);
                reinterpret_cast<unsigned*>(dptr + dcode_delta)[0] = en0.y;
                reinterpret_cast<unsigned*>(dptr + dcode_delta)[kDRow] = en1.y;
                dptr += 2 * kDRow;
            }
            if (e + G <= t) {
                const uint2 en0 = ent[e];
                LaneT g0;
                g0.template load_shared<HALF>(gs_lane + (en0.y & kRowMask));
                if (dptr > dlast1) reduce_slots();
                acc.axpy(__uint_as_float(en0.x), g0);
                dptr[0] = xr.dot(g0);
                reinterpret_cast<unsigned*>(dptr + dcode_delta)[0] = en0.y;
                dptr += kDRow;
                e += G;
            }
            if (e < t) {  // the run's last step has entries for the first t - e groups only
                uint2 en0 = make_uint2(0u, kPadCode);
                LaneT g0;
                g0.zero();
                if (grp < t - e) {
                    en0 = ent[e];
                    g0.template load_shared<HALF>(gs_lane + (en0.y & kRowMask));
                }
                if (dptr > dlast1) reduce_slots();
                acc.axpy(__uint_as_float(en0.x), g0);
                dptr[0] = xr.dot(g0);
                reinterpret_cast<unsigned*>(dptr + dcode_delta)[0] = en0.y;
                dptr += kDRow;
                e = t;
            }
            tmem_store_sums(taddr0 + j * COLS, acc);
        }
        if (dptr != dlane) reduce_slots();
        tmem_wait_store();

        __pipeline_wait_prior(0);  // this thread's staged weights of the next chunk are in place
        widen_staged(buf ^ 1, staged_cnt);

        // Every segChunks chunks the running grad_x sums go out as one partial and restart from zero.
        const long long done = c - c_begin + 1;
        if (done % p.segChunks == 0 || c + 1 == c_end) {
            const int seg = static_cast<int>((done - 1) / p.segChunks);
            if constexpr (VPL == 8) {
                for (int j = 0; j < NI; ++j) {
                    const int i = i_lo + warp * NI + j;
                    unsigned av[8], zero[8];
                    tmem_load8(taddr0 + j * 16, av);
    #pragma unroll
                    for (int m = 0; m < 8; ++m) zero[m] = 0u;
                    tmem_wait_load(av, zero);
                    tmem_store8(taddr0 + j * 16, zero);
                    float out[8];
    #pragma unroll
                    for (int m = 0; m < 8; ++m) {
                        out[m] = __uint_as_float(av[m]);
    #pragma unroll
                        for (int off = 16; off >= LG; off /= 2) out[m] += __shfl_xor_sync(0xffffffffu, out[m], off);  // the groups
                    }
                    if (i < N && grp == 0) {
                        // One partial per range: the first segment stores, the later ones add to what this lane
                        // stored before (a handful of fp32 additions of segment sums; the long sums stay inside
                        // the segments, and the ranges are added in fp64 afterwards).
                        float* dst = p.partial + (static_cast<size_t>(r) * N + i) * p.Bpad + 4 * q;
                        if (seg > 0) {
                            const float4 a = *reinterpret_cast<const float4*>(dst);
                            const float4 b = *reinterpret_cast<const float4*>(dst + BT / 2);
                            out[0] += a.x, out[1] += a.y, out[2] += a.z, out[3] += a.w;
                            out[4] += b.x, out[5] += b.y, out[6] += b.z, out[7] += b.w;
                        }
                        *reinterpret_cast<float4*>(dst) = make_float4(out[0], out[1], out[2], out[3]);
                        *reinterpret_cast<float4*>(dst + BT / 2) = make_float4(out[4], out[5], out[6], out[7]);
                    }
                }
            } else {
                for (int j = 0; j < NI; ++j) {
                    const int i = i_lo + warp * NI + j;
                    unsigned av[VPL], zero[VPL];
    #pragma unroll
                    for (int m = 0; m < VPL; ++m) zero[m] = 0u;
                    tmem_load_cols<VPL>(taddr0 + j * COLS, av);
                    tmem_store_cols<VPL>(taddr0 + j * COLS, zero);
                    float out[VPL];
    #pragma unroll
                    for (int m = 0; m < VPL; ++m) {
                        out[m] = __uint_as_float(av[m]);
    #pragma unroll
                        for (int off = 16; off >= LG; off /= 2) out[m] += __shfl_xor_sync(0xffffffffu, out[m], off);  // the groups
                    }
                    if (i < N && grp == 0) {
                        // One partial per range: the first segment stores, the later ones add to what this lane
                        // stored before (a handful of fp32 additions of segment sums; the long sums stay inside
                        // the segments, and the ranges are added in fp64 afterwards).
                        float* dst = p.partial + (static_cast<size_t>(r) * N + i) * p.Bpad + 4 * q;
    #pragma unroll
                        for (int h = 0; h < VPL / 4; ++h) {
                            if (seg > 0) {
                                const float4 a = *reinterpret_cast<const float4*>(dst + h * (BT / 2));
                                out[4 * h] += a.x, out[4 * h + 1] += a.y, out[4 * h + 2] += a.z, out[4 * h + 3] += a.w;
                            }
                            *reinterpret_cast<float4*>(dst + h * (BT / 2)) =
                                make_float4(out[4 * h], out[4 * h + 1], out[4 * h + 2], out[4 * h + 3]);
                        }
                    }
                }
            }
            tmem_wait_store();
        }
    }

    // A range without chunks still owns a partial: zeros.
    if (c_begin >= c_end) {
        for (int j = 0; j < NI; ++j) {
            const int i = i_lo + warp * NI + j;
            if (i < N && grp == 0) {
                float* dst = p.partial + (static_cast<size_t>(r) * N + i) * p.Bpad + 4 * q;
                *reinterpret_cast<float4*>(dst) = make_float4(0.f, 0.f, 0.f, 0.f);
                if constexpr (VPL == 8) *reinterpret_cast<float4*>(dst + BT / 2) = make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
    }

    // A thread that gave up waits once more, again bounded, for the copy it abandoned (the chunk it recorded
    // when the copy was issued) before the CTA releases its shared memory.
    if (pending >= 0) mbar_wait_bounded(g_bar, static_cast<unsigned>(pending - c_begin) & 1u);
    tmem_fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, kTmemCols);
}

struct FusedConfig {
    int bpl, ni, iparts, Bpad, R, entCap, segChunks, S;
    int groups;  // lane groups per warp of the group kernel (2: batch 33..128, 4: batch <= 32), 0: ffi_bwd_fused_kernel
    int vpl;     // batch elements per lane of the group kernel: 8 (batch 65..128) or 4
    size_t smem;
};

constexpr int kGroupThreads = 512, kGroupNI = 8;  // (1024 threads x 4 inputs was measured: 10 % slower)

bool fused_config(const ffi_plan* plan, int64_t B, const DeviceInfo& dev, FusedConfig* c) {
    if (!plan || !plan->has_chunks || B > 128) return false;
    if (plan->K >= (1 << (32 - kKShift))) return false;  // k shares the entry's code word with the row offset
    // the group kernel's entry code holds the position within the chunk in 14 bits
    const bool group_kernel = static_cast<long long>(plan->chunk_rows) * plan->K <= (1 << (32 - kKShift));
    c->groups = group_kernel ? (B > 32 ? 2 : 4) : 0;
    c->vpl = group_kernel && B <= 64 ? 4 : 8;
    c->bpl = group_kernel ? (B > 64 ? 4 : 2) : (B <= 32 ? 1 : (B <= 64 ? 2 : 4));
    // ffi_bwd_fused_kernel: 32 accumulator + 32 x registers per lane; the group kernel: 512 TMEM columns per lane quarter
    c->ni = group_kernel ? (c->vpl == 4 ? 2 * kGroupNI : kGroupNI) : 32 / c->bpl;
    const int BT = group_kernel ? c->vpl * (32 / c->groups) : 32 * c->bpl;
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
    // the group kernel adds its segments into one partial per range; the register kernel keeps one per segment
    c->S = group_kernel ? 1 : static_cast<int>(ceil_div(ceil_div(plan->n_chunks, R), seg));
    const int stat = width <= 128 ? 0 : (width <= 256 ? 1 : 2);
    const size_t cap = static_cast<size_t>((plan->max_slice_entries[stat] + 7) / 8 * 8 + 8);
    const size_t T = static_cast<size_t>(plan->chunk_rows);
    if (T * BT * 4 > (size_t{1} << kKShift)) return false;
    // the group kernel buffers 32 / groups steps per warp; + its barrier, TMEM slot and alignment slack
    const size_t slots = group_kernel ? 32 / c->groups : kSlots;
    const size_t total = T * BT * 4 + 2 * cap * 8 + static_cast<size_t>(kWarps) * slots * kDRow * 4 +
                         2 * (kWarps * c->ni + 1) * 4 + 16 + (group_kernel ? 1024 : 0);
    if (total > static_cast<size_t>(dev.max_smem_optin)) return false;  // unusually dense slice or large K: separate kernels
    c->entCap = static_cast<int>(cap);
    c->smem = total;
    return true;
}

// cuTensorMapEncodeTiled through the runtime's driver entry point (the library does not link libcuda).
int encode_g_map(CUtensorMap* map, const float* gT, int64_t L, int64_t ldg, int chunk_rows, int BT) {
    using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeFn encode = nullptr;
    if (!encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        FFI_CUDA_CHECK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q));
        if (q != cudaDriverEntryPointSuccess || !fn) return fail(FFI_ERR_CUDA, "cuTensorMapEncodeTiled is not available");
        encode = reinterpret_cast<EncodeFn>(fn);
    }
    if (reinterpret_cast<uintptr_t>(gT) % 16 != 0 || chunk_rows > 256 || (BT != 32 && BT != 64 && BT != 128))
        return fail(FFI_ERR_INVALID_ARGUMENT, "transposed gradient must be 16-byte aligned, chunks at most 256 rows");
    // the stored rows may be narrower than the tile (batch <= 32 keeps 32 columns): the box's columns past them
    // are filled with zeros, like its rows past L
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(ldg < BT ? ldg : BT), static_cast<cuuint64_t>(L)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ldg) * 4};
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(BT), static_cast<cuuint32_t>(chunk_rows)};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(gT), dims, strides, box, elem,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(FFI_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", static_cast<int>(r));
    return FFI_OK;
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

// True when the one-pass backward of this shape is the group kernel, which also reads bf16 x and W.
bool backward_fused_takes_bf16(const ffi_plan* plan, int64_t B) {
    DeviceInfo dev;
    if (get_device_info(&dev) != FFI_OK) return false;
    FusedConfig c;
    return fused_config(plan, B, dev, &c) && c.groups != 0;
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

// grad_x (always), grad_W (when gW != nullptr) and grad_bias (when gbias != nullptr, from gT) in one
// kernel (grad_bias by a separate pass over gT where the pair kernel does not apply).  xT is x as [N][ldx].
int launch_backward_fused(const GradXArgs& a, const void* xT, int64_t ldx, float* gW, float* gbias,
                          cudaStream_t stream) {
    DeviceInfo dev;
    int rc = get_device_info(&dev);
    if (rc != FFI_OK) return rc;
    FusedConfig c;
    if (!fused_config(a.plan, a.B, dev, &c)) return fail(FFI_ERR_UNSUPPORTED, "fused backward does not cover this shape");
    const size_t need = static_cast<size_t>(c.R) * c.S * a.N * c.Bpad * 4;
    if (!a.workspace || a.workspace_bytes < need || reinterpret_cast<uintptr_t>(a.workspace) % 16 != 0)
        return fail(FFI_ERR_WORKSPACE, "fused backward needs %zu bytes of 16-byte aligned workspace", need);
    // the group kernel's tile copy fills the columns past a narrower stored row with zeros
    const int64_t min_ldg = c.groups ? round_up(a.B, 32) : c.Bpad;
    if (!a.gT || a.ldg < min_ldg || a.ldg % 32 != 0 || !xT)
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
    p.gbias = nullptr;
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
    const bool pairs = c.groups != 0;
    if (a.w_bf16 && !pairs) return fail(FFI_ERR_UNSUPPORTED, "this fused backward kernel reads fp32 x and W");
    if (gbias && !pairs) {  // the other kernels leave grad_bias to a pass over gT
        rc = launch_bias_grad_rows(a.gT, a.ldg, a.L, gbias, stream);
        if (rc != FFI_OK) return rc;
    }
    if (pairs) {
        p.gbias = gbias;
        // gT as a 2-D tensor [L rows][BT columns] with row pitch ldg; one box = the g tile of a chunk
        CUtensorMap g_map;
        rc = encode_g_map(&g_map, a.gT, a.L, a.ldg, a.plan->chunk_rows, c.Bpad);
        if (rc != FFI_OK) return rc;
        dim3 grid(static_cast<unsigned>(c.R), static_cast<unsigned>(c.iparts), 1);
        auto launch_group = [&](auto kern) -> int {
            FFI_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(c.smem)));
            kern<<<grid, kGroupThreads, c.smem, stream>>>(p, g_map);
            return FFI_OK;
        };
        if (c.groups == 2 && c.vpl == 8 && !a.w_bf16) rc = launch_group(ffi_bwd_pairs_kernel<kGroupNI, kGroupThreads, 16, 2, float>);
        else if (c.groups == 2 && c.vpl == 8) rc = launch_group(ffi_bwd_pairs_kernel<kGroupNI, kGroupThreads, 16, 2, __nv_bfloat16>);
        else if (c.groups == 2 && c.vpl == 4 && !a.w_bf16) rc = launch_group(ffi_bwd_pairs_kernel<2 * kGroupNI, kGroupThreads, 16, 2, float, 4>);
        else if (c.groups == 2 && c.vpl == 4) rc = launch_group(ffi_bwd_pairs_kernel<2 * kGroupNI, kGroupThreads, 16, 2, __nv_bfloat16, 4>);
        else if (!a.w_bf16) rc = launch_group(ffi_bwd_pairs_kernel<2 * kGroupNI, kGroupThreads, 8, 4, float, 4>);
        else rc = launch_group(ffi_bwd_pairs_kernel<2 * kGroupNI, kGroupThreads, 8, 4, __nv_bfloat16, 4>);
        if (rc != FFI_OK) return rc;
        FFI_LAUNCH_CHECK("ffi_bwd_pairs_kernel");
        rc = FFI_OK;
    }
    else if (c.bpl == 4) rc = launch_fused_t<8, 4>(p, c, stream);
    else if (c.bpl == 2) rc = launch_fused_t<16, 2>(p, c, stream);
    else rc = launch_fused_t<32, 1>(p, c, stream);
    if (rc != FFI_OK) return rc;
    return reduce_range_partials(p.partial, a.gx, c.R * c.S, a.N, a.B, c.Bpad, a.x_transposed, stream);
}

}  // namespace ffi

// Test hook: how long (clock64 ticks of the current device, about 0.5 ns each) the bounded device-side waits
// may last before they give up.  The default is about two seconds; a test of the give-up path lowers it.
extern "C" int ffi_set_wait_limit_ticks(int64_t ticks) {
    if (ticks < 1000) return ffi::fail(FFI_ERR_INVALID_ARGUMENT, "the wait limit must be at least 1000 ticks");
    const long long t = ticks;
    FFI_CUDA_CHECK(cudaMemcpyToSymbol(ffi::g_wait_limit, &t, sizeof(t)));
    return ffi::set_peer_wait_limit(t);
}

// Number of bounded device-side waits that gave up since the library was loaded (0 in a healthy
// run; any other value means the results of the affected call are void).  Synchronises the device.
extern "C" int ffi_wait_timeouts(int* out) {
    if (!out) return ffi::fail(FFI_ERR_INVALID_ARGUMENT, "NULL output passed to ffi_wait_timeouts");
    FFI_CUDA_CHECK(cudaMemcpyFromSymbol(out, ffi::g_wait_timeouts, sizeof(int)));
    int peers = 0;
    const int rc = ffi::peer_wait_timeouts(&peers);
    if (rc != FFI_OK) return rc;
    *out += peers;
    return FFI_OK;
}
