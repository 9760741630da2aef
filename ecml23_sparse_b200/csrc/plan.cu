// Transposed (CSR-by-input) index of an FFI index table, built on the device.
//
// The reference has no such structure: its grad_x scatters with atomicAdd
// (tfsparse/cc/kernels/backward.cu.h:119-182).  Definition (bit-exact contract):
// flat position p = o*K + k; `perm` lists all positions ordered by key idx[p]
// ascending, ties by p ascending; rowptr[i] = number of positions with key < i.
//
// Build: a stable least-significant-digit radix sort of (key, position) pairs, 8 bits
// per pass, one warp per 1024-element tile (per-tile digit histogram, global exclusive
// scan, stable in-tile ranking with warp match).  From the canonical form a chunked
// form is derived for the narrow-input grad_x kernel: the outputs are cut into chunks
// of T rows, and chunk c stores its T*K positions ordered by (key, position) in
// cperm[c*T*K ...], with cptr[c][i] the offset of input i's run inside the chunk.
// Concatenating, for each input i, its runs over the chunks in chunk order gives back
// exactly row i of the canonical form (chunks are ascending ranges of p).
#include <atomic>
#include <cstdlib>

#include "ffi_common.cuh"

namespace ffi {
namespace {

constexpr int kTile = 1024;      // elements per warp tile
constexpr int kSortWarps = 4;    // warps per block in the sort kernels

__global__ void validate_idx_kernel(const int* __restrict__ idx, long long n, int N, int* bad) {
    long long e = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    bool any = false;
    for (; e < n; e += stride) {
        unsigned v = static_cast<unsigned>(idx[e]);
        any |= v >= static_cast<unsigned>(N);
    }
    if (any) *bad = 1;
}

// counts[d * nTiles + tile] = number of elements of `tile` whose digit is d.
__global__ void radix_hist_kernel(const int* __restrict__ keys, long long n, int shift,
                                  int* __restrict__ counts, long long nTiles) {
    __shared__ int h[kSortWarps][256];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long long tile = static_cast<long long>(blockIdx.x) * kSortWarps + warp;
    for (int d = lane; d < 256; d += 32) h[warp][d] = 0;
    __syncwarp();
    if (tile < nTiles) {
        const long long base = tile * kTile;
        for (int r = 0; r < kTile / 32; ++r) {
            long long e = base + r * 32 + lane;
            if (e < n) atomicAdd(&h[warp][(keys[e] >> shift) & 255], 1);
        }
        __syncwarp();
        for (int d = lane; d < 256; d += 32) counts[static_cast<long long>(d) * nTiles + tile] = h[warp][d];
    }
}

// In-place exclusive scan of `data[0..n)`: int64 running totals, int32 output (totals are bounded by
// L*K < 2^31).  Three phases: every block adds up its segment of kScanSeg consecutive elements, one block
// scans the segment totals, every block rescans its segment from its offset.
constexpr int kScanThreads = 256;
constexpr int kScanPer = 16;                          // consecutive elements per thread
constexpr int kScanSeg = kScanThreads * kScanPer;     // elements per block

__device__ __forceinline__ long long block_exclusive_scan(long long v, long long* sh, long long* total) {
    // exclusive scan of one value per thread over the block (kScanThreads threads); *total = block sum
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    long long incl = v;
#pragma unroll
    for (int off = 1; off < 32; off *= 2) {
        const long long up = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl += up;
    }
    if (lane == 31) sh[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        long long w = lane < kScanThreads / 32 ? sh[lane] : 0;
        long long wi = w;
#pragma unroll
        for (int off = 1; off < 32; off *= 2) {
            const long long up = __shfl_up_sync(0xffffffffu, wi, off);
            if (lane >= off) wi += up;
        }
        if (lane < kScanThreads / 32) sh[lane] = wi - w;
        if (lane == kScanThreads / 32 - 1) sh[kScanThreads / 32] = wi;
    }
    __syncthreads();
    *total = sh[kScanThreads / 32];
    const long long res = sh[warp] + incl - v;
    __syncthreads();
    return res;
}

__global__ void __launch_bounds__(kScanThreads) scan_segment_sums_kernel(const int* __restrict__ data, long long n,
                                                                        long long* __restrict__ seg_sums) {
    __shared__ long long sh[kScanThreads / 32 + 1];
    const long long base = static_cast<long long>(blockIdx.x) * kScanSeg + static_cast<long long>(threadIdx.x) * kScanPer;
    long long s = 0;
#pragma unroll
    for (int u = 0; u < kScanPer; ++u)
        if (base + u < n) s += data[base + u];
    long long total;
    block_exclusive_scan(s, sh, &total);
    if (threadIdx.x == 0) seg_sums[blockIdx.x] = total;
}

// exclusive scan of the segment totals by one block (a few thousand values)
__global__ void __launch_bounds__(kScanThreads) scan_totals_kernel(long long* __restrict__ seg_sums, long long nseg) {
    __shared__ long long sh[kScanThreads / 32 + 1];
    long long carry = 0;
    for (long long b0 = 0; b0 < nseg; b0 += kScanThreads) {
        const long long i = b0 + threadIdx.x;
        const long long v = i < nseg ? seg_sums[i] : 0;
        long long total;
        const long long ex = block_exclusive_scan(v, sh, &total);
        if (i < nseg) seg_sums[i] = carry + ex;
        carry += total;
    }
}

__global__ void __launch_bounds__(kScanThreads) scan_apply_kernel(int* __restrict__ data, long long n,
                                                                 const long long* __restrict__ seg_offsets) {
    __shared__ long long sh[kScanThreads / 32 + 1];
    const long long base = static_cast<long long>(blockIdx.x) * kScanSeg + static_cast<long long>(threadIdx.x) * kScanPer;
    int v[kScanPer];
    long long s = 0;
#pragma unroll
    for (int u = 0; u < kScanPer; ++u) {
        v[u] = base + u < n ? data[base + u] : 0;
        s += v[u];
    }
    long long total;
    long long run = seg_offsets[blockIdx.x] + block_exclusive_scan(s, sh, &total);
#pragma unroll
    for (int u = 0; u < kScanPer; ++u) {
        if (base + u < n) data[base + u] = static_cast<int>(run);
        run += v[u];
    }
}

// The same scan by one block, for short arrays (the self-check export's N + 1 row totals).
__global__ void small_exclusive_scan_kernel(int* __restrict__ data, long long n) {
    __shared__ long long sums[1024];
    const int t = threadIdx.x;
    const long long chunk = (n + blockDim.x - 1) / blockDim.x;
    const long long lo = min(n, t * chunk), hi = min(n, lo + chunk);
    long long s = 0;
    for (long long e = lo; e < hi; ++e) s += data[e];
    sums[t] = s;
    __syncthreads();
    if (t == 0) {
        long long run = 0;
        for (int j = 0; j < blockDim.x; ++j) {
            long long v = sums[j];
            sums[j] = run;
            run += v;
        }
    }
    __syncthreads();
    long long run = sums[t];
    for (long long e = lo; e < hi; ++e) {
        int v = data[e];
        data[e] = static_cast<int>(run);
        run += v;
    }
}

// `seg_scratch` holds ceil(n / kScanSeg) int64 values.
int launch_exclusive_scan(int* data, long long n, long long* seg_scratch, cudaStream_t stream) {
    const long long nseg = ceil_div(n, kScanSeg);
    scan_segment_sums_kernel<<<static_cast<unsigned>(nseg), kScanThreads, 0, stream>>>(data, n, seg_scratch);
    scan_totals_kernel<<<1, kScanThreads, 0, stream>>>(seg_scratch, nseg);
    scan_apply_kernel<<<static_cast<unsigned>(nseg), kScanThreads, 0, stream>>>(data, n, seg_scratch);
    FFI_LAUNCH_CHECK("exclusive scan");
    return FFI_OK;
}

// Stable scatter of one digit pass. vals_in == nullptr means "value = element index".
__global__ void radix_scatter_kernel(const int* __restrict__ keys_in, const int* __restrict__ vals_in,
                                     int* __restrict__ keys_out, int* __restrict__ vals_out,
                                     long long n, int shift, const int* __restrict__ offsets,
                                     long long nTiles) {
    __shared__ int base[kSortWarps][256];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long long tile = static_cast<long long>(blockIdx.x) * kSortWarps + warp;
    if (tile >= nTiles) return;
    for (int d = lane; d < 256; d += 32) base[warp][d] = offsets[static_cast<long long>(d) * nTiles + tile];
    __syncwarp();
    const long long first = tile * kTile;
    const unsigned lt = (1u << lane) - 1u;
    for (int r = 0; r < kTile / 32; ++r) {
        const long long e = first + r * 32 + lane;
        const bool valid = e < n;
        const unsigned active = __ballot_sync(0xffffffffu, valid);
        if (valid) {
            const int key = keys_in[e];
            const int val = vals_in ? vals_in[e] : static_cast<int>(e);
            const int d = (key >> shift) & 255;
            const unsigned same = __match_any_sync(active, d);
            const int rank = __popc(same & lt);
            const int dst = base[warp][d] + rank;
            __syncwarp(active);
            if (rank == 0) base[warp][d] += __popc(same);
            keys_out[dst] = key;
            vals_out[dst] = val;
        }
        __syncwarp();
    }
}

// rowptr[i] = lower_bound(sorted_keys, i), i in [0, N].
__global__ void rowptr_kernel(const int* __restrict__ sorted_keys, long long n, int N,
                              int* __restrict__ rowptr) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i > N) return;
    long long lo = 0, hi = n;
    while (lo < hi) {
        long long mid = (lo + hi) >> 1;
        if (sorted_keys[mid] < i) lo = mid + 1;
        else hi = mid;
    }
    rowptr[i] = static_cast<int>(lo);
}

// lb[c][i] = first position e in row i of the canonical form with perm[e] >= c*T*K.
__global__ void chunk_bounds_kernel(const int* __restrict__ rowptr, const int* __restrict__ perm,
                                    int N, long long chunkEntries, long long nChunks,
                                    int* __restrict__ lb) {
    const long long id = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (id >= (nChunks + 1) * N) return;
    const long long c = id / N;
    const int i = static_cast<int>(id - c * N);
    const long long target = c * chunkEntries;
    int lo = rowptr[i], hi = rowptr[i + 1];
    while (lo < hi) {
        int mid = (lo + hi) >> 1;
        if (perm[mid] < target) lo = mid + 1;
        else hi = mid;
    }
    lb[id] = lo;
}

// One block per chunk: cptr[c][0..N] = exclusive scan over i of the run lengths, and the
// runs themselves are copied into cperm.
__global__ void chunk_fill_kernel(const int* __restrict__ perm, const int* __restrict__ lb, int N,
                                  long long chunkEntries, int* __restrict__ cptr,
                                  int* __restrict__ cperm) {
    extern __shared__ int run_off[];  // N + 1
    const long long c = blockIdx.x;
    const int* lb0 = lb + c * N;
    const int* lb1 = lb + (c + 1) * N;
    if (threadIdx.x == 0) {
        int run = 0;
        for (int i = 0; i < N; ++i) {
            run_off[i] = run;
            run += lb1[i] - lb0[i];
        }
        run_off[N] = run;
    }
    __syncthreads();
    for (int i = threadIdx.x; i <= N; i += blockDim.x) cptr[c * (N + 1) + i] = run_off[i];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    int* dst = cperm + c * chunkEntries;
    for (int i = warp; i < N; i += nwarps) {
        const int s = lb0[i], len = lb1[i] - s, off = run_off[i];
        for (int r = lane; r < len; r += 32) dst[off + r] = perm[s + r];
    }
}

// stats[j] = max over chunks c and slices s of (entries of chunk c whose input lies in
// [s*w, (s+1)*w)), w = 128 << j.  Integer max is order independent.
__global__ void slice_stats_kernel(const int* __restrict__ cptr, int N, long long nChunks, int* __restrict__ stats) {
    const long long c = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (c >= nChunks) return;
    const int* row = cptr + c * (N + 1);
    for (int j = 0; j < 4; ++j) {
        const int w = 128 << j;
        int best = 0;
        for (int lo = 0; lo < N; lo += w) best = max(best, row[min(N, lo + w)] - row[lo]);
        atomicMax(stats + j, best);
    }
}

// Self-check export: rebuild the canonical form from (cptr, cperm).
__global__ void chunked_row_totals_kernel(const int* __restrict__ cptr, int N, long long nChunks,
                                          int* __restrict__ totals) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i > N) return;
    if (i == N) {
        totals[N] = 0;
        return;
    }
    long long s = 0;
    for (long long c = 0; c < nChunks; ++c) s += cptr[c * (N + 1) + i + 1] - cptr[c * (N + 1) + i];
    totals[i] = static_cast<int>(s);
}

__global__ void chunked_gather_kernel(const int* __restrict__ cptr, const int* __restrict__ cperm,
                                      const int* __restrict__ rowptr, int N, long long nChunks,
                                      long long chunkEntries, int* __restrict__ perm_out) {
    const int lane = threadIdx.x & 31;
    const int i = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (i >= N) return;
    long long run = rowptr[i];
    for (long long c = 0; c < nChunks; ++c) {
        const int s = cptr[c * (N + 1) + i], len = cptr[c * (N + 1) + i + 1] - s;
        const int* src = cperm + c * chunkEntries + s;
        for (int r = lane; r < len; r += 32) perm_out[run + r] = src[r];
        run += len;
    }
}

int significant_bits(int64_t n) {
    int bits = 0;
    while ((static_cast<int64_t>(1) << bits) < n) ++bits;
    return bits < 1 ? 1 : bits;
}

struct DeviceBuffer {
    void* ptr = nullptr;
    ~DeviceBuffer() {
        if (ptr) cudaFree(ptr);
    }
    cudaError_t alloc(size_t bytes) { return cudaMalloc(&ptr, bytes ? bytes : 4); }
    template <class T>
    T* as() {
        return static_cast<T*>(ptr);
    }
};

}  // namespace

// Rows per chunk of the chunked lists: the grad_x kernel keeps, per chunk, a g tile of
// T x 128 floats and up to T*K staged (weight, row) pairs in shared memory.
int plan_chunk_rows(int64_t K) {
    const int64_t budget = 200 * 1024;
    int64_t T = budget / (512 + 8 * K);
    if (T > 256) T = 256;
    T = T / 8 * 8;
    return static_cast<int>(T);
}

constexpr int64_t kNarrowMaxN = 2048;  // inputs the register-accumulator grad_x kernel covers

}  // namespace ffi

using namespace ffi;

namespace ffi {
namespace {

constexpr size_t kScratchAlign = 256;
size_t scratch_up(size_t v) { return (v + kScratchAlign - 1) / kScratchAlign * kScratchAlign; }

// Geometry of a plan and the carving of its build scratch (one allocation).
struct PlanLayout {
    long long n, nTiles, scan_segs, nChunks, cptrBytes;
    int T;
    bool chunks;
    size_t off_kA, off_vA, off_kB, off_vB, off_counts, off_bad, off_segs, off_lb, off_stats, total;
};

PlanLayout plan_layout(int64_t L, int64_t K, int64_t N) {
    PlanLayout g;
    g.n = L * K;
    g.nTiles = ceil_div(g.n, kTile);
    g.scan_segs = ceil_div(256 * g.nTiles > N + 1 ? 256 * g.nTiles : N + 1, kScanSeg);
    g.T = plan_chunk_rows(K);
    g.nChunks = ceil_div(L, g.T > 0 ? g.T : 1);
    g.cptrBytes = g.nChunks * (N + 1) * 4;
    g.chunks = g.T >= 8 && N <= kNarrowMaxN && g.cptrBytes <= (512LL << 20) && static_cast<long long>(g.T) * K <= 65536;
    size_t off = 0;
    auto take = [&](size_t bytes) {
        const size_t at = off;
        off += scratch_up(bytes ? bytes : 4);
        return at;
    };
    g.off_kA = take(g.n * 4);
    g.off_vA = take(g.n * 4);
    g.off_kB = take(g.n * 4);
    g.off_vB = take(g.n * 4);
    g.off_counts = take(256 * g.nTiles * 4);
    g.off_bad = take(4);
    g.off_segs = take(g.scan_segs * 8);
    g.off_lb = take(g.chunks ? (g.nChunks + 1) * N * 4 : 4);
    g.off_stats = take(4 * sizeof(int));
    g.total = off;
    return g;
}

// Fills the (already allocated) arrays of `plan` from `idx`; `scratch` holds plan_layout(...).total bytes.
// Synchronises the stream (index validation, slice statistics).
int plan_build(ffi_plan* plan, const int32_t* idx, unsigned char* scratch, cudaStream_t stream) {
    const int64_t L = plan->L, K = plan->K, N = plan->N;
    const PlanLayout g = plan_layout(L, K, N);
    const long long n = g.n, nTiles = g.nTiles;
    int* kA = reinterpret_cast<int*>(scratch + g.off_kA);
    int* vA = reinterpret_cast<int*>(scratch + g.off_vA);
    int* kB = reinterpret_cast<int*>(scratch + g.off_kB);
    int* vB = reinterpret_cast<int*>(scratch + g.off_vB);
    int* counts = reinterpret_cast<int*>(scratch + g.off_counts);
    int* bad = reinterpret_cast<int*>(scratch + g.off_bad);
    long long* segs = reinterpret_cast<long long*>(scratch + g.off_segs);
    int* lb = reinterpret_cast<int*>(scratch + g.off_lb);
    int* stats = reinterpret_cast<int*>(scratch + g.off_stats);

    FFI_CUDA_CHECK(cudaMemsetAsync(bad, 0, 4, stream));
    validate_idx_kernel<<<1024, 256, 0, stream>>>(idx, n, static_cast<int>(N), bad);
    int h_bad = 0;
    FFI_CUDA_CHECK(cudaMemcpyAsync(&h_bad, bad, 4, cudaMemcpyDeviceToHost, stream));
    FFI_CUDA_CHECK(cudaStreamSynchronize(stream));
    if (h_bad) return fail(FFI_ERR_INDEX_RANGE, "idx holds a value outside [0, %lld)", (long long)N);

    const int passes = (significant_bits(N) + 7) / 8;
    const unsigned sortBlocks = static_cast<unsigned>(ceil_div(nTiles, kSortWarps));
    const int* kin = idx;
    const int* vin = nullptr;
    int* kout = kA;
    int* vout = vA;
    for (int pass = 0; pass < passes; ++pass) {
        const int shift = 8 * pass;
        radix_hist_kernel<<<sortBlocks, 32 * kSortWarps, 0, stream>>>(kin, n, shift, counts, nTiles);
        const int src = launch_exclusive_scan(counts, 256 * nTiles, segs, stream);
        if (src != FFI_OK) return src;
        radix_scatter_kernel<<<sortBlocks, 32 * kSortWarps, 0, stream>>>(kin, vin, kout, vout, n, shift, counts, nTiles);
        kin = kout;
        vin = vout;
        const bool toB = (kout == kA);
        kout = toB ? kB : kA;
        vout = toB ? vB : vA;
    }
    FFI_LAUNCH_CHECK("radix sort");
    rowptr_kernel<<<static_cast<unsigned>(ceil_div(N + 1, 256)), 256, 0, stream>>>(kin, n, static_cast<int>(N),
                                                                                   plan->rowptr);
    FFI_CUDA_CHECK(cudaMemcpyAsync(plan->perm, vin, n * 4, cudaMemcpyDeviceToDevice, stream));
    FFI_LAUNCH_CHECK("rowptr_kernel");

    // Chunked lists for the narrow-input grad_x kernel.
    if (g.chunks) {
        const long long chunkEntries = static_cast<long long>(g.T) * K;
        const long long nb = (g.nChunks + 1) * N;
        chunk_bounds_kernel<<<static_cast<unsigned>(ceil_div(nb, 256)), 256, 0, stream>>>(
            plan->rowptr, plan->perm, static_cast<int>(N), chunkEntries, g.nChunks, lb);
        chunk_fill_kernel<<<static_cast<unsigned>(g.nChunks), 256, (N + 1) * sizeof(int), stream>>>(
            plan->perm, lb, static_cast<int>(N), chunkEntries, plan->cptr, plan->cperm);
        FFI_LAUNCH_CHECK("chunk kernels");
        // slice statistics for the kernels that stage one slice of a chunk in shared memory
        FFI_CUDA_CHECK(cudaMemsetAsync(stats, 0, 4 * sizeof(int), stream));
        slice_stats_kernel<<<static_cast<unsigned>(ceil_div(g.nChunks, 256)), 256, 0, stream>>>(
            plan->cptr, static_cast<int>(N), g.nChunks, stats);
        FFI_LAUNCH_CHECK("slice_stats_kernel");
        FFI_CUDA_CHECK(cudaMemcpyAsync(plan->max_slice_entries, stats, 4 * sizeof(int), cudaMemcpyDeviceToHost, stream));
        plan->chunk_rows = g.T;
        plan->n_chunks = g.nChunks;
        plan->has_chunks = true;
    }
    FFI_CUDA_CHECK(cudaStreamSynchronize(stream));
    return FFI_OK;
}

}  // namespace
}  // namespace ffi

namespace ffi {
namespace {
__device__ int g_bounds_bad = 0;
std::atomic<int> g_debug_bounds{-1};  // -1: not decided yet (environment), 0: off, 1: on
}  // namespace

bool debug_bounds_enabled() {
    int v = g_debug_bounds.load();
    if (v < 0) {
        const char* e = std::getenv("FFI_DEBUG_BOUNDS");
        v = (e && e[0] != '\0' && e[0] != '0') ? 1 : 0;
        g_debug_bounds.store(v);
    }
    return v == 1;
}

int check_index_range(const int32_t* idx, int64_t n, int64_t N, cudaStream_t stream) {
    int zero = 0, h_bad = 0;
    FFI_CUDA_CHECK(cudaMemcpyToSymbolAsync(g_bounds_bad, &zero, sizeof(int), 0, cudaMemcpyHostToDevice, stream));
    int* bad = nullptr;
    FFI_CUDA_CHECK(cudaGetSymbolAddress(reinterpret_cast<void**>(&bad), g_bounds_bad));
    validate_idx_kernel<<<1024, 256, 0, stream>>>(idx, n, static_cast<int>(N), bad);
    FFI_LAUNCH_CHECK("validate_idx_kernel");
    FFI_CUDA_CHECK(cudaMemcpyAsync(&h_bad, bad, sizeof(int), cudaMemcpyDeviceToHost, stream));
    FFI_CUDA_CHECK(cudaStreamSynchronize(stream));
    if (h_bad) return fail(FFI_ERR_INDEX_RANGE, "debug bounds: idx holds a value outside [0, %lld)", (long long)N);
    return FFI_OK;
}
}  // namespace ffi

extern "C" int ffi_set_debug_bounds(int on) {
    ffi::g_debug_bounds.store(on ? 1 : 0);
    return FFI_OK;
}

extern "C" int ffi_plan_create(const int32_t* idx, int64_t L, int64_t K, int64_t N, void* stream_v,
                               ffi_plan** out_plan) {
    FFI_TRACE("ffi_plan_create");
    if (!out_plan) return fail(FFI_ERR_INVALID_ARGUMENT, "out_plan is NULL");
    *out_plan = nullptr;
    if (!idx) return fail(FFI_ERR_INVALID_ARGUMENT, "idx is NULL");
    if (L <= 0 || K <= 0 || N <= 0) return fail(FFI_ERR_INVALID_ARGUMENT, "L, K, N must be positive");
    if (N >= (1LL << 31) || L * K >= (1LL << 31) - kTile)
        return fail(FFI_ERR_UNSUPPORTED, "L*K=%lld (or N) does not fit 32-bit positions", (long long)(L * K));
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);

    // Owns the half-built plan: every early return below (the CUDA check macros included) frees
    // the plan and its device arrays; success hands it to the caller.
    struct PlanOwner {
        ffi_plan* p;
        ~PlanOwner() {
            if (p) ffi_plan_destroy(p);
        }
    } owner{new ffi_plan()};
    ffi_plan* plan = owner.p;
    plan->L = L;
    plan->K = K;
    plan->N = N;
    FFI_CUDA_CHECK(cudaGetDevice(&plan->device));
    const PlanLayout g = plan_layout(L, K, N);

    if (cudaMalloc(&plan->rowptr, (N + 1) * sizeof(int)) != cudaSuccess ||
        cudaMalloc(&plan->perm, g.n * sizeof(int)) != cudaSuccess) {
        cudaGetLastError();
        return fail(FFI_ERR_ALLOC, "cudaMalloc of the transposed index failed");
    }
    plan->device_bytes = (N + 1) * sizeof(int) + g.n * sizeof(int);
    if (g.chunks) {
        if (cudaMalloc(&plan->cptr, g.cptrBytes) != cudaSuccess || cudaMalloc(&plan->cperm, g.n * 4) != cudaSuccess) {
            cudaGetLastError();
            return fail(FFI_ERR_ALLOC, "cudaMalloc of the chunked index failed");
        }
        plan->device_bytes += g.cptrBytes + g.n * 4;
    }
    DeviceBuffer scratch;
    if (scratch.alloc(g.total) != cudaSuccess) {
        cudaGetLastError();
        return fail(FFI_ERR_ALLOC, "cudaMalloc of sort scratch failed");
    }
    const int rc = plan_build(plan, idx, scratch.as<unsigned char>(), stream);
    if (rc != FFI_OK) return rc;
    owner.p = nullptr;
    *out_plan = plan;
    return FFI_OK;
}

extern "C" int ffi_plan_rebuild(ffi_plan* plan, const int32_t* idx, void* stream_v) {
    FFI_TRACE("ffi_plan_rebuild");
    if (!plan || !idx) return fail(FFI_ERR_INVALID_ARGUMENT, "NULL argument to ffi_plan_rebuild");
    int rc = check_plan_device(plan);
    if (rc != FFI_OK) return rc;
    const PlanLayout g = plan_layout(plan->L, plan->K, plan->N);
    if (!plan->build_scratch) {
        if (cudaMalloc(&plan->build_scratch, g.total) != cudaSuccess) {
            cudaGetLastError();
            plan->build_scratch = nullptr;
            return fail(FFI_ERR_ALLOC, "cudaMalloc of the plan's sort scratch failed");
        }
        plan->device_bytes += g.total;
    }
    return plan_build(plan, idx, static_cast<unsigned char*>(plan->build_scratch), static_cast<cudaStream_t>(stream_v));
}

extern "C" int ffi_plan_destroy(ffi_plan* plan) {
    if (!plan) return FFI_OK;
    if (plan->rowptr) cudaFree(plan->rowptr);
    if (plan->perm) cudaFree(plan->perm);
    if (plan->cperm) cudaFree(plan->cperm);
    if (plan->cptr) cudaFree(plan->cptr);
    if (plan->build_scratch) cudaFree(plan->build_scratch);
    delete plan;
    return FFI_OK;
}

extern "C" int ffi_plan_info(const ffi_plan* plan, int64_t* L, int64_t* K, int64_t* N, int64_t* chunk_rows,
                             int64_t* n_chunks, int64_t* device_bytes) {
    if (!plan) return fail(FFI_ERR_INVALID_ARGUMENT, "plan is NULL");
    if (L) *L = plan->L;
    if (K) *K = plan->K;
    if (N) *N = plan->N;
    if (chunk_rows) *chunk_rows = plan->has_chunks ? plan->chunk_rows : 0;
    if (n_chunks) *n_chunks = plan->has_chunks ? plan->n_chunks : 0;
    if (device_bytes) *device_bytes = static_cast<int64_t>(plan->device_bytes);
    return FFI_OK;
}

extern "C" int ffi_plan_export(const ffi_plan* plan, int32_t* rowptr, int32_t* perm, void* stream_v) {
    if (!plan || !rowptr || !perm) return fail(FFI_ERR_INVALID_ARGUMENT, "NULL argument to ffi_plan_export");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    FFI_CUDA_CHECK(cudaMemcpyAsync(rowptr, plan->rowptr, (plan->N + 1) * 4, cudaMemcpyDeviceToDevice, stream));
    FFI_CUDA_CHECK(cudaMemcpyAsync(perm, plan->perm, plan->L * plan->K * 4, cudaMemcpyDeviceToDevice, stream));
    return FFI_OK;
}

extern "C" int ffi_plan_export_chunked(const ffi_plan* plan, int32_t* rowptr, int32_t* perm, void* stream_v) {
    if (!plan || !rowptr || !perm)
        return fail(FFI_ERR_INVALID_ARGUMENT, "NULL argument to ffi_plan_export_chunked");
    if (!plan->has_chunks) return fail(FFI_ERR_UNSUPPORTED, "plan has no chunked lists (wide N)");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    const int N = static_cast<int>(plan->N);
    chunked_row_totals_kernel<<<static_cast<unsigned>(ceil_div(N + 1, 256)), 256, 0, stream>>>(
        plan->cptr, N, plan->n_chunks, rowptr);
    small_exclusive_scan_kernel<<<1, 1024, 0, stream>>>(rowptr, N + 1);
    chunked_gather_kernel<<<static_cast<unsigned>(ceil_div(N, 4)), 128, 0, stream>>>(
        plan->cptr, plan->cperm, rowptr, N, plan->n_chunks,
        static_cast<long long>(plan->chunk_rows) * plan->K, perm);
    FFI_LAUNCH_CHECK("chunked export");
    return FFI_OK;
}
