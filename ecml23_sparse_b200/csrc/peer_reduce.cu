// One-shot sum of the per-GPU grad_x partials over peer memory (label-sharded layer, one process per GPU).
//
// The label dimension is sharded, so every GPU ends its backward with a partial grad_x of B*N floats
// (0.4 MB at the headline shape): a message small enough that a library all-reduce is pure latency.
// Here every rank leaves its partial in a buffer the other ranks can read (peer pointers of a
// symmetric allocation the caller made), raises a flag in each peer's flag array, waits until all
// ranks have raised theirs, and adds the world's partials itself, in rank order, so that every GPU
// gets the same bits.  One launch per step; no counterpart in the reference, which is single-GPU.
//
// Waiting on another GPU is bounded: a wait that lasts longer than about two seconds is counted
// (ffi_wait_timeouts) and the kernel goes on with whatever it finds, so a lost peer can never hang
// the device.  Flags carry the step number (monotonic), so nothing has to be reset; buffers are
// used alternately (step parity), so a fast rank cannot overwrite what a slow rank still reads: a
// rank writes slot p again two steps later, after it has seen every peer's flag of the step in
// between, which a peer raises only after it finished reading slot p.
#include "ffi_common.cuh"

namespace ffi {
namespace {

__device__ int g_peer_timeouts = 0;  // waits on other GPUs that gave up (added into ffi_wait_timeouts)
__device__ long long g_peer_wait_limit = 4000000000ll;  // clock64 ticks a wait may last (about two seconds)

constexpr int kMaxPeers = 16;

struct PeerParams {
    const float* bufs[kMaxPeers];   // peer r's buffer: [2][n] floats
    unsigned* flags[kMaxPeers];     // peer r's flags: [2][world] words, flags[r][p * world + s] = last step rank s finished
    float* out;
    long long n;
    int rank, world;
    unsigned step;
};

__device__ __forceinline__ unsigned load_flag(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void store_flag(unsigned* p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// out[i] = sum over ranks of their partial, in rank order; all WORLD loads of an element are issued before
// the first add, so one round trip over NVLink covers them all.
template <int WORLD>
__device__ __forceinline__ void add_partials(const PeerParams& p, int par) {
    const long long n4 = p.n / 4;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4; i += stride) {
        float4 v[WORLD];
#pragma unroll
        for (int r = 0; r < WORLD; ++r)
            v[r] = reinterpret_cast<const float4*>(p.bufs[r] + static_cast<size_t>(par) * p.n)[i];
        float4 s = v[0];
#pragma unroll
        for (int r = 1; r < WORLD; ++r) s.x += v[r].x, s.y += v[r].y, s.z += v[r].z, s.w += v[r].w;
        reinterpret_cast<float4*>(p.out)[i] = s;
    }
}

__global__ void __launch_bounds__(256) peer_sum_kernel(PeerParams p) {
    const int par = static_cast<int>(p.step & 1u);
    // 1. tell every rank (myself included) that my partial of this step is in place
    if (blockIdx.x == 0 && static_cast<int>(threadIdx.x) < p.world) {
        __threadfence_system();
        store_flag(p.flags[threadIdx.x] + par * p.world + p.rank, p.step);
    }
    // 2. wait (bounded) until every rank has said so in MY flag array
    if (static_cast<int>(threadIdx.x) < p.world) {
        const unsigned* f = p.flags[p.rank] + par * p.world + threadIdx.x;
        if (static_cast<int>(load_flag(f) - p.step) < 0) {
            const long long start = clock64();
            const long long limit = g_peer_wait_limit;
            while (static_cast<int>(load_flag(f) - p.step) < 0) {
                if (clock64() - start > limit) {
                    atomicAdd(&g_peer_timeouts, 1);
                    break;
                }
            }
        }
    }
    __syncthreads();
    // 3. add the partials in rank order (0 + v0 + v1 + ... with the first term exact: same bits as a running sum)
    switch (p.world) {
        case 1: add_partials<1>(p, par); break;
        case 2: add_partials<2>(p, par); break;
        case 4: add_partials<4>(p, par); break;
        case 8: add_partials<8>(p, par); break;
        default: {
            const long long n4 = p.n / 4;
            const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
            for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4; i += stride) {
                float4 s = reinterpret_cast<const float4*>(p.bufs[0] + static_cast<size_t>(par) * p.n)[i];
                for (int r = 1; r < p.world; ++r) {
                    const float4 v = reinterpret_cast<const float4*>(p.bufs[r] + static_cast<size_t>(par) * p.n)[i];
                    s.x += v.x, s.y += v.y, s.z += v.z, s.w += v.w;
                }
                reinterpret_cast<float4*>(p.out)[i] = s;
            }
        }
    }
}

}  // namespace

int peer_wait_timeouts(int* out) {
    FFI_CUDA_CHECK(cudaMemcpyFromSymbol(out, g_peer_timeouts, sizeof(int)));
    return FFI_OK;
}

int set_peer_wait_limit(long long ticks) {
    FFI_CUDA_CHECK(cudaMemcpyToSymbol(g_peer_wait_limit, &ticks, sizeof(ticks)));
    return FFI_OK;
}

}  // namespace ffi

using namespace ffi;

extern "C" int ffi_peer_sum(const void* const* peer_bufs, void* const* peer_flags, int rank, int world, int64_t n,
                            uint32_t step, float* out, void* stream_v) {
    FFI_TRACE("ffi_peer_sum");
    if (!peer_bufs || !peer_flags || !out) return fail(FFI_ERR_INVALID_ARGUMENT, "NULL argument passed to ffi_peer_sum");
    if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world)
        return fail(FFI_ERR_INVALID_ARGUMENT, "ffi_peer_sum supports 1..%d ranks", kMaxPeers);
    if (n <= 0 || n % 4 != 0) return fail(FFI_ERR_INVALID_ARGUMENT, "the element count must be a positive multiple of 4");
    if (step == 0) return fail(FFI_ERR_INVALID_ARGUMENT, "steps are numbered from 1 (flags start at 0)");
    PeerParams p;
    for (int r = 0; r < world; ++r) {
        if (!peer_bufs[r] || !peer_flags[r] || reinterpret_cast<uintptr_t>(peer_bufs[r]) % 16 != 0)
            return fail(FFI_ERR_INVALID_ARGUMENT, "peer buffer %d is NULL or not 16-byte aligned", r);
        p.bufs[r] = static_cast<const float*>(peer_bufs[r]);
        p.flags[r] = static_cast<unsigned*>(peer_flags[r]);
    }
    p.out = out;
    p.n = n;
    p.rank = rank;
    p.world = world;
    p.step = step;
    const long long n4 = n / 4;
    long long blocks = (n4 + 255) / 256;
    if (blocks > 128) blocks = 128;  // all blocks resident at once (fewer than SMs): none of them waits for another block
    peer_sum_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream_v)>>>(p);
    FFI_LAUNCH_CHECK("peer_sum_kernel");
    return FFI_OK;
}
