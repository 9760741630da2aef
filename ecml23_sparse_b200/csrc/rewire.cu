// One rewiring step of the fixed-fan-in layer, on the device.
//
// Replaces the TensorFlow graph the reference runs every `rewire_interval` steps:
//   * FixedFractionSelector.select (sparse/layer.py:62-86): threshold = the num_selected-th
//     smallest |w| over all L*K weights (tf.nn.top_k of -|w|), selected = |w| < threshold, strictly;
//   * StratifiedRewireLayerV2._rewire (sparse/custom_layer.py:32-43): every selected connection gets
//     a new source drawn uniformly from [0, n_in); its weight is kept;
//   * _update_sparse_kernel / SparseAdam.update_sparse (custom_layer.py:20-30, sparse/optimizer.py:14-23):
//     the Adam moments m and v are zeroed at the selected positions.
//
// The k-th smallest |w| is found by a radix select over the fp32 bit patterns (|w| >= 0, so the order
// of the values is the order of their bits with the sign cleared): four passes, most significant byte
// first; each pass histograms the byte of the elements that match the prefix found so far (integer
// atomics: order independent) and one small block picks the bin that holds the k-th element.  No host
// round trip: prefix and remaining rank live in the caller's workspace.  The new sources come from a
// counter-based hash of (seed, position), so a step is reproducible and can be restated on the host
// bit for bit.
#include "ffi_common.cuh"

namespace ffi {
namespace {

struct SelectState {
    unsigned prefix;      // bits of the k-th smallest |w| found so far (high bytes)
    unsigned remaining;   // rank of the wanted element among those that match the prefix (1-based)
    unsigned count;       // number of rewired positions (output of the apply kernel)
    unsigned pad;
    unsigned hist[4][256];
};

__device__ __forceinline__ unsigned abs_bits(float w) { return __float_as_uint(w) & 0x7fffffffu; }

__global__ void rewire_init_kernel(SelectState* st, unsigned k) {
    for (int i = threadIdx.x; i < 4 * 256; i += blockDim.x) st->hist[i / 256][i % 256] = 0u;
    if (threadIdx.x == 0) {
        st->prefix = 0u;
        st->remaining = k;
        st->count = 0u;
    }
}

// pass p looks at byte (3 - p) of the elements whose higher bytes equal the prefix
__global__ void __launch_bounds__(256) rewire_hist_kernel(const float* __restrict__ w, long long n, int pass,
                                                          SelectState* st) {
    __shared__ unsigned h[256];
    h[threadIdx.x] = 0u;
    __syncthreads();
    const int shift = 24 - 8 * pass;
    const unsigned prefix = st->prefix;
    const unsigned mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long e = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; e < n; e += stride) {
        const unsigned b = abs_bits(w[e]);
        if ((b & mask) == prefix) atomicAdd(&h[(b >> shift) & 255u], 1u);
    }
    __syncthreads();
    if (h[threadIdx.x]) atomicAdd(&st->hist[pass][threadIdx.x], h[threadIdx.x]);
}

__global__ void rewire_pick_kernel(SelectState* st, int pass) {
    if (threadIdx.x != 0) return;
    const int shift = 24 - 8 * pass;
    unsigned rem = st->remaining, run = 0u;
    int d = 0;
    for (; d < 255; ++d) {
        const unsigned c = st->hist[pass][d];
        if (run + c >= rem) break;
        run += c;
    }
    st->prefix |= static_cast<unsigned>(d) << shift;
    st->remaining = rem - run;
}

// splitmix64 finaliser over (seed, position): the generator of the package's seeded inputs
__device__ __forceinline__ unsigned long long hash64(unsigned long long base, unsigned long long counter) {
    unsigned long long z = counter * 0x9E3779B97F4A7C15ull + base;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

__global__ void __launch_bounds__(256) rewire_apply_kernel(const float* __restrict__ w, int* __restrict__ idx,
                                                           float* __restrict__ m, float* __restrict__ v, long long n,
                                                           unsigned n_in, unsigned long long base, SelectState* st,
                                                           float* __restrict__ threshold_out) {
    const unsigned thr = st->prefix;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    unsigned local = 0u;
    for (long long e = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; e < n; e += stride) {
        if (abs_bits(w[e]) < thr) {
            idx[e] = static_cast<int>((hash64(base, static_cast<unsigned long long>(e)) >> 1) % n_in);
            if (m) m[e] = 0.f;
            if (v) v[e] = 0.f;
            ++local;
        }
    }
#pragma unroll
    for (int off = 16; off >= 1; off /= 2) local += __shfl_xor_sync(0xffffffffu, local, off);
    if ((threadIdx.x & 31) == 0 && local) atomicAdd(&st->count, local);
    if (blockIdx.x == 0 && threadIdx.x == 0 && threshold_out) *threshold_out = __uint_as_float(thr);
}

__global__ void rewire_finish_kernel(const SelectState* st, int* count_out) {
    if (threadIdx.x == 0 && count_out) *count_out = static_cast<int>(st->count);
}

}  // namespace
}  // namespace ffi

using namespace ffi;

extern "C" size_t ffi_rewire_workspace_bytes(void) { return sizeof(SelectState); }

extern "C" int ffi_rewire(const float* w, int32_t* idx, float* m, float* v, int64_t n, int64_t n_in,
                          int64_t num_selected, uint64_t seed, float* threshold_out, int32_t* count_out,
                          void* workspace, size_t workspace_bytes, void* stream_v) {
    FFI_TRACE("ffi_rewire");
    if (!w || !idx) return fail(FFI_ERR_INVALID_ARGUMENT, "NULL tensor passed to ffi_rewire");
    if ((m == nullptr) != (v == nullptr)) return fail(FFI_ERR_INVALID_ARGUMENT, "m and v must both be given or both be NULL");
    if (n <= 0 || n >= (1LL << 31) || n_in <= 0 || n_in >= (1LL << 31))
        return fail(FFI_ERR_INVALID_ARGUMENT, "n and n_in must be positive and fit 31 bits");
    if (num_selected < 0 || num_selected > n)
        return fail(FFI_ERR_INVALID_ARGUMENT, "num_selected must lie in [0, n]");
    if (!workspace || workspace_bytes < sizeof(SelectState) || reinterpret_cast<uintptr_t>(workspace) % 16 != 0)
        return fail(FFI_ERR_WORKSPACE, "ffi_rewire needs %zu bytes of 16-byte aligned workspace", sizeof(SelectState));
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    SelectState* st = static_cast<SelectState*>(workspace);
    DeviceInfo dev;
    int rc = get_device_info(&dev);
    if (rc != FFI_OK) return rc;
    if (num_selected == 0) {  // nothing is below "the 0-th smallest": no connection moves
        if (threshold_out) FFI_CUDA_CHECK(cudaMemsetAsync(threshold_out, 0, sizeof(float), stream));
        if (count_out) FFI_CUDA_CHECK(cudaMemsetAsync(count_out, 0, sizeof(int), stream));
        return FFI_OK;
    }
    long long want = (n + 255) / 256;
    const unsigned blocks = static_cast<unsigned>(want < dev.sm_count * 8 ? want : dev.sm_count * 8);
    rewire_init_kernel<<<1, 256, 0, stream>>>(st, static_cast<unsigned>(num_selected));
    for (int pass = 0; pass < 4; ++pass) {
        rewire_hist_kernel<<<blocks, 256, 0, stream>>>(w, n, pass, st);
        rewire_pick_kernel<<<1, 32, 0, stream>>>(st, pass);
    }
    // base of the hash stream: as the package's generators derive it from (seed, stream 0)
    const unsigned long long base = static_cast<unsigned long long>(seed) * 0x632BE59BD9B4E019ull;
    rewire_apply_kernel<<<blocks, 256, 0, stream>>>(w, idx, m, v, n, static_cast<unsigned>(n_in), base, st, threshold_out);
    rewire_finish_kernel<<<1, 32, 0, stream>>>(st, count_out);
    FFI_LAUNCH_CHECK("rewire kernels");
    return FFI_OK;
}
