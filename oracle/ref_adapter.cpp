// TEST INFRASTRUCTURE ONLY (part of the parity oracle; never linked into the product).
//
// C entry points around the reference's own CPU functors.  This file is compiled
// together with the reference sources tfsparse/cc/kernels/forward.cpp and
// backward.cpp (taken from where they lie, not copied) against the stand-in headers
// in ref_shim/.  It plays the role of the reference's testing/cpu.cpp:34-39
// (`run_cpu_kernel`): build a thread-pool device, wrap raw buffers in MatrixType
// views, call the functor.
#include "common.h"

#include <cstdint>
#include <thread>

namespace {

template <bool Transposed>
void forward_impl(const float* features, const std::int32_t* lookup, const float* weights,
                  float* output, std::int64_t batch, std::int64_t n_in, std::int64_t units,
                  std::int64_t fan_in, int threads) {
    CPUDevice device(threads);
    MatrixType<const float> f(features, Transposed ? n_in : batch, Transposed ? batch : n_in);
    MatrixType<const std::int32_t> l(lookup, units, fan_in);
    MatrixType<const float> w(weights, units, fan_in);
    MatrixType<float> o(output, batch, units);
    FixedFanInSparseMatmulKernel<CPUDevice, float, std::int32_t, ForwardImplementations::CPU, Transposed> kernel;
    kernel(device, f, l, w, o);
}

template <bool Transposed>
void backward_impl(const float* features, const std::int32_t* lookup, const float* weights,
                   const float* out_grad, float* feature_grad, float* weight_grad,
                   std::int64_t batch, std::int64_t n_in, std::int64_t units, std::int64_t fan_in,
                   int threads) {
    CPUDevice device(threads);
    MatrixType<const float> f(features, Transposed ? n_in : batch, Transposed ? batch : n_in);
    MatrixType<const std::int32_t> l(lookup, units, fan_in);
    MatrixType<const float> w(weights, units, fan_in);
    MatrixType<const float> g(out_grad, batch, units);
    MatrixType<float> fg(feature_grad, Transposed ? n_in : batch, Transposed ? batch : n_in);
    MatrixType<float> wg(weight_grad, units, fan_in);
    FixedFanInSparseMatmulGradKernel<CPUDevice, float, std::int32_t, BackwardImplementations::CPU, Transposed> kernel;
    kernel(device, f, l, w, g, fg, wg);
}

int pick_threads(int threads) {
    if (threads > 0) return threads;
    unsigned hw = std::thread::hardware_concurrency();
    return hw == 0 ? 1 : static_cast<int>(hw);
}

}  // namespace

extern "C" {

// threads <= 0 means "all hardware threads", as testing/cpu.cpp:36-37 does.
void ref_forward(const float* features, const std::int32_t* lookup, const float* weights,
                 float* output, std::int64_t batch, std::int64_t n_in, std::int64_t units,
                 std::int64_t fan_in, int transposed, int threads) {
    threads = pick_threads(threads);
    if (transposed)
        forward_impl<true>(features, lookup, weights, output, batch, n_in, units, fan_in, threads);
    else
        forward_impl<false>(features, lookup, weights, output, batch, n_in, units, fan_in, threads);
}

void ref_backward(const float* features, const std::int32_t* lookup, const float* weights,
                  const float* out_grad, float* feature_grad, float* weight_grad,
                  std::int64_t batch, std::int64_t n_in, std::int64_t units, std::int64_t fan_in,
                  int transposed, int threads) {
    threads = pick_threads(threads);
    if (transposed)
        backward_impl<true>(features, lookup, weights, out_grad, feature_grad, weight_grad, batch, n_in,
                            units, fan_in, threads);
    else
        backward_impl<false>(features, lookup, weights, out_grad, feature_grad, weight_grad, batch, n_in,
                             units, fan_in, threads);
}

int ref_hardware_threads() { return pick_threads(0); }

}  // extern "C"
