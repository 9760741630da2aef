// TEST INFRASTRUCTURE ONLY (part of the parity oracle; never linked into the product).
//
// Stand-in for TensorFlow's op_kernel.h so that the reference's CPU kernel sources
// (tfsparse/cc/kernels/forward.cpp and backward.cpp) compile unchanged without a
// TensorFlow installation.  Those two files only need the `tensorflow` namespace to
// exist (tfsparse/cc/kernels/common.h:12 has `using namespace tensorflow;`).
#pragma once
#include <cstdint>
#include <type_traits>
namespace tensorflow {}
