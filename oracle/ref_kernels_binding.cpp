// Binding for the reference's own elementwise CUDA kernels, compiled for sm_100a from the sources
// where they lie in the reference checkout (csrc/multi_pointwise.cu, csrc/multi_pad_fusion.cu).
// It exists so that GPU parity tests can compare this repository's kernels byte-for-byte with the
// reference's kernels running on the same B200.  It replaces the reference's csrc/ops.cu:9-16
// (which also binds the Hopper-only CUTLASS GEMM that cannot be built for sm_100a).
// TEST INFRASTRUCTURE ONLY: built into oracle/_ref/, never imported by the product package.
#include <torch/extension.h>

#include "multi_pad_fusion.h"
#include "multi_pointwise.h"

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("multi_quantize", &fp8_gmm::MultiQuantize);
  m.def("multi_scale_mul", &fp8_gmm::MultiScaleMul);
  m.def("multi_pad_transpose", &fp8_gmm::MultiPadTranspose);
  m.def("multi_pad_cast_transpose", &fp8_gmm::MultiPadCastTranspose);
  m.def("multi_pad_cast_transpose_dgelu", &fp8_gmm::MultiPadCastTransposeDgelu);
}
