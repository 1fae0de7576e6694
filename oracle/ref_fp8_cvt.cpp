// Builds into oracle/_ref/: calls the CUDA toolkit's own host-side FP8 constructors, the very
// converter the reference's kernels invoke as `OType(scale * x)` (csrc/utils.cuh:11-12 aliases
// fp8e4m3/fp8e5m2 to __nv_fp8_e4m3/__nv_fp8_e5m2).  Used only to pin the oracle's converter.
#include <cuda_fp8.h>
#include <cstdint>

extern "C" void ref_fp8_cvt_array(const float* x, uint8_t* out, int64_t n, int format) {
  for (int64_t i = 0; i < n; ++i) {
    if (format == 0) {
      __nv_fp8_e4m3 v(x[i]);
      out[i] = v.__x;
    } else {
      __nv_fp8_e5m2 v(x[i]);
      out[i] = v.__x;
    }
  }
}
