// Shared device/host helpers for the fp8_gmm_b200 kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/fp8_gmm_b200.h"

namespace fp8gmm {

// ---- host-side error plumbing ---------------------------------------------------------------
void set_error(const char* fmt, ...);
int cuda_fail(cudaError_t err, const char* what);
int sm_count();              // SMs of the current device (cached per device)
int* device_status_word();   // device address of the per-device status word (kernels report timeouts here)
void count_launch();         // bumps the process-wide launch counter (fp8gmm_launch_count)
unsigned long long gemm_wait_limit_ns();  // limit of the GEMM kernels' mbarrier waits (fp8gmm_set_wait_limits)
unsigned long long peer_wait_limit_ns();  // limit of fp8gmm_peer_wait's spin on the sequence numbers

#define FP8GMM_CHECK_ARG(cond, ...)       \
  do {                                    \
    if (!(cond)) {                        \
      ::fp8gmm::set_error(__VA_ARGS__);   \
      return FP8GMM_INVALID_ARGUMENT;     \
    }                                     \
  } while (0)

#define FP8GMM_CHECK_CUDA(expr)                                        \
  do {                                                                 \
    cudaError_t err__ = (expr);                                        \
    if (err__ != cudaSuccess) return ::fp8gmm::cuda_fail(err__, #expr); \
  } while (0)

// ---- device helpers --------------------------------------------------------------------------
#ifdef __CUDACC__

// Two fp32 -> two fp8 bytes packed in 16 bits (lo in bits 0-7), round-to-nearest-even, saturating to
// the largest finite value: the same instruction the toolkit's __nv_fp8_e4m3/__nv_fp8_e5m2
// constructors use on the device, which is what the reference's `OType(x)` compiles to.
template <int kFormat>
__device__ __forceinline__ uint32_t cvt_fp8x2(float lo, float hi) {
  uint16_t r;
  if constexpr (kFormat == FP8GMM_E4M3) {
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  } else {
    asm("cvt.rn.satfinite.e5m2x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  }
  return r;
}

template <int kFormat>
__device__ __forceinline__ uint32_t cvt_fp8x4(float a, float b, float c, float d) {
  return cvt_fp8x2<kFormat>(a, b) | (cvt_fp8x2<kFormat>(c, d) << 16);
}

__device__ __forceinline__ float bf16_lo(uint32_t packed) { return __uint_as_float(packed << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t packed) { return __uint_as_float(packed & 0xFFFF0000u); }

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
  return v;
}

// max-merge of a non-negative float through integer atomicMax (exact and order independent).
__device__ __forceinline__ void atomic_max_nonneg(float* addr, float v) {
  atomicMax(reinterpret_cast<int*>(addr), __float_as_int(v));
}

// Streaming 16-byte / 8-byte global accesses (data is touched once: keep it out of L1).
__device__ __forceinline__ uint4 ld_stream16(const void* p) { return __ldcs(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ uint2 ld_stream8(const void* p) { return __ldcs(reinterpret_cast<const uint2*>(p)); }
__device__ __forceinline__ void st_stream16(void* p, uint4 v) { __stcs(reinterpret_cast<uint4*>(p), v); }
__device__ __forceinline__ void st_stream8(void* p, uint2 v) { __stcs(reinterpret_cast<uint2*>(p), v); }

// Largest t in [0, n) with table[t] <= x, for a non-decreasing table with table[0] <= x < table[n].
__device__ __forceinline__ int upper_slot(const int* table, int n, int x) {
  int lo = 0, hi = n;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (table[mid] <= x) lo = mid; else hi = mid;
  }
  return lo;
}

#endif  // __CUDACC__

}  // namespace fp8gmm
