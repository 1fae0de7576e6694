// Multi-tensor streaming kernels: bf16 -> fp8 quantise + amax, and the in-place two-scale multiply.
//
// HBM-bound: 3 bytes per element for quantise (2 read + 1 written), 4 for scale-mul.  One launch
// covers up to kMaxTensors tensors; the descriptor table travels in the kernel parameter block, a
// block finds its tensor by binary search over a tile prefix-sum, and every tensor is cut into
// tiles of kTileElems elements so that work is balanced by bytes rather than by tensor.
// Semantics follow reference csrc/multi_pointwise.cu:34-97 (quantise) and :99-151 (scale-mul);
// compiled with --use_fast_math like the reference (setup.py:21) so flush-to-zero behaviour matches.
#include <vector>

#include "common.cuh"

namespace fp8gmm {
namespace {

constexpr int kThreads = 256;
constexpr int kElemsPerThread = 32;
constexpr int kTileElems = kThreads * kElemsPerThread;  // 8192 elements = 16 KiB of bf16
constexpr int kMaxTensors = 320;

struct QuantDesc {
  const uint16_t* in;
  uint8_t* out;
  const float* scale;
  float* amax;
  int64_t numel;
};

struct QuantArgs {
  int num;
  int tile_start[kMaxTensors + 1];
  QuantDesc d[kMaxTensors];
};

struct ScaleMulDesc {
  uint16_t* data;
  const float* s1;
  const float* s2;
  int64_t numel;
};

struct ScaleMulArgs {
  int num;
  int tile_start[kMaxTensors + 1];
  ScaleMulDesc d[kMaxTensors];
};

template <int kFormat>
__global__ void __launch_bounds__(kThreads) multi_quantize_kernel(const __grid_constant__ QuantArgs args) {
  const int tile = blockIdx.x;
  const int t = upper_slot(args.tile_start, args.num, tile);
  const QuantDesc& d = args.d[t];
  const int64_t base = static_cast<int64_t>(tile - args.tile_start[t]) * kTileElems;
  const float scale = d.scale ? *d.scale : 1.0f;
  const int tid = threadIdx.x;
  float amax = 0.f;

  const bool full = base + kTileElems <= d.numel;
  const bool aligned = ((reinterpret_cast<uintptr_t>(d.in) | reinterpret_cast<uintptr_t>(d.out)) & 15) == 0;
  if (full && aligned) {
    // Two chunks of 16 elements per thread; a warp reads 1 KiB contiguous and writes 512 B contiguous.
    uint4 v[2][2];
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      const uint16_t* p = d.in + base + (c * kThreads + tid) * 16;
      v[c][0] = ld_stream16(p);
      v[c][1] = ld_stream16(p + 8);
    }
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      uint32_t w[8] = {v[c][0].x, v[c][0].y, v[c][0].z, v[c][0].w, v[c][1].x, v[c][1].y, v[c][1].z, v[c][1].w};
      uint32_t q[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float a = bf16_lo(w[2 * i]), b = bf16_hi(w[2 * i]), c2 = bf16_lo(w[2 * i + 1]), e = bf16_hi(w[2 * i + 1]);
        amax = fmaxf(fmaxf(fabsf(a), fabsf(b)), fmaxf(fmaxf(fabsf(c2), fabsf(e)), amax));
        q[i] = cvt_fp8x4<kFormat>(a * scale, b * scale, c2 * scale, e * scale);
      }
      if (d.out) st_stream16(d.out + base + (c * kThreads + tid) * 16, make_uint4(q[0], q[1], q[2], q[3]));
    }
  } else {
    for (int i = 0; i < kElemsPerThread; ++i) {
      const int64_t idx = base + i * kThreads + tid;
      if (idx < d.numel) {
        const float a = __uint_as_float(static_cast<uint32_t>(d.in[idx]) << 16);
        amax = fmaxf(fabsf(a), amax);
        if (d.out) d.out[idx] = static_cast<uint8_t>(cvt_fp8x2<kFormat>(a * scale, 0.f) & 0xFF);
      }
    }
  }

  if (d.amax) {
    __shared__ float staging[kThreads / 32];
    amax = warp_max(amax);
    if ((tid & 31) == 0) staging[tid >> 5] = amax;
    __syncthreads();
    if (tid < 32) {
      float m = tid < kThreads / 32 ? staging[tid] : 0.f;
      m = warp_max(m);
      if (tid == 0) atomic_max_nonneg(d.amax, m);
    }
  }
}

__global__ void __launch_bounds__(kThreads) multi_scale_mul_kernel(const __grid_constant__ ScaleMulArgs args) {
  const int tile = blockIdx.x;
  const int t = upper_slot(args.tile_start, args.num, tile);
  const ScaleMulDesc& d = args.d[t];
  const int64_t base = static_cast<int64_t>(tile - args.tile_start[t]) * kTileElems;
  const float s1 = d.s1 ? *d.s1 : 1.0f;
  const float s2 = d.s2 ? *d.s2 : 1.0f;
  const int tid = threadIdx.x;
  const bool full = base + kTileElems <= d.numel;
  const bool aligned = (reinterpret_cast<uintptr_t>(d.data) & 15) == 0;
  if (full && aligned) {
    uint4 v[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) v[c] = *reinterpret_cast<const uint4*>(d.data + base + (c * kThreads + tid) * 8);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t w[4] = {v[c].x, v[c].y, v[c].z, v[c].w};
#pragma unroll
      for (int i = 0; i < 4; ++i) w[i] = pack_bf16x2(bf16_lo(w[i]) * s1 * s2, bf16_hi(w[i]) * s1 * s2);
      *reinterpret_cast<uint4*>(d.data + base + (c * kThreads + tid) * 8) = make_uint4(w[0], w[1], w[2], w[3]);
    }
  } else {
    for (int i = 0; i < kElemsPerThread; ++i) {
      const int64_t idx = base + i * kThreads + tid;
      if (idx < d.numel) {
        const float a = __uint_as_float(static_cast<uint32_t>(d.data[idx]) << 16);
        const __nv_bfloat16 r = __float2bfloat16_rn(a * s1 * s2);
        d.data[idx] = *reinterpret_cast<const uint16_t*>(&r);
      }
    }
  }
}

}  // namespace
}  // namespace fp8gmm

extern "C" {

int fp8gmm_multi_quantize(const fp8gmm_tensor_desc* descs, int count, int out_format, void* stream) {
  using namespace fp8gmm;
  FP8GMM_CHECK_ARG(count >= 0 && (count == 0 || descs != nullptr), "multi_quantize: bad descriptor list");
  FP8GMM_CHECK_ARG(out_format == FP8GMM_E4M3 || out_format == FP8GMM_E5M2, "multi_quantize: bad fp8 format %d",
                   out_format);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  QuantArgs args;
  int i = 0;
  while (i < count) {
    args.num = 0;
    args.tile_start[0] = 0;
    for (; i < count && args.num < kMaxTensors; ++i) {
      const fp8gmm_tensor_desc& t = descs[i];
      FP8GMM_CHECK_ARG(t.rows >= 0 && t.cols >= 0, "multi_quantize: tensor %d has a negative size", i);
      const int64_t numel = t.rows * t.cols;
      if (numel == 0) continue;
      FP8GMM_CHECK_ARG(t.in != nullptr, "multi_quantize: tensor %d has a NULL input", i);
      const int64_t tiles = (numel + kTileElems - 1) / kTileElems;
      if (tiles + args.tile_start[args.num] > INT32_MAX) break;  // start a new launch
      QuantDesc& q = args.d[args.num];
      q.in = static_cast<const uint16_t*>(t.in);
      q.out = static_cast<uint8_t*>(t.out);
      q.scale = t.scale;
      q.amax = t.amax;
      q.numel = numel;
      args.tile_start[args.num + 1] = args.tile_start[args.num] + static_cast<int>(tiles);
      ++args.num;
    }
    if (args.num == 0) {
      FP8GMM_CHECK_ARG(i >= count, "multi_quantize: tensor %d is too large for one launch", i);
      continue;
    }
    const int grid = args.tile_start[args.num];
    if (out_format == FP8GMM_E4M3)
      multi_quantize_kernel<FP8GMM_E4M3><<<grid, kThreads, 0, s>>>(args);
    else
      multi_quantize_kernel<FP8GMM_E5M2><<<grid, kThreads, 0, s>>>(args);
    FP8GMM_CHECK_CUDA(cudaGetLastError());
    count_launch();
  }
  return FP8GMM_OK;
}

int fp8gmm_multi_scale_mul(const fp8gmm_scale_mul_desc* descs, int count, void* stream) {
  using namespace fp8gmm;
  FP8GMM_CHECK_ARG(count >= 0 && (count == 0 || descs != nullptr), "multi_scale_mul: bad descriptor list");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  ScaleMulArgs args;
  int i = 0;
  while (i < count) {
    args.num = 0;
    args.tile_start[0] = 0;
    for (; i < count && args.num < kMaxTensors; ++i) {
      const fp8gmm_scale_mul_desc& t = descs[i];
      FP8GMM_CHECK_ARG(t.numel >= 0, "multi_scale_mul: tensor %d has a negative size", i);
      if (t.numel == 0) continue;
      FP8GMM_CHECK_ARG(t.data != nullptr, "multi_scale_mul: tensor %d has a NULL pointer", i);
      const int64_t tiles = (t.numel + kTileElems - 1) / kTileElems;
      if (tiles + args.tile_start[args.num] > INT32_MAX) break;
      ScaleMulDesc& q = args.d[args.num];
      q.data = static_cast<uint16_t*>(t.data);
      q.s1 = t.scale1;
      q.s2 = t.scale2;
      q.numel = t.numel;
      args.tile_start[args.num + 1] = args.tile_start[args.num] + static_cast<int>(tiles);
      ++args.num;
    }
    if (args.num == 0) {
      FP8GMM_CHECK_ARG(i >= count, "multi_scale_mul: tensor %d is too large for one launch", i);
      continue;
    }
    multi_scale_mul_kernel<<<args.tile_start[args.num], kThreads, 0, s>>>(args);
    FP8GMM_CHECK_CUDA(cudaGetLastError());
    count_launch();
  }
  return FP8GMM_OK;
}

}  // extern "C"
