// Router-side row permutation of an MoE block (HBM-bound, no tensor cores).
//
// The reference's example takes these steps from megablocks (fp8_gmm/example.py:26-32: sort + histogram +
// inclusive_cumsum; :52 / :87 / :118 gather; :59 / :92 / :121 scatter).  They sit on both sides of the grouped GEMMs:
// rows have to be sorted by expert before GroupedLinear / GroupedMlp see them and un-sorted (and mixed with the router
// weights) afterwards.  megablocks is not a dependency here, so the same contract is provided natively:
//   sort     top_expert (n = tokens * top_k int32 expert ids)  ->  indices (the stable argsort: indices[i] is the flat
//            (token, slot) position held by sorted row i), bin_ids (expert of sorted row i), bins (inclusive cumsum of
//            the histogram), tokens_per_expert (histogram), and the inverse permutation
//   gather   out[i] = x[indices[i] / top_k]                          (optionally scaled by weights[indices[i]])
//   scatter  out[t] = sum_k weights[t * top_k + k] * x[inverse[t * top_k + k]]     (fp32 accumulate, k ascending)
//   rowdot   d_weights[p] = <grad[p / top_k], x[inverse[p]]>         (gradient of scatter w.r.t. the router weights)
// The sort is a stable counting sort with one CTA per expert: every CTA scans the id list (at most a few hundred
// KB, L2 resident) and compacts the positions that carry its expert, so equal ids keep their order and the result
// does not depend on scheduling.
#include "common.cuh"

namespace fp8gmm {
namespace {

constexpr int kSortThreads = 1024;
constexpr int kStatusBadExpertId = 0x200;   // an expert id outside [0, num_experts), or a row index it left unset

// Number of entries equal to `expert`, one CTA per expert.
__global__ void __launch_bounds__(kSortThreads) moe_count_kernel(const int32_t* __restrict__ ids, int64_t n, int num_experts,
                                                                 int64_t* __restrict__ counts, int* __restrict__ status) {
  __shared__ int warp_sums[kSortThreads / 32];
  const int expert = blockIdx.x;
  int local = 0;
  bool bad = false;
  for (int64_t i = threadIdx.x; i < n; i += kSortThreads) {
    const int32_t id = ids[i];
    local += id == expert;
    bad |= id < 0 || id >= num_experts;
  }
  // Ids outside the range match no CTA, so their rows would stay unsorted: report them (the first CTA looks).
  if (expert == 0 && __syncthreads_or(bad) && threadIdx.x == 0) atomicOr(status, kStatusBadExpertId);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) local += __shfl_xor_sync(0xFFFFFFFFu, local, o);
  if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = local;
  __syncthreads();
  if (threadIdx.x < 32) {
    int v = warp_sums[threadIdx.x];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    if (threadIdx.x == 0) counts[expert] = v;
  }
}

// bins = inclusive cumsum of counts (one thread: the list has at most a few hundred entries).
__global__ void moe_bins_kernel(const int64_t* __restrict__ counts, int num_experts, int64_t* __restrict__ bins) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    int64_t run = 0;
    for (int e = 0; e < num_experts; ++e) {
      run += counts[e];
      bins[e] = run;
    }
  }
}

// Stable placement: CTA `expert` walks the id list in strips of kSortThreads and writes the positions that carry its
// expert to indices[start + rank], where rank counts earlier matches.
__global__ void __launch_bounds__(kSortThreads) moe_place_kernel(const int32_t* __restrict__ ids, int64_t n,
                                                                 const int64_t* __restrict__ bins, int32_t* __restrict__ indices,
                                                                 int32_t* __restrict__ bin_ids, int32_t* __restrict__ inverse) {
  __shared__ int warp_sums[kSortThreads / 32];
  __shared__ int strip_total;
  const int expert = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int64_t base = expert == 0 ? 0 : bins[expert - 1];
  for (int64_t i0 = 0; i0 < n; i0 += kSortThreads) {
    const int64_t i = i0 + threadIdx.x;
    const bool hit = i < n && ids[i] == expert;
    const unsigned ballot = __ballot_sync(0xFFFFFFFFu, hit);
    const int in_warp = __popc(ballot & ((1u << lane) - 1u));
    if (lane == 0) warp_sums[warp] = __popc(ballot);
    __syncthreads();
    if (warp == 0) {
      const int v = warp_sums[lane];
      int incl = v;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int up = __shfl_up_sync(0xFFFFFFFFu, incl, o);
        if (lane >= o) incl += up;
      }
      warp_sums[lane] = incl - v;  // exclusive prefix of the warp totals
      if (lane == 31) strip_total = incl;
    }
    __syncthreads();
    if (hit) {
      const int64_t dst = base + warp_sums[warp] + in_warp;
      indices[dst] = static_cast<int32_t>(i);
      bin_ids[dst] = expert;
      inverse[i] = static_cast<int32_t>(dst);
    }
    base += strip_total;
    __syncthreads();
  }
}

__device__ __forceinline__ void unpack8(uint4 v, float (&f)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) f[2 * j] = bf16_lo(w[j]), f[2 * j + 1] = bf16_hi(w[j]);
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  return make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
}
__device__ __forceinline__ float bf16_to_float(uint16_t v) { return __uint_as_float(static_cast<uint32_t>(v) << 16); }
__device__ __forceinline__ uint16_t float_to_bf16(float f) {
  const __nv_bfloat16 b = __float2bfloat16_rn(f);
  return *reinterpret_cast<const uint16_t*>(&b);
}

// out[r] = scale_r * x[indices[r] / top_k]; one thread per 16-byte chunk (kVec) or per element.
template <bool kVec>
__global__ void __launch_bounds__(256) moe_gather_kernel(const uint16_t* __restrict__ x, const int32_t* __restrict__ indices,
                                                         const float* __restrict__ weights, int top_k, int64_t rows, int64_t cols,
                                                         uint16_t* __restrict__ out, int* __restrict__ status) {
  const int64_t per_row = kVec ? cols / 8 : cols;
  const int64_t total = rows * per_row;
  for (int64_t id = blockIdx.x * 256ll + threadIdx.x; id < total; id += 256ll * gridDim.x) {
    const int64_t r = id / per_row, c = id - r * per_row;
    const int32_t slot = indices[r];
    if (slot < 0 || slot >= rows) {   // not a permutation entry (the sort saw an invalid expert id): skip, report
      if (c == 0) atomicOr(status, kStatusBadExpertId);
      continue;
    }
    const int64_t src = slot / top_k;
    if (kVec) {
      uint4 v = __ldg(reinterpret_cast<const uint4*>(x + src * cols) + c);
      if (weights != nullptr) {
        const float w = weights[slot];
        float f[8];
        unpack8(v, f);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] *= w;
        v = pack8(f);
      }
      st_stream16(reinterpret_cast<uint4*>(out + r * cols) + c, v);
    } else {
      const float w = weights != nullptr ? weights[slot] : 1.f;
      const uint16_t v = x[src * cols + c];
      out[r * cols + c] = weights != nullptr ? float_to_bf16(bf16_to_float(v) * w) : v;
    }
  }
}

// out[t] = sum_k weights[t * top_k + k] * x[inverse[t * top_k + k]], accumulated in fp32 with k ascending.
template <bool kVec>
__global__ void __launch_bounds__(256) moe_scatter_kernel(const uint16_t* __restrict__ x, const int32_t* __restrict__ inverse,
                                                          const float* __restrict__ weights, int top_k, int64_t tokens, int64_t cols,
                                                          uint16_t* __restrict__ out, int* __restrict__ status) {
  const int64_t per_row = kVec ? cols / 8 : cols;
  const int64_t total = tokens * per_row;
  const int64_t n_rows = tokens * top_k;
  for (int64_t id = blockIdx.x * 256ll + threadIdx.x; id < total; id += 256ll * gridDim.x) {
    const int64_t t = id / per_row, c = id - t * per_row;
    if (kVec) {
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
      for (int k = 0; k < top_k; ++k) {
        const int64_t p = t * top_k + k;
        const float w = weights != nullptr ? weights[p] : 1.f;
        const int64_t src = inverse[p];
        if (src < 0 || src >= n_rows) {   // position the sort never placed: contributes nothing, reported
          if (c == 0) atomicOr(status, kStatusBadExpertId);
          continue;
        }
        float f[8];
        unpack8(ld_stream16(reinterpret_cast<const uint4*>(x + src * cols) + c), f);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = fmaf(w, f[j], acc[j]);
      }
      *(reinterpret_cast<uint4*>(out + t * cols) + c) = pack8(acc);
    } else {
      float acc = 0.f;
      for (int k = 0; k < top_k; ++k) {
        const int64_t p = t * top_k + k;
        const float w = weights != nullptr ? weights[p] : 1.f;
        const int64_t src = inverse[p];
        if (src < 0 || src >= n_rows) {
          if (c == 0) atomicOr(status, kStatusBadExpertId);
          continue;
        }
        acc = fmaf(w, bf16_to_float(x[src * cols + c]), acc);
      }
      out[t * cols + c] = float_to_bf16(acc);
    }
  }
}

// d_weights[p] = <grad[p / top_k], x[inverse[p]]>, one warp per (token, slot) position.
__global__ void __launch_bounds__(256) moe_rowdot_kernel(const uint16_t* __restrict__ grad, const uint16_t* __restrict__ x,
                                                         const int32_t* __restrict__ inverse, int top_k, int64_t n, int64_t cols,
                                                         float* __restrict__ d_weights, int* __restrict__ status) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = (256ll * gridDim.x) >> 5;
  for (int64_t p = (blockIdx.x * 256ll + threadIdx.x) >> 5; p < n; p += warps) {
    const int64_t src = inverse[p];
    if (src < 0 || src >= n) {
      if (lane == 0) {
        atomicOr(status, kStatusBadExpertId);
        d_weights[p] = 0.f;
      }
      continue;
    }
    const uint16_t* g = grad + (p / top_k) * cols;
    const uint16_t* v = x + src * cols;
    float acc = 0.f;
    if (cols % 8 == 0 && (reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(v)) % 16 == 0) {
      for (int64_t c = lane; c < cols / 8; c += 32) {
        float a[8], b[8];
        unpack8(__ldg(reinterpret_cast<const uint4*>(g) + c), a);
        unpack8(ld_stream16(reinterpret_cast<const uint4*>(v) + c), b);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc = fmaf(a[j], b[j], acc);
      }
    } else {
      for (int64_t c = lane; c < cols; c += 32) acc = fmaf(bf16_to_float(g[c]), bf16_to_float(v[c]), acc);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, o);
    if (lane == 0) d_weights[p] = acc;
  }
}

// Router: softmax over the expert logits in fp32, then the top_k largest probabilities (descending; equal values
// keep the lower expert id first), optionally renormalised to sum to one (reference fp8_gmm/example.py:14-23).
// One warp per token; lane l holds experts l, l + 32, ...
constexpr int kTopkMaxPerLane = 32;   // up to 1024 experts
template <typename T>
__device__ __forceinline__ float logit_to_float(T v);
template <>
__device__ __forceinline__ float logit_to_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ float logit_to_float<uint16_t>(uint16_t v) { return bf16_to_float(v); }

template <typename T>
__global__ void __launch_bounds__(256) moe_topk_kernel(const T* __restrict__ logits, int64_t tokens, int num_experts, int top_k,
                                                       int renorm, float* __restrict__ probs, float* __restrict__ weights,
                                                       int32_t* __restrict__ experts) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = (256ll * gridDim.x) >> 5;
  for (int64_t t = (blockIdx.x * 256ll + threadIdx.x) >> 5; t < tokens; t += warps) {
    const T* row = logits + t * num_experts;
    float v[kTopkMaxPerLane];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < kTopkMaxPerLane; ++i) {
      const int e = lane + 32 * i;
      v[i] = e < num_experts ? logit_to_float<T>(row[e]) : -INFINITY;
      mx = fmaxf(mx, v[i]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < kTopkMaxPerLane; ++i) {
      v[i] = lane + 32 * i < num_experts ? expf(v[i] - mx) : 0.f;
      sum += v[i];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o);
#pragma unroll
    for (int i = 0; i < kTopkMaxPerLane; ++i) {
      v[i] = __fdiv_rn(v[i], sum);
      const int e = lane + 32 * i;
      if (probs != nullptr && e < num_experts) probs[t * num_experts + e] = v[i];
    }
    float picked_sum = 0.f;
    float my_weight = 0.f;   // lane r keeps the r-th pick until the renormalisation is known
    int my_expert = 0;
    for (int r = 0; r < top_k; ++r) {
      float best = -1.f;
      int best_e = INT32_MAX;
#pragma unroll
      for (int i = 0; i < kTopkMaxPerLane; ++i) {
        const int e = lane + 32 * i;
        if (e < num_experts && v[i] > best) best = v[i], best_e = e;   // ascending e: the first maximum wins
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xFFFFFFFFu, best, o);
        const int oe = __shfl_xor_sync(0xFFFFFFFFu, best_e, o);
        if (ob > best || (ob == best && oe < best_e)) best = ob, best_e = oe;
      }
      if ((best_e & 31) == lane) {
#pragma unroll
        for (int i = 0; i < kTopkMaxPerLane; ++i)
          if (i == (best_e >> 5)) v[i] = -2.f;   // taken
      }
      picked_sum += best;
      if (lane == (r & 31)) my_weight = best, my_expert = best_e;
      if ((r & 31) == 31 || r == top_k - 1) {
        // top_k may exceed 32: flush this batch of picks (renormalisation then needs a second pass, below)
        const int base = r & ~31;
        if (lane <= (r & 31)) {
          weights[t * top_k + base + lane] = my_weight;
          experts[t * top_k + base + lane] = my_expert;
        }
      }
    }
    if (renorm) {
      __syncwarp();
      for (int r = lane; r < top_k; r += 32) weights[t * top_k + r] = __fdiv_rn(weights[t * top_k + r], picked_sum);
    }
  }
}

int row_grid(int64_t work_items) {
  const int64_t blocks = (work_items + 255) / 256;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
  return static_cast<int>(blocks < 1 ? 1 : blocks < cap ? blocks : cap);
}

}  // namespace
}  // namespace fp8gmm

extern "C" {

int fp8gmm_moe_sort(const int32_t* expert_ids, int64_t n, int num_experts, int32_t* indices, int32_t* bin_ids,
                    int32_t* inverse, int64_t* bins, int64_t* tokens_per_expert, void* stream) {
  using namespace fp8gmm;
  FP8GMM_CHECK_ARG(n >= 0 && n <= INT32_MAX && num_experts > 0 && num_experts <= 65535, "moe_sort: bad sizes");
  FP8GMM_CHECK_ARG(bins != nullptr && tokens_per_expert != nullptr, "moe_sort: NULL histogram output");
  FP8GMM_CHECK_ARG(n == 0 || (expert_ids && indices && bin_ids && inverse), "moe_sort: NULL pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int* status = device_status_word();
  FP8GMM_CHECK_ARG(status != nullptr, "moe_sort: cannot resolve the device status word");
  if (n > 0) {
    // positions that no CTA places (ids out of range) keep -1, which the gather / scatter kernels recognise
    FP8GMM_CHECK_CUDA(cudaMemsetAsync(indices, 0xFF, static_cast<size_t>(n) * sizeof(int32_t), s));
    FP8GMM_CHECK_CUDA(cudaMemsetAsync(inverse, 0xFF, static_cast<size_t>(n) * sizeof(int32_t), s));
  }
  moe_count_kernel<<<num_experts, kSortThreads, 0, s>>>(expert_ids, n, num_experts, tokens_per_expert, status);
  moe_bins_kernel<<<1, 32, 0, s>>>(tokens_per_expert, num_experts, bins);
  if (n > 0) moe_place_kernel<<<num_experts, kSortThreads, 0, s>>>(expert_ids, n, bins, indices, bin_ids, inverse);
  FP8GMM_CHECK_CUDA(cudaGetLastError());
  count_launch();
  count_launch();
  if (n > 0) count_launch();
  return FP8GMM_OK;
}

int fp8gmm_moe_topk(const void* logits, int logits_are_bf16, int64_t tokens, int num_experts, int top_k, int renormalize,
                    float* probs, float* weights, int32_t* experts, void* stream) {
  using namespace fp8gmm;
  FP8GMM_CHECK_ARG(tokens >= 0 && num_experts > 0 && num_experts <= 32 * kTopkMaxPerLane, "moe_topk: num_experts must be in [1, %d]",
                   32 * kTopkMaxPerLane);
  FP8GMM_CHECK_ARG(top_k > 0 && top_k <= num_experts, "moe_topk: top_k must be in [1, num_experts]");
  if (tokens == 0) return FP8GMM_OK;
  FP8GMM_CHECK_ARG(logits && weights && experts, "moe_topk: NULL pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int grid = row_grid(tokens * 32);
  if (logits_are_bf16)
    moe_topk_kernel<uint16_t><<<grid, 256, 0, s>>>(static_cast<const uint16_t*>(logits), tokens, num_experts, top_k, renormalize,
                                                   probs, weights, experts);
  else
    moe_topk_kernel<float><<<grid, 256, 0, s>>>(static_cast<const float*>(logits), tokens, num_experts, top_k, renormalize, probs,
                                                weights, experts);
  FP8GMM_CHECK_CUDA(cudaGetLastError());
  count_launch();
  return FP8GMM_OK;
}

int fp8gmm_moe_gather(const void* x, const int32_t* indices, const float* weights, int top_k, int64_t rows, int64_t cols,
                      void* out, void* stream) {
  using namespace fp8gmm;
  FP8GMM_CHECK_ARG(top_k > 0 && rows >= 0 && cols >= 0, "moe_gather: bad sizes");
  if (rows == 0 || cols == 0) return FP8GMM_OK;
  FP8GMM_CHECK_ARG(x && indices && out, "moe_gather: NULL pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int* status = device_status_word();
  FP8GMM_CHECK_ARG(status != nullptr, "moe_gather: cannot resolve the device status word");
  const bool vec = cols % 8 == 0 && (reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) % 16 == 0;
  if (vec)
    moe_gather_kernel<true><<<row_grid(rows * (cols / 8)), 256, 0, s>>>(static_cast<const uint16_t*>(x), indices, weights, top_k,
                                                                       rows, cols, static_cast<uint16_t*>(out), status);
  else
    moe_gather_kernel<false><<<row_grid(rows * cols), 256, 0, s>>>(static_cast<const uint16_t*>(x), indices, weights, top_k, rows,
                                                                  cols, static_cast<uint16_t*>(out), status);
  FP8GMM_CHECK_CUDA(cudaGetLastError());
  count_launch();
  return FP8GMM_OK;
}

int fp8gmm_moe_scatter(const void* x, const int32_t* inverse, const float* weights, int top_k, int64_t tokens, int64_t cols,
                       void* out, void* stream) {
  using namespace fp8gmm;
  FP8GMM_CHECK_ARG(top_k > 0 && tokens >= 0 && cols >= 0, "moe_scatter: bad sizes");
  if (tokens == 0 || cols == 0) return FP8GMM_OK;
  FP8GMM_CHECK_ARG(x && inverse && out, "moe_scatter: NULL pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int* status = device_status_word();
  FP8GMM_CHECK_ARG(status != nullptr, "moe_scatter: cannot resolve the device status word");
  const bool vec = cols % 8 == 0 && (reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) % 16 == 0;
  if (vec)
    moe_scatter_kernel<true><<<row_grid(tokens * (cols / 8)), 256, 0, s>>>(static_cast<const uint16_t*>(x), inverse, weights, top_k,
                                                                          tokens, cols, static_cast<uint16_t*>(out), status);
  else
    moe_scatter_kernel<false><<<row_grid(tokens * cols), 256, 0, s>>>(static_cast<const uint16_t*>(x), inverse, weights, top_k,
                                                                     tokens, cols, static_cast<uint16_t*>(out), status);
  FP8GMM_CHECK_CUDA(cudaGetLastError());
  count_launch();
  return FP8GMM_OK;
}

int fp8gmm_moe_rowdot(const void* grad, const void* x, const int32_t* inverse, int top_k, int64_t n, int64_t cols,
                      float* d_weights, void* stream) {
  using namespace fp8gmm;
  FP8GMM_CHECK_ARG(top_k > 0 && n >= 0 && cols >= 0, "moe_rowdot: bad sizes");
  if (n == 0) return FP8GMM_OK;
  FP8GMM_CHECK_ARG(grad && x && inverse && d_weights, "moe_rowdot: NULL pointer");
  int* status = device_status_word();
  FP8GMM_CHECK_ARG(status != nullptr, "moe_rowdot: cannot resolve the device status word");
  moe_rowdot_kernel<<<row_grid(n * 32), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint16_t*>(grad), static_cast<const uint16_t*>(x), inverse, top_k, n, cols, d_weights, status);
  FP8GMM_CHECK_CUDA(cudaGetLastError());
  count_launch();
  return FP8GMM_OK;
}

}  // extern "C"
