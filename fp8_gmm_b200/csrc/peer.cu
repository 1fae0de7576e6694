// Peer-memory plumbing for the expert-parallel row exchange (dispatch / combine) on one NVSwitch node.
//
// The reference has no multi-GPU exchange at all (its example permutes rows on one device with megablocks,
// fp8_gmm/example.py:52-59); this file is the transport under fp8_gmm_b200/ep.py.  Design:
//   * every rank owns receive buffers obtained from cudaMalloc here and exported with CUDA IPC, so that each
//     peer maps them into its own address space once, at set-up;
//   * rows travel as plain device-to-device copies (cudaMemcpyAsync on a side stream): the copy engines
//     move them over NVLink, no SM is taken from the GEMMs that run meanwhile;
//   * completion is announced with one 32-bit sequence number per (receiver, sender) pair, written into the
//     receiver's memory by a one-warp kernel that is stream-ordered after the sender's copies, and awaited
//     by a one-warp kernel on the receiver's compute stream.  Sequence numbers only grow, so nothing is
//     ever reset.  The wait is bounded (two seconds unless fp8gmm_set_wait_limits changed it): when it runs
//     out the kernel records a code in the device status word and returns, it never hangs the GPU.
// A waiting kernel and the kernel that releases it always run on different GPUs.
#include <cstring>

#include "common.cuh"

namespace fp8gmm {
namespace {

constexpr int kMaxPeers = 64;
constexpr int kStatusPeerTimeout = 0x100;

struct SignalParams {
  uint32_t* flags[kMaxPeers];
  int count;
  uint32_t value;
};

__global__ void peer_signal_kernel(const SignalParams p) {
  const int i = threadIdx.x;
  if (i < p.count && p.flags[i] != nullptr) {
    // everything this stream did before (the copies) is complete; make the number visible system-wide
    __threadfence_system();
    *reinterpret_cast<volatile uint32_t*>(p.flags[i]) = p.value;
    __threadfence_system();
  }
}

__device__ __forceinline__ unsigned long long peer_global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// Lane i waits until flags[i] has reached `value` (sequence numbers compare modulo 2^32).
__global__ void peer_wait_kernel(const uint32_t* flags, int count, uint32_t value, int* status, unsigned long long limit_ns) {
  const int i = threadIdx.x;
  if (i >= count) return;
  const volatile uint32_t* f = flags + i;
  const unsigned long long t0 = peer_global_ns();
  for (;;) {
    for (int spin = 0; spin < 64; ++spin) {
      const uint32_t v = *f;
      if (static_cast<int32_t>(v - value) >= 0) {
        __threadfence_system();
        return;
      }
    }
    if (peer_global_ns() - t0 > limit_ns) {
      atomicOr(status, kStatusPeerTimeout);
      return;
    }
    __nanosleep(200);
  }
}

// ---------------------------------------------------------------------------------------------
// Block permutation of rows in local memory (HBM-bound).  The expert-parallel forward receives a chunk's rows
// source-major (one large copy per sending rank) and the grouped GEMM wants them expert-major; the rows have to be
// copied out of the receive buffer once anyway (the fc1 weight gradient needs them after the buffer has been reused),
// so that copy applies the permutation.  Blocks are runs of consecutive rows; a CTA takes 32 KB pieces of the
// concatenated blocks, 16-byte vectors, eight loads in flight per thread.
// ---------------------------------------------------------------------------------------------
constexpr int kPermMaxBlocks = 160;   // per launch (the parameter block stays below 4 KB)
constexpr int kPermUnroll = 8;

struct PermParams {
  const uint8_t* src[kPermMaxBlocks];
  uint8_t* dst[kPermMaxBlocks];
  unsigned int vec_start[kPermMaxBlocks + 1];   // prefix sums of the blocks' 16-byte vector counts
  int count;
};

__global__ void __launch_bounds__(256) block_permute_kernel(const __grid_constant__ PermParams p) {
  const unsigned int total = p.vec_start[p.count];
  const unsigned int per_piece = 256u * kPermUnroll;
  const unsigned int pieces = (total + per_piece - 1) / per_piece;
  for (unsigned int c = blockIdx.x; c < pieces; c += gridDim.x) {
    const unsigned int base = c * per_piece;
    int b = upper_slot(reinterpret_cast<const int*>(p.vec_start), p.count, static_cast<int>(base));
    uint4 v[kPermUnroll];
    int blk[kPermUnroll];
#pragma unroll
    for (int u = 0; u < kPermUnroll; ++u) {
      const unsigned int i = base + u * 256u + threadIdx.x;
      blk[u] = -1;
      if (i < total) {
        while (i >= p.vec_start[b + 1]) ++b;
        blk[u] = b;
        v[u] = ld_stream16(p.src[b] + static_cast<size_t>(i - p.vec_start[b]) * 16);
      }
    }
#pragma unroll
    for (int u = 0; u < kPermUnroll; ++u) {
      const unsigned int i = base + u * 256u + threadIdx.x;
      if (blk[u] >= 0) *reinterpret_cast<uint4*>(p.dst[blk[u]] + static_cast<size_t>(i - p.vec_start[blk[u]]) * 16) = v[u];
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Sum of a bf16 buffer over the ranks of a tensor-parallel group, over peer memory (plain peer loads; no
// multimem, no TMA).  The reference all-reduces the input gradient of its MLP with NCCL after the fc1 data-gradient
// GEMM (fp8_gmm/grouped_mlp.py:300-303,323-324); here the GEMM writes its partial rows into a peer-mapped staging
// buffer chunk by chunk and two light kernels per chunk finish the sum while the next chunk's GEMM runs:
//   reduce-scatter  rank r sums slice r of the chunk over all ranks' staging buffers (fp32, ranks in ascending
//                   order, one rounding to bf16) and stores it in its own staging buffer;
//   all-gather      every rank reads slice s from rank s's staging buffer into its result tensor (local memory).
// Every element is summed exactly once, by one rank, so all ranks end with identical bits.
// ---------------------------------------------------------------------------------------------
struct ReduceParams {
  const uint4* bufs[kMaxPeers];  // staging buffer of every rank as mapped here
  uint4* out;                    // reduce-scatter: this rank's staging buffer; all-gather: the result tensor
  long long begin;               // first 16-byte vector of the chunk
  long long vectors;             // 16-byte vectors in the chunk
  long long per_rank;            // vectors per slice (the last slice may be shorter)
  int world;
  int rank;
};

__device__ __forceinline__ void accumulate8(float (&acc)[8], uint4 v) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    acc[2 * j] += bf16_lo(w[j]);
    acc[2 * j + 1] += bf16_hi(w[j]);
  }
}

constexpr int kReduceBatch = 4;   // independent 16-byte loads a thread keeps in flight per rank (peer latency is microseconds)

__global__ void __launch_bounds__(256) peer_reduce_scatter_kernel(const ReduceParams p) {
  const long long lo = p.begin + p.rank * p.per_rank;
  const long long end = p.begin + p.vectors;
  const long long hi = lo + p.per_rank < end ? lo + p.per_rank : end;
  const long long stride = 256ll * gridDim.x;
  for (long long i0 = lo + blockIdx.x * 256ll + threadIdx.x; i0 < hi; i0 += stride * kReduceBatch) {
    float acc[kReduceBatch][8];
#pragma unroll
    for (int u = 0; u < kReduceBatch; ++u)
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[u][j] = 0.f;
    for (int r = 0; r < p.world; ++r) {
      uint4 v[kReduceBatch];
#pragma unroll
      for (int u = 0; u < kReduceBatch; ++u) {
        const long long i = i0 + u * stride;
        v[u] = i < hi ? __ldcv(p.bufs[r] + i) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int u = 0; u < kReduceBatch; ++u) accumulate8(acc[u], v[u]);
    }
#pragma unroll
    for (int u = 0; u < kReduceBatch; ++u) {
      const long long i = i0 + u * stride;
      if (i < hi)
        p.out[i] = make_uint4(pack_bf16x2(acc[u][0], acc[u][1]), pack_bf16x2(acc[u][2], acc[u][3]),
                              pack_bf16x2(acc[u][4], acc[u][5]), pack_bf16x2(acc[u][6], acc[u][7]));
    }
  }
}

__global__ void __launch_bounds__(256) peer_all_gather_kernel(const ReduceParams p) {
  const long long stride = 256ll * gridDim.x;
  for (long long v0 = blockIdx.x * 256ll + threadIdx.x; v0 < p.vectors; v0 += stride * kReduceBatch) {
    uint4 v[kReduceBatch];
#pragma unroll
    for (int u = 0; u < kReduceBatch; ++u) {
      const long long i = v0 + u * stride;
      if (i < p.vectors) v[u] = __ldcv(p.bufs[static_cast<int>(i / p.per_rank)] + p.begin + i);
    }
#pragma unroll
    for (int u = 0; u < kReduceBatch; ++u) {
      const long long i = v0 + u * stride;
      if (i < p.vectors) p.out[p.begin + i] = v[u];
    }
  }
}

int fill_reduce_params(ReduceParams* p, void* const* bufs, int world, int rank, int64_t elem_offset, int64_t numel, void* out,
                       const char* name) {
  FP8GMM_CHECK_ARG(bufs != nullptr && world >= 1 && world <= kMaxPeers && rank >= 0 && rank < world, "%s: bad group", name);
  FP8GMM_CHECK_ARG(elem_offset >= 0 && numel >= 0 && elem_offset % 8 == 0 && numel % 8 == 0,
                   "%s: offset and length must be multiples of 8 elements", name);
  memset(p, 0, sizeof(*p));
  for (int r = 0; r < world; ++r) {
    FP8GMM_CHECK_ARG(bufs[r] != nullptr && reinterpret_cast<uintptr_t>(bufs[r]) % 16 == 0, "%s: buffer %d is NULL or unaligned", name, r);
    p->bufs[r] = static_cast<const uint4*>(bufs[r]);
  }
  FP8GMM_CHECK_ARG(out != nullptr && reinterpret_cast<uintptr_t>(out) % 16 == 0, "%s: output is NULL or unaligned", name);
  p->out = static_cast<uint4*>(out);
  p->begin = elem_offset / 8;
  p->vectors = numel / 8;
  p->per_rank = (p->vectors + world - 1) / world;
  if (p->per_rank == 0) p->per_rank = 1;
  p->world = world;
  p->rank = rank;
  return FP8GMM_OK;
}

int reduce_grid(long long vectors, int max_ctas) {
  const long long want = (vectors + 255) / 256;
  const long long cap = max_ctas > 0 ? max_ctas : 64;
  return static_cast<int>(want < 1 ? 1 : want < cap ? want : cap);
}

}  // namespace
}  // namespace fp8gmm

extern "C" {

int fp8gmm_peer_reduce_scatter_bf16(void* const* bufs, int world, int rank, int64_t elem_offset, int64_t numel, int max_ctas,
                                    void* stream) {
  using namespace fp8gmm;
  ReduceParams p;
  const int rc = fill_reduce_params(&p, bufs, world, rank, elem_offset, numel, bufs ? bufs[rank < world && rank >= 0 ? rank : 0] : nullptr,
                                    "peer_reduce_scatter_bf16");
  if (rc != FP8GMM_OK) return rc;
  if (numel == 0) return FP8GMM_OK;
  peer_reduce_scatter_kernel<<<reduce_grid(p.per_rank, max_ctas), 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  FP8GMM_CHECK_CUDA(cudaGetLastError());
  count_launch();
  return FP8GMM_OK;
}

int fp8gmm_peer_all_gather_bf16(void* const* bufs, int world, int rank, int64_t elem_offset, int64_t numel, void* out, int max_ctas,
                                void* stream) {
  using namespace fp8gmm;
  ReduceParams p;
  const int rc = fill_reduce_params(&p, bufs, world, rank, elem_offset, numel, out, "peer_all_gather_bf16");
  if (rc != FP8GMM_OK) return rc;
  if (numel == 0) return FP8GMM_OK;
  peer_all_gather_kernel<<<reduce_grid(p.vectors, max_ctas), 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  FP8GMM_CHECK_CUDA(cudaGetLastError());
  count_launch();
  return FP8GMM_OK;
}

int fp8gmm_peer_alloc(size_t bytes, void** ptr, void* handle) {
  using namespace fp8gmm;
  FP8GMM_CHECK_ARG(ptr != nullptr && handle != nullptr && bytes > 0, "peer_alloc: bad arguments");
  static_assert(sizeof(cudaIpcMemHandle_t) == FP8GMM_PEER_HANDLE_BYTES, "IPC handle size");
  void* p = nullptr;
  FP8GMM_CHECK_CUDA(cudaMalloc(&p, bytes));
  cudaIpcMemHandle_t h;
  cudaError_t err = cudaIpcGetMemHandle(&h, p);
  if (err != cudaSuccess) {
    cudaFree(p);
    return cuda_fail(err, "cudaIpcGetMemHandle");
  }
  err = cudaMemset(p, 0, bytes < 4096 ? bytes : 4096);  // flag pages start at zero; data buffers need no clearing
  if (err != cudaSuccess) {
    cudaFree(p);
    return cuda_fail(err, "cudaMemset");
  }
  memcpy(handle, &h, sizeof(h));
  *ptr = p;
  return FP8GMM_OK;
}

int fp8gmm_peer_free(void* ptr) {
  if (ptr != nullptr) FP8GMM_CHECK_CUDA(cudaFree(ptr));
  return FP8GMM_OK;
}

int fp8gmm_peer_open(const void* handle, void** ptr) {
  using namespace fp8gmm;
  FP8GMM_CHECK_ARG(ptr != nullptr && handle != nullptr, "peer_open: bad arguments");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  FP8GMM_CHECK_CUDA(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return FP8GMM_OK;
}

int fp8gmm_peer_close(void* ptr) {
  if (ptr != nullptr) FP8GMM_CHECK_CUDA(cudaIpcCloseMemHandle(ptr));
  return FP8GMM_OK;
}

int fp8gmm_peer_copy_blocks(const fp8gmm_copy_block* blocks, int count, void* stream) {
  using namespace fp8gmm;
  FP8GMM_CHECK_ARG(count >= 0 && (count == 0 || blocks != nullptr), "peer_copy_blocks: bad arguments");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  for (int i = 0; i < count; ++i) {
    if (blocks[i].bytes == 0) continue;
    FP8GMM_CHECK_ARG(blocks[i].dst != nullptr && blocks[i].src != nullptr, "peer_copy_blocks: NULL pointer in block %d", i);
    FP8GMM_CHECK_CUDA(cudaMemcpyAsync(blocks[i].dst, blocks[i].src, blocks[i].bytes, cudaMemcpyDeviceToDevice, s));
  }
  return FP8GMM_OK;
}

int fp8gmm_block_permute_rows(const void* src, void* dst, const int64_t* src_start, const int64_t* dst_start,
                              const int64_t* rows, int64_t num_blocks, int64_t row_bytes, void* stream) {
  using namespace fp8gmm;
  FP8GMM_CHECK_ARG(num_blocks >= 0 && row_bytes > 0 && row_bytes % 16 == 0, "block_permute_rows: row_bytes must be a positive multiple of 16");
  if (num_blocks == 0) return FP8GMM_OK;
  FP8GMM_CHECK_ARG(src && dst && src_start && dst_start && rows, "block_permute_rows: NULL pointer");
  FP8GMM_CHECK_ARG((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) % 16 == 0, "block_permute_rows: unaligned buffer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  PermParams p;
  p.count = 0;
  p.vec_start[0] = 0;
  auto flush = [&]() -> int {
    if (p.count == 0) return FP8GMM_OK;
    const unsigned int pieces = (p.vec_start[p.count] + 256u * kPermUnroll - 1) / (256u * kPermUnroll);
    const unsigned int cap = static_cast<unsigned int>(sm_count()) * 8u;
    block_permute_kernel<<<static_cast<int>(pieces < cap ? pieces : cap), 256, 0, s>>>(p);
    FP8GMM_CHECK_CUDA(cudaGetLastError());
    count_launch();
    p.count = 0;
    return FP8GMM_OK;
  };
  for (int64_t i = 0; i < num_blocks; ++i) {
    FP8GMM_CHECK_ARG(rows[i] >= 0 && src_start[i] >= 0 && dst_start[i] >= 0, "block_permute_rows: negative entry in block %lld", (long long)i);
    if (rows[i] == 0) continue;
    const uint64_t vecs = static_cast<uint64_t>(rows[i]) * static_cast<uint64_t>(row_bytes) / 16;
    FP8GMM_CHECK_ARG(vecs <= 0x3FFFFFFFull, "block_permute_rows: block %lld is too large", (long long)i);
    if (p.count == kPermMaxBlocks || static_cast<uint64_t>(p.vec_start[p.count]) + vecs > 0x7FFFFFFFull) {
      const int rc = flush();
      if (rc != FP8GMM_OK) return rc;
    }
    p.src[p.count] = static_cast<const uint8_t*>(src) + src_start[i] * row_bytes;
    p.dst[p.count] = static_cast<uint8_t*>(dst) + dst_start[i] * row_bytes;
    p.vec_start[p.count + 1] = p.vec_start[p.count] + static_cast<unsigned int>(vecs);
    ++p.count;
  }
  return flush();
}

int fp8gmm_peer_signal(uint32_t* const* flags, int count, uint32_t value, void* stream) {
  using namespace fp8gmm;
  FP8GMM_CHECK_ARG(count >= 0 && count <= kMaxPeers && (count == 0 || flags != nullptr), "peer_signal: bad arguments");
  if (count == 0) return FP8GMM_OK;
  SignalParams p;
  memset(&p, 0, sizeof(p));
  for (int i = 0; i < count; ++i) p.flags[i] = flags[i];
  p.count = count;
  p.value = value;
  peer_signal_kernel<<<1, kMaxPeers, 0, static_cast<cudaStream_t>(stream)>>>(p);
  FP8GMM_CHECK_CUDA(cudaGetLastError());
  count_launch();
  return FP8GMM_OK;
}

int fp8gmm_peer_wait(const uint32_t* flags, int count, uint32_t value, void* stream) {
  using namespace fp8gmm;
  FP8GMM_CHECK_ARG(count >= 0 && count <= kMaxPeers && (count == 0 || flags != nullptr), "peer_wait: bad arguments");
  if (count == 0) return FP8GMM_OK;
  int* status = device_status_word();
  FP8GMM_CHECK_ARG(status != nullptr, "peer_wait: cannot resolve the device status word");
  peer_wait_kernel<<<1, kMaxPeers, 0, static_cast<cudaStream_t>(stream)>>>(flags, count, value, status, peer_wait_limit_ns());
  FP8GMM_CHECK_CUDA(cudaGetLastError());
  count_launch();
  return FP8GMM_OK;
}

}  // extern "C"
