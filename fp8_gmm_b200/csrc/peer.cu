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

}  // namespace
}  // namespace fp8gmm

extern "C" {

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
