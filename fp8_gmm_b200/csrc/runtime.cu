// Host-side plumbing of the C ABI: error strings, device queries, the per-device status word that
// kernels use to report a bounded wait that ran out, and the delayed-scaling recipe update kernel.
#include <atomic>
#include <cmath>
#include <cstring>
#include <mutex>

#include "common.cuh"

namespace fp8gmm {

namespace {
thread_local char g_error[512] = "";
constexpr int kMaxDevices = 64;
int g_sm_count[kMaxDevices] = {0};
int* g_status_addr[kMaxDevices] = {nullptr};
std::mutex g_mutex;
std::atomic<uint64_t> g_launches{0};
// Bounded waits: a GEMM role gives up on an mbarrier after the first limit, fp8gmm_peer_wait on its sequence
// numbers after the second (defaults 1 s and 2 s; fp8gmm_set_wait_limits).
std::atomic<unsigned long long> g_gemm_wait_ns{1000ull * 1000ull * 1000ull};
std::atomic<unsigned long long> g_peer_wait_ns{2000ull * 1000ull * 1000ull};

// One status word per device that loads the library (a __device__ variable is instantiated per device).
__device__ int g_device_status = 0;
}  // namespace

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

int cuda_fail(cudaError_t err, const char* what) {
  set_error("CUDA error %d (%s) in %s", static_cast<int>(err), cudaGetErrorString(err), what);
  return FP8GMM_CUDA_ERROR;
}

static int current_device() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 0;
  return dev;
}

void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }
unsigned long long gemm_wait_limit_ns() { return g_gemm_wait_ns.load(std::memory_order_relaxed); }
unsigned long long peer_wait_limit_ns() { return g_peer_wait_ns.load(std::memory_order_relaxed); }

int sm_count() {
  const int dev = current_device();
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_sm_count[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    g_sm_count[dev] = n;
  }
  return g_sm_count[dev];
}

int* device_status_word() {
  const int dev = current_device();
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_status_addr[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_device_status) != cudaSuccess) return nullptr;
    g_status_addr[dev] = static_cast<int*>(p);
  }
  return g_status_addr[dev];
}

// --------------------------------------------------------------------------------------------
// Delayed-scaling update: one thread per meta slot walks its history column.
// --------------------------------------------------------------------------------------------
__global__ void delayed_scaling_update_kernel(float* __restrict__ hist, float* __restrict__ scale,
                                              float* __restrict__ scale_inv, int len, int n, float fp8_max,
                                              float inv_pow2_margin, int algo) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float amax;
  if (algo == 0) {
    amax = 0.f;
    for (int r = 0; r < len; ++r) {
      const float h = hist[(size_t)r * n + i];
      // torch.max semantics: NaN propagates, so a NaN amax leaves the scale unchanged below.
      amax = (h != h || amax != amax) ? NAN : fmaxf(amax, h);
    }
  } else {
    amax = hist[i];
  }
  float s = scale[i];
  if (amax > 0.f && isfinite(amax)) s = __fdiv_rn(fp8_max, amax) * inv_pow2_margin;
  scale[i] = s;
  scale_inv[i] = __fdiv_rn(1.0f, s);
  // roll(-1) along the history axis, then zero row 0: new[r] = old[r+1] for r < len-1, new[len-1] = old[0].
  if (len > 1) {
    const float first = hist[i];
    for (int r = 0; r + 1 < len; ++r) hist[(size_t)r * n + i] = hist[(size_t)(r + 1) * n + i];
    hist[(size_t)(len - 1) * n + i] = first;
  }
  hist[i] = 0.f;
}

}  // namespace fp8gmm

extern "C" {

int fp8gmm_version(void) { return 1000; }

uint64_t fp8gmm_launch_count(void) { return fp8gmm::g_launches.load(std::memory_order_relaxed); }

const char* fp8gmm_last_error(void) { return fp8gmm::g_error; }

int fp8gmm_device_status(void* stream) {
  int* word = fp8gmm::device_status_word();
  if (word == nullptr) {
    fp8gmm::set_error("cannot resolve the device status word");
    return FP8GMM_CUDA_ERROR;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  FP8GMM_CHECK_CUDA(cudaStreamSynchronize(s));
  int host = 0;
  FP8GMM_CHECK_CUDA(cudaMemcpy(&host, word, sizeof(int), cudaMemcpyDeviceToHost));
  if (host != 0) {
    const int zero = 0;
    FP8GMM_CHECK_CUDA(cudaMemcpy(word, &zero, sizeof(int), cudaMemcpyHostToDevice));
    fp8gmm::set_error("a kernel gave up on a bounded wait (code 0x%x)", host);
    return FP8GMM_DEVICE_TIMEOUT;
  }
  return FP8GMM_OK;
}

int fp8gmm_device_status_async(int* host_word, void* stream) {
  FP8GMM_CHECK_ARG(host_word != nullptr, "device_status_async: NULL destination");
  int* word = fp8gmm::device_status_word();
  if (word == nullptr) {
    fp8gmm::set_error("cannot resolve the device status word");
    return FP8GMM_CUDA_ERROR;
  }
  FP8GMM_CHECK_CUDA(cudaMemcpyAsync(host_word, word, sizeof(int), cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream)));
  return FP8GMM_OK;
}

int fp8gmm_set_wait_limits(int64_t gemm_wait_ns, int64_t peer_wait_ns) {
  FP8GMM_CHECK_ARG(gemm_wait_ns >= 0 && peer_wait_ns >= 0, "set_wait_limits: limits must not be negative (0 keeps the current one)");
  if (gemm_wait_ns > 0) fp8gmm::g_gemm_wait_ns.store(static_cast<unsigned long long>(gemm_wait_ns), std::memory_order_relaxed);
  if (peer_wait_ns > 0) fp8gmm::g_peer_wait_ns.store(static_cast<unsigned long long>(peer_wait_ns), std::memory_order_relaxed);
  return FP8GMM_OK;
}

int fp8gmm_delayed_scaling_update(float* amax_history, float* scale, float* scale_inv, int history_len, int n,
                                  float fp8_max, float margin, int algo, void* stream) {
  FP8GMM_CHECK_ARG(amax_history && scale && scale_inv, "delayed_scaling_update: NULL pointer");
  FP8GMM_CHECK_ARG(history_len >= 1 && n >= 0, "delayed_scaling_update: bad sizes");
  FP8GMM_CHECK_ARG(algo == 0 || algo == 1, "delayed_scaling_update: algo must be 0 (max) or 1 (most recent)");
  if (n == 0) return FP8GMM_OK;
  const float inv_pow2 = 1.0f / std::exp2(margin);
  fp8gmm::delayed_scaling_update_kernel<<<(n + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      amax_history, scale, scale_inv, history_len, n, fp8_max, inv_pow2, algo);
  FP8GMM_CHECK_CUDA(cudaGetLastError());
  fp8gmm::count_launch();
  return FP8GMM_OK;
}

}  // extern "C"
