// Error reporting, version and device-error word of the C ABI.
#include <mutex>
#include <string.h>

#include "common.cuh"
#include "ptx.cuh"

namespace b200q {

static thread_local char tl_error[512] = "";

int fail(int status, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(tl_error, sizeof(tl_error), fmt, ap);
  va_end(ap);
  return status;
}

void clear_error() { tl_error[0] = 0; }

int sm_count() {
  static std::mutex mu;
  static int cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  std::lock_guard<std::mutex> lock(mu);
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

// Mirror of the device error word in mapped pinned host memory, one per device, created on request.
// Returns the host pointer of the current device's word (nullptr when there is none and `create` is false
// or the mapping failed).
unsigned int* host_error_word(bool create) {
  static std::mutex mu;
  static unsigned int* words[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (words[dev] == nullptr && create) {
    unsigned int* h = nullptr;
    unsigned int* d = nullptr;
    if (cudaHostAlloc(reinterpret_cast<void**>(&h), sizeof(unsigned int), cudaHostAllocMapped) != cudaSuccess ||
        cudaHostGetDevicePointer(reinterpret_cast<void**>(&d), h, 0) != cudaSuccess) {
      cudaGetLastError();
      return nullptr;
    }
    *h = 0;
    if (cudaMemcpyToSymbol(g_host_error_word, &d, sizeof(d)) != cudaSuccess) {
      cudaGetLastError();
      cudaFreeHost(h);
      return nullptr;
    }
    words[dev] = h;
  }
  return words[dev];
}

// Self-test of the bounded wait: one warp waits on an mbarrier that nothing will ever arrive on.  The wait must
// run out after `limit_ns`, record kDevTimeoutSelfTest and let the kernel return normally.
__global__ void expire_wait_kernel(unsigned long long limit_ns) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_flag = 0;
    fence_mbar_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) mbar_wait(&bar, 0, &abort_flag, kDevTimeoutSelfTest, limit_ns);
  __syncthreads();
}

}  // namespace b200q


extern "C" {

int b200q_version(void) { return 100; }

const char* b200q_last_error(void) { return b200q::tl_error; }

const char* b200q_status_string(int status) {
  switch (status) {
    case B200Q_OK: return "ok";
    case B200Q_ERR_BAD_ARG: return "bad argument";
    case B200Q_ERR_UNSUPPORTED: return "unsupported";
    case B200Q_ERR_LAUNCH: return "launch failure";
    case B200Q_ERR_WORKSPACE: return "workspace too small";
    case B200Q_ERR_DEVICE: return "device-side error";
    default: return "unknown status";
  }
}

int b200q_device_error(unsigned int* code, int reset) {
  B200Q_REQUIRE(code != nullptr, B200Q_ERR_BAD_ARG, "b200q_device_error: code is NULL");
  unsigned int v = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, b200q::g_device_error, sizeof(v));
  if (e != cudaSuccess) return b200q::fail(B200Q_ERR_LAUNCH, "b200q_device_error: %s", cudaGetErrorString(e));
  *code = v;
  if (reset && v != 0) {
    unsigned int z = 0;
    e = cudaMemcpyToSymbol(b200q::g_device_error, &z, sizeof(z));
    if (e != cudaSuccess) return b200q::fail(B200Q_ERR_LAUNCH, "b200q_device_error: %s", cudaGetErrorString(e));
    if (unsigned int* h = b200q::host_error_word(false)) *reinterpret_cast<volatile unsigned int*>(h) = 0;
  }
  return v == 0 ? B200Q_OK : B200Q_ERR_DEVICE;
}

int b200q_enable_host_error_word(void) {
  b200q::clear_error();
  return b200q::host_error_word(true) != nullptr
             ? B200Q_OK
             : b200q::fail(B200Q_ERR_LAUNCH, "b200q_enable_host_error_word: could not map a pinned host word");
}

unsigned int b200q_peek_device_error(void) {
  unsigned int* h = b200q::host_error_word(false);
  return h ? *reinterpret_cast<volatile unsigned int*>(h) : 0u;
}

int b200q_selftest_expire_wait(uint64_t limit_ns, void* stream) {
  b200q::clear_error();
  B200Q_REQUIRE(limit_ns > 0 && limit_ns <= 1000000000ULL, B200Q_ERR_BAD_ARG,
                "b200q_selftest_expire_wait: limit must be between 1 ns and 1 s");
  b200q::expire_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(limit_ns);
  return b200q::check_launch("selftest_expire_wait");
}

}  // extern "C"
