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
  }
  return v == 0 ? B200Q_OK : B200Q_ERR_DEVICE;
}

}  // extern "C"
