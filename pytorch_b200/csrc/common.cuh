// Host-side helpers shared by the C-ABI translation units.
#pragma once
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>

#include <mutex>

#include "../../include/b200q.h"

namespace b200q {

// Stores the calling thread's last error message and returns `status`.
int fail(int status, const char* fmt, ...);
void clear_error();

// Number of SMs of the current device (cached per device).
int sm_count();

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

#define B200Q_REQUIRE(cond, status, ...)            \
  do {                                              \
    if (!(cond)) return ::b200q::fail((status), __VA_ARGS__); \
  } while (0)

// Call after a kernel launch: turns a launch error into B200Q_ERR_LAUNCH.
inline int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(B200Q_ERR_LAUNCH, "%s: %s", what, cudaGetErrorString(e));
  return B200Q_OK;
}

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// Raises the dynamic shared-memory limit of kernel `Kern` to `bytes`, once per device.  The per-device
// record is guarded by a mutex, so concurrent first calls from several host threads are safe.
template <auto Kern>
int ensure_dynamic_smem(int bytes, const char* what) {
  static std::mutex mu;
  static bool done[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = -1;
  std::lock_guard<std::mutex> lock(mu);
  if (dev >= 0 && done[dev]) return B200Q_OK;
  cudaError_t err = cudaFuncSetAttribute(Kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (err != cudaSuccess) return fail(B200Q_ERR_LAUNCH, "%s: cudaFuncSetAttribute: %s", what, cudaGetErrorString(err));
  if (dev >= 0) done[dev] = true;
  return B200Q_OK;
}

}  // namespace b200q
