// Host-side construction of TMA tensor maps.  The driver entry point is looked up at
// run time through the CUDA runtime, so the library has no link-time dependency on libcuda.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <mutex>

#include "common.cuh"

namespace b200q {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// Row-major 2-D tensor [outer, inner] of `elem_bytes`-wide elements with a row pitch of
// pitch_bytes; box [box_outer, box_inner]; out-of-range elements read as zero.
// Requirements checked here: base 16-byte aligned, pitch a multiple of 16 bytes, inner box
// extent a multiple of 16 bytes and (for 128-byte swizzle) at most 128 bytes, boxes <= 256.
inline int make_tmap_2d(CUtensorMap* out, CUtensorMapDataType dt, int elem_bytes, const void* base, uint64_t inner,
                        uint64_t outer, uint64_t pitch_bytes, uint32_t box_inner, uint32_t box_outer,
                        CUtensorMapSwizzle swz, const char* what) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return fail(B200Q_ERR_LAUNCH, "%s: cuTensorMapEncodeTiled is not available from this driver", what);
  if (!aligned(base, 16) || pitch_bytes % 16 != 0 || (uint64_t)box_inner * elem_bytes % 16 != 0 || box_inner > 256 ||
      box_outer > 256 || (swz == CU_TENSOR_MAP_SWIZZLE_128B && (uint64_t)box_inner * elem_bytes > 128))
    return fail(B200Q_ERR_BAD_ARG, "%s: operand does not meet the TMA alignment rules", what);
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {pitch_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(B200Q_ERR_LAUNCH, "%s: cuTensorMapEncodeTiled failed (CUresult %d)", what, (int)r);
  return B200Q_OK;
}

// Same, through a small cache keyed by every argument: a weight is used with the same map call after
// call, and encoding a map costs more than looking it up.  Thread-safe (one mutex); 256 direct-mapped
// entries, a colliding key simply replaces the entry.
inline int make_tmap_2d_cached(CUtensorMap* out, CUtensorMapDataType dt, int elem_bytes, const void* base,
                               uint64_t inner, uint64_t outer, uint64_t pitch_bytes, uint32_t box_inner,
                               uint32_t box_outer, CUtensorMapSwizzle swz, const char* what) {
  struct Entry {
    const void* base;
    uint64_t inner, outer, pitch;
    uint32_t box_inner, box_outer;
    int dt, elem_bytes, swz;
    bool valid;
    CUtensorMap map;
  };
  static std::mutex mu;
  static Entry table[256];
  uint64_t h = reinterpret_cast<uint64_t>(base) * 0x9E3779B97F4A7C15ull;
  h ^= (inner * 31 + outer) * 0xC2B2AE3D27D4EB4Full + pitch_bytes * 0x165667B19E3779F9ull + box_outer * 131 + box_inner;
  Entry& e = table[(h >> 24) & 255];
  {
    std::lock_guard<std::mutex> lock(mu);
    if (e.valid && e.base == base && e.inner == inner && e.outer == outer && e.pitch == pitch_bytes &&
        e.box_inner == box_inner && e.box_outer == box_outer && e.dt == (int)dt && e.elem_bytes == elem_bytes &&
        e.swz == (int)swz) {
      *out = e.map;
      return B200Q_OK;
    }
  }
  if (int rc = make_tmap_2d(out, dt, elem_bytes, base, inner, outer, pitch_bytes, box_inner, box_outer, swz, what)) return rc;
  std::lock_guard<std::mutex> lock(mu);
  e.base = base; e.inner = inner; e.outer = outer; e.pitch = pitch_bytes;
  e.box_inner = box_inner; e.box_outer = box_outer; e.dt = (int)dt; e.elem_bytes = elem_bytes; e.swz = (int)swz;
  e.map = *out;
  e.valid = true;
  return B200Q_OK;
}

}  // namespace b200q
