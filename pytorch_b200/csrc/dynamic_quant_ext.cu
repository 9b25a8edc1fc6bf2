// npu_dynamic_quant with group_index (one smooth-scale row per group of tokens, as in a
// mixture-of-experts layer) and npu_dynamic_quant_asymmetric.  Same row-per-CTA structure as
// dynamic_quant.cu (the row stays in registers, 2 B in + 1 B out per element); this file holds
// the variants outside the W8A8 hot path so that the symmetric kernel keeps its tight code.
//
// Asymmetric: per row, xs = x * smooth (fp32), scale = (max(xs) - min(xs)) / 255,
// offset = 127 - max(xs) / scale, y = clamp(rint(xs / scale + offset), -128, 127);
// a constant row gives scale 0, offset 0 and y 0.  The fast path forms fma(xs, 1/scale, offset)
// and redoes a vector with IEEE division and a separate sum only when one of its values lies
// within 1e-4 of a rounding boundary, where the two could round differently (they differ by less
// than 4e-5: |xs/scale| <= 255, three roundings of 2^-24 relative each).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"

namespace b200q {
namespace {

// Floats ordered like unsigned integers: flip all bits of negatives, the sign bit of the rest.
__device__ __forceinline__ uint32_t f32_ordered(float f) {
  const uint32_t b = __float_as_uint(f);
  return b ^ ((b >> 31) ? 0xFFFFFFFFu : 0x80000000u);
}
__device__ __forceinline__ float f32_unordered(uint32_t u) {
  return __uint_as_float(u ^ ((u >> 31) ? 0x80000000u : 0xFFFFFFFFu));
}

// Maximum and minimum over the CTA (red: 2 x 32 words of shared memory).
__device__ __forceinline__ void block_max_min(float& mx, float& mn, uint32_t* red) {
  const uint32_t wmax = __reduce_max_sync(0xffffffffu, f32_ordered(mx));
  const uint32_t wmin = __reduce_min_sync(0xffffffffu, f32_ordered(mn));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = (blockDim.x + 31) >> 5;
  if (lane == 0) { red[warp] = wmax; red[32 + warp] = wmin; }
  __syncthreads();
  const uint32_t a = lane < nwarps ? red[lane] : 0u;
  const uint32_t b = lane < nwarps ? red[32 + lane] : 0xFFFFFFFFu;
  mx = f32_unordered(__reduce_max_sync(0xffffffffu, a));
  mn = f32_unordered(__reduce_min_sync(0xffffffffu, b));
}

__device__ __forceinline__ uint2 pack8_low_bytes(const uint32_t (&u)[8]) {
  uint2 o;
  o.x = __byte_perm(__byte_perm(u[0], u[1], 0x0040), __byte_perm(u[2], u[3], 0x0040), 0x5410);
  o.y = __byte_perm(__byte_perm(u[4], u[5], 0x0040), __byte_perm(u[6], u[7], 0x0040), 0x5410);
  return o;
}

__device__ __forceinline__ int quant_asym_exact(float f, float scale, float offset) {
  const int q = __float2int_rn(__fadd_rn(__fdiv_rn(f, scale), offset));
  return max(-128, min(127, q));
}

// Eight values -> eight int8, bit-exact with clamp(rint(xs / scale + offset)): the correctly rounded quotient by
// the same two-FMA refinement as the symmetric kernel (quantize8), one rounded addition of the offset, then the
// 1.5 * 2^23 addition that rounds to the nearest-even integer and leaves its low byte in the mantissa.  The
// result lies in [-128, 127] by construction (offset = 127 - max/scale, scale = (max - min)/255) as long as the
// offset is moderate, which the caller checks, so no clamp.
// Packed two-wide fp32 instructions; a constant row (scale 0) gives 0, a scale too small for a finite
// reciprocal (inv is NaN) takes true divisions.
// MODE 0: packed path; 1: true divisions with the clamp; 2: constant row (scale 0), all zeros.  The mode is the
// same for a whole row, so the caller branches once per row, not once per vector.
template <int MODE>
__device__ __forceinline__ uint2 quantize8_asym(const float (&f)[8], float scale, float inv, float offset) {
  uint32_t u[8];
  if (MODE == 2) {
#pragma unroll
    for (int j = 0; j < 8; ++j) u[j] = 0u;
  } else if (MODE == 0) {
    const float2 inv2 = make_float2(inv, inv), nscale2 = make_float2(-scale, -scale), off2 = make_float2(offset, offset);
    const float2 magic2 = make_float2(12582912.0f, 12582912.0f);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 x = make_float2(f[2 * j], f[2 * j + 1]);
      const float2 q0 = __fmul2_rn(x, inv2);
      const float2 r = __ffma2_rn(q0, nscale2, x);
      const float2 q = __ffma2_rn(r, inv2, q0);
      const float2 m = __fadd2_rn(__fadd2_rn(q, off2), magic2);
      u[2 * j] = __float_as_uint(m.x);
      u[2 * j + 1] = __float_as_uint(m.y);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) u[j] = (uint32_t)quant_asym_exact(f[j], scale, offset);
  }
  return pack8_low_bytes(u);
}

// Group of a row: group_index holds the sorted, cumulative end rows of the groups
// (test/onnx/test_wrapper_onnx_ops.py:1345-1354); rows past the last entry use the last group.
__device__ __forceinline__ int group_of_row(const int32_t* __restrict__ gidx, int ngroups, int64_t row) {
  int g = 0;
  while (g < ngroups - 1 && row >= gidx[g]) ++g;
  return g;
}

template <typename T, typename ST, int ITERS, bool ASYM>
__global__ void __launch_bounds__(512)
dynamic_quant_ext_rows(const T* __restrict__ x, const ST* __restrict__ smooth, const int32_t* __restrict__ gidx,
                       int ngroups, int8_t* __restrict__ y, float* __restrict__ scale_out,
                       float* __restrict__ offset_out, int64_t rows, int k) {
  __shared__ uint32_t red[2][64];
  const int nvec = k >> 3;
  uint4 raw[ITERS];
  // A thread's vector past the end of the row is replaced by the row's last vector: it adds nothing
  // new to the maximum and minimum, needs no predicates in the arithmetic, and is not stored.
  auto load_row = [&](int64_t row) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * k);
#pragma unroll
    for (int i = 0; i < ITERS; ++i) raw[i] = ld_stream(xr + min((int)(threadIdx.x + i * blockDim.x), nvec - 1));
  };
  int par = 0;
  if ((int64_t)blockIdx.x < rows) load_row(blockIdx.x);
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x, par ^= 1) {
    const ST* sm_row = smooth;
    if (smooth != nullptr && gidx != nullptr) sm_row = smooth + (int64_t)group_of_row(gidx, ngroups, row) * k;
    float f[ITERS][8];
    float mx = -INFINITY, mn = INFINITY;
#pragma unroll
    for (int i = 0; i < ITERS; ++i) {
      const int v = min((int)(threadIdx.x + i * blockDim.x), nvec - 1);
      const uint32_t w[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
      float2 sm[4];
      if (smooth != nullptr) load_smooth8(sm_row + v * 8, sm);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 pr = unpack2<T>(w[j]);
        if (smooth != nullptr) pr = __fmul2_rn(pr, sm[j]);
        f[i][2 * j] = pr.x;
        f[i][2 * j + 1] = pr.y;
        mx = fmaxf(mx, fmaxf(f[i][2 * j], f[i][2 * j + 1]));
        mn = fminf(mn, fminf(f[i][2 * j], f[i][2 * j + 1]));
      }
    }
    if (row + gridDim.x < rows) load_row(row + gridDim.x);   // in flight during the reduction and quantisation
    block_max_min(mx, mn, red[par]);
    uint2* yr = reinterpret_cast<uint2*>(y + row * k) + threadIdx.x;
    if (ASYM) {
      const float scale = __fdiv_rn(__fsub_rn(mx, mn), 255.0f);
      const float offset = scale == 0.0f ? 0.0f : __fsub_rn(127.0f, __fdiv_rn(mx, scale));
      if (threadIdx.x == 0) { scale_out[row] = scale; offset_out[row] = offset; }
      // A row whose values sit far from zero compared with their spread has a huge offset; the sum with the
      // offset then rounds coarsely and can leave [-128, 127], which only the clamping path handles.
      const float inv = fabsf(offset) < 30000.0f ? quant_inverse(scale) : __int_as_float(0x7fc00000);
      if (scale == 0.0f) {
#pragma unroll
        for (int i = 0; i < ITERS; ++i)
          if (threadIdx.x + i * blockDim.x < nvec) st_stream(yr + i * blockDim.x, quantize8_asym<2>(f[i], scale, inv, offset));
      } else if (inv == inv) {
#pragma unroll
        for (int i = 0; i < ITERS; ++i)
          if (threadIdx.x + i * blockDim.x < nvec) st_stream(yr + i * blockDim.x, quantize8_asym<0>(f[i], scale, inv, offset));
      } else {
#pragma unroll
        for (int i = 0; i < ITERS; ++i)
          if (threadIdx.x + i * blockDim.x < nvec) st_stream(yr + i * blockDim.x, quantize8_asym<1>(f[i], scale, inv, offset));
      }
    } else {
      const float amax = fmaxf(fabsf(mx), fabsf(mn));
      const float scale = scale_of_amax(amax);
      if (threadIdx.x == 0) scale_out[row] = scale;
      const float inv = quant_inverse(scale);
      if (inv == inv) {
#pragma unroll
        for (int i = 0; i < ITERS; ++i)
          if (threadIdx.x + i * blockDim.x < nvec) st_stream(yr + i * blockDim.x, quantize8<false>(f[i], scale, inv));
      } else {
#pragma unroll
        for (int i = 0; i < ITERS; ++i)
          if (threadIdx.x + i * blockDim.x < nvec) st_stream(yr + i * blockDim.x, quantize8<true>(f[i], scale, inv));
      }
    }
  }
}

// Any k, any alignment: the row is read twice (second pass from L2).
template <typename T, typename ST, bool ASYM>
__global__ void dynamic_quant_ext_generic(const T* __restrict__ x, const ST* __restrict__ smooth,
                                          const int32_t* __restrict__ gidx, int ngroups, int8_t* __restrict__ y,
                                          float* __restrict__ scale_out, float* __restrict__ offset_out, int64_t k) {
  __shared__ uint32_t red[64];
  const int64_t row = blockIdx.x;
  const T* xr = x + row * k;
  const ST* sm_row = smooth;
  if (smooth != nullptr && gidx != nullptr) sm_row = smooth + (int64_t)group_of_row(gidx, ngroups, row) * k;
  float mx = -INFINITY, mn = INFINITY;
  for (int64_t c = threadIdx.x; c < k; c += blockDim.x) {
    float f = to_f32<T>(xr[c]);
    if (smooth != nullptr) f = __fmul_rn(f, to_f32<ST>(sm_row[c]));
    mx = fmaxf(mx, f);
    mn = fminf(mn, f);
  }
  block_max_min(mx, mn, red);
  float scale, offset = 0.0f;
  if (ASYM) {
    scale = __fdiv_rn(__fsub_rn(mx, mn), 255.0f);
    offset = scale == 0.0f ? 0.0f : __fsub_rn(127.0f, __fdiv_rn(mx, scale));
    if (threadIdx.x == 0) { scale_out[row] = scale; offset_out[row] = offset; }
  } else {
    scale = __fdiv_rn(fmaxf(fabsf(mx), fabsf(mn)), 127.0f);
    if (threadIdx.x == 0) scale_out[row] = scale;
  }
  for (int64_t c = threadIdx.x; c < k; c += blockDim.x) {
    float f = to_f32<T>(xr[c]);
    if (smooth != nullptr) f = __fmul_rn(f, to_f32<ST>(sm_row[c]));
    int q = 0;
    if (scale != 0.0f)
      q = ASYM ? quant_asym_exact(f, scale, offset) : max(-128, min(127, __float2int_rn(__fdiv_rn(f, scale))));
    y[row * k + c] = static_cast<int8_t>(q);
  }
}

template <typename T, typename ST, bool ASYM>
int launch_dq_ext(const void* x, const void* smooth, const int32_t* gidx, int ngroups, int8_t* y, float* scale,
                  float* offset, int64_t rows, int64_t k, cudaStream_t st) {
  const T* xp = static_cast<const T*>(x);
  const ST* sp = static_cast<const ST*>(smooth);
  const bool vec = (k % 8 == 0) && aligned(x, 16) && aligned(y, 8) && k <= 8 * 512 * 16 &&
                   (smooth == nullptr || aligned(smooth, 16));
  if (!vec) {
    dynamic_quant_ext_generic<T, ST, ASYM><<<(unsigned)rows, 256, 0, st>>>(xp, sp, gidx, ngroups, y, scale, offset, k);
    return check_launch("dynamic_quant (generic)");
  }
  const int nvec = (int)(k / 8);
  int iters = 1;
  while (iters < 4 && nvec > iters * 256) iters *= 2;
  if (nvec > 4 * 512)                                    // at most 512 threads: the row's fp32 products need the registers
    while (iters < 16 && nvec > iters * 512) iters *= 2;
  int threads = (int)ceil_div(nvec, iters);
  threads = (int)ceil_div(threads, 32) * 32;
  int per_sm = 1;
#define B200Q_DQX_CASE(I)                                                                                   \
  case I: {                                                                                                  \
    auto kern = dynamic_quant_ext_rows<T, ST, I, ASYM>;                                                      \
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, threads, 0);                                \
    const int64_t cap = (int64_t)sm_count() * (per_sm > 0 ? per_sm : 1);                                     \
    kern<<<(unsigned)(rows < cap ? rows : cap), threads, 0, st>>>(xp, sp, gidx, ngroups, y, scale, offset,   \
                                                                  rows, (int)k);                             \
  } break;
  switch (iters) {
    B200Q_DQX_CASE(1)
    B200Q_DQX_CASE(2)
    B200Q_DQX_CASE(4)
    B200Q_DQX_CASE(8)
    B200Q_DQX_CASE(16)
  }
#undef B200Q_DQX_CASE
  return check_launch("dynamic_quant (grouped / asymmetric)");
}

template <bool ASYM>
int dq_ext_dispatch(const void* x, int x_dtype, const void* smooth, int smooth_dtype, const int32_t* gidx, int ngroups,
                    int8_t* y, float* scale, float* offset, int64_t rows, int64_t k, cudaStream_t st) {
  const bool sm_f32 = smooth == nullptr || smooth_dtype == B200Q_F32;
  if (x_dtype == B200Q_BF16) {
    if (sm_f32) return launch_dq_ext<__nv_bfloat16, float, ASYM>(x, smooth, gidx, ngroups, y, scale, offset, rows, k, st);
    return launch_dq_ext<__nv_bfloat16, __nv_bfloat16, ASYM>(x, smooth, gidx, ngroups, y, scale, offset, rows, k, st);
  }
  if (sm_f32) return launch_dq_ext<__half, float, ASYM>(x, smooth, gidx, ngroups, y, scale, offset, rows, k, st);
  return launch_dq_ext<__half, __half, ASYM>(x, smooth, gidx, ngroups, y, scale, offset, rows, k, st);
}

}  // namespace
}  // namespace b200q

extern "C" int b200q_dynamic_quant_ext(const void* x, int x_dtype, const void* smooth, int smooth_dtype,
                                       const int32_t* group_index, int64_t n_groups, int8_t* y, float* scale,
                                       float* offset, int64_t rows, int64_t k, void* stream) {
  using namespace b200q;
  clear_error();
  B200Q_REQUIRE(rows >= 0 && k >= 0 && n_groups >= 0, B200Q_ERR_BAD_ARG, "dynamic_quant: negative size");
  B200Q_REQUIRE(x_dtype == B200Q_BF16 || x_dtype == B200Q_F16, B200Q_ERR_UNSUPPORTED,
                "dynamic_quant: input must be bf16 or f16 (dtype enum %d)", x_dtype);
  B200Q_REQUIRE(group_index == nullptr || (smooth != nullptr && n_groups >= 1 && n_groups <= 0x7fffffffLL),
                B200Q_ERR_BAD_ARG, "dynamic_quant: group_index needs smooth_scales of shape [groups, k]");
  if (rows == 0) return B200Q_OK;
  B200Q_REQUIRE(rows <= 0x7fffffffLL, B200Q_ERR_UNSUPPORTED, "dynamic_quant: more than 2^31-1 rows");
  B200Q_REQUIRE(scale != nullptr, B200Q_ERR_BAD_ARG, "dynamic_quant: scale is NULL");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (k == 0) {
    cudaError_t e = cudaMemsetAsync(scale, 0, rows * sizeof(float), st);
    if (e == cudaSuccess && offset) e = cudaMemsetAsync(offset, 0, rows * sizeof(float), st);
    return e == cudaSuccess ? B200Q_OK : fail(B200Q_ERR_LAUNCH, "dynamic_quant: %s", cudaGetErrorString(e));
  }
  B200Q_REQUIRE(x != nullptr && y != nullptr, B200Q_ERR_BAD_ARG, "dynamic_quant: x or y is NULL");
  B200Q_REQUIRE(aligned(x, 2) && aligned(scale, 4) && aligned(offset, 4) && aligned(group_index, 4), B200Q_ERR_BAD_ARG,
                "dynamic_quant: misaligned buffer");
  B200Q_REQUIRE(smooth == nullptr || smooth_dtype == B200Q_F32 || smooth_dtype == x_dtype, B200Q_ERR_UNSUPPORTED,
                "dynamic_quant: smooth_scales must be f32 or the input's dtype");
  if (offset != nullptr)
    return dq_ext_dispatch<true>(x, x_dtype, smooth, smooth_dtype, group_index, (int)n_groups, y, scale, offset, rows, k, st);
  return dq_ext_dispatch<false>(x, x_dtype, smooth, smooth_dtype, group_index, (int)n_groups, y, scale, nullptr, rows, k, st);
}
