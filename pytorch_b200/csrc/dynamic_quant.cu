// npu_dynamic_quant: per-token symmetric int8 quantisation (memory-bound row kernel).
//
// One CTA works on one row at a time (persistent CTAs stride over the rows).  Every thread keeps
// its slice of the row in registers (ITERS 128-bit loads, all issued before the first use, the next
// row's loads in flight during the arithmetic), so x is read from HBM exactly once:
// 2 B in + 1 B out per element.  The row maximum is a warp-shuffle reduction followed by
// one exchange through shared memory.  Quantisation is bit-exact with
// rint(xs / scale) under IEEE division: the fast path multiplies by 1/scale and only a
// vector with an element within 1e-4 of a rounding boundary (where the two could differ)
// is redone with a true division.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <stdlib.h>

#include "common.cuh"

namespace b200q {
namespace {

template <typename T>
__device__ __forceinline__ float2 unpack2(uint32_t v);
template <>
__device__ __forceinline__ float2 unpack2<__nv_bfloat16>(uint32_t v) {
  // bf16 -> fp32 is a 16-bit shift
  return make_float2(__uint_as_float(v << 16), __uint_as_float(v & 0xFFFF0000u));
}
template <>
__device__ __forceinline__ float2 unpack2<__half>(uint32_t v) {
  return __half22float2(*reinterpret_cast<const __half2*>(&v));
}
template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <>
__device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }

__device__ __forceinline__ uint4 ld_stream(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ void st_stream(uint2* p, uint2 v) {
  asm volatile("st.global.cs.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(v.x), "r"(v.y) : "memory");
}

// Eight consecutive smooth-scale values as four fp32 pairs (the vector is re-read by every row and
// stays in L1/L2).
__device__ __forceinline__ void load_smooth8(const float* p, float2 (&s)[4]) {
  const float4 a = __ldg(reinterpret_cast<const float4*>(p)), b = __ldg(reinterpret_cast<const float4*>(p) + 1);
  s[0] = make_float2(a.x, a.y), s[1] = make_float2(a.z, a.w), s[2] = make_float2(b.x, b.y), s[3] = make_float2(b.z, b.w);
}
template <typename ST>
__device__ __forceinline__ void load_smooth8(const ST* p, float2 (&s)[4]) {
  const uint4 a = __ldg(reinterpret_cast<const uint4*>(p));
  const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) s[j] = unpack2<ST>(w[j]);
}

// Reciprocal of a row's scale for quantize8.  0 for an all-zero row (every product is then 0); NaN marks
// a scale so small that its reciprocal overflows or the refinement's residual could underflow: such a
// row is quantised with true divisions instead (the same decision for every thread of the row).
__device__ __forceinline__ float quant_inverse(float scale) {
  if (scale == 0.0f) return 0.0f;
  if (scale < 1e-30f) return __int_as_float(0x7fc00000);
  return __frcp_rn(scale);
}

// Eight values (four fp32 pairs) -> eight int8 (packed), bit-exact with clamp(rint(xs / scale)).
// With y = RN(1/scale): q0 = RN(f*y) is within one ulp of the quotient, r = f - q0*scale is exact in one
// fused multiply-add, and RN(q0 + r*y) is then the correctly rounded IEEE quotient (Markstein's division
// refinement; it needs y correctly rounded, which __frcp_rn gives, and no overflow or underflow, which
// quant_inverse rules out).  Adding 1.5 * 2^23 rounds that quotient to the nearest-even integer and leaves its
// two's-complement low byte in the low mantissa byte; |xs/scale| <= 127.0001 because scale = amax/127,
// so no clamp is needed.  No branch, no division; the four steps are packed two-wide fp32 instructions
// (fma.rn.f32x2 and friends of sm_100), each lane rounded exactly like the scalar instruction, which halves
// the issue slots of a kernel that is bound by instruction issue, not by arithmetic.
// EXACT = false: the refinement above (inv is a finite reciprocal or 0); EXACT = true: true divisions (inv is
// NaN).  The choice is the same for a whole row, so callers branch once per row, not once per vector.
template <bool EXACT>
__device__ __forceinline__ uint2 quantize8(const float2 (&f)[4], float scale, float inv) {
  uint32_t u[8];
  if (!EXACT) {
    const float2 inv2 = make_float2(inv, inv), nscale2 = make_float2(-scale, -scale);
    const float2 magic2 = make_float2(12582912.0f, 12582912.0f);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 q0 = __fmul2_rn(f[j], inv2);
      const float2 r = __ffma2_rn(q0, nscale2, f[j]);
      const float2 q = __ffma2_rn(r, inv2, q0);
      const float2 m = __fadd2_rn(q, magic2);
      u[2 * j] = __float_as_uint(m.x);
      u[2 * j + 1] = __float_as_uint(m.y);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      u[2 * j] = (uint32_t)__float2int_rn(__fdiv_rn(f[j].x, scale));
      u[2 * j + 1] = (uint32_t)__float2int_rn(__fdiv_rn(f[j].y, scale));
    }
  }
  uint2 o;
  o.x = __byte_perm(__byte_perm(u[0], u[1], 0x0040), __byte_perm(u[2], u[3], 0x0040), 0x5410);
  o.y = __byte_perm(__byte_perm(u[4], u[5], 0x0040), __byte_perm(u[6], u[7], 0x0040), 0x5410);
  return o;
}

// The same for callers that hold eight separate floats.
template <bool EXACT>
__device__ __forceinline__ uint2 quantize8(const float (&f)[8], float scale, float inv) {
  const float2 g[4] = {{f[0], f[1]}, {f[2], f[3]}, {f[4], f[5]}, {f[6], f[7]}};
  return quantize8<EXACT>(g, scale, inv);
}

// RN(amax / 127), the row's scale, without the division routine: the same refinement with the constant
// reciprocal.  Equal to the IEEE quotient for every float from 1e-30 up (checked exhaustively on the host);
// smaller maxima take the division.
__device__ __forceinline__ float scale_of_amax(float amax) {
  if (amax < 1e-30f) return __fdiv_rn(amax, 127.0f);
  const float r = __uint_as_float(0x3C010204u);          // RN(1/127)
  const float q0 = __fmul_rn(amax, r);
  return __fmaf_rn(__fmaf_rn(-q0, 127.0f, amax), r, q0);
}

template <typename ST>
__device__ __forceinline__ void load_smooth8(const ST* p, float (&s)[8]) {
  float2 t[4];
  load_smooth8(p, t);
#pragma unroll
  for (int j = 0; j < 4; ++j) s[2 * j] = t[j].x, s[2 * j + 1] = t[j].y;
}

// x*smooth for the four pairs of one vector, and the running maximum of their magnitudes.
template <typename T, bool SMOOTH>
__device__ __forceinline__ void products8(const uint4& raw, const float2 (&sm)[4], float2 (&f)[4], float& amax) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 pr = unpack2<T>(w[j]);
    f[j] = SMOOTH ? __fmul2_rn(pr, sm[j]) : pr;
    amax = fmaxf(amax, fmaxf(fabsf(f[j].x), fabsf(f[j].y)));
  }
}

// Maximum of a non-negative value over the CTA.  Non-negative floats order like their bit patterns,
// so each warp reduces with one integer redux instruction; one exchange through shared memory joins
// the warps.
__device__ __forceinline__ float block_max(float v, float* red) {
  const unsigned w = __reduce_max_sync(0xffffffffu, __float_as_uint(v));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = (blockDim.x + 31) >> 5;
  if (lane == 0) red[warp] = __uint_as_float(w);
  __syncthreads();
  const unsigned m = __float_as_uint((lane < nwarps) ? red[lane] : 0.0f);
  return __uint_as_float(__reduce_max_sync(0xffffffffu, m));
}

// Vector path: k % 8 == 0 and 16-byte aligned rows.  Thread t owns vectors t, t+blockDim, ...
// Persistent CTAs walk the rows with a stride of gridDim.x; the packed 16-bit loads of the CTA's
// next row are issued before the arithmetic of the current one.  The fp32 products x*smooth are
// formed once, in the max pass, and kept in registers for the quantisation pass.  FULL means that
// every thread's every vector is inside the row (k == 8 * ITERS * blockDim): no bounds predicates.
// TH is the CTA size when it is one of the common ones (then every load, store and smooth-scale address is a
// per-thread base plus a compile-time offset), else 0 (taken from blockDim).
template <typename T, typename ST, int ITERS, bool SMOOTH, bool FULL, int TH = 0>
__global__ void __launch_bounds__(TH ? TH : (ITERS == 4 ? 1024 : 512), TH == 256 ? 4 : 1)
dynamic_quant_rows(const T* __restrict__ x, const ST* __restrict__ smooth, int8_t* __restrict__ y,
                   float* __restrict__ scale_out, int64_t rows, int k) {
  __shared__ float red[2][32];
  const int nvec = k >> 3;
  const int nth = TH ? TH : (int)blockDim.x;
  uint4 nxt[ITERS];
  float2 f[ITERS][4];
  const ST* sm_base = smooth + (int64_t)threadIdx.x * 8;
  auto load_row = [&](int64_t row) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * k) + threadIdx.x;
#pragma unroll
    for (int i = 0; i < ITERS; ++i)
      nxt[i] = (FULL || threadIdx.x + i * nth < nvec) ? ld_stream(xr + i * nth) : make_uint4(0, 0, 0, 0);
  };
  int64_t row = blockIdx.x;
  if (row < rows) load_row(row);
  int par = 0;
  for (; row < rows; row += gridDim.x, par ^= 1) {
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < ITERS; ++i) {
      const int v = threadIdx.x + i * nth;
      float2 sm[4] = {{1.0f, 1.0f}, {1.0f, 1.0f}, {1.0f, 1.0f}, {1.0f, 1.0f}};     // past the row: 0 * 1
      if (SMOOTH && (FULL || v < nvec)) load_smooth8(sm_base + i * nth * 8, sm);
      products8<T, SMOOTH>(nxt[i], sm, f[i], amax);
    }
    if (row + gridDim.x < rows) load_row(row + gridDim.x);   // in flight during the reduction and quantisation
    amax = block_max(amax, red[par]);
    const float scale = scale_of_amax(amax);
    if (threadIdx.x == 0) scale_out[row] = scale;
    const float inv = quant_inverse(scale);
    uint2* yr = reinterpret_cast<uint2*>(y + row * k) + threadIdx.x;
    if (inv == inv) {
#pragma unroll
      for (int i = 0; i < ITERS; ++i)
        if (FULL || threadIdx.x + i * nth < nvec) st_stream(yr + i * nth, quantize8<false>(f[i], scale, inv));
    } else {
#pragma unroll
      for (int i = 0; i < ITERS; ++i)
        if (FULL || threadIdx.x + i * nth < nvec) st_stream(yr + i * nth, quantize8<true>(f[i], scale, inv));
    }
  }
}

// Generic path: any k, any alignment; the row is read twice (second pass from L2).
template <typename T, typename ST, bool SMOOTH>
__global__ void dynamic_quant_rows_generic(const T* __restrict__ x, const ST* __restrict__ smooth,
                                           int8_t* __restrict__ y, float* __restrict__ scale_out, int64_t k) {
  __shared__ float red[32];
  const int64_t row = blockIdx.x;
  const T* xr = x + row * k;
  float amax = 0.0f;
  for (int64_t c = threadIdx.x; c < k; c += blockDim.x) {
    float f = to_f32<T>(xr[c]);
    if (SMOOTH) f = __fmul_rn(f, to_f32<ST>(smooth[c]));
    amax = fmaxf(amax, fabsf(f));
  }
  amax = block_max(amax, red);
  const float scale = __fdiv_rn(amax, 127.0f);
  if (threadIdx.x == 0) scale_out[row] = scale;
  for (int64_t c = threadIdx.x; c < k; c += blockDim.x) {
    float f = to_f32<T>(xr[c]);
    if (SMOOTH) f = __fmul_rn(f, to_f32<ST>(smooth[c]));
    int q = 0;
    if (scale != 0.0f) q = max(-128, min(127, __float2int_rn(rintf(__fdiv_rn(f, scale)))));
    y[row * k + c] = static_cast<int8_t>(q);
  }
}

template <typename T, typename ST, bool SMOOTH>
int launch_dq(const void* x, const void* smooth, int8_t* y, float* scale, int64_t rows, int64_t k,
              cudaStream_t st) {
  const T* xp = static_cast<const T*>(x);
  const ST* sp = static_cast<const ST*>(smooth);
  const bool vec = (k % 8 == 0) && aligned(x, 16) && aligned(y, 8) && k <= 8 * 512 * 16 &&
                   (!SMOOTH || aligned(smooth, 16));
  if (!vec) {
    dynamic_quant_rows_generic<T, ST, SMOOTH><<<(unsigned)rows, 256, 0, st>>>(xp, sp, y, scale, k);
    return check_launch("dynamic_quant (generic)");
  }
  const int nvec = (int)(k / 8);
  // Up to four 128-bit loads per thread (32 fp32 products kept in registers) with <= 256 threads where
  // the row allows it (k <= 8192); longer rows widen the CTA up to 1024 threads (k <= 32768), then take
  // 8 and 16 loads per thread with 512 threads.
  int iters = 1;
  while (iters < 4 && nvec > iters * 256) iters *= 2;
  if (nvec > 4 * 1024)                                   // k > 32768: more loads per thread
    while (iters < 16 && nvec > iters * 512) iters *= 2;
  if (const char* env = getenv("B200Q_DQ_ITERS")) {       // tuning aid: force the loads per thread
    const int v = atoi(env);
    if ((v == 1 || v == 2 || v == 4 || v == 8 || v == 16) && ceil_div(nvec, v) <= (v == 4 ? 1024 : 512)) iters = v;
  }
  int threads = (int)ceil_div(nvec, iters);
  threads = (int)ceil_div(threads, 32) * 32;
  const bool full = (int64_t)threads * iters == nvec;
  int per_sm = 1;
#define B200Q_DQ_LAUNCH(I, F, TH)                                                                             \
  {                                                                                                            \
    auto kern = dynamic_quant_rows<T, ST, I, SMOOTH, F, TH>;                                                   \
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, threads, 0);                                  \
    const int64_t cap = (int64_t)sm_count() * (per_sm > 0 ? per_sm : 1);                                       \
    kern<<<(unsigned)(rows < cap ? rows : cap), threads, 0, st>>>(xp, sp, y, scale, rows, (int)k);            \
  }
#define B200Q_DQ_CASE(I)                                  \
  case I:                                                 \
    if (full) B200Q_DQ_LAUNCH(I, true, 0) else B200Q_DQ_LAUNCH(I, false, 0) \
    break;
  // The common full-row shapes (k = 2048 * iters, 7168 * iters, 8192 * iters) with the CTA size compiled in.
  if (full && iters == 4 && threads == 256) B200Q_DQ_LAUNCH(4, true, 256)
  else if (full && iters == 4 && threads == 896) B200Q_DQ_LAUNCH(4, true, 896)
  else if (full && iters == 4 && threads == 1024) B200Q_DQ_LAUNCH(4, true, 1024)
  else if (full && iters == 2 && threads == 256) B200Q_DQ_LAUNCH(2, true, 256)
  else switch (iters) {
    B200Q_DQ_CASE(1)
    B200Q_DQ_CASE(2)
    B200Q_DQ_CASE(4)
    B200Q_DQ_CASE(8)
    B200Q_DQ_CASE(16)
  }
#undef B200Q_DQ_CASE
#undef B200Q_DQ_LAUNCH
  return check_launch("dynamic_quant");
}

}  // namespace
}  // namespace b200q

extern "C" int b200q_dynamic_quant(const void* x, int x_dtype, const void* smooth, int smooth_dtype, int8_t* y,
                                   float* scale, int64_t rows, int64_t k, void* stream) {
  using namespace b200q;
  clear_error();
  B200Q_REQUIRE(rows >= 0 && k >= 0, B200Q_ERR_BAD_ARG, "dynamic_quant: negative size");
  B200Q_REQUIRE(x_dtype == B200Q_BF16 || x_dtype == B200Q_F16, B200Q_ERR_UNSUPPORTED,
                "dynamic_quant: input must be bf16 or f16 (dtype enum %d)", x_dtype);
  if (rows == 0) return B200Q_OK;
  B200Q_REQUIRE(rows <= 0x7fffffffLL, B200Q_ERR_UNSUPPORTED, "dynamic_quant: more than 2^31-1 rows");
  B200Q_REQUIRE(scale != nullptr, B200Q_ERR_BAD_ARG, "dynamic_quant: scale is NULL");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (k == 0) {
    cudaError_t e = cudaMemsetAsync(scale, 0, rows * sizeof(float), st);
    return e == cudaSuccess ? B200Q_OK : fail(B200Q_ERR_LAUNCH, "dynamic_quant: %s", cudaGetErrorString(e));
  }
  B200Q_REQUIRE(x != nullptr && y != nullptr, B200Q_ERR_BAD_ARG, "dynamic_quant: x or y is NULL");
  B200Q_REQUIRE(aligned(x, 2) && aligned(scale, 4), B200Q_ERR_BAD_ARG, "dynamic_quant: misaligned buffer");
  if (smooth == nullptr) {
    if (x_dtype == B200Q_BF16) return launch_dq<__nv_bfloat16, float, false>(x, nullptr, y, scale, rows, k, st);
    return launch_dq<__half, float, false>(x, nullptr, y, scale, rows, k, st);
  }
  B200Q_REQUIRE(smooth_dtype == B200Q_F32 || smooth_dtype == x_dtype, B200Q_ERR_UNSUPPORTED,
                "dynamic_quant: smooth_scales must be f32 or the input's dtype");
  if (x_dtype == B200Q_BF16) {
    if (smooth_dtype == B200Q_F32) return launch_dq<__nv_bfloat16, float, true>(x, smooth, y, scale, rows, k, st);
    return launch_dq<__nv_bfloat16, __nv_bfloat16, true>(x, smooth, y, scale, rows, k, st);
  }
  if (smooth_dtype == B200Q_F32) return launch_dq<__half, float, true>(x, smooth, y, scale, rows, k, st);
  return launch_dq<__half, __half, true>(x, smooth, y, scale, rows, k, st);
}
