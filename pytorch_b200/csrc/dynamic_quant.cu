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

// Eight consecutive smooth-scale values as fp32 (the vector is re-read by every row and
// stays in L1/L2).
__device__ __forceinline__ void load_smooth8(const float* p, float (&s)[8]) {
  const float4 a = __ldg(reinterpret_cast<const float4*>(p)), b = __ldg(reinterpret_cast<const float4*>(p) + 1);
  s[0] = a.x, s[1] = a.y, s[2] = a.z, s[3] = a.w, s[4] = b.x, s[5] = b.y, s[6] = b.z, s[7] = b.w;
}
template <typename ST>
__device__ __forceinline__ void load_smooth8(const ST* p, float (&s)[8]) {
  const uint4 a = __ldg(reinterpret_cast<const uint4*>(p));
  const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 f = unpack2<ST>(w[j]);
    s[2 * j] = f.x, s[2 * j + 1] = f.y;
  }
}

// Reciprocal of a row's scale for quantize8.  0 for an all-zero row (every product is then 0); NaN marks
// a scale so small that its reciprocal overflows or the refinement's residual could underflow: such a
// row is quantised with true divisions instead (the same decision for every thread of the row).
__device__ __forceinline__ float quant_inverse(float scale) {
  if (scale == 0.0f) return 0.0f;
  if (scale < 1e-30f) return __int_as_float(0x7fc00000);
  return __frcp_rn(scale);
}

// Eight values -> eight int8 (packed), bit-exact with clamp(rint(xs / scale)).
// With y = RN(1/scale): q0 = RN(f*y) is within one ulp of the quotient, r = f - q0*scale is exact in one
// fused multiply-add, and RN(q0 + r*y) is then the correctly rounded IEEE quotient (Markstein's division
// refinement; it needs y correctly rounded, which __frcp_rn gives, and no overflow or underflow, which
// quant_inverse rules out).  Adding 1.5 * 2^23 rounds that quotient to the nearest-even integer and leaves its
// two's-complement low byte in the low mantissa byte; |xs/scale| <= 127.0001 because scale = amax/127,
// so no clamp is needed.  No branch, no division.
__device__ __forceinline__ uint2 quantize8(const float (&f)[8], float scale, float inv) {
  constexpr float kMagic = 12582912.0f;
  uint32_t u[8];
  if (inv == inv) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float q0 = __fmul_rn(f[j], inv);
      const float r = __fmaf_rn(-q0, scale, f[j]);
      const float q = __fmaf_rn(r, inv, q0);
      u[j] = __float_as_uint(__fadd_rn(q, kMagic));
    }
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) u[j] = (uint32_t)__float2int_rn(__fdiv_rn(f[j], scale));
  }
  uint2 o;
  o.x = __byte_perm(__byte_perm(u[0], u[1], 0x0040), __byte_perm(u[2], u[3], 0x0040), 0x5410);
  o.y = __byte_perm(__byte_perm(u[4], u[5], 0x0040), __byte_perm(u[6], u[7], 0x0040), 0x5410);
  return o;
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
template <typename T, typename ST, int ITERS, bool SMOOTH, bool FULL>
__global__ void __launch_bounds__(ITERS == 4 ? 1024 : 512) dynamic_quant_rows(const T* __restrict__ x, const ST* __restrict__ smooth,
                                                         int8_t* __restrict__ y, float* __restrict__ scale_out,
                                                         int64_t rows, int k) {
  __shared__ float red[2][32];
  const int nvec = k >> 3;
  uint4 nxt[ITERS];
  float f[ITERS][8];
  auto load_row = [&](int64_t row) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * k) + threadIdx.x;
#pragma unroll
    for (int i = 0; i < ITERS; ++i)
      nxt[i] = (FULL || threadIdx.x + i * blockDim.x < nvec) ? ld_stream(xr + i * blockDim.x) : make_uint4(0, 0, 0, 0);
  };
  int64_t row = blockIdx.x;
  if (row < rows) load_row(row);
  int par = 0;
  for (; row < rows; row += gridDim.x, par ^= 1) {
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < ITERS; ++i) {
      const int v = threadIdx.x + i * blockDim.x;
      const uint32_t w[4] = {nxt[i].x, nxt[i].y, nxt[i].z, nxt[i].w};
      float sm[8];
      if (SMOOTH && (FULL || v < nvec)) load_smooth8(smooth + v * 8, sm);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 pr = unpack2<T>(w[j]);
        f[i][2 * j] = (SMOOTH && (FULL || v < nvec)) ? __fmul_rn(pr.x, sm[2 * j]) : pr.x;
        f[i][2 * j + 1] = (SMOOTH && (FULL || v < nvec)) ? __fmul_rn(pr.y, sm[2 * j + 1]) : pr.y;
        amax = fmaxf(amax, fmaxf(fabsf(f[i][2 * j]), fabsf(f[i][2 * j + 1])));
      }
    }
    if (row + gridDim.x < rows) load_row(row + gridDim.x);   // in flight during the reduction and quantisation
    amax = block_max(amax, red[par]);
    const float scale = __fdiv_rn(amax, 127.0f);
    if (threadIdx.x == 0) scale_out[row] = scale;
    const float inv = quant_inverse(scale);
    uint2* yr = reinterpret_cast<uint2*>(y + row * k) + threadIdx.x;
#pragma unroll
    for (int i = 0; i < ITERS; ++i)
      if (FULL || threadIdx.x + i * blockDim.x < nvec) st_stream(yr + i * blockDim.x, quantize8(f[i], scale, inv));
  }
}

// Staged kernel.  Persistent CTAs stride over the rows; thread 0 keeps `stages` rows in flight with one
// bulk copy per row into a shared-memory ring, each completing on its own mbarrier.  Per row: wait for the
// row, pull this thread's ITERS vectors out of shared memory, form the fp32 products x*smooth once and
// keep them in registers, reduce the row maximum (the __syncthreads inside also tells thread 0 that every
// thread has finished reading the stage, so it refills it with the row `stages` ahead at once), quantise
// from registers, stream the int8 out.  x is read from HBM exactly once and never waits on registers.
template <typename T, typename ST, int ITERS, bool SMOOTH>
__global__ void __launch_bounds__(512) dynamic_quant_staged(const T* __restrict__ x, const ST* __restrict__ smooth,
                                                           int8_t* __restrict__ y, float* __restrict__ scale_out,
                                                           int64_t rows, int k, int stages) {
  extern __shared__ __align__(128) uint8_t dq_smem[];
  __shared__ float red[2][32];
  __shared__ uint64_t full[12];
  __shared__ int abort_flag;
  const int nvec = k >> 3;
  const uint32_t row_bytes = (uint32_t)k * 2u;
  const uint32_t ring = smem_u32(dq_smem);
  if (threadIdx.x == 0) {
    for (int i = 0; i < stages; ++i) mbar_init(&full[i], 1);
    abort_flag = 0;
    fence_mbar_init();
  }
  __syncthreads();
  const uint64_t pol = policy_evict_first();
  auto fetch = [&](int64_t row, int stage) {          // thread 0 only
    mbar_arrive_expect_tx(&full[stage], row_bytes);
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
        ::"r"(ring + (uint32_t)stage * row_bytes), "l"(x + row * k), "r"(row_bytes), "r"(smem_u32(&full[stage])), "l"(pol)
        : "memory");
  };
  if (threadIdx.x == 0) {
    int64_t r = blockIdx.x;
    for (int i = 0; i < stages && r < rows; ++i, r += gridDim.x) fetch(r, i);
  }
  // The smooth scales of this thread's columns are the same for every row: keep them in registers when
  // they fit (ITERS <= 2), else re-read them (they stay in L1).
  float smk[ITERS <= 2 ? ITERS : 1][8];
  if (SMOOTH && ITERS <= 2) {
#pragma unroll
    for (int i = 0; i < ITERS; ++i) {
      const int v = threadIdx.x + i * blockDim.x;
      if (v < nvec) load_smooth8(smooth + v * 8, smk[i]);
    }
  }
  int stage = 0, par = 0;
  uint32_t phase = 0;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x, par ^= 1) {
    // A wait that gives up must end the loop for the whole CTA at the same place: the thread contributes a
    // sentinel above every float to the maximum reduction below, which every thread then sees.
    const bool got = mbar_wait(&full[stage], phase, &abort_flag, kDevTimeoutProducer);
    const uint32_t src = ring + (uint32_t)stage * row_bytes + threadIdx.x * 16;
    float f[ITERS][8];
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < ITERS; ++i) {
      const int v = threadIdx.x + i * blockDim.x;
      const bool in = got && v < nvec;
      const uint4 raw = in ? ld_shared_v4(src + i * blockDim.x * 16) : make_uint4(0, 0, 0, 0);
      const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
      float sm[8];
      if (SMOOTH && ITERS > 2 && in) load_smooth8(smooth + v * 8, sm);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 pr = unpack2<T>(w[j]);
        const float s0 = !SMOOTH ? 1.0f : (ITERS <= 2 ? smk[ITERS <= 2 ? i : 0][2 * j] : sm[2 * j]);
        const float s1 = !SMOOTH ? 1.0f : (ITERS <= 2 ? smk[ITERS <= 2 ? i : 0][2 * j + 1] : sm[2 * j + 1]);
        f[i][2 * j] = (SMOOTH && in) ? __fmul_rn(pr.x, s0) : pr.x;
        f[i][2 * j + 1] = (SMOOTH && in) ? __fmul_rn(pr.y, s1) : pr.y;
        amax = fmaxf(amax, fmaxf(fabsf(f[i][2 * j]), fabsf(f[i][2 * j + 1])));
      }
    }
    amax = block_max(got ? amax : __uint_as_float(0xFFFFFFFFu), red[par]);   // every thread has read its part of the stage
    if (__float_as_uint(amax) == 0xFFFFFFFFu) break;
    if (threadIdx.x == 0) {
      const int64_t nxt = row + (int64_t)stages * gridDim.x;
      if (nxt < rows) fetch(nxt, stage);
    }
    const float scale = __fdiv_rn(amax, 127.0f);
    if (threadIdx.x == 0) scale_out[row] = scale;
    const float inv = quant_inverse(scale);
    uint2* yr = reinterpret_cast<uint2*>(y + row * k) + threadIdx.x;
#pragma unroll
    for (int i = 0; i < ITERS; ++i)
      if (threadIdx.x + i * blockDim.x < nvec) st_stream(yr + i * blockDim.x, quantize8(f[i], scale, inv));
    if (++stage == stages) { stage = 0; phase ^= 1; }
  }
  // Copies still in flight when a wait gave up must land before the shared memory is released.
  if (abort_flag && threadIdx.x == 0)
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  __syncthreads();
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
  if (k >= 1024 && k <= 32768) {
    // Staged kernel: the fewest vectors per thread that keep the CTA at 384 threads or fewer (eight vectors
    // and up to 512 threads for the longest rows); as many CTAs per SM as 64 KB (rows up to 16 KB), 96 KB
    // (up to 32 KB) or 200 KB rings allow.
    int it = 1;
    while (it < 8 && ceil_div(nvec, it) > (it == 4 ? 512 : 384)) it *= 2;
    int threads = (int)ceil_div(ceil_div(nvec, it), 32) * 32;
    const int64_t row_bytes = k * 2;
    const int64_t budget = row_bytes <= 16384 ? 65536 : row_bytes <= 32768 ? 98304 : 204800;
    int stages = (int)(budget / row_bytes);
    stages = stages > 12 ? 12 : stages < 2 ? 2 : stages;
    const int smem = (int)(stages * row_bytes);
    int per_sm = 1;
#define B200Q_DQS_LAUNCH(I)                                                                                    \
  {                                                                                                            \
    constexpr auto kern = dynamic_quant_staged<T, ST, I, SMOOTH>;                                             \
    if (int rc = ensure_dynamic_smem<kern>(204800, "dynamic_quant")) return rc;                               \
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, threads, smem);                               \
    const int64_t cap = (int64_t)sm_count() * (per_sm > 0 ? per_sm : 1);                                       \
    kern<<<(unsigned)(rows < cap ? rows : cap), threads, smem, st>>>(xp, sp, y, scale, rows, (int)k, stages); \
  }
    switch (it) {
      case 1: B200Q_DQS_LAUNCH(1) break;
      case 2: B200Q_DQS_LAUNCH(2) break;
      case 4: B200Q_DQS_LAUNCH(4) break;
      default: B200Q_DQS_LAUNCH(8) break;
    }
#undef B200Q_DQS_LAUNCH
    return check_launch("dynamic_quant (staged)");
  }
  // Up to four 128-bit loads per thread (32 fp32 products kept in registers) with <= 256 threads where
  // the row allows it (k <= 8192); longer rows widen the CTA up to 1024 threads (k <= 32768), then take
  // 8 and 16 loads per thread with 512 threads.
  int iters = 1;
  while (iters < 4 && nvec > iters * 256) iters *= 2;
  if (nvec > 4 * 1024)                                   // k > 32768: more loads per thread
    while (iters < 16 && nvec > iters * 512) iters *= 2;
  int threads = (int)ceil_div(nvec, iters);
  threads = (int)ceil_div(threads, 32) * 32;
  const bool full = (int64_t)threads * iters == nvec;
  int per_sm = 1;
#define B200Q_DQ_LAUNCH(I, F)                                                                                 \
  {                                                                                                            \
    auto kern = dynamic_quant_rows<T, ST, I, SMOOTH, F>;                                                       \
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, threads, 0);                                  \
    const int64_t cap = (int64_t)sm_count() * (per_sm > 0 ? per_sm : 1);                                       \
    kern<<<(unsigned)(rows < cap ? rows : cap), threads, 0, st>>>(xp, sp, y, scale, rows, (int)k);            \
  }
#define B200Q_DQ_CASE(I)                                  \
  case I:                                                 \
    if (full) B200Q_DQ_LAUNCH(I, true) else B200Q_DQ_LAUNCH(I, false) \
    break;
  switch (iters) {
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
