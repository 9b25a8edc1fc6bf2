// npu_swiglu_quant (dynamic mode): the step between the gate/up projection and the down projection
// of a quantised MLP block in one pass.  x [rows, 2F] holds the two halves side by side;
// act = silu(a) * b with a the activated half (npu_swiglu activates the left one:
// torch_npu/_inductor/decomposition.py:186-188), xs = act * smooth, then the per-token symmetric
// int8 quantisation of npu_dynamic_quant.  Unfused, the activation would be written as bf16 and read
// back (4 B per output element); fused, the kernel reads 4 B and writes 1 B per output element and
// the activation never leaves fp32 registers.  Same row-per-CTA structure as dynamic_quant.cu.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"
#include "ptx.cuh"

namespace b200q {
namespace {

// Hardware reciprocal for operands in [1, 2^126]: the result is a normal number, so the flush-to-zero form
// (which skips the rescaling of the full-range form) returns the same value.
__device__ __forceinline__ float rcp_approx(float d) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(d));
  return y;
}

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// (silu(a.x) * b.x, silu(a.y) * b.y) with silu(a) = a * (1 / (1 + exp(-a))).  exp(-a) is the hardware
// 2^x of -a * log2(e) (what __expf computes, without its rescaling for results below the normal range, which
// vanish next to the 1 they are added to); the exponent is capped at 115 = 80 * log2(e), so the sum stays a
// normal number (for a < -80 the result is below 2e-33 in magnitude either way).  The reciprocal of a normal
// number: the hardware approximation (within one ulp) and one Newton step in two fused multiply-adds, which
// rounds like an IEEE division of 1 by the sum without that routine's checks for special operands.  Sums,
// products and the Newton step run as packed two-wide fp32 instructions.
__device__ __forceinline__ float2 silu_mul2(float2 a, float2 b) {
  const float2 one = make_float2(1.0f, 1.0f);
  const float2 t = __fmul2_rn(a, make_float2(-1.4426950408889634f, -1.4426950408889634f));
  const float2 d = __fadd2_rn(one, make_float2(ex2_approx(fminf(t.x, 115.0f)), ex2_approx(fminf(t.y, 115.0f))));
  const float2 y0 = make_float2(rcp_approx(d.x), rcp_approx(d.y));
  const float2 err = __ffma2_rn(make_float2(-d.x, -d.y), y0, one);
  const float2 s = __ffma2_rn(y0, err, y0);
  return __fmul2_rn(__fmul2_rn(a, s), b);
}

template <typename T, typename ST, int ITERS, bool WIDE>
__global__ void __launch_bounds__(WIDE ? 1024 : 512)
swiglu_quant_rows(const T* __restrict__ x, const ST* __restrict__ smooth, int8_t* __restrict__ y,
                  float* __restrict__ scale_out, int64_t rows, int f, int act_offset, int gate_offset) {
  __shared__ float red[2][32];
  const int nvec = f >> 3;
  // Rows up to 16384 outputs wide keep the next row's packed loads in flight during the arithmetic of
  // the current one.  Wider rows (WIDE: up to 1024 threads with four vectors each, 64 registers) need
  // the registers for the fp32 activations and load as they go; the larger CTA hides the latency.
  constexpr bool PREFETCH = !WIDE;
  uint4 ra[PREFETCH ? ITERS : 1], rb[PREFETCH ? ITERS : 1];
  // A thread's vector past the end of the row repeats the row's last vector (not stored).
  auto load_row = [&](int64_t row) {
    if (!PREFETCH) return;
    const uint4* xa = reinterpret_cast<const uint4*>(x + row * 2 * f + act_offset);
    const uint4* xb = reinterpret_cast<const uint4*>(x + row * 2 * f + gate_offset);
#pragma unroll
    for (int i = 0; i < (PREFETCH ? ITERS : 1); ++i) {
      const int v = min((int)(threadIdx.x + i * blockDim.x), nvec - 1);
      ra[i] = ld_stream(xa + v);
      rb[i] = ld_stream(xb + v);
    }
  };
  int par = 0;
  if ((int64_t)blockIdx.x < rows) load_row(blockIdx.x);
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x, par ^= 1) {
    float2 act[ITERS][4];
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < ITERS; ++i) {
      const int v = min((int)(threadIdx.x + i * blockDim.x), nvec - 1);
      uint4 qa, qb;
      if (PREFETCH) {
        qa = ra[PREFETCH ? i : 0];
        qb = rb[PREFETCH ? i : 0];
      } else {
        qa = ld_stream(reinterpret_cast<const uint4*>(x + row * 2 * f + act_offset) + v);
        qb = ld_stream(reinterpret_cast<const uint4*>(x + row * 2 * f + gate_offset) + v);
      }
      const uint32_t wa[4] = {qa.x, qa.y, qa.z, qa.w};
      const uint32_t wb[4] = {qb.x, qb.y, qb.z, qb.w};
      float2 sm[4];
      if (smooth != nullptr) load_smooth8(smooth + v * 8, sm);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 r = silu_mul2(unpack2<T>(wa[j]), unpack2<T>(wb[j]));
        if (smooth != nullptr) r = __fmul2_rn(r, sm[j]);
        act[i][j] = r;
        amax = fmaxf(amax, fmaxf(fabsf(r.x), fabsf(r.y)));
      }
    }
    if (row + gridDim.x < rows) {
      load_row(row + gridDim.x);                             // in flight during the reduction and quantisation
      if (!PREFETCH && (threadIdx.x & 7) == 0) {
        // Wide rows: no registers to spare for the next row, so its lines are at least brought into L2 while this
        // row is reduced and quantised (one prefetch per 128-byte line, by every eighth thread).
        const char* na = reinterpret_cast<const char*>(x + (row + gridDim.x) * 2 * f + act_offset);
        const char* nb = reinterpret_cast<const char*>(x + (row + gridDim.x) * 2 * f + gate_offset);
#pragma unroll
        for (int i = 0; i < ITERS; ++i) {
          const int v = threadIdx.x + i * blockDim.x;
          if (v < nvec) {
            prefetch_l2(na + (int64_t)v * 16);
            prefetch_l2(nb + (int64_t)v * 16);
          }
        }
      }
    }
    amax = block_max(amax, red[par]);
    const float scale = scale_of_amax(amax);
    if (threadIdx.x == 0) scale_out[row] = scale;
    const float inv = quant_inverse(scale);
    uint2* yr = reinterpret_cast<uint2*>(y + row * f) + threadIdx.x;
    if (inv == inv) {
#pragma unroll
      for (int i = 0; i < ITERS; ++i)
        if (threadIdx.x + i * blockDim.x < nvec) st_stream(yr + i * blockDim.x, quantize8<false>(act[i], scale, inv));
    } else {
#pragma unroll
      for (int i = 0; i < ITERS; ++i)
        if (threadIdx.x + i * blockDim.x < nvec) st_stream(yr + i * blockDim.x, quantize8<true>(act[i], scale, inv));
    }
  }
}

template <typename T, typename ST>
int launch_swiglu_quant(const void* x, const void* smooth, int8_t* y, float* scale, int64_t rows, int64_t f,
                        bool activate_left, cudaStream_t st) {
  const T* xp = static_cast<const T*>(x);
  const ST* sp = static_cast<const ST*>(smooth);
  const int nvec = (int)(f / 8);
  int iters = 1;
  while (iters < 4 && nvec > iters * 256) iters *= 2;
  const bool wide = nvec > 4 * 512;                      // four vectors per thread, up to 1024 threads
  int threads = (int)ceil_div(nvec, iters);
  threads = (int)ceil_div(threads, 32) * 32;
  const int act_off = activate_left ? 0 : (int)f, gate_off = activate_left ? (int)f : 0;
  int per_sm = 1;
#define B200Q_SGQ_CASE(I, W)                                                                                 \
  {                                                                                                          \
    auto kern = swiglu_quant_rows<T, ST, I, W>;                                                              \
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, threads, 0);                                \
    const int64_t cap = (int64_t)sm_count() * (per_sm > 0 ? per_sm : 1);                                     \
    kern<<<(unsigned)(rows < cap ? rows : cap), threads, 0, st>>>(xp, sp, y, scale, rows, (int)f, act_off,   \
                                                                  gate_off);                                 \
  }
  if (wide) B200Q_SGQ_CASE(4, true)
  else if (iters == 1) B200Q_SGQ_CASE(1, false)
  else if (iters == 2) B200Q_SGQ_CASE(2, false)
  else B200Q_SGQ_CASE(4, false)
#undef B200Q_SGQ_CASE
  return check_launch("swiglu_quant");
}

}  // namespace
}  // namespace b200q

extern "C" int b200q_swiglu_quant(const void* x, int x_dtype, const void* smooth, int smooth_dtype, int activate_left,
                                  int8_t* y, float* scale, int64_t rows, int64_t f, void* stream) {
  using namespace b200q;
  clear_error();
  B200Q_REQUIRE(rows >= 0 && f >= 0, B200Q_ERR_BAD_ARG, "swiglu_quant: negative size");
  B200Q_REQUIRE(x_dtype == B200Q_BF16 || x_dtype == B200Q_F16, B200Q_ERR_UNSUPPORTED,
                "swiglu_quant: input must be bf16 or f16 (dtype enum %d)", x_dtype);
  if (rows == 0) return B200Q_OK;
  B200Q_REQUIRE(rows <= 0x7fffffffLL, B200Q_ERR_UNSUPPORTED, "swiglu_quant: more than 2^31-1 rows");
  B200Q_REQUIRE(scale != nullptr, B200Q_ERR_BAD_ARG, "swiglu_quant: scale is NULL");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (f == 0) {
    cudaError_t e = cudaMemsetAsync(scale, 0, rows * sizeof(float), st);
    return e == cudaSuccess ? B200Q_OK : fail(B200Q_ERR_LAUNCH, "swiglu_quant: %s", cudaGetErrorString(e));
  }
  B200Q_REQUIRE(x != nullptr && y != nullptr, B200Q_ERR_BAD_ARG, "swiglu_quant: x or y is NULL");
  B200Q_REQUIRE(f % 8 == 0 && f <= 8 * 1024 * 4, B200Q_ERR_UNSUPPORTED,
                "swiglu_quant: the output width (%lld) must be a multiple of 8 and at most 32768", (long long)f);
  B200Q_REQUIRE(aligned(x, 16) && aligned(y, 8) && aligned(scale, 4) && (smooth == nullptr || aligned(smooth, 16)),
                B200Q_ERR_BAD_ARG, "swiglu_quant: x and smooth_scales must be 16-byte aligned, y 8-byte aligned");
  B200Q_REQUIRE(smooth == nullptr || smooth_dtype == B200Q_F32 || smooth_dtype == x_dtype, B200Q_ERR_UNSUPPORTED,
                "swiglu_quant: smooth_scales must be f32 or the input's dtype");
  const bool sm_f32 = smooth == nullptr || smooth_dtype == B200Q_F32;
  const bool left = activate_left != 0;
  if (x_dtype == B200Q_BF16) {
    if (sm_f32) return launch_swiglu_quant<__nv_bfloat16, float>(x, smooth, y, scale, rows, f, left, st);
    return launch_swiglu_quant<__nv_bfloat16, __nv_bfloat16>(x, smooth, y, scale, rows, f, left, st);
  }
  if (sm_f32) return launch_swiglu_quant<__half, float>(x, smooth, y, scale, rows, f, left, st);
  return launch_swiglu_quant<__half, __half>(x, smooth, y, scale, rows, f, left, st);
}
