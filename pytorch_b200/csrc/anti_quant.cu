// npu_anti_quant: int8 / packed int4 -> fp16 / bf16, out = cast((float(x) + offset) * scale)
// with per-column fp32 (or bf16) scale and offset.  Memory-bound element kernel: 1 B (int8) or
// 0.5 B (int4) in and 2 B out per element; scale and offset are re-read by every row and stay in L1.
// The sum and the product are separate fp32 roundings (no fused multiply-add), then one
// round-to-nearest-even cast, exactly as the reference's golden composes them
// (test/custom_ops/test_npu_anti_quant.py:29-42).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"

namespace b200q {
namespace {

template <typename PT>
__device__ __forceinline__ float aq_param(const PT* p, int64_t i);
template <>
__device__ __forceinline__ float aq_param<float>(const float* p, int64_t i) { return __ldg(p + i); }
template <>
__device__ __forceinline__ float aq_param<__nv_bfloat16>(const __nv_bfloat16* p, int64_t i) {
  return __bfloat162float(p[i]);
}

// Sixteen consecutive per-column parameters as fp32 (16-byte aligned source).
__device__ __forceinline__ void aq_load16(const float* p, float (&s)[16]) {
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const float4 v = __ldg(reinterpret_cast<const float4*>(p) + q);
    s[4 * q] = v.x, s[4 * q + 1] = v.y, s[4 * q + 2] = v.z, s[4 * q + 3] = v.w;
  }
}
__device__ __forceinline__ void aq_load16(const __nv_bfloat16* p, float (&s)[16]) {
#pragma unroll
  for (int q = 0; q < 2; ++q) {
    const uint4 v = __ldg(reinterpret_cast<const uint4*>(p) + q);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      s[8 * q + 2 * j] = __uint_as_float(w[j] << 16);
      s[8 * q + 2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
    }
  }
}

template <typename OT>
__device__ __forceinline__ uint32_t aq_pack(float a, float b);
template <>
__device__ __forceinline__ uint32_t aq_pack<__half>(float a, float b) {
  __half2 r = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&r);
}
template <>
__device__ __forceinline__ uint32_t aq_pack<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 r = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&r);
}
template <typename OT>
__device__ __forceinline__ OT aq_cast(float a);
template <>
__device__ __forceinline__ __half aq_cast<__half>(float a) { return __float2half_rn(a); }
template <>
__device__ __forceinline__ __nv_bfloat16 aq_cast<__nv_bfloat16>(float a) { return __float2bfloat16_rn(a); }

__device__ __forceinline__ float aq_one(float x, float sc, float of, bool has_off) {
  return __fmul_rn(has_off ? __fadd_rn(x, of) : x, sc);
}

// Integers placed in the mantissa of 2^23 and one exact subtraction: cheaper than the
// quarter-rate integer-to-float conversion.  int8: byte b of the word, biased by 128.
__device__ __forceinline__ float aq_byte_to_float(uint32_t w_biased, int b) {
  // selector 0x7440 | b: result bytes (b, 4, 4, 7) of {w_biased, 0x4B000000} = 0x4B0000bb
  return __fsub_rn(__uint_as_float(__byte_perm(w_biased, 0x4B000000u, 0x7440 | b)), 8388736.0f);
}
__device__ __forceinline__ float aq_nibble_to_float(uint32_t w_biased, int j) {
  return __fsub_rn(__uint_as_float(((w_biased >> (4 * j)) & 0xFu) | 0x4B000000u), 8388616.0f);
}

// Vector path: n % 16 == 0, all buffers 16-byte aligned.  A thread owns 16 consecutive columns
// (its scale and offset values stay in registers) and walks down the rows: per row one 128-bit
// (int8) or 64-bit (int4, value j of a word in bits [4j, 4j+4)) load and two 128-bit stores, the
// loads of UNROLL rows issued before the first use so that enough bytes are in flight to cover
// the HBM latency.  Without an offset the sum adds 0.0, which leaves the integer unchanged.
template <int BITS, typename PT, typename OT>
__global__ void __launch_bounds__(256, 3) anti_quant_vec_kernel(const void* __restrict__ x, const PT* __restrict__ scale,
                                                                const PT* __restrict__ offset, OT* __restrict__ out,
                                                                int64_t rows, int vec_per_row) {
  constexpr int UNROLL = 4;
  const int cv = blockIdx.x * blockDim.x + threadIdx.x;
  if (cv >= vec_per_row) return;
  float sc[16], of[16];
  aq_load16(scale + cv * 16, sc);
  if (offset != nullptr) {
    aq_load16(offset + cv * 16, of);
  } else {
#pragma unroll
    for (int j = 0; j < 16; ++j) of[j] = 0.0f;
  }
  const int64_t rstep = gridDim.y;
  for (int64_t r0 = blockIdx.y; r0 < rows; r0 += rstep * UNROLL) {
    uint4 q[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int64_t r = r0 + u * rstep;
      q[u] = make_uint4(0, 0, 0, 0);
      if (r < rows) {
        const int64_t v = r * vec_per_row + cv;
        if (BITS == 8) q[u] = __ldcs(static_cast<const uint4*>(x) + v);
        else { const uint2 t = __ldcs(static_cast<const uint2*>(x) + v); q[u].x = t.x; q[u].y = t.y; }
      }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int64_t r = r0 + u * rstep;
      if (r >= rows) break;
      uint32_t o[8];
      if (BITS == 8) {
        const uint32_t w[4] = {q[u].x ^ 0x80808080u, q[u].y ^ 0x80808080u, q[u].z ^ 0x80808080u, q[u].w ^ 0x80808080u};
#pragma unroll
        for (int j = 0; j < 16; j += 2) {
          // packed two-wide fp32: exact subtraction of the bias, rounded sum with the offset, rounded product
          const float2 raw = make_float2(__uint_as_float(__byte_perm(w[j >> 2], 0x4B000000u, 0x7440 | (j & 3))),
                                         __uint_as_float(__byte_perm(w[j >> 2], 0x4B000000u, 0x7440 | ((j & 3) + 1))));
          const float2 v = __fadd2_rn(raw, make_float2(-8388736.0f, -8388736.0f));
          const float2 r = __fmul2_rn(__fadd2_rn(v, make_float2(of[j], of[j + 1])), make_float2(sc[j], sc[j + 1]));
          o[j >> 1] = aq_pack<OT>(r.x, r.y);
        }
      } else {
        const uint32_t w[2] = {q[u].x ^ 0x88888888u, q[u].y ^ 0x88888888u};
#pragma unroll
        for (int j = 0; j < 16; j += 2) {
          const float2 raw = make_float2(__uint_as_float(((w[j >> 3] >> (4 * (j & 7))) & 0xFu) | 0x4B000000u),
                                         __uint_as_float(((w[j >> 3] >> (4 * ((j & 7) + 1))) & 0xFu) | 0x4B000000u));
          const float2 v = __fadd2_rn(raw, make_float2(-8388616.0f, -8388616.0f));
          const float2 r = __fmul2_rn(__fadd2_rn(v, make_float2(of[j], of[j + 1])), make_float2(sc[j], sc[j + 1]));
          o[j >> 1] = aq_pack<OT>(r.x, r.y);
        }
      }
      uint4* dst = reinterpret_cast<uint4*>(out) + 2 * (r * vec_per_row + cv);
      __stcs(dst, make_uint4(o[0], o[1], o[2], o[3]));
      __stcs(dst + 1, make_uint4(o[4], o[5], o[6], o[7]));
    }
  }
}

// Any n (int4: any multiple of 8), any alignment: one thread per output element.
template <int BITS, typename PT, typename OT>
__global__ void anti_quant_generic_kernel(const void* __restrict__ x, const PT* __restrict__ scale,
                                          const PT* __restrict__ offset, OT* __restrict__ out, int64_t total,
                                          int64_t n) {
  const bool has_off = offset != nullptr;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t c = i % n;
    float xv;
    if (BITS == 8) {
      xv = (float)static_cast<const int8_t*>(x)[i];
    } else {
      const uint32_t w = static_cast<const uint32_t*>(x)[i >> 3];
      xv = (float)(((int32_t)(w << (28 - 4 * (i & 7)))) >> 28);
    }
    out[i] = aq_cast<OT>(aq_one(xv, aq_param<PT>(scale, c), has_off ? aq_param<PT>(offset, c) : 0.0f, has_off));
  }
}

template <int BITS, typename PT, typename OT>
int launch_anti_quant(const void* x, const void* scale, const void* offset, void* out, int64_t rows, int64_t n,
                      cudaStream_t st) {
  const int64_t total = rows * n;
  const bool vec = n % 16 == 0 && aligned(x, 16) && aligned(out, 16) && aligned(scale, 16) &&
                   (offset == nullptr || aligned(offset, 16));
  if (vec) {
    const int vpr = (int)(n / 16);
    const int threads = vpr >= 256 ? 256 : (int)ceil_div(vpr, 32) * 32;
    const unsigned gx = (unsigned)ceil_div(vpr, threads);
    // about three CTAs of 256 threads per SM; every CTA takes at least UNROLL rows
    int64_t gy = ceil_div((int64_t)sm_count() * 3 * 256, (int64_t)gx * threads);
    const int64_t max_gy = ceil_div(rows, 4);
    if (gy > max_gy) gy = max_gy;
    if (gy > 65535) gy = 65535;
    if (gy < 1) gy = 1;
    anti_quant_vec_kernel<BITS, PT, OT><<<dim3(gx, (unsigned)gy), threads, 0, st>>>(
        x, static_cast<const PT*>(scale), static_cast<const PT*>(offset), static_cast<OT*>(out), rows, vpr);
    return check_launch("anti_quant");
  }
  const int64_t want = ceil_div(total, 256);
  const int blocks = (int)(want < (int64_t)sm_count() * 16 ? want : (int64_t)sm_count() * 16);
  anti_quant_generic_kernel<BITS, PT, OT><<<blocks, 256, 0, st>>>(x, static_cast<const PT*>(scale),
                                                                   static_cast<const PT*>(offset), static_cast<OT*>(out),
                                                                   total, n);
  return check_launch("anti_quant (generic)");
}

template <int BITS, typename PT>
int anti_quant_out(int out_dtype, const void* x, const void* scale, const void* offset, void* out, int64_t rows,
                   int64_t n, cudaStream_t st) {
  if (out_dtype == B200Q_F16) return launch_anti_quant<BITS, PT, __half>(x, scale, offset, out, rows, n, st);
  return launch_anti_quant<BITS, PT, __nv_bfloat16>(x, scale, offset, out, rows, n, st);
}

}  // namespace
}  // namespace b200q

extern "C" int b200q_anti_quant(const void* x, int src_bits, const void* scale, const void* offset, int param_dtype,
                                void* out, int out_dtype, int64_t rows, int64_t n, void* stream) {
  using namespace b200q;
  clear_error();
  B200Q_REQUIRE(rows >= 0 && n >= 0, B200Q_ERR_BAD_ARG, "anti_quant: negative size");
  B200Q_REQUIRE(src_bits == 8 || src_bits == 4, B200Q_ERR_UNSUPPORTED, "anti_quant: src_bits must be 8 or 4, got %d",
                src_bits);
  B200Q_REQUIRE(src_bits == 8 || n % 8 == 0, B200Q_ERR_BAD_ARG,
                "anti_quant: packed int4 input needs a last dimension that is a multiple of 8");
  B200Q_REQUIRE(param_dtype == B200Q_F32 || param_dtype == B200Q_BF16, B200Q_ERR_UNSUPPORTED,
                "anti_quant: scale and offset must be f32 or bf16 (dtype enum %d)", param_dtype);
  B200Q_REQUIRE(out_dtype == B200Q_F16 || out_dtype == B200Q_BF16, B200Q_ERR_UNSUPPORTED,
                "anti_quant: dst_dtype must be f16 or bf16 (dtype enum %d)", out_dtype);
  if (rows == 0 || n == 0) return B200Q_OK;
  B200Q_REQUIRE(x != nullptr && scale != nullptr && out != nullptr, B200Q_ERR_BAD_ARG, "anti_quant: NULL buffer");
  B200Q_REQUIRE(aligned(out, 2) && (src_bits == 8 || aligned(x, 4)), B200Q_ERR_BAD_ARG, "anti_quant: misaligned buffer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (src_bits == 8) {
    if (param_dtype == B200Q_F32) return anti_quant_out<8, float>(out_dtype, x, scale, offset, out, rows, n, st);
    return anti_quant_out<8, __nv_bfloat16>(out_dtype, x, scale, offset, out, rows, n, st);
  }
  if (param_dtype == B200Q_F32) return anti_quant_out<4, float>(out_dtype, x, scale, offset, out, rows, n, st);
  return anti_quant_out<4, __nv_bfloat16>(out_dtype, x, scale, offset, out, rows, n, st);
}
