// npu_convert_weight_to_int4pack and npu_trans_quant_param: small layout kernels.
#include "common.cuh"
#include "ptx.cuh"

namespace b200q {
namespace {

// One thread packs eight int32-held int4 values (two 128-bit loads) into one int32; value j of a
// group lands in bits [4j, 4j+4).  Grid-stride over the output words.  A value outside [-8, 7] has no
// int4 representation: its low nibble is packed, and the kernel records kDevInt4Range in the device
// error word so that the caller learns about it (the CPU golden raises in the same situation).
__global__ void int4pack_kernel(const int4* __restrict__ w, int32_t* __restrict__ packed, int64_t nwords) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < nwords;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int4 a = __ldcs(w + 2 * i), b = __ldcs(w + 2 * i + 1);
    // v in [-8, 7]  <=>  (v + 8) has no bit above bit 3
    const uint32_t high = ((uint32_t)(a.x + 8) | (uint32_t)(a.y + 8) | (uint32_t)(a.z + 8) | (uint32_t)(a.w + 8) |
                           (uint32_t)(b.x + 8) | (uint32_t)(b.y + 8) | (uint32_t)(b.z + 8) | (uint32_t)(b.w + 8)) & ~0xFu;
    if (high) record_device_error(kDevInt4Range);
    const uint32_t v = (a.x & 0xF) | ((a.y & 0xF) << 4) | ((a.z & 0xF) << 8) | ((a.w & 0xF) << 12) |
                       ((b.x & 0xF) << 16) | ((b.y & 0xF) << 20) | ((b.z & 0xF) << 24) |
                       ((uint32_t)(b.w & 0xF) << 28);
    __stcs(packed + i, (int32_t)v);
  }
}

__global__ void trans_quant_param_kernel(const float* __restrict__ scale, int64_t scale_len,
                                         int64_t* __restrict__ out, int64_t out_len) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < out_len;
       i += (int64_t)gridDim.x * blockDim.x) {
    out[i] = (int64_t)(uint64_t)__float_as_uint(scale[scale_len == 1 ? 0 : i]);
  }
}

}  // namespace
}  // namespace b200q

extern "C" int b200q_int4pack(const int32_t* w, int32_t* packed, int64_t rows, int64_t cols, void* stream) {
  using namespace b200q;
  clear_error();
  B200Q_REQUIRE(rows >= 0 && cols >= 0, B200Q_ERR_BAD_ARG, "int4pack: negative size");
  B200Q_REQUIRE(cols % 8 == 0, B200Q_ERR_BAD_ARG, "int4pack: last dimension (%lld) must be a multiple of 8",
                (long long)cols);
  const int64_t nwords = rows * (cols / 8);
  if (nwords == 0) return B200Q_OK;
  B200Q_REQUIRE(w != nullptr && packed != nullptr, B200Q_ERR_BAD_ARG, "int4pack: NULL buffer");
  B200Q_REQUIRE(aligned(w, 16) && aligned(packed, 4), B200Q_ERR_BAD_ARG, "int4pack: misaligned buffer");
  const int threads = 256;
  const int64_t want = ceil_div(nwords, threads);
  const int blocks = (int)(want < (int64_t)sm_count() * 16 ? want : (int64_t)sm_count() * 16);
  int4pack_kernel<<<blocks, threads, 0, static_cast<cudaStream_t>(stream)>>>(reinterpret_cast<const int4*>(w),
                                                                             packed, nwords);
  return check_launch("int4pack");
}

extern "C" int b200q_trans_quant_param(const float* scale, int64_t scale_len, int64_t* out, int64_t out_len,
                                       void* stream) {
  using namespace b200q;
  clear_error();
  B200Q_REQUIRE(scale_len >= 1 && out_len >= 0, B200Q_ERR_BAD_ARG, "trans_quant_param: bad length");
  B200Q_REQUIRE(scale_len == 1 || scale_len == out_len, B200Q_ERR_BAD_ARG,
                "trans_quant_param: scale has %lld elements, output %lld", (long long)scale_len, (long long)out_len);
  if (out_len == 0) return B200Q_OK;
  B200Q_REQUIRE(scale != nullptr && out != nullptr, B200Q_ERR_BAD_ARG, "trans_quant_param: NULL buffer");
  const int threads = 256;
  const int blocks = (int)(ceil_div(out_len, threads) < 1024 ? ceil_div(out_len, threads) : 1024);
  trans_quant_param_kernel<<<blocks, threads, 0, static_cast<cudaStream_t>(stream)>>>(scale, scale_len, out,
                                                                                      out_len);
  return check_launch("trans_quant_param");
}
