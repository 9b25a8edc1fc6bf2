// npu_weight_quant_batchmatmul (placeholder entry points; replaced by the fused kernel).
#include "common.cuh"

extern "C" size_t b200q_weight_quant_matmul_workspace_bytes(int64_t, int64_t, int64_t, int) { return 0; }

extern "C" int b200q_weight_quant_matmul(const b200q_weight_quant_matmul_args*, void*) {
  return b200q::fail(B200Q_ERR_UNSUPPORTED, "weight_quant_matmul: kernel not built");
}
