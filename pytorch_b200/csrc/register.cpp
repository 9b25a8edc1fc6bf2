// PyTorch registration of the quantized-inference operators under the reference's own
// operator names: torch.ops.npu.npu_dynamic_quant, npu_quant_matmul,
// npu_weight_quant_batchmatmul, npu_convert_weight_to_int4pack, npu_trans_quant_param.
//
// This translation unit takes the place of the generated registration of the reference
// (torchnpugen/templates/CustomRegisterSchema.cpp:43-55: TORCH_LIBRARY(npu) schema definitions
// plus a per-op wrapper that checks devices, sets a device guard and forwards to
// op_plugin::<op>) and of the op-plugin OpApi functions behind it.  Each implementation
// validates its arguments, allocates outputs and workspace from PyTorch's CUDA caching allocator
// and calls the C ABI of include/b200q.h on the current stream.  Only the CUDA and Meta
// dispatch keys are registered: a CPU tensor reaches no kernel and raises.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include <mutex>

#include "b200q.h"

namespace {

using at::Tensor;
using c10::optional;

int dtype_enum(at::ScalarType t) {
  switch (t) {
    case at::kBFloat16: return B200Q_BF16;
    case at::kHalf: return B200Q_F16;
    case at::kFloat: return B200Q_F32;
    case at::kChar: return B200Q_I8;
    case at::kInt: return B200Q_I32;
    case at::kLong: return B200Q_I64;
    default: return 99;
  }
}

void check_status(int status, const char* op) {
  TORCH_CHECK(status == B200Q_OK, op, ": ", b200q_last_error(), " (", b200q_status_string(status), ")");
}

// A kernel that gives up a bounded wait returns early and leaves its output unfinished.  The library mirrors
// the device's error word into pinned host memory, so every operator call can look at it for free and raise
// (the error belongs to an earlier launch on this device; like the reference, which reports asynchronous
// launch failures at the next call, torch_npu/csrc/framework/OpParamMaker.cpp:258-264).  The mirror is set up
// on the first operator call on a device.
void surface_device_error(const char* op, const Tensor& t) {
  static std::once_flag once[64];
  const int dev = t.device().index();
  if (dev >= 0 && dev < 64) std::call_once(once[dev], [] { b200q_enable_host_error_word(); });
  const unsigned int code = b200q_peek_device_error();
  if (code != 0) {
    unsigned int seen = 0;
    b200q_device_error(&seen, 1);      // synchronises and clears, so that the next call can proceed
    TORCH_CHECK(false, op, ": an earlier kernel on ", t.device(), " gave up a bounded wait (device error code 0x", std::hex,
                code, "); its output is incomplete");
  }
}

// Same rule and message as the reference's generated wrapper (torchnpugen/custom_functions.py:137-208;
// expected text in test/custom_ops/test_npu_anti_quant.py:86-88).
void check_same_device(const char* op, const Tensor& first, std::initializer_list<const optional<Tensor>*> rest) {
  for (const optional<Tensor>* t : rest) {
    if (t->has_value() && (*t)->defined()) {
      TORCH_CHECK((*t)->device() == first.device(), op,
                  ": Expected all tensors to be on the same device, but found at least two devices, ",
                  first.device(), " and ", (*t)->device(), "!");
    }
  }
}

void* stream_of(const Tensor& t) { return at::cuda::getCurrentCUDAStream(t.device().index()).stream(); }

// ---------------------------------------------------------------------------------------------
// npu_dynamic_quant(input, *, smooth_scales=None, group_index=None, dst_type=None) -> (y, scale)
std::tuple<Tensor, Tensor> dynamic_quant_check(const Tensor& input, const optional<Tensor>& smooth,
                                               const optional<Tensor>& group_index,
                                               optional<at::ScalarType> dst_type) {
  TORCH_CHECK(input.dim() >= 1, "npu_dynamic_quant: input must have at least one dimension");
  TORCH_CHECK(input.scalar_type() == at::kBFloat16 || input.scalar_type() == at::kHalf,
              "npu_dynamic_quant: input must be float16 or bfloat16, got ", input.scalar_type());
  TORCH_CHECK(!dst_type.has_value() || *dst_type == at::kChar,
              "npu_dynamic_quant: dst_type must be torch.int8, got ", *dst_type);
  if (group_index.has_value()) {
    // One smooth-scale row per group of tokens (test/onnx/test_wrapper_onnx_ops.py:1345-1354).
    TORCH_CHECK(smooth.has_value(), "npu_dynamic_quant: group_index needs smooth_scales of shape [groups, k]");
    TORCH_CHECK(group_index->dim() == 1 && (group_index->scalar_type() == at::kInt || group_index->scalar_type() == at::kLong),
                "npu_dynamic_quant: group_index must be a 1-D int32 or int64 tensor");
    TORCH_CHECK(smooth->dim() == 2 && smooth->size(0) == group_index->size(0) && smooth->size(1) == input.size(-1),
                "npu_dynamic_quant: with group_index, smooth_scales must have shape [", group_index->size(0), ", ",
                input.size(-1), "]");
  } else if (smooth.has_value()) {
    TORCH_CHECK(smooth->dim() == 1 && smooth->size(0) == input.size(-1),
                "npu_dynamic_quant: smooth_scales must have shape [", input.size(-1), "]");
  }
  if (smooth.has_value())
    TORCH_CHECK(smooth->scalar_type() == at::kFloat || smooth->scalar_type() == input.scalar_type(),
                "npu_dynamic_quant: smooth_scales must be float32 or the input's dtype");
  auto scale_shape = input.sizes().vec();
  scale_shape.pop_back();
  return {at::empty(input.sizes(), input.options().dtype(at::kChar)),
          at::empty(scale_shape, input.options().dtype(at::kFloat))};
}

std::tuple<Tensor, Tensor> dynamic_quant_cuda(const Tensor& input, const optional<Tensor>& smooth,
                                              const optional<Tensor>& group_index,
                                              optional<at::ScalarType> dst_type) {
  check_same_device("npu_dynamic_quant", input, {&smooth, &group_index});
  c10::cuda::CUDAGuard guard(input.device());
  surface_device_error(__func__, input);
  auto [y, scale] = dynamic_quant_check(input, smooth, group_index, dst_type);
  Tensor x = input.contiguous();
  Tensor sm = smooth.has_value() ? smooth->contiguous() : Tensor();
  const int64_t k = x.size(-1);
  const int64_t rows = k ? x.numel() / k : scale.numel();
  if (group_index.has_value()) {
    Tensor gi = group_index->to(at::kInt).contiguous();
    check_status(b200q_dynamic_quant_ext(x.data_ptr(), dtype_enum(x.scalar_type()), sm.data_ptr(),
                                         dtype_enum(sm.scalar_type()), static_cast<const int32_t*>(gi.data_ptr()),
                                         gi.numel(), static_cast<int8_t*>(y.data_ptr()),
                                         static_cast<float*>(scale.data_ptr()), nullptr, rows, k, stream_of(x)),
                 "npu_dynamic_quant");
    return {y, scale};
  }
  check_status(b200q_dynamic_quant(x.data_ptr(), dtype_enum(x.scalar_type()), sm.defined() ? sm.data_ptr() : nullptr,
                                   sm.defined() ? dtype_enum(sm.scalar_type()) : B200Q_NONE,
                                   static_cast<int8_t*>(y.data_ptr()), static_cast<float*>(scale.data_ptr()), rows, k,
                                   stream_of(x)),
               "npu_dynamic_quant");
  return {y, scale};
}

// npu_dynamic_quant_asymmetric(input, *, smooth_scales=None, group_index=None, dst_type=None) -> (y, scale, offset)
std::tuple<Tensor, Tensor, Tensor> dynamic_quant_asym_cuda(const Tensor& input, const optional<Tensor>& smooth,
                                                           const optional<Tensor>& group_index,
                                                           optional<at::ScalarType> dst_type) {
  check_same_device("npu_dynamic_quant_asymmetric", input, {&smooth, &group_index});
  c10::cuda::CUDAGuard guard(input.device());
  surface_device_error(__func__, input);
  auto [y, scale] = dynamic_quant_check(input, smooth, group_index, dst_type);
  Tensor offset = at::empty_like(scale);
  Tensor x = input.contiguous();
  Tensor sm = smooth.has_value() ? smooth->contiguous() : Tensor();
  Tensor gi = group_index.has_value() ? group_index->to(at::kInt).contiguous() : Tensor();
  const int64_t k = x.size(-1);
  const int64_t rows = k ? x.numel() / k : scale.numel();
  check_status(b200q_dynamic_quant_ext(x.data_ptr(), dtype_enum(x.scalar_type()), sm.defined() ? sm.data_ptr() : nullptr,
                                       sm.defined() ? dtype_enum(sm.scalar_type()) : B200Q_NONE,
                                       gi.defined() ? static_cast<const int32_t*>(gi.data_ptr()) : nullptr,
                                       gi.defined() ? gi.numel() : 0, static_cast<int8_t*>(y.data_ptr()),
                                       static_cast<float*>(scale.data_ptr()), static_cast<float*>(offset.data_ptr()),
                                       rows, k, stream_of(x)),
               "npu_dynamic_quant_asymmetric");
  return {y, scale, offset};
}

std::tuple<Tensor, Tensor, Tensor> dynamic_quant_asym_meta(const Tensor& input, const optional<Tensor>& smooth,
                                                           const optional<Tensor>& group_index,
                                                           optional<at::ScalarType> dst_type) {
  auto [y, scale] = dynamic_quant_check(input, smooth, group_index, dst_type);
  return {y, scale, at::empty_like(scale)};
}

// ---------------------------------------------------------------------------------------------
// npu_swiglu_quant(x, *, smooth_scales=None, offsets=None, group_index=None, activate_left=False, quant_mode=0,
//                  group_list_type=0, dst_type=None) -> (y, scale); only the dynamic mode (quant_mode=1) is built.
std::tuple<Tensor, Tensor> swiglu_quant_check(const Tensor& x, const optional<Tensor>& smooth,
                                              const optional<Tensor>& offsets, const optional<Tensor>& group_index,
                                              int64_t quant_mode, optional<at::ScalarType> dst_type) {
  TORCH_CHECK(x.dim() >= 1 && x.size(-1) % 2 == 0, "npu_swiglu_quant: the last dimension of x must be even");
  TORCH_CHECK(x.scalar_type() == at::kBFloat16 || x.scalar_type() == at::kHalf,
              "npu_swiglu_quant: x must be float16 or bfloat16, got ", x.scalar_type());
  TORCH_CHECK(quant_mode == 1, "npu_swiglu_quant: only quant_mode=1 (dynamic, per token) is implemented, got ", quant_mode);
  TORCH_CHECK(!offsets.has_value() && !group_index.has_value(),
              "npu_swiglu_quant: offsets and group_index are not supported");
  TORCH_CHECK(!dst_type.has_value() || *dst_type == at::kChar, "npu_swiglu_quant: dst_type must be torch.int8");
  const int64_t f = x.size(-1) / 2;
  if (smooth.has_value()) {
    TORCH_CHECK(smooth->numel() == f, "npu_swiglu_quant: smooth_scales must have ", f, " elements");
    TORCH_CHECK(smooth->scalar_type() == at::kFloat || smooth->scalar_type() == x.scalar_type(),
                "npu_swiglu_quant: smooth_scales must be float32 or the input's dtype");
  }
  auto shape = x.sizes().vec();
  shape.back() = f;
  auto scale_shape = shape;
  scale_shape.pop_back();
  return {at::empty(shape, x.options().dtype(at::kChar)), at::empty(scale_shape, x.options().dtype(at::kFloat))};
}

std::tuple<Tensor, Tensor> swiglu_quant_cuda(const Tensor& x, const optional<Tensor>& smooth,
                                             const optional<Tensor>& offsets, const optional<Tensor>& group_index,
                                             bool activate_left, int64_t quant_mode, int64_t /*group_list_type*/,
                                             optional<at::ScalarType> dst_type) {
  check_same_device("npu_swiglu_quant", x, {&smooth, &offsets, &group_index});
  c10::cuda::CUDAGuard guard(x.device());
  surface_device_error(__func__, x);
  auto [y, scale] = swiglu_quant_check(x, smooth, offsets, group_index, quant_mode, dst_type);
  Tensor xc = x.contiguous();
  Tensor sm = smooth.has_value() ? smooth->contiguous() : Tensor();
  const int64_t f = xc.size(-1) / 2;
  const int64_t rows = f ? xc.numel() / (2 * f) : scale.numel();
  check_status(b200q_swiglu_quant(xc.data_ptr(), dtype_enum(xc.scalar_type()), sm.defined() ? sm.data_ptr() : nullptr,
                                  sm.defined() ? dtype_enum(sm.scalar_type()) : B200Q_NONE, activate_left ? 1 : 0,
                                  static_cast<int8_t*>(y.data_ptr()), static_cast<float*>(scale.data_ptr()), rows, f,
                                  stream_of(x)),
               "npu_swiglu_quant");
  return {y, scale};
}

std::tuple<Tensor, Tensor> swiglu_quant_meta(const Tensor& x, const optional<Tensor>& smooth,
                                             const optional<Tensor>& offsets, const optional<Tensor>& group_index,
                                             bool, int64_t quant_mode, int64_t, optional<at::ScalarType> dst_type) {
  return swiglu_quant_check(x, smooth, offsets, group_index, quant_mode, dst_type);
}

// ---------------------------------------------------------------------------------------------
// npu_anti_quant(x, scale, *, offset=None, dst_dtype=None, src_dtype=None) -> Tensor
// x int8 [..., n], or int32 words of eight int4 values [..., n/8]; scale/offset [n] float32 or bfloat16.
std::vector<int64_t> anti_quant_check(const Tensor& x, const Tensor& scale, const optional<Tensor>& offset,
                                      optional<at::ScalarType> dst_dtype, optional<at::ScalarType> src_dtype) {
  TORCH_CHECK(x.scalar_type() == at::kChar || x.scalar_type() == at::kInt,
              "npu_anti_quant: x must be int8, or int32 holding eight int4 values per element, got ", x.scalar_type());
  TORCH_CHECK(x.dim() >= 1, "npu_anti_quant: x must have at least one dimension");
  TORCH_CHECK(!dst_dtype.has_value() || *dst_dtype == at::kHalf || *dst_dtype == at::kBFloat16,
              "The argument 'dst_dtype' must be torch.float16 or torch.bfloat16.");
  TORCH_CHECK(!src_dtype.has_value() || *src_dtype == at::kChar || *src_dtype == at::kQUInt4x2,
              "The argument 'src_dtype' must be torch.int8 or torch.quint4x2.");
  auto shape = x.sizes().vec();
  if (x.scalar_type() == at::kInt) shape.back() *= 8;
  TORCH_CHECK(scale.scalar_type() == at::kFloat || scale.scalar_type() == at::kBFloat16,
              "npu_anti_quant: scale must be float32 or bfloat16, got ", scale.scalar_type());
  TORCH_CHECK(scale.numel() == shape.back() || scale.numel() == 1, "npu_anti_quant: scale must have ", shape.back(),
              " elements (or one), got ", scale.numel());
  if (offset.has_value()) {
    TORCH_CHECK(offset->scalar_type() == scale.scalar_type(), "npu_anti_quant: offset must have the dtype of scale");
    TORCH_CHECK(offset->numel() == scale.numel(), "npu_anti_quant: offset must have the shape of scale");
  }
  return shape;
}

Tensor anti_quant_cuda(const Tensor& x, const Tensor& scale, const optional<Tensor>& offset,
                       optional<at::ScalarType> dst_dtype, optional<at::ScalarType> src_dtype) {
  check_same_device("npu_anti_quant", x, {&offset});
  TORCH_CHECK(scale.device() == x.device(), "Expected all tensors to be on the same device, but found at least two devices, ",
              x.device(), " and ", scale.device(), "! (npu_anti_quant)");
  c10::cuda::CUDAGuard guard(x.device());
  surface_device_error(__func__, x);
  auto shape = anti_quant_check(x, scale, offset, dst_dtype, src_dtype);
  const at::ScalarType out_t = dst_dtype.value_or(at::kHalf);
  Tensor out = at::empty(shape, x.options().dtype(out_t));
  const int64_t n = shape.back();
  const int64_t rows = n ? out.numel() / n : 0;
  Tensor xc = x.contiguous();
  Tensor sc = (scale.numel() == n ? scale : scale.expand({n})).contiguous();
  Tensor of = offset.has_value() ? (offset->numel() == n ? *offset : offset->expand({n})).contiguous() : Tensor();
  check_status(b200q_anti_quant(xc.data_ptr(), x.scalar_type() == at::kInt ? 4 : 8, sc.data_ptr(),
                                of.defined() ? of.data_ptr() : nullptr, dtype_enum(sc.scalar_type()), out.data_ptr(),
                                dtype_enum(out_t), rows, n, stream_of(x)),
               "npu_anti_quant");
  return out;
}

Tensor anti_quant_meta(const Tensor& x, const Tensor& scale, const optional<Tensor>& offset,
                       optional<at::ScalarType> dst_dtype, optional<at::ScalarType> src_dtype) {
  auto shape = anti_quant_check(x, scale, offset, dst_dtype, src_dtype);
  return at::empty(shape, x.options().dtype(dst_dtype.value_or(at::kHalf)));
}

// ---------------------------------------------------------------------------------------------
// npu_quant_matmul(x1, x2, scale, *, offset, pertoken_scale, bias, output_dtype) -> Tensor
struct QmmShape {
  std::vector<int64_t> out_shape;
  int64_t batch_x2, m_total, m_per_batch, k, n;
};

QmmShape quant_matmul_check(const Tensor& x1, const Tensor& x2, const Tensor& scale, const optional<Tensor>& offset,
                            const optional<Tensor>& pertoken, const optional<Tensor>& bias, at::ScalarType out_dtype) {
  TORCH_CHECK(!(x1.scalar_type() == at::kInt || x2.scalar_type() == at::kInt),
              "npu_quant_matmul: int32 (int4-packed A4W4) inputs are not supported");
  TORCH_CHECK(x1.scalar_type() == at::kChar && x2.scalar_type() == at::kChar,
              "npu_quant_matmul: x1 and x2 must be int8, got ", x1.scalar_type(), " and ", x2.scalar_type());
  TORCH_CHECK(x1.dim() >= 2 && (x2.dim() == 2 || x2.dim() == 3),
              "npu_quant_matmul: x1 must have >= 2 dimensions and x2 2 or 3, got ", x1.dim(), " and ", x2.dim());
  QmmShape s;
  s.k = x1.size(-1);
  s.n = x2.size(-1);
  TORCH_CHECK(x2.size(-2) == s.k, "npu_quant_matmul: inner dimensions differ: x1 [..., ", s.k, "] and x2 [", x2.size(-2),
              ", ", s.n, "]");
  TORCH_CHECK(scale.scalar_type() == at::kFloat || scale.scalar_type() == at::kBFloat16 ||
                  scale.scalar_type() == at::kLong,
              "npu_quant_matmul: scale should be torch.int64, torch.float32 or torch.bfloat16 datatype, but now it is ",
              scale.scalar_type());
  TORCH_CHECK(scale.numel() == 1 || scale.numel() == s.n, "npu_quant_matmul: scale must have 1 or n=", s.n, " elements");
  if (offset.has_value()) {
    TORCH_CHECK(offset->scalar_type() == at::kFloat, "npu_quant_matmul: offset should be torch.float32 datatype");
    TORCH_CHECK(offset->numel() == 1 || offset->numel() == s.n, "npu_quant_matmul: offset must have 1 or n elements");
  }
  TORCH_CHECK(out_dtype == at::kChar || out_dtype == at::kHalf || out_dtype == at::kBFloat16 || out_dtype == at::kInt,
              "npu_quant_matmul: output_dtype should be torch.int8, torch.float16, torch.bfloat16 or torch.int32, but now it is ",
              out_dtype);
  s.batch_x2 = x2.dim() == 3 ? x2.size(0) : 1;
  s.out_shape = x1.sizes().vec();
  s.out_shape.back() = s.n;
  if (x2.dim() == 3) {
    TORCH_CHECK(x1.dim() <= 3, "npu_quant_matmul: a 3-D x2 takes a 2-D or 3-D x1");
    const int64_t b1 = x1.dim() == 3 ? x1.size(0) : 1;
    TORCH_CHECK(b1 == s.batch_x2 || b1 == 1 || s.batch_x2 == 1, "npu_quant_matmul: batch dimensions ", b1, " and ",
                s.batch_x2, " do not broadcast");
    s.out_shape = {std::max(b1, s.batch_x2), x1.size(-2), s.n};
  }
  s.m_total = 1;
  for (size_t i = 0; i + 1 < s.out_shape.size(); ++i) s.m_total *= s.out_shape[i];
  // A 3-D x2 with a single batch is one weight for every row of x1: the batches of x1 fold into m.
  s.m_per_batch = (x2.dim() == 3 && s.batch_x2 > 1) ? x1.size(-2) : s.m_total;
  if (pertoken.has_value()) {
    TORCH_CHECK(pertoken->scalar_type() == at::kFloat, "npu_quant_matmul: pertoken_scale should be torch.float32 datatype");
    TORCH_CHECK(pertoken->numel() == s.m_total || pertoken->numel() == 1, "npu_quant_matmul: pertoken_scale must have ",
                s.m_total, " elements, got ", pertoken->numel());
  }
  if (bias.has_value()) {
    const auto bt = bias->scalar_type();
    TORCH_CHECK(bt == at::kInt || bt == at::kBFloat16 || bt == at::kHalf || bt == at::kFloat,
                "npu_quant_matmul: bias should be torch.int32, torch.bfloat16, torch.float16 or torch.float32 datatype");
    TORCH_CHECK(bias->size(-1) == s.n && (bias->numel() == s.n || bias->numel() == s.n * s.batch_x2),
                "npu_quant_matmul: bias must be [n] or [batch, 1, n]");
    TORCH_CHECK(out_dtype != at::kInt || bt == at::kInt, "npu_quant_matmul: int32 output takes an int32 bias");
  }
  return s;
}

Tensor quant_matmul_cuda(const Tensor& x1, const Tensor& x2, const Tensor& scale, const optional<Tensor>& offset,
                         const optional<Tensor>& pertoken, const optional<Tensor>& bias,
                         optional<at::ScalarType> output_dtype) {
  const optional<Tensor> x2o(x2), so(scale);
  check_same_device("npu_quant_matmul", x1, {&x2o, &so, &offset, &pertoken, &bias});
  c10::cuda::CUDAGuard guard(x1.device());
  surface_device_error(__func__, x1);
  const at::ScalarType out_dtype = output_dtype.value_or(at::kChar);
  QmmShape s = quant_matmul_check(x1, x2, scale, offset, pertoken, bias, out_dtype);
  Tensor out = at::empty(s.out_shape, x1.options().dtype(out_dtype));
  if (out.numel() == 0) return out;

  Tensor a = x1.contiguous();
  if (x2.dim() == 3 && x1.dim() == 3 && x1.size(0) == 1 && s.batch_x2 > 1) a = a.expand({s.batch_x2, -1, -1}).contiguous();
  Tensor sc = scale.contiguous();
  Tensor of = offset.has_value() ? offset->contiguous() : Tensor();
  Tensor pt = pertoken.has_value() ? pertoken->contiguous() : Tensor();
  if (pt.defined() && pt.numel() == 1 && s.m_total != 1) pt = pt.expand({s.m_total}).contiguous();
  Tensor bs = bias.has_value() ? bias->contiguous() : Tensor();
  const int64_t nb = (x2.dim() == 3 && s.batch_x2 > 1) ? s.batch_x2 : 1;
  const bool a_batched = nb > 1 && a.dim() == 3 && a.size(0) == nb;
  const bool bias_batched = bs.defined() && bs.numel() == s.n * nb && nb > 1;

  for (int64_t b = 0; b < nb; ++b) {
    Tensor w = x2.dim() == 3 ? x2.select(0, x2.size(0) == 1 ? 0 : b) : x2;
    // Fast layouts: the transposed view of an [n,k] weight, or a contiguous [k,n] one.
    const bool kmajor = w.stride(0) == 1 && w.stride(1) >= s.k;
    const bool nmajor = w.stride(1) == 1 && w.stride(0) == s.n;
    if (!kmajor && !nmajor) w = w.contiguous();
    b200q_quant_matmul_args args{};
    args.x1 = static_cast<const int8_t*>(a.data_ptr()) + (a_batched ? b * s.m_per_batch * s.k : 0);
    args.x2 = static_cast<const int8_t*>(w.data_ptr());
    args.m = s.m_per_batch; args.k = s.k; args.n = s.n;
    args.x2_stride_k = w.stride(0); args.x2_stride_n = w.stride(1);
    args.scale = sc.data_ptr(); args.scale_dtype = dtype_enum(sc.scalar_type()); args.scale_len = sc.numel();
    if (of.defined()) { args.offset = static_cast<const float*>(of.data_ptr()); args.offset_len = of.numel(); }
    if (pt.defined()) args.pertoken_scale = static_cast<const float*>(pt.data_ptr()) + (nb > 1 ? b * s.m_per_batch : 0);
    args.bias_dtype = B200Q_NONE;
    if (bs.defined()) {
      args.bias = static_cast<const char*>(bs.data_ptr()) + (bias_batched ? b * s.n * bs.element_size() : 0);
      args.bias_dtype = dtype_enum(bs.scalar_type());
    }
    args.out = static_cast<char*>(out.data_ptr()) + (nb > 1 ? b * s.m_per_batch * s.n * out.element_size() : 0);
    args.out_dtype = dtype_enum(out_dtype);
    const size_t need = b200q_quant_matmul_workspace_bytes(args.m, args.k, args.n, args.x2_stride_k, args.x2_stride_n);
    Tensor ws;
    if (need) {
      ws = at::empty({static_cast<int64_t>(need)}, x1.options().dtype(at::kByte));
      args.workspace = ws.data_ptr();
      args.workspace_bytes = need;
    }
    check_status(b200q_quant_matmul(&args, stream_of(x1)), "npu_quant_matmul");
  }
  return out;
}

Tensor quant_matmul_meta(const Tensor& x1, const Tensor& x2, const Tensor& scale, const optional<Tensor>& offset,
                         const optional<Tensor>& pertoken, const optional<Tensor>& bias,
                         optional<at::ScalarType> output_dtype) {
  // Shape rule of the reference's meta kernel (test/test_fake_tensor.py:1884-1925), including int4-packed
  // int32 operands whose last dimension of x2 counts eight values per element.
  const at::ScalarType out_dtype = output_dtype.value_or(at::kChar);
  if (x1.scalar_type() == at::kInt && x2.scalar_type() == at::kInt) {
    auto shape = x1.sizes().vec();
    shape.back() = x2.size(-1) * 8;
    return at::empty(shape, x1.options().dtype(out_dtype));
  }
  QmmShape s = quant_matmul_check(x1, x2, scale, offset, pertoken, bias, out_dtype);
  return at::empty(s.out_shape, x1.options().dtype(out_dtype));
}

// ---------------------------------------------------------------------------------------------
// npu_weight_quant_batchmatmul(x, weight, antiquant_scale, antiquant_offset, quant_scale, quant_offset,
//                              bias, antiquant_group_size, inner_precise, *, weight_dtype) -> Tensor
struct WqShape {
  std::vector<int64_t> out_shape;
  int64_t m, k, n, groups;
  int bits;
};

WqShape weight_quant_check(const Tensor& x, const Tensor& weight, const Tensor& scale, const optional<Tensor>& offset,
                           const optional<Tensor>& quant_scale, const optional<Tensor>& quant_offset,
                           const optional<Tensor>& bias, int64_t group_size, int64_t inner_precise,
                           optional<at::ScalarType> weight_dtype) {
  TORCH_CHECK(x.scalar_type() == at::kBFloat16 || x.scalar_type() == at::kHalf,
              "npu_weight_quant_batchmatmul: x must be float16 or bfloat16, got ", x.scalar_type());
  TORCH_CHECK(x.dim() >= 2 && weight.dim() == 2, "npu_weight_quant_batchmatmul: x must have >= 2 dimensions and weight 2");
  TORCH_CHECK(weight.scalar_type() == at::kChar || weight.scalar_type() == at::kInt,
              "npu_weight_quant_batchmatmul: weight must be int8 or int32 (eight int4 per element), got ",
              weight.scalar_type());
  TORCH_CHECK(!quant_scale.has_value() && !quant_offset.has_value(),
              "npu_weight_quant_batchmatmul: quant_scale / quant_offset (int8 re-quantised output) are not supported");
  TORCH_CHECK(inner_precise == 0, "npu_weight_quant_batchmatmul: inner_precise must be 0");
  TORCH_CHECK(!weight_dtype.has_value(), "npu_weight_quant_batchmatmul: weight_dtype is not supported");
  WqShape s;
  s.bits = weight.scalar_type() == at::kInt ? 4 : 8;
  s.k = x.size(-1);
  s.n = weight.size(1) * (s.bits == 4 ? 8 : 1);
  TORCH_CHECK(weight.size(0) == s.k, "npu_weight_quant_batchmatmul: x [..., ", s.k, "] and weight [", weight.size(0),
              ", ...] do not match");
  TORCH_CHECK(group_size >= 0, "npu_weight_quant_batchmatmul: antiquant_group_size must be >= 0");
  s.groups = group_size > 0 ? (s.k + group_size - 1) / group_size : 1;
  auto check_param = [&](const Tensor& p, const char* name) {
    TORCH_CHECK(p.scalar_type() == x.scalar_type(), "npu_weight_quant_batchmatmul: ", name, " must have x's dtype");
    TORCH_CHECK(p.size(-1) == s.n && p.numel() == s.groups * s.n, "npu_weight_quant_batchmatmul: ", name, " must be [",
                s.groups, ", ", s.n, "]", s.groups == 1 ? " or [n]" : "");
  };
  check_param(scale, "antiquant_scale");
  if (offset.has_value()) check_param(*offset, "antiquant_offset");
  if (bias.has_value())
    TORCH_CHECK(bias->numel() == s.n && bias->scalar_type() == x.scalar_type(),
                "npu_weight_quant_batchmatmul: bias must be [n] in x's dtype");
  s.out_shape = x.sizes().vec();
  s.out_shape.back() = s.n;
  s.m = s.k ? x.numel() / s.k : 0;
  return s;
}

Tensor weight_quant_cuda(const Tensor& x, const Tensor& weight, const Tensor& scale, const optional<Tensor>& offset,
                         const optional<Tensor>& quant_scale, const optional<Tensor>& quant_offset,
                         const optional<Tensor>& bias, int64_t group_size, int64_t inner_precise,
                         optional<at::ScalarType> weight_dtype) {
  const optional<Tensor> wo(weight), so(scale);
  check_same_device("npu_weight_quant_batchmatmul", x, {&wo, &so, &offset, &quant_scale, &quant_offset, &bias});
  c10::cuda::CUDAGuard guard(x.device());
  surface_device_error(__func__, x);
  WqShape s = weight_quant_check(x, weight, scale, offset, quant_scale, quant_offset, bias, group_size, inner_precise,
                                 weight_dtype);
  Tensor out = at::empty(s.out_shape, x.options());
  if (out.numel() == 0) return out;
  Tensor xc = x.contiguous();
  Tensor w = s.bits == 4 ? weight.contiguous() : weight;
  Tensor sc = scale.contiguous();
  Tensor of = offset.has_value() ? offset->contiguous() : Tensor();
  Tensor bs = bias.has_value() ? bias->contiguous() : Tensor();
  b200q_weight_quant_matmul_args args{};
  args.x = xc.data_ptr(); args.x_dtype = dtype_enum(x.scalar_type());
  args.weight = w.data_ptr(); args.weight_bits = s.bits;
  args.m = s.m; args.k = s.k; args.n = s.n;
  args.w_stride_k = s.bits == 8 ? w.stride(0) : 0; args.w_stride_n = s.bits == 8 ? w.stride(1) : 0;
  args.antiquant_scale = sc.data_ptr();
  args.antiquant_offset = of.defined() ? of.data_ptr() : nullptr;
  args.group_size = group_size;
  args.bias = bs.defined() ? bs.data_ptr() : nullptr;
  args.out = out.data_ptr();
  const size_t need = b200q_weight_quant_matmul_workspace_bytes(s.m, s.k, s.n, s.bits);
  Tensor ws;
  if (need) {
    ws = at::empty({static_cast<int64_t>(need)}, x.options().dtype(at::kByte));
    args.workspace = ws.data_ptr();
    args.workspace_bytes = need;
  }
  check_status(b200q_weight_quant_matmul(&args, stream_of(x)), "npu_weight_quant_batchmatmul");
  return out;
}

Tensor weight_quant_meta(const Tensor& x, const Tensor& weight, const Tensor& scale, const optional<Tensor>& offset,
                         const optional<Tensor>& quant_scale, const optional<Tensor>& quant_offset,
                         const optional<Tensor>& bias, int64_t group_size, int64_t inner_precise,
                         optional<at::ScalarType> weight_dtype) {
  WqShape s = weight_quant_check(x, weight, scale, offset, quant_scale, quant_offset, bias, group_size, inner_precise,
                                 weight_dtype);
  return at::empty(s.out_shape, x.options());
}

// ---------------------------------------------------------------------------------------------
std::vector<int64_t> int4pack_shape(const Tensor& weight) {
  TORCH_CHECK(weight.scalar_type() == at::kInt, "npu_convert_weight_to_int4pack: weight must be int32 (one int4 value per element)");
  TORCH_CHECK(weight.dim() >= 1 && weight.size(-1) % 8 == 0,
              "npu_convert_weight_to_int4pack: the last dimension must be a multiple of 8");
  auto shape = weight.sizes().vec();
  shape.back() /= 8;
  return shape;
}

Tensor int4pack_cuda(const Tensor& weight, int64_t /*inner_k_tiles*/) {
  c10::cuda::CUDAGuard guard(weight.device());
  surface_device_error(__func__, weight);
  Tensor out = at::empty(int4pack_shape(weight), weight.options());
  Tensor w = weight.contiguous();
  const int64_t cols = w.size(-1);
  check_status(b200q_int4pack(static_cast<const int32_t*>(w.data_ptr()), static_cast<int32_t*>(out.data_ptr()),
                              cols ? w.numel() / cols : 0, cols, stream_of(w)),
               "npu_convert_weight_to_int4pack");
  return out;
}

Tensor int4pack_meta(const Tensor& weight, int64_t) { return at::empty(int4pack_shape(weight), weight.options()); }

// npu_trans_quant_param(scale, offset=None) -> int64 with the broadcast shape of scale and offset
std::vector<int64_t> trans_shape(const Tensor& scale, const optional<Tensor>& offset) {
  TORCH_CHECK(scale.scalar_type() == at::kFloat, "npu_trans_quant_param: scale must be float32");
  if (!offset.has_value()) return scale.sizes().vec();
  TORCH_CHECK(offset->scalar_type() == at::kFloat, "npu_trans_quant_param: offset must be float32");
  TORCH_CHECK(scale.numel() == 1 || offset->numel() == 1 || scale.numel() == offset->numel(),
              "npu_trans_quant_param: scale and offset do not broadcast");
  return scale.numel() >= offset->numel() ? scale.sizes().vec() : offset->sizes().vec();
}

Tensor trans_quant_param_cuda(const Tensor& scale, const optional<Tensor>& offset) {
  check_same_device("npu_trans_quant_param", scale, {&offset});
  c10::cuda::CUDAGuard guard(scale.device());
  surface_device_error(__func__, scale);
  Tensor out = at::empty(trans_shape(scale, offset), scale.options().dtype(at::kLong));
  Tensor sc = scale.contiguous();
  check_status(b200q_trans_quant_param(static_cast<const float*>(sc.data_ptr()), sc.numel(),
                                       static_cast<int64_t*>(out.data_ptr()), out.numel(), stream_of(sc)),
               "npu_trans_quant_param");
  return out;
}

Tensor trans_quant_param_meta(const Tensor& scale, const optional<Tensor>& offset) {
  return at::empty(trans_shape(scale, offset), scale.options().dtype(at::kLong));
}

std::tuple<Tensor, Tensor> dynamic_quant_meta(const Tensor& input, const optional<Tensor>& smooth,
                                              const optional<Tensor>& group_index, optional<at::ScalarType> dst_type) {
  return dynamic_quant_check(input, smooth, group_index, dst_type);
}

}  // namespace

TORCH_LIBRARY(npu, m) {
  m.def("npu_dynamic_quant(Tensor input, *, Tensor? smooth_scales=None, Tensor? group_index=None, "
        "ScalarType? dst_type=None) -> (Tensor, Tensor)");
  m.def("npu_quant_matmul(Tensor x1, Tensor x2, Tensor scale, *, Tensor? offset=None, Tensor? pertoken_scale=None, "
        "Tensor? bias=None, ScalarType? output_dtype=None) -> Tensor");
  m.def("npu_weight_quant_batchmatmul(Tensor x, Tensor weight, Tensor antiquant_scale, Tensor? antiquant_offset=None, "
        "Tensor? quant_scale=None, Tensor? quant_offset=None, Tensor? bias=None, int antiquant_group_size=0, "
        "int inner_precise=0, *, ScalarType? weight_dtype=None) -> Tensor");
  m.def("npu_convert_weight_to_int4pack(Tensor weight, int inner_k_tiles=0) -> Tensor");
  m.def("npu_dynamic_quant_asymmetric(Tensor input, *, Tensor? smooth_scales=None, Tensor? group_index=None, "
        "ScalarType? dst_type=None) -> (Tensor, Tensor, Tensor)");
  m.def("npu_swiglu_quant(Tensor x, *, Tensor? smooth_scales=None, Tensor? offsets=None, Tensor? group_index=None, "
        "bool activate_left=False, int quant_mode=0, int group_list_type=0, ScalarType? dst_type=None) "
        "-> (Tensor, Tensor)");
  m.def("npu_anti_quant(Tensor x, Tensor scale, *, Tensor? offset=None, ScalarType? dst_dtype=None, "
        "ScalarType? src_dtype=None) -> Tensor");
  m.def("npu_trans_quant_param(Tensor scale, Tensor? offset=None) -> Tensor");
}

TORCH_LIBRARY_IMPL(npu, CUDA, m) {
  m.impl("npu_dynamic_quant", TORCH_FN(dynamic_quant_cuda));
  m.impl("npu_quant_matmul", TORCH_FN(quant_matmul_cuda));
  m.impl("npu_weight_quant_batchmatmul", TORCH_FN(weight_quant_cuda));
  m.impl("npu_convert_weight_to_int4pack", TORCH_FN(int4pack_cuda));
  m.impl("npu_dynamic_quant_asymmetric", TORCH_FN(dynamic_quant_asym_cuda));
  m.impl("npu_anti_quant", TORCH_FN(anti_quant_cuda));
  m.impl("npu_swiglu_quant", TORCH_FN(swiglu_quant_cuda));
  m.impl("npu_trans_quant_param", TORCH_FN(trans_quant_param_cuda));
}

TORCH_LIBRARY_IMPL(npu, Meta, m) {
  m.impl("npu_dynamic_quant", TORCH_FN(dynamic_quant_meta));
  m.impl("npu_quant_matmul", TORCH_FN(quant_matmul_meta));
  m.impl("npu_weight_quant_batchmatmul", TORCH_FN(weight_quant_meta));
  m.impl("npu_convert_weight_to_int4pack", TORCH_FN(int4pack_meta));
  m.impl("npu_dynamic_quant_asymmetric", TORCH_FN(dynamic_quant_asym_meta));
  m.impl("npu_anti_quant", TORCH_FN(anti_quant_meta));
  m.impl("npu_swiglu_quant", TORCH_FN(swiglu_quant_meta));
  m.impl("npu_trans_quant_param", TORCH_FN(trans_quant_param_meta));
}
