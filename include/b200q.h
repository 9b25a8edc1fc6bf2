/* b200q.h - C ABI of the B200 (sm_100a) quantized-inference kernels.
 *
 * These entry points are what a binding of torch_npu's quantized-inference operator
 * path calls in place of the op-plugin OpApi functions and the aclnn kernels behind
 * them.  Reference interfaces are cited by the path of the file inside Ascend/pytorch.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer unless it says "host"; tensors are row-major;
 *   - `stream` is a cudaStream_t passed as void*; work is enqueued, never synchronised;
 *   - functions return a b200q_status; b200q_last_error() gives the thread's last message;
 *   - the library allocates no device memory: scratch is passed in by the caller and sized
 *     by the matching *_workspace_bytes() query;
 *   - there is no CPU fallback: without a CUDA device every compute call fails.
 */
#ifndef B200Q_H_
#define B200Q_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  B200Q_OK = 0,
  B200Q_ERR_BAD_ARG = 1,      /* null pointer, negative size, misaligned buffer, bad enum   */
  B200Q_ERR_UNSUPPORTED = 2,  /* valid request outside what the path implements            */
  B200Q_ERR_LAUNCH = 3,       /* CUDA reported an error at launch                           */
  B200Q_ERR_WORKSPACE = 4,    /* workspace missing or smaller than *_workspace_bytes()      */
  B200Q_ERR_DEVICE = 5        /* a kernel recorded a device-side error (see device_error)   */
} b200q_status;

typedef enum {
  B200Q_BF16 = 0,
  B200Q_F16 = 1,
  B200Q_F32 = 2,
  B200Q_I8 = 3,
  B200Q_I32 = 4,
  B200Q_I64 = 5,  /* npu_trans_quant_param encoding: fp32 bit pattern in the low word */
  B200Q_NONE = -1
} b200q_dtype;

/* Library version (major*10000 + minor*100 + patch) and the last error text of the calling thread. */
int b200q_version(void);
const char* b200q_last_error(void);
const char* b200q_status_string(int status);

/* Reads (and, if `reset` != 0, clears) the device-side error word of the current device.
 * 0 means no kernel gave up a bounded wait.  Synchronises the device. */
int b200q_device_error(unsigned int* code, int reset);

/* Optional mirror of the error word in mapped pinned host memory.  After b200q_enable_host_error_word()
 * (once per device, with that device current; it allocates one pinned host word and synchronises), a
 * kernel that records an error also writes the code to the mirror, and b200q_peek_device_error() reads
 * it without touching the device: a host layer can check it at every call for free.  0 = no error.
 * The same role as the reference's asynchronous error surfacing at the next call
 * (torch_npu/csrc/framework/OpParamMaker.cpp:258-264). */
int b200q_enable_host_error_word(void);
unsigned int b200q_peek_device_error(void);

/* Self-test of the bounded waits: launches one warp that waits on a barrier nothing will ever arrive on,
 * with a budget of limit_ns (1 ns .. 1 s).  The kernel returns by itself; afterwards b200q_device_error
 * reports code 0x1FF.  Nothing faults or traps.  Counterpart of the reference's watchdog test, which
 * lets a collective time out on purpose (test/distributed/test_watchdog.py:15-32). */
int b200q_selftest_expire_wait(uint64_t limit_ns, void* stream);

/* npu_dynamic_quant(input, smooth_scales=None) -> (int8 y, fp32 scale)
 *   replaces op_plugin::npu_dynamic_quant / aclnn DynamicQuant, reached from
 *   torch_npu/onnx/wrapper_onnx_ops.py:743-745; output contract test/test_fake_tensor.py:1671-1686.
 * x [rows,k] bf16 or f16; smooth [k] (f32 or x's dtype) or NULL; y int8 [rows,k]; scale f32 [rows].
 * Per row: xs = x*smooth (fp32), scale = max|xs| / 127, y = clamp(rint(xs/scale), -128, 127);
 * an all-zero row gives scale 0 and y 0. */
int b200q_dynamic_quant(const void* x, int x_dtype, const void* smooth, int smooth_dtype, int8_t* y,
                        float* scale, int64_t rows, int64_t k, void* stream);

/* npu_dynamic_quant(input, smooth_scales, group_index) and
 * npu_dynamic_quant_asymmetric(input, smooth_scales, group_index) -> (int8 y, f32 scale, f32 offset)
 *   replace op_plugin::npu_dynamic_quant / npu_dynamic_quant_asymmetric (aclnnDynamicQuantV2), reached from
 *   torch_npu/onnx/wrapper_onnx_ops.py:743-745 and :762-767; output contracts test/test_fake_tensor.py:1671-1709,
 *   group_index usage test/onnx/test_wrapper_onnx_ops.py:1335-1392.
 * group_index (or NULL): int32 [n_groups], sorted cumulative end rows; row r uses smooth row g, the first g
 * with r < group_index[g] (rows past the last entry use the last row); smooth is then [n_groups, k].
 * offset == NULL: symmetric, as b200q_dynamic_quant.  offset != NULL: asymmetric, per row
 * scale = (max(xs) - min(xs)) / 255, offset = 127 - max(xs) / scale,
 * y = clamp(rint(xs / scale + offset), -128, 127); a constant row gives scale 0, offset 0, y 0. */
int b200q_dynamic_quant_ext(const void* x, int x_dtype, const void* smooth, int smooth_dtype,
                            const int32_t* group_index, int64_t n_groups, int8_t* y, float* scale, float* offset,
                            int64_t rows, int64_t k, void* stream);

/* npu_swiglu_quant(x, *, smooth_scales=None, ..., activate_left, quant_mode=1 (dynamic)) -> (int8 y, f32 scale)
 *   replaces op_plugin::npu_swiglu_quant / aclnnSwiGluQuant (named in docs/zh/release_notes.md:303; the
 *   activation is the reference's npu_swiglu, torch_npu/_inductor/decomposition.py:186-188).
 * x [rows, 2f] bf16 or f16; act = silu(a) * b in fp32 with a = x[:, :f] when activate_left, else x[:, f:];
 * xs = act * smooth (smooth [f], f32 or x's dtype, or NULL); then per row scale = max|xs| / 127,
 * y = clamp(rint(xs / scale), -128, 127) as b200q_dynamic_quant.  f must be a multiple of 8, at most 32768. */
int b200q_swiglu_quant(const void* x, int x_dtype, const void* smooth, int smooth_dtype, int activate_left,
                       int8_t* y, float* scale, int64_t rows, int64_t f, void* stream);

/* npu_quant_matmul(x1, x2, scale, *, offset, pertoken_scale, bias, output_dtype)
 *   replaces op_plugin::npu_quant_matmul / aclnnQuantMatmulV3-V4, reached from
 *   torch_npu/contrib/module/linear_quant.py:110-112 and linear_a8w8_quant.py:117-120.
 * out[m,n] = cast( float(sum_k x1[m,k]*x2[k,n] + bias_i32[n]) * scale[n] * pertoken[m]
 *                  + bias_float[n] + offset[n] );  int32 output returns the accumulator. */
typedef struct {
  const int8_t* x1;        /* [m,k], row stride k                                             */
  const int8_t* x2;        /* element (k_,n_) at x2[k_*x2_stride_k + n_*x2_stride_n]          */
  int64_t m, k, n;
  int64_t x2_stride_k;     /* 1 for the transposed view of an [n,k] weight (what the modules  */
  int64_t x2_stride_n;     /*   pass); n and 1 for a contiguous [k,n] weight                  */
  const void* scale;       /* [scale_len], scale_len = 1 or n; f32, bf16 or i64               */
  int scale_dtype;
  int64_t scale_len;
  const float* offset;     /* [offset_len] (1 or n) or NULL                                   */
  int64_t offset_len;
  const float* pertoken_scale; /* [m] or NULL                                                 */
  const void* bias;        /* [n] or NULL; i32 joins the accumulator, bf16/f16/f32 are added
                              after the scales                                                */
  int bias_dtype;
  void* out;               /* [m,n], row stride out_row_stride (n when that field is 0)       */
  int out_dtype;           /* B200Q_I8, B200Q_F16, B200Q_BF16, B200Q_I32 (accumulator) or
                              B200Q_F32 (dequantised value before the output cast)            */
  void* workspace;         /* >= b200q_quant_matmul_workspace_bytes(), 256-byte aligned       */
  size_t workspace_bytes;
  int64_t out_row_stride;  /* elements between rows of out; 0 means n.  A larger stride lets a
                              column shard be written straight into its place in an [m, N] matrix */
  /* Multi-GPU epilogues: the GEMM itself stores finished tiles into peers' memory (peer-mapped device
   * pointers, plain 128-bit stores over NVLink, full 128-byte lines), so the exchange overlaps the main
   * loop tile by tile.  They take the place of the collective that follows the matmul in the reference:
   * hcclAllGather of a column-sharded output (torch_npu/csrc/distributed/ProcessGroupHCCL.cpp:5896-5956) and
   * the reduce-scatter inside npu_mm_reduce_scatter_base (torch_npu/distributed/tensor/_matrix_ops.py:556-561).
   *   replicate (route_rows == 0, n_peer_out = 1..8): every element written to out[...] is also written to
   *     the same offset from peer_out[i], the address of the same block in peer i's matrix.
   *   routed (route_rows > 0): row r goes to row r % route_rows of peer_out[r / route_rows]
   *     (ceil(m / route_rows) <= 8 entries, one of which may be local memory; row stride out_row_stride);
   *     `out` is ignored.  With out_dtype B200Q_F32 this is the scatter half of a reduce-scatter.
   * Needs out_dtype bf16/f16/f32/i32, n*size a multiple of 128 bytes, 16-byte aligned destinations and
   * operands that meet the TMA rules; the caller orders a cross-rank barrier after the call. */
  void* const* peer_out;   /* HOST array of device pointers, or NULL                                   */
  int n_peer_out;
  int64_t route_rows;
} b200q_quant_matmul_args;

size_t b200q_quant_matmul_workspace_bytes(int64_t m, int64_t k, int64_t n, int64_t x2_stride_k,
                                          int64_t x2_stride_n);
int b200q_quant_matmul(const b200q_quant_matmul_args* args, void* stream);

/* b200q_quant_matmul for callers that cannot allocate device memory.  (No counterpart in the
 * reference: its operators always draw workspace from the framework's allocator.)
 *   Who needs it: a host that cannot call cudaMalloc or torch's allocator when the matmul runs, e.g. a
 *   server that has already given all free HBM to its KV-cache pool, a plugin living inside another
 *   runtime's fixed memory plan, or a code path where an allocation, which may synchronise the device,
 *   is not allowed.  Such a caller has nothing to put into args->workspace.
 *   What it does: same arguments, same kernels and bit-identical results as b200q_quant_matmul, but
 *   args->workspace / workspace_bytes are ignored and the scratch (split-K accumulators, weight
 *   re-layout) comes from an array of b200q_static_scratch_bytes() = 16 MiB built into the library.
 *   Every GPU that loads the library holds that array until the process exits.  It calls no
 *   cudaMalloc/cudaFree and no allocating library routine.
 *   Limit: shapes whose b200q_quant_matmul_workspace_bytes() exceeds 16 MiB are refused with
 *   B200Q_ERR_WORKSPACE (nothing is launched); use b200q_quant_matmul for those.
 *   First call on a device: looks up the array's device address (cudaGetSymbolAddress, once per device,
 *   cached).  Make that first call before starting any stream capture.
 *   Sharing: all calls on a device use the same array and it keeps its last contents; the part that
 *   must start at zero is cleared on `stream` inside every call.  Two calls that overlap on the GPU
 *   (different streams without an ordering between them) race on the array: serialise them. */
size_t b200q_static_scratch_bytes(void);
int b200q_quant_matmul_static_scratch(const b200q_quant_matmul_args* args, void* stream);

/* npu_weight_quant_batchmatmul(x, weight, antiquant_scale, antiquant_offset, ..., antiquant_group_size)
 *   replaces op_plugin::npu_weight_quant_batchmatmul / aclnnWeightQuantBatchMatmulV2, reached from
 *   torch_npu/contrib/module/linear_weight_quant.py:106-109.
 * out = x @ ((w + antiquant_offset) * antiquant_scale) (+ bias), result in x's dtype. */
typedef struct {
  const void* x;           /* [m,k] bf16 or f16, row stride k                                 */
  int x_dtype;
  const void* weight;      /* int8: element (k_,n_) at weight[k_*w_stride_k + n_*w_stride_n];
                              int4: int32 [k, n/8] contiguous, 8 values per word, value j of a
                              word in bits [4j, 4j+4)                                         */
  int weight_bits;         /* 8 or 4                                                          */
  int64_t m, k, n;
  int64_t w_stride_k, w_stride_n; /* int8 only                                                */
  const void* antiquant_scale;    /* [groups, n] in x's dtype, row stride n; groups = 1 or k/group_size */
  const void* antiquant_offset;   /* same shape or NULL                                       */
  int64_t group_size;      /* 0 = per channel                                                 */
  const void* bias;        /* [n] in x's dtype, or NULL                                       */
  void* out;               /* [m,n] in x's dtype                                              */
  void* workspace;
  size_t workspace_bytes;
} b200q_weight_quant_matmul_args;

size_t b200q_weight_quant_matmul_workspace_bytes(int64_t m, int64_t k, int64_t n, int weight_bits);
int b200q_weight_quant_matmul(const b200q_weight_quant_matmul_args* args, void* stream);

/* npu_convert_weight_to_int4pack(weight): int32 [rows, cols] holding one int4 value each
 * -> int32 [rows, cols/8]; value j of each group of eight goes to bits [4j, 4j+4).
 *   The operator does not occur in the reference tree; the nibble order is the one its
 *   unpack helper expects, test/custom_ops/test_npu_anti_quant.py:12-24. */
int b200q_int4pack(const int32_t* w, int32_t* packed, int64_t rows, int64_t cols, void* stream);

/* npu_anti_quant(x, scale, *, offset=None, dst_dtype=None, src_dtype=None)
 *   replaces op_plugin::npu_anti_quant / aclnnAscendAntiQuant (wrapper torch_npu/onnx/wrapper_onnx_ops.py:824-828;
 *   golden test/custom_ops/test_npu_anti_quant.py:29-42, contract test/test_fake_tensor.py:1949-1959).
 * x: int8 [rows, n] (src_bits 8) or int32 words of eight int4 values [rows, n/8] (src_bits 4, value j of a
 * word in bits [4j, 4j+4)); scale, offset: [n] f32 or bf16 (offset may be NULL); out [rows, n] f16 or bf16.
 * out = cast((float(x) + offset) * scale): fp32 sum, fp32 product, one rounding to the output type. */
int b200q_anti_quant(const void* x, int src_bits, const void* scale, const void* offset, int param_dtype,
                     void* out, int out_dtype, int64_t rows, int64_t n, void* stream);

/* Exchange step of the column-sharded linear: pushes bytes [col_offset, col_offset + block_bytes) of
 * every row of the local [rows, row_stride_bytes] matrix `src` to the same place in each of the
 * `n_peers` matrices `peer_dst[i]` (HOST array of device pointers into peers' memory, mapped for
 * peer access by the caller, e.g. through CUDA IPC or torch symmetric memory).  Plain 128-bit stores
 * over NVLink; the caller runs a cross-rank barrier afterwards.
 *   replaces hcclAllGather in ProcessGroupHCCL::_allgather_base
 *   (torch_npu/csrc/distributed/ProcessGroupHCCL.cpp:5896-5956) for this path. */
int b200q_scatter_columns(const void* src, void* const* peer_dst, int n_peers, int64_t rows,
                          int64_t row_stride_bytes, int64_t col_offset_bytes, int64_t block_bytes, void* stream);

/* The same exchange on the copy engines: one strided device-to-device copy per peer (cudaMemcpy2DAsync) of
 * bytes [col_offset, col_offset + block_bytes) of every row, queued on `stream` in the order of `peer_dst`.
 * No SM is used, so a side stream can carry the exchange of one step while the kernels of the next one run;
 * the caller orders it after the producing GEMM with an event and runs the cross-rank barrier behind it on
 * the same stream.  Same arguments as b200q_scatter_columns; no alignment rule.
 *   replaces hcclAllGather in ProcessGroupHCCL::_allgather_base
 *   (torch_npu/csrc/distributed/ProcessGroupHCCL.cpp:5896-5956) for this path. */
int b200q_copy_columns(const void* src, void* const* peer_dst, int n_peers, int64_t rows, int64_t row_stride_bytes,
                       int64_t col_offset_bytes, int64_t block_bytes, void* stream);

/* Cross-rank barrier for the multi-GPU epilogues above: `flags` is a HOST array of `world` device
 * pointers, flags[i] = rank i's array of `world` zero-initialised uint32 words, mapped for peer access.
 * Rank `rank` announces `epoch` (1, 2, 3 ... the same on every rank for the same barrier) to every peer
 * and waits until every peer has announced it; everything the stream wrote before (pushes included) is
 * ordered before the announcement.  The wait is bounded by timeout_ns (0 = 10 s): when a peer does not
 * arrive the kernel records code 0x104 in the device error word and returns, it never traps.
 *   replaces the synchronisation inside hcclAllGather / HcclReduceScatter for this path. */
int b200q_peer_barrier(void* const* flags, int world, int rank, uint32_t epoch, uint64_t timeout_ns, void* stream);

/* Reduce half of npu_mm_reduce_scatter_base / npu_mm_all_reduce_base (golden:
 * test/distributed/tensor/test_matrix_ops.py:86-110, partial products added in rank order in fp32):
 * out[r,c] = cast(slots[0][r][c] + slots[1][r][c] + ... ), slots f32 [n_slots, rows, n] contiguous, out
 * [rows, n] bf16/f16/f32; the result is also stored at the same offset of each peer_out[i] (HOST array of
 * n_peer_out device pointers into peers' memory, or NULL/0).  rows*n must be a multiple of 4. */
int b200q_reduce_slots(const float* slots, int n_slots, int64_t rows, int64_t n, void* out, int out_dtype,
                       void* const* peer_out, int n_peer_out, void* stream);

/* npu_trans_quant_param(scale, offset=None): fp32 scale -> int64 dequant parameter
 *   (torch_npu/contrib/module/linear_quant.py:107-108; contract test/test_fake_tensor.py:1929-1943).
 * out[i] = bit pattern of scale[i % scale_len] in the low word, upper word 0. */
int b200q_trans_quant_param(const float* scale, int64_t scale_len, int64_t* out, int64_t out_len, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200Q_H_ */
