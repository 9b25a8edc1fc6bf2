// Exchange step of the column-sharded linear over NVLink peer memory.
//
// Every rank holds an [rows, N] output matrix in memory its peers can address.  After its GEMM has
// written the rank's own column block into the local matrix, this kernel pushes that block into the
// same place of every peer's matrix with plain 128-bit stores: each warp reads 512 contiguous bytes
// of a row once and writes them to all peers (one read, g-1 remote writes), so the NVLink packets
// are full cache lines and no re-interleaving copy is needed afterwards.  It takes the place of
// hcclAllGather in the reference's sharded linear (torch_npu/csrc/distributed/ProcessGroupHCCL.cpp:5896-5956).
// No TMA, no multicast, no waits: the caller orders it on a stream after the GEMM and runs a
// cross-rank barrier after it.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"
#include "ptx.cuh"

namespace b200q {
namespace {

constexpr int kMaxPeers = 15;

struct PeerList {
  void* dst[kMaxPeers];
  int count;
};

// Each thread moves kUnroll 16-byte vectors per trip (loads first, then all remote stores), so that a
// partly occupied SM - the kernel usually shares the GPU with the next GEMM - still keeps enough
// stores in flight to fill the links.
constexpr int kUnroll = 4;

__global__ void __launch_bounds__(256) scatter_columns_kernel(const uint8_t* __restrict__ src, PeerList peers,
                                                             int64_t rows, int64_t row_stride, int64_t col_offset,
                                                             int64_t vecs_per_row) {
  const int64_t total = rows * vecs_per_row;
  const int64_t step = (int64_t)gridDim.x * blockDim.x;
  for (int64_t base = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; base < total; base += step * kUnroll) {
    uint4 val[kUnroll];
    int64_t off[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t i = base + u * step;
      off[u] = -1;
      if (i < total) {
        const int64_t r = i / vecs_per_row, v = i - r * vecs_per_row;
        off[u] = r * row_stride + col_offset + v * 16;
        val[u] = __ldcs(reinterpret_cast<const uint4*>(src + off[u]));
      }
    }
#pragma unroll 1
    for (int p = 0; p < peers.count; ++p) {
      uint8_t* dst = static_cast<uint8_t*>(peers.dst[p]);
#pragma unroll
      for (int u = 0; u < kUnroll; ++u)
        if (off[u] >= 0) *reinterpret_cast<uint4*>(dst + off[u]) = val[u];
    }
  }
}

// Cross-rank barrier over peer-mapped flag words.  flags.dst[i] is rank i's array of `world` 32-bit words.
// Lane p tells rank p "rank `rank` has reached barrier `epoch`" by storing the epoch into word `rank` of
// p's array, then waits until word p of its own array has reached the epoch.  Epochs only grow, so the
// words never need clearing; the comparison is on the signed distance, which survives wrap-around.  A
// system-scope fence before the stores orders everything this stream wrote earlier (the pushes of the
// preceding kernels included) before the flag.  The wait has a time budget: when a peer does not show
// up, the kernel records kDevTimeoutBarrier in the device error word and returns; it never traps.
__global__ void peer_barrier_kernel(PeerList flags, int world, int rank, uint32_t epoch, unsigned long long limit_ns) {
  const int p = threadIdx.x;
  if (p >= world || p == rank) return;
  __threadfence_system();
  uint32_t* theirs = static_cast<uint32_t*>(flags.dst[p]) + rank;
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(theirs), "r"(epoch) : "memory");
  const uint32_t* mine = static_cast<const uint32_t*>(flags.dst[rank]) + p;
  const unsigned long long t0 = global_timer_ns();
  for (;;) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
    if ((int32_t)(v - epoch) >= 0) return;
    if (global_timer_ns() - t0 > limit_ns) {
      record_device_error(kDevTimeoutBarrier);
      return;
    }
    __nanosleep(100);
  }
}

// Sum of n_slots fp32 [rows, n] slices in slot order (the order the reference's golden adds the ranks'
// partial products in), one rounding to the output type; optionally the result also goes to the same
// offset of every peer destination (the all-gather half of an all-reduce).  Four elements per thread.
template <typename OT>
__device__ __forceinline__ void store4(OT* p, float4 v);
template <>
__device__ __forceinline__ void store4<float>(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
template <>
__device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, float4 v) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 u;
  u.x = *reinterpret_cast<uint32_t*>(&a);
  u.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = u;
}
template <>
__device__ __forceinline__ void store4<__half>(__half* p, float4 v) {
  __half2 a = __floats2half2_rn(v.x, v.y), b = __floats2half2_rn(v.z, v.w);
  uint2 u;
  u.x = *reinterpret_cast<uint32_t*>(&a);
  u.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = u;
}

template <typename OT>
__global__ void __launch_bounds__(256) reduce_slots_kernel(const float* __restrict__ slots, int n_slots, int64_t quads,
                                                          OT* __restrict__ out, PeerList peers) {
  const int64_t step = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < quads; i += step) {
    float4 acc = __ldcs(reinterpret_cast<const float4*>(slots) + i);
    for (int s = 1; s < n_slots; ++s) {
      const float4 v = __ldcs(reinterpret_cast<const float4*>(slots) + (int64_t)s * quads + i);
      acc.x = __fadd_rn(acc.x, v.x);
      acc.y = __fadd_rn(acc.y, v.y);
      acc.z = __fadd_rn(acc.z, v.z);
      acc.w = __fadd_rn(acc.w, v.w);
    }
    store4<OT>(out + 4 * i, acc);
    for (int p = 0; p < peers.count; ++p) store4<OT>(static_cast<OT*>(peers.dst[p]) + 4 * i, acc);
  }
}

}  // namespace
}  // namespace b200q

extern "C" int b200q_peer_barrier(void* const* flags, int world, int rank, uint32_t epoch, uint64_t timeout_ns,
                                  void* stream) {
  using namespace b200q;
  clear_error();
  B200Q_REQUIRE(world >= 1 && world <= kMaxPeers && rank >= 0 && rank < world, B200Q_ERR_BAD_ARG,
                "peer_barrier: world %d / rank %d out of range (at most %d ranks)", world, rank, kMaxPeers);
  B200Q_REQUIRE(timeout_ns <= 10000000000ULL, B200Q_ERR_BAD_ARG, "peer_barrier: timeout above 10 s");
  if (world == 1) return B200Q_OK;
  B200Q_REQUIRE(flags != nullptr, B200Q_ERR_BAD_ARG, "peer_barrier: flags is NULL");
  PeerList fl{};
  fl.count = world;
  for (int i = 0; i < world; ++i) {
    B200Q_REQUIRE(flags[i] != nullptr && aligned(flags[i], 4), B200Q_ERR_BAD_ARG, "peer_barrier: flag array %d is NULL or misaligned", i);
    fl.dst[i] = flags[i];
  }
  peer_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(fl, world, rank, epoch,
                                                                      timeout_ns ? timeout_ns : 10000000000ULL);
  return check_launch("peer_barrier");
}

extern "C" int b200q_reduce_slots(const float* slots, int n_slots, int64_t rows, int64_t n, void* out, int out_dtype,
                                  void* const* peer_out, int n_peer_out, void* stream) {
  using namespace b200q;
  clear_error();
  B200Q_REQUIRE(n_slots >= 1 && rows >= 0 && n >= 0, B200Q_ERR_BAD_ARG, "reduce_slots: bad size");
  B200Q_REQUIRE(n_peer_out >= 0 && n_peer_out <= kMaxPeers, B200Q_ERR_BAD_ARG, "reduce_slots: 0..%d peers", kMaxPeers);
  B200Q_REQUIRE(out_dtype == B200Q_BF16 || out_dtype == B200Q_F16 || out_dtype == B200Q_F32, B200Q_ERR_UNSUPPORTED,
                "reduce_slots: output must be bf16, f16 or f32");
  if (rows == 0 || n == 0) return B200Q_OK;
  B200Q_REQUIRE(slots != nullptr && out != nullptr, B200Q_ERR_BAD_ARG, "reduce_slots: NULL buffer");
  B200Q_REQUIRE((rows * n) % 4 == 0 && aligned(slots, 16) && aligned(out, 16), B200Q_ERR_BAD_ARG,
                "reduce_slots: rows*n must be a multiple of 4 and the buffers 16-byte aligned");
  PeerList peers{};
  peers.count = n_peer_out;
  for (int i = 0; i < n_peer_out; ++i) {
    B200Q_REQUIRE(peer_out != nullptr && peer_out[i] != nullptr && aligned(peer_out[i], 16), B200Q_ERR_BAD_ARG,
                  "reduce_slots: peer %d pointer is NULL or misaligned", i);
    peers.dst[i] = peer_out[i];
  }
  const int64_t quads = rows * n / 4;
  const int64_t want = ceil_div(quads, 256);
  const int blocks = (int)(want < (int64_t)sm_count() * 8 ? want : (int64_t)sm_count() * 8);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (out_dtype == B200Q_BF16)
    reduce_slots_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(slots, n_slots, quads, static_cast<__nv_bfloat16*>(out), peers);
  else if (out_dtype == B200Q_F16)
    reduce_slots_kernel<__half><<<blocks, 256, 0, st>>>(slots, n_slots, quads, static_cast<__half*>(out), peers);
  else
    reduce_slots_kernel<float><<<blocks, 256, 0, st>>>(slots, n_slots, quads, static_cast<float*>(out), peers);
  return check_launch("reduce_slots");
}

extern "C" int b200q_scatter_columns(const void* src, void* const* peer_dst, int n_peers, int64_t rows,
                                     int64_t row_stride_bytes, int64_t col_offset_bytes, int64_t block_bytes,
                                     void* stream) {
  using namespace b200q;
  clear_error();
  B200Q_REQUIRE(n_peers >= 0 && n_peers <= kMaxPeers, B200Q_ERR_BAD_ARG, "scatter_columns: 0..%d peers, got %d",
                kMaxPeers, n_peers);
  B200Q_REQUIRE(rows >= 0 && block_bytes >= 0 && col_offset_bytes >= 0 &&
                    col_offset_bytes + block_bytes <= row_stride_bytes,
                B200Q_ERR_BAD_ARG, "scatter_columns: column block does not fit the row");
  if (n_peers == 0 || rows == 0 || block_bytes == 0) return B200Q_OK;
  B200Q_REQUIRE(src != nullptr && peer_dst != nullptr, B200Q_ERR_BAD_ARG, "scatter_columns: NULL pointer");
  B200Q_REQUIRE(aligned(src, 16) && row_stride_bytes % 16 == 0 && col_offset_bytes % 16 == 0 && block_bytes % 16 == 0,
                B200Q_ERR_BAD_ARG, "scatter_columns: base, row stride, column offset and block must be 16-byte multiples");
  PeerList peers{};
  peers.count = n_peers;
  for (int i = 0; i < n_peers; ++i) {
    B200Q_REQUIRE(peer_dst[i] != nullptr && aligned(peer_dst[i], 16), B200Q_ERR_BAD_ARG,
                  "scatter_columns: peer %d pointer is NULL or misaligned", i);
    peers.dst[i] = peer_dst[i];
  }
  const int64_t vecs_per_row = block_bytes / 16;
  const int64_t want = ceil_div(rows * vecs_per_row, 256 * kUnroll);
  const int64_t cap = (int64_t)sm_count() * 4;
  scatter_columns_kernel<<<(unsigned)(want < cap ? want : cap), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(src), peers, rows, row_stride_bytes, col_offset_bytes, vecs_per_row);
  return check_launch("scatter_columns");
}

extern "C" int b200q_copy_columns(const void* src, void* const* peer_dst, int n_peers, int64_t rows,
                                  int64_t row_stride_bytes, int64_t col_offset_bytes, int64_t block_bytes,
                                  void* stream) {
  using namespace b200q;
  clear_error();
  B200Q_REQUIRE(n_peers >= 0 && n_peers <= kMaxPeers, B200Q_ERR_BAD_ARG, "copy_columns: 0..%d peers, got %d", kMaxPeers,
                n_peers);
  B200Q_REQUIRE(rows >= 0 && block_bytes >= 0 && col_offset_bytes >= 0 &&
                    col_offset_bytes + block_bytes <= row_stride_bytes,
                B200Q_ERR_BAD_ARG, "copy_columns: column block does not fit the row");
  if (n_peers == 0 || rows == 0 || block_bytes == 0) return B200Q_OK;
  B200Q_REQUIRE(src != nullptr && peer_dst != nullptr, B200Q_ERR_BAD_ARG, "copy_columns: NULL pointer");
  const uint8_t* from = static_cast<const uint8_t*>(src) + col_offset_bytes;
  for (int i = 0; i < n_peers; ++i) {
    B200Q_REQUIRE(peer_dst[i] != nullptr, B200Q_ERR_BAD_ARG, "copy_columns: peer %d pointer is NULL", i);
    cudaError_t err = cudaMemcpy2DAsync(static_cast<uint8_t*>(peer_dst[i]) + col_offset_bytes, (size_t)row_stride_bytes,
                                        from, (size_t)row_stride_bytes, (size_t)block_bytes, (size_t)rows,
                                        cudaMemcpyDeviceToDevice, static_cast<cudaStream_t>(stream));
    if (err != cudaSuccess) return fail(B200Q_ERR_LAUNCH, "copy_columns: peer %d: %s", i, cudaGetErrorString(err));
  }
  return B200Q_OK;
}
