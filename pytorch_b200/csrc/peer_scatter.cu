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
#include "common.cuh"

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

}  // namespace
}  // namespace b200q

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
