// npu_quant_matmul: int8 x int8 -> int32 GEMM on tcgen05 (kind::i8) with a fused
// dequantisation epilogue.
//
// Both operands are consumed K-major (x1 [M,K]; the weight as [N,K], which is the memory
// the reference's modules hand over as a transposed view).  One persistent CTA per SM:
//   warp 0      TMA producer: 128x128-byte operand tiles, 128B swizzle, STAGES-deep ring
//   warp 1      MMA issuer: tcgen05.mma.cta_group::1.kind::i8, M=128, N=BN, K=32 per instruction,
//               accumulators in TMEM, two accumulator buffers so the epilogue of one tile
//               overlaps the main loop of the next
//   warps 2-5   epilogue: tcgen05.ld -> registers -> float(acc+bias)*scale*pertoken+offset -> store
// Two operand assignments share the kernel:
//   normal (M > 128)  A = x1 rows (tokens), B = weight rows (channels)
//   swapped (M <= 128) A = weight rows, B = x1 rows padded to BN in {16,32,64,128}: the weight, which
//               dominates the traffic, fills the 128-row MMA axis; K is split across CTAs so
//               that every SM streams weights, partial sums meet in an int32 scratch through
//               integer atomics (exact in any order) and a small kernel applies the epilogue.
// Every mbarrier wait is bounded; on a timeout the CTA records an error code and winds down.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <stdlib.h>

#include <mutex>
#include <type_traits>

#include "common.cuh"
#include "ptx.cuh"
#include "tensormap.cuh"

namespace b200q {
namespace {

constexpr int kBK = 128;            // K bytes per pipeline stage = one 128B swizzle row
constexpr int kTileA = 128;         // rows of the A operand per tile = UMMA M
constexpr int kATileBytes = kTileA * kBK;
constexpr int kEpiThreads = 128;
constexpr int kThreads = 64 + kEpiThreads;

enum EpiFlags : uint32_t {
  kHasPt = 1, kHasOff = 2, kHasIntBias = 4, kHasFloatBias = 8,
  kOutVec = 16   // rows of `out` are 16-byte aligned: a thread may store 128-bit vectors
};

constexpr int kMaxDest = 8;   // GPUs of one node

struct Epi {
  const void* scale;
  const float* offset;
  const float* pertoken;
  const void* bias;
  void* out;
  int32_t* acc_ws;  // split-K: raw accumulators are added here instead of writing `out`
  int64_t m, n;
  int64_t ldo;      // row stride of `out` in elements (>= n)
  int scale_dtype, scale_bcast, offset_bcast, bias_dtype, out_dtype;
  uint32_t flags;
  // Multi-GPU epilogues (peer-mapped destinations, plain stores over NVLink):
  //   replicate (n_dest > 0, route_rows == 0): every finished element also goes to the same offset of
  //       dest[0..n_dest), the peers' copies of `out`;
  //   routed (route_rows > 0): row mm goes to row mm % route_rows of dest[mm / route_rows] (one of them
  //       may be local memory); `out` is not written.
  void* dest[kMaxDest];
  int n_dest;
  int64_t route_rows;
};

struct Sched {
  int tiles_a, tiles_b, splits, kblocks, kb_per_split, units;
};

__device__ __forceinline__ float load_scale(const Epi& e, int64_t n) {
  const int64_t i = e.scale_bcast ? 0 : n;
  if (e.scale_dtype == B200Q_F32) return __ldg(static_cast<const float*>(e.scale) + i);
  if (e.scale_dtype == B200Q_BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(e.scale)[i]);
  return __uint_as_float(static_cast<uint32_t>(static_cast<const unsigned long long*>(e.scale)[i]));
}
__device__ __forceinline__ float load_offset(const Epi& e, int64_t n) {
  return (e.flags & kHasOff) ? __ldg(e.offset + (e.offset_bcast ? 0 : n)) : 0.0f;
}
__device__ __forceinline__ int load_int_bias(const Epi& e, int64_t n) {
  return (e.flags & kHasIntBias) ? __ldg(static_cast<const int*>(e.bias) + n) : 0;
}
__device__ __forceinline__ float load_float_bias(const Epi& e, int64_t n) {
  if (!(e.flags & kHasFloatBias)) return 0.0f;
  if (e.bias_dtype == B200Q_F32) return __ldg(static_cast<const float*>(e.bias) + n);
  if (e.bias_dtype == B200Q_BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(e.bias)[n]);
  return __half2float(static_cast<const __half*>(e.bias)[n]);
}

// One rounding per step, no fused multiply-add: the CPU oracle does the same five operations.
__device__ __forceinline__ float dequant(int acc, int ib, float sc, float pt, float fb, float off, uint32_t flags) {
  float v = __int2float_rn(acc + ib);
  v = __fmul_rn(v, sc);
  if (flags & kHasPt) v = __fmul_rn(v, pt);
  if (flags & kHasFloatBias) v = __fadd_rn(v, fb);
  if (flags & kHasOff) v = __fadd_rn(v, off);
  return v;
}

__device__ __forceinline__ uint32_t to_bits16(float v, int out_dtype) {
  if (out_dtype == B200Q_BF16) return __bfloat16_as_ushort(__float2bfloat16_rn(v));
  return __half_as_ushort(__float2half_rn(v));
}
__device__ __forceinline__ int to_int8(float v) { return max(-128, min(127, __float2int_rn(v))); }

// Stores one finished element.
__device__ __forceinline__ void store_one(const Epi& e, int64_t idx, int acc, int ib, float v) {
  switch (e.out_dtype) {
    case B200Q_I32: static_cast<int*>(e.out)[idx] = acc + ib; break;
    case B200Q_F32: static_cast<float*>(e.out)[idx] = v; break;
    case B200Q_I8: static_cast<int8_t*>(e.out)[idx] = (int8_t)to_int8(v); break;
    default: static_cast<unsigned short*>(e.out)[idx] = (unsigned short)to_bits16(v, e.out_dtype); break;
  }
}

template <int N>
__device__ __forceinline__ void tmem_ld_chunk(uint32_t taddr, uint32_t (&r)[N]);
template <>
__device__ __forceinline__ void tmem_ld_chunk<32>(uint32_t taddr, uint32_t (&r)[32]) { tmem_ld_x32(taddr, r); }
template <>
__device__ __forceinline__ void tmem_ld_chunk<16>(uint32_t taddr, uint32_t (&r)[16]) { tmem_ld_x16(taddr, r); }

// AND-reduction of a predicate over the epilogue warps (named barrier 2).  Every epilogue
// thread calls it once per tile, so the decision to stop is taken by all of them together.
__device__ __forceinline__ bool epilogue_all(bool pred) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 p, %1, 0;\n\t"
      "bar.red.and.pred q, 2, %2, p;\n\t"
      "selp.u32 %0, 1, 0, q;\n\t}"
      : "=r"(r)
      : "r"((uint32_t)pred), "r"(kEpiThreads)
      : "memory");
  return r != 0;
}

// Epilogue of one accumulator tile whose rows are tokens and whose columns are channels: the calling
// thread owns row `mm` (TMEM lane taddr>>16 + lane) and walks the BN columns CH at a time; its CH results
// are contiguous in the output row.  Column parameters come from shared memory (broadcast reads).
// Must be called by all 32 lanes of the warp (tcgen05.ld is warp-collective).
template <int BN, int CH>
__device__ __forceinline__ void store_token_rows(const Epi& e, uint32_t taddr, int64_t mm, int64_t n_tile0,
                                                 const float* col_f0, const float* col_f1, const float* col_f2,
                                                 const int* col_i) {
  const bool mv = mm < e.m;
  const float pt = (mv && (e.flags & kHasPt)) ? __ldg(e.pertoken + mm) : 1.0f;
  const bool vec = (e.flags & kOutVec) != 0;
#pragma unroll 1
  for (int c = 0; c < BN / CH; ++c) {
    uint32_t r[CH];
    __syncwarp();
    tmem_ld_chunk<CH>(taddr + c * CH, r);
    tmem_ld_wait();
    const int64_t n0 = n_tile0 + c * CH;
    if (!mv || n0 >= e.n) continue;
    if (e.acc_ws) {
#pragma unroll
      for (int j = 0; j < CH; ++j)
        if (n0 + j < e.n) atomicAdd(e.acc_ws + mm * e.n + n0 + j, (int)r[j]);
    } else if (vec && n0 + CH <= e.n) {
      // 128-bit stores
      if (e.out_dtype == B200Q_I32) {
        uint4* dst = reinterpret_cast<uint4*>(static_cast<int*>(e.out) + mm * e.ldo + n0);
#pragma unroll
        for (int q = 0; q < CH / 4; ++q)
          dst[q] = make_uint4(r[4 * q] + col_i[c * CH + 4 * q], r[4 * q + 1] + col_i[c * CH + 4 * q + 1],
                              r[4 * q + 2] + col_i[c * CH + 4 * q + 2], r[4 * q + 3] + col_i[c * CH + 4 * q + 3]);
      } else if (e.out_dtype == B200Q_F32) {
        uint4* dst = reinterpret_cast<uint4*>(static_cast<float*>(e.out) + mm * e.ldo + n0);
#pragma unroll
        for (int q = 0; q < CH / 4; ++q) {
          uint32_t w[4];
#pragma unroll
          for (int b = 0; b < 4; ++b) {
            const int cj = c * CH + 4 * q + b;
            w[b] = __float_as_uint(dequant((int)r[4 * q + b], col_i[cj], col_f0[cj], pt, col_f2[cj], col_f1[cj], e.flags));
          }
          dst[q] = make_uint4(w[0], w[1], w[2], w[3]);
        }
      } else if (e.out_dtype == B200Q_I8) {
        uint32_t packed[CH / 4];
#pragma unroll
        for (int j = 0; j < CH; j += 4) {
          uint32_t w = 0;
#pragma unroll
          for (int b = 0; b < 4; ++b) {
            const int cj = c * CH + j + b;
            const float v = dequant((int)r[j + b], col_i[cj], col_f0[cj], pt, col_f2[cj], col_f1[cj], e.flags);
            w |= (uint32_t)(to_int8(v) & 0xFF) << (8 * b);
          }
          packed[j / 4] = w;
        }
        uint4* dst = reinterpret_cast<uint4*>(static_cast<int8_t*>(e.out) + mm * e.ldo + n0);
#pragma unroll
        for (int q = 0; q < CH / 16; ++q)
          dst[q] = make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
      } else {
        uint32_t packed[CH / 2];
#pragma unroll
        for (int j = 0; j < CH; j += 2) {
          const int cj = c * CH + j;
          const float v0 = dequant((int)r[j], col_i[cj], col_f0[cj], pt, col_f2[cj], col_f1[cj], e.flags);
          const float v1 =
              dequant((int)r[j + 1], col_i[cj + 1], col_f0[cj + 1], pt, col_f2[cj + 1], col_f1[cj + 1], e.flags);
          packed[j / 2] = to_bits16(v0, e.out_dtype) | (to_bits16(v1, e.out_dtype) << 16);
        }
        uint4* dst = reinterpret_cast<uint4*>(static_cast<unsigned short*>(e.out) + mm * e.ldo + n0);
#pragma unroll
        for (int q = 0; q < CH / 8; ++q)
          dst[q] = make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < CH; ++j) {
        if (n0 + j < e.n) {
          const int cj = c * CH + j;
          const int acc = (int)r[j];
          store_one(e, mm * e.ldo + n0 + j, acc, col_i[cj],
                    dequant(acc, col_i[cj], col_f0[cj], pt, col_f2[cj], col_f1[cj], e.flags));
        }
      }
    }
  }
}

// Epilogue of one accumulator tile for the multi-GPU forms (Epi::dest).  The calling warp owns the 32 token
// rows starting at row0 (lane = row).  Results pass through a 4 KB shared-memory staging area private to
// the warp, 128 bytes of every row at a time (64 16-bit or 32 32-bit outputs), so that eight lanes then
// write one full 128-byte line of a row and a warp instruction covers four rows: full lines keep the
// NVLink packets of the remote stores dense (256-byte runs with a correspondingly larger staging area and one
// pipeline stage less were measured slower: 0.45 against 0.42 ms for a link-bound 235 MB push to one peer).  16-byte chunks are XOR-swizzled by the row so that both
// the row-wise writes and the line-wise reads are free of bank conflicts.  Requires out_dtype in
// {bf16, f16, f32, i32}, n a multiple of the 128-byte slab and 16-byte aligned destinations.
constexpr int kPushStageBytes = 32 * 128;                  // per epilogue warp

template <int BN>
__device__ __forceinline__ void store_token_rows_push(const Epi& e, uint32_t taddr, int64_t row0, int lane,
                                                      int64_t n_tile0, const float* col_f0, const float* col_f1,
                                                      const float* col_f2, const int* col_i, uint32_t stage) {
  const int64_t mm = row0 + lane;
  const bool mv = mm < e.m;
  const float pt = (mv && (e.flags & kHasPt)) ? __ldg(e.pertoken + mm) : 1.0f;
  const bool wide = e.out_dtype == B200Q_F32 || e.out_dtype == B200Q_I32;
  const int ob = wide ? 4 : 2;
  const int slab = wide ? 32 : 64;                       // columns per 128-byte slab
#pragma unroll 1
  for (int c0 = 0; c0 < BN; c0 += slab) {
    if (n_tile0 + c0 >= e.n) break;                      // same decision in every lane
    uint32_t w[32];                                      // this row's 128 bytes
    if (wide) {
      uint32_t r[32];
      __syncwarp();
      tmem_ld_x32(taddr + c0, r);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const int cj = c0 + j;
        w[j] = e.out_dtype == B200Q_I32
                   ? r[j] + (uint32_t)col_i[cj]
                   : __float_as_uint(dequant((int)r[j], col_i[cj], col_f0[cj], pt, col_f2[cj], col_f1[cj], e.flags));
      }
    } else {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint32_t r[32];
        __syncwarp();
        tmem_ld_x32(taddr + c0 + 32 * h, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          const int cj = c0 + 32 * h + j;
          const float v0 = dequant((int)r[j], col_i[cj], col_f0[cj], pt, col_f2[cj], col_f1[cj], e.flags);
          const float v1 = dequant((int)r[j + 1], col_i[cj + 1], col_f0[cj + 1], pt, col_f2[cj + 1], col_f1[cj + 1], e.flags);
          w[16 * h + j / 2] = to_bits16(v0, e.out_dtype) | (to_bits16(v1, e.out_dtype) << 16);
        }
      }
    }
    __syncwarp();                                        // the previous slab has been read out
#pragma unroll
    for (int c = 0; c < 8; ++c)
      st_shared_v4(stage + lane * 128 + ((c ^ (lane & 7)) << 4), make_uint4(w[4 * c], w[4 * c + 1], w[4 * c + 2], w[4 * c + 3]));
    __syncwarp();
    const int ch = lane & 7;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int rr = 4 * i + (lane >> 3);
      const uint4 v = ld_shared_v4(stage + rr * 128 + ((ch ^ (rr & 7)) << 4));
      const int64_t row = row0 + rr;
      if (row >= e.m) continue;
      if (e.route_rows > 0) {
        const int64_t d = row / e.route_rows, lr = row - d * e.route_rows;
        *reinterpret_cast<uint4*>(static_cast<uint8_t*>(e.dest[d]) + (lr * e.ldo + n_tile0 + c0) * ob + ch * 16) = v;
      } else {
        const int64_t off = (row * e.ldo + n_tile0 + c0) * ob + ch * 16;
        *reinterpret_cast<uint4*>(static_cast<uint8_t*>(e.out) + off) = v;
#pragma unroll 1
        for (int p = 0; p < e.n_dest; ++p) *reinterpret_cast<uint4*>(static_cast<uint8_t*>(e.dest[p]) + off) = v;
      }
    }
  }
}

// Replicating epilogue through TMA stores (16-bit outputs, CTA-pair kernel): the four epilogue warps write a
// 128-row x 64-column chunk of the tile into a 128B-swizzled staging buffer, one thread issues a bulk tensor
// store of the chunk into the local matrix and into every peer's, and the warps go on to the next chunk in
// another buffer.  The accumulator buffer in tensor memory is released as soon as its last chunk is in shared
// memory, so the MMAs of the next tile overlap the stores over NVLink.  Rows beyond m and columns beyond n are
// clipped by the tensor maps.
constexpr int kTmaStoreBufs = 3;
constexpr int kTmaStoreBufBytes = 128 * 128;               // 128 rows x 64 two-byte columns
struct OutMaps {
  CUtensorMap m[kMaxDest + 1];                             // [0] the local matrix, [1..n_dest] the peers'
};
struct NoOutMaps {};

template <int BN>
__device__ __forceinline__ void store_token_rows_tma(const Epi& e, const OutMaps& om, uint32_t taddr, int64_t cta_row0,
                                                     int quad, int lane, bool issuer, int64_t n_tile0,
                                                     const float* col_f0, const float* col_f1, const float* col_f2,
                                                     const int* col_i, uint32_t stage_base, uint32_t& chunk) {
  const int64_t mm = cta_row0 + quad * 32 + lane;
  const float pt = (mm < e.m && (e.flags & kHasPt)) ? __ldg(e.pertoken + mm) : 1.0f;
  const uint32_t row = (uint32_t)(quad * 32 + lane);
#pragma unroll 1
  for (int c0 = 0; c0 < BN; c0 += 64) {
    if (n_tile0 + c0 >= e.n) break;                        // same decision in every thread
    uint32_t w[32];                                        // this row's 128 bytes
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      uint32_t r[32];
      __syncwarp();
      tmem_ld_x32(taddr + c0 + 32 * h, r);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; j += 2) {
        const int cj = c0 + 32 * h + j;
        const float v0 = dequant((int)r[j], col_i[cj], col_f0[cj], pt, col_f2[cj], col_f1[cj], e.flags);
        const float v1 = dequant((int)r[j + 1], col_i[cj + 1], col_f0[cj + 1], pt, col_f2[cj + 1], col_f1[cj + 1], e.flags);
        w[16 * h + j / 2] = to_bits16(v0, e.out_dtype) | (to_bits16(v1, e.out_dtype) << 16);
      }
    }
    const uint32_t buf = stage_base + (chunk % kTmaStoreBufs) * kTmaStoreBufBytes;
    named_barrier_sync(2, kEpiThreads);                    // the issuer has seen this buffer's last stores read it
#pragma unroll
    for (int c = 0; c < 8; ++c)
      st_shared_v4(buf + row * 128 + ((c ^ (row & 7)) << 4), make_uint4(w[4 * c], w[4 * c + 1], w[4 * c + 2], w[4 * c + 3]));
    fence_proxy_async_smem();
    named_barrier_sync(3, kEpiThreads);
    if (issuer) {
      if (cta_row0 < e.m)                                  // a box that starts beyond the last row is not issued at all
        for (int d = 0; d <= e.n_dest; ++d) tma_store_2d(&om.m[d], buf, (int)(n_tile0 + c0), (int)cta_row0);
      bulk_commit_group();
      bulk_wait_group_read<kTmaStoreBufs - 1>();           // the buffer of the next chunk is free again
    }
    ++chunk;
  }
}

// Per-channel parameters of the BN columns starting at n_tile0 -> shared memory, by the epilogue threads.
template <int BN>
__device__ __forceinline__ void stage_channel_params(const Epi& e, int64_t n_tile0, int et, float* col_f0, float* col_f1,
                                                     float* col_f2, int* col_i) {
  for (int i = et; i < BN; i += kEpiThreads) {
    const int64_t nn = n_tile0 + i;
    const bool v = nn < e.n;
    col_f0[i] = v ? load_scale(e, nn) : 0.0f;
    col_f1[i] = v ? load_offset(e, nn) : 0.0f;
    col_f2[i] = v ? load_float_bias(e, nn) : 0.0f;
    col_i[i] = v ? load_int_bias(e, nn) : 0;
  }
}

template <int BN, int STAGES, bool PUSH = false>
struct SmemLayout {
  static constexpr int kBTileBytes = BN * kBK;
  static constexpr int kStageBytes = kATileBytes + kBTileBytes;
  static constexpr int kTiles = STAGES * kStageBytes;
  static constexpr int kBarOff = kTiles;                       // full[S], empty[S], tfull[2], tempty[2]
  static constexpr int kMiscOff = kBarOff + (2 * STAGES + 4) * 8;   // tmem base, abort flag
  static constexpr int kColOff = kMiscOff + 16;                // 4 x BN 32-bit column parameters
  static constexpr int kPushOff = (kColOff + 4 * BN * 4 + 127) & ~127;   // staging per epilogue warp (multi-GPU epilogue)
  static constexpr int kTotal = kPushOff + (PUSH ? (kEpiThreads / 32) * kPushStageBytes : 0);
  static constexpr int kDynamic = kTotal + 1024;               // slack to align the tiles to 1024 B
};

// PUSH: the token-row epilogue of the multi-GPU forms (a separate instantiation, so that the single-GPU kernel
// carries neither its staging areas nor its registers).
template <int BN, int STAGES, bool SWAP, bool PUSH = false>
__global__ void __launch_bounds__(kThreads, 1)
w8a8_umma_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const Epi e,
                 const Sched s) {
  using L = SmemLayout<BN, STAGES, PUSH>;
  static_assert(!(SWAP && PUSH), "the swapped epilogue does not store to peers");
  constexpr int CH = BN < 32 ? 16 : 32;                 // accumulator columns per tcgen05.ld
  constexpr uint32_t kTmemCols = (2 * BN < 32) ? 32 : 2 * BN;
  static_assert(kTmemCols <= 512 && (kTmemCols & (kTmemCols - 1)) == 0, "TMEM columns: power of two <= 512");
  static_assert(kTmemCols <= 256 || L::kDynamic > 116 * 1024, "two resident CTAs must not both want >256 TMEM columns");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * kATileBytes;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* empty = full + STAGES;
  uint64_t* tfull = empty + STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(smem + L::kMiscOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kMiscOff + 4);
  float* col_f0 = reinterpret_cast<float*>(smem + L::kColOff);   // normal: scale[n]   swapped: pertoken[m]
  float* col_f1 = col_f0 + BN;                                     // normal: offset[n]
  float* col_f2 = col_f1 + BN;                                     // normal: float bias[n]
  int* col_i = reinterpret_cast<int*>(col_f2 + BN);                // normal: int bias[n]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull[i], 1);
      mbar_init(&tempty[i], kEpiThreads / 32);
    }
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tensormap(&tmA);
    prefetch_tensormap(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < s.units && ok; u += gridDim.x) {
        const int ta = u % s.tiles_a, rest = u / s.tiles_a;
        const int tb = rest % s.tiles_b, sp = rest / s.tiles_b;
        const int kb0 = sp * s.kb_per_split, kb1 = min(s.kblocks, kb0 + s.kb_per_split);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag, kDevTimeoutProducer)) { ok = false; break; }
          mbar_arrive_expect_tx(&full[stage], L::kStageBytes);
          tma_load_2d(sA + stage * kATileBytes, &tmA, &full[stage], kb * kBK, ta * kTileA);
          tma_load_2d(sB + stage * L::kBTileBytes, &tmB, &full[stage], kb * kBK, tb * BN);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        // Give copies that are still in flight time to land before shared memory is released.
        for (int i = 0; i < 200; ++i) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(2 /*s32*/, 1 /*s8*/, 1 /*s8*/, 0, 0, kTileA, BN);
      int stage = 0, buf = 0;
      uint32_t phase = 0, tphase = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < s.units && ok; u += gridDim.x) {
        const int sp = (u / s.tiles_a) / s.tiles_b;
        const int kb0 = sp * s.kb_per_split, kb1 = min(s.kblocks, kb0 + s.kb_per_split);
        if (!mbar_wait(&tempty[buf], tphase ^ 1, abort_flag, kDevTimeoutMma)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full[stage], phase, abort_flag, kDevTimeoutMma)) { ok = false; break; }
          tc_fence_after();
          const uint64_t adesc = make_smem_desc(smem_u32(sA + stage * kATileBytes), 16, 1024, kSwizzle128B);
          const uint64_t bdesc = make_smem_desc(smem_u32(sB + stage * L::kBTileBytes), 16, 1024, kSwizzle128B);
#pragma unroll
          for (int k4 = 0; k4 < kBK / 32; ++k4)   // +32 bytes along K inside the swizzle row = +2 in the address field
            umma_i8(d_tmem, adesc + 2 * k4, bdesc + 2 * k4, idesc, (kb > kb0 || k4 > 0) ? 1u : 0u);
          umma_commit(&empty[stage]);             // stage is free once these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&tfull[buf]);                 // accumulator complete
        if (++buf == 2) { buf = 0; tphase ^= 1; }
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int et = threadIdx.x - 64;                 // 0..127
    const int quad = warp & 3;                       // TMEM lane quadrant this warp may read
    const int row_in_tile = quad * 32 + lane;
    int buf = 0;
    uint32_t tphase = 0;
    bool ok = true;
    for (int u = blockIdx.x; u < s.units && ok; u += gridDim.x) {
      const int ta = u % s.tiles_a, tb = (u / s.tiles_a) % s.tiles_b;
      // Column parameters of this tile -> shared memory (read back as broadcasts).
      named_barrier_sync(1, kEpiThreads);
      if (SWAP) {
        for (int i = et; i < BN; i += kEpiThreads) {
          const int64_t mm = (int64_t)tb * BN + i;
          col_f0[i] = ((e.flags & kHasPt) && mm < e.m) ? __ldg(e.pertoken + mm) : 1.0f;
        }
      } else {
        stage_channel_params<BN>(e, (int64_t)tb * BN, et, col_f0, col_f1, col_f2, col_i);
      }
      named_barrier_sync(1, kEpiThreads);

      if (!epilogue_all(mbar_wait(&tfull[buf], tphase, abort_flag, kDevTimeoutEpilogue))) { ok = false; break; }
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + buf * BN;

      if (SWAP) {
        // D rows are channels (n), D columns are tokens (m): lanes write consecutive n.
        const int64_t n = (int64_t)ta * kTileA + row_in_tile;
        const bool nv = n < e.n;
        const float sc = nv ? load_scale(e, n) : 0.0f, off = nv ? load_offset(e, n) : 0.0f;
        const float fb = nv ? load_float_bias(e, n) : 0.0f;
        const int ib = nv ? load_int_bias(e, n) : 0;
#pragma unroll 1
        for (int c = 0; c < BN / CH; ++c) {
          uint32_t r[CH];
          __syncwarp();
          tmem_ld_chunk<CH>(taddr + c * CH, r);
          tmem_ld_wait();
          if (nv) {
#pragma unroll
            for (int j = 0; j < CH; ++j) {
              const int64_t mm = (int64_t)tb * BN + c * CH + j;
              if (mm < e.m) {
                const int acc = (int)r[j];
                if (e.acc_ws) {
                  atomicAdd(e.acc_ws + mm * e.n + n, acc);
                } else {
                  store_one(e, mm * e.ldo + n, acc, ib, dequant(acc, ib, sc, col_f0[c * CH + j], fb, off, e.flags));
                }
              }
            }
          }
        }
      } else {
        // D rows are tokens (m), D columns are channels (n).
        if constexpr (PUSH) {
          store_token_rows_push<BN>(e, taddr, (int64_t)ta * kTileA + quad * 32, lane, (int64_t)tb * BN, col_f0, col_f1,
                                    col_f2, col_i, smem_u32(smem + L::kPushOff) + (warp - 2) * kPushStageBytes);
        } else {
          store_token_rows<BN, CH>(e, taddr, (int64_t)ta * kTileA + row_in_tile, (int64_t)tb * BN, col_f0, col_f1, col_f2,
                                   col_i);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[buf]);
      if (++buf == 2) { buf = 0; tphase ^= 1; }
    }
  }

  // Teardown: every role arrives here whether it finished or aborted.
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---------------------------------------------------------------------------------------------
// Two-CTA variant for large M (cluster of two CTAs on neighbouring SMs, tcgen05 cta_group::2).
// The pair owns a 256 x 256 output tile: each CTA loads 128 token rows of A and 128 channel rows of B
// (its half of the B operand) per K block, so shared-memory fill and operand traffic per MMA drop by a
// third against the one-CTA tile; the leader CTA (rank 0) issues M=256, N=256 MMAs that read both
// halves and write 128 accumulator rows into each CTA's TMEM.  Both CTAs' TMA loads count on the
// leader's `full` barrier; the leader's tcgen05.commit arrives on both CTAs' `empty` / `tfull`
// barriers (one commit per CTA, no multicast); both epilogues arrive on the leader's `tempty`.
// EPI: 0 plain stores to `out`; 1 plain stores to `out` and the peers (any output type, routed form);
// 2 TMA stores to `out` and the peers (16-bit outputs, replicate form).
template <int STAGES, int EPI = 0>
struct PairLayout {
  static constexpr int kBN = 256;
  static constexpr int kBHalfBytes = 128 * kBK;
  static constexpr int kStageBytes = kATileBytes + kBHalfBytes;
  static constexpr int kTiles = STAGES * kStageBytes;
  static constexpr int kBarOff = kTiles;
  static constexpr int kMiscOff = kBarOff + (2 * STAGES + 4) * 8;
  static constexpr int kColOff = kMiscOff + 16;
  static constexpr int kPushOff = (kColOff + 4 * kBN * 4 + 1023) & ~1023;
  static constexpr int kTotal = kPushOff + (EPI == 1 ? (kEpiThreads / 32) * kPushStageBytes
                                            : EPI == 2 ? kTmaStoreBufs * kTmaStoreBufBytes : 0);
  static constexpr int kDynamic = kTotal + 1024;
};

template <int STAGES, int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
w8a8_umma_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const Epi e,
                      const Sched s, const __grid_constant__ std::conditional_t<EPI == 2, OutMaps, NoOutMaps> om) {
  using L = PairLayout<STAGES, EPI>;
  constexpr int BN = L::kBN, CH = 32;
  constexpr uint32_t kTmemCols = 512;
  static_assert(L::kDynamic > 116 * 1024 && L::kDynamic <= 227 * 1024, "one CTA per SM; shared memory budget");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * kATileBytes;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* empty = full + STAGES;
  uint64_t* tfull = empty + STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(smem + L::kMiscOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kMiscOff + 4);
  float* col_f0 = reinterpret_cast<float*>(smem + L::kColOff);
  float* col_f1 = col_f0 + BN;
  float* col_f2 = col_f1 + BN;
  int* col_i = reinterpret_cast<int*>(col_f2 + BN);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();                 // 0 = leader
  const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull[i], 1);
      mbar_init(&tempty[i], 2 * (kEpiThreads / 32));       // epilogue warps of both CTAs
    }
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tensormap(&tmA);
    prefetch_tensormap(&tmB);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_holder, kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                                      // the peer's barriers exist before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int u = pair; u < s.units && ok; u += npairs) {
        const int ta = u % s.tiles_a, tb = u / s.tiles_a;
        for (int kb = 0; kb < s.kblocks; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag, kDevTimeoutProducer)) { ok = false; break; }
          if (rank == 0) mbar_arrive_expect_tx(&full[stage], 2 * L::kStageBytes);   // bytes of both CTAs
          const uint32_t leader_full = map_to_cta(smem_u32(&full[stage]), 0);
          tma_load_2d_pair(sA + stage * kATileBytes, &tmA, leader_full, kb * kBK, ta * 256 + (int)rank * 128);
          tma_load_2d_pair(sB + stage * L::kBHalfBytes, &tmB, leader_full, kb * kBK, tb * 256 + (int)rank * 128);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok)
        for (int i = 0; i < 200; ++i) __nanosleep(1000);
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer (leader only)
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = make_idesc(2 /*s32*/, 1 /*s8*/, 1 /*s8*/, 0, 0, 256, BN);
      int stage = 0, buf = 0;
      uint32_t phase = 0, tphase = 0;
      bool ok = true;
      for (int u = pair; u < s.units && ok; u += npairs) {
        if (!mbar_wait(&tempty[buf], tphase ^ 1, abort_flag, kDevTimeoutMma)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = 0; kb < s.kblocks; ++kb) {
          if (!mbar_wait(&full[stage], phase, abort_flag, kDevTimeoutMma)) { ok = false; break; }
          tc_fence_after();
          const uint64_t adesc = make_smem_desc(smem_u32(sA + stage * kATileBytes), 16, 1024, kSwizzle128B);
          const uint64_t bdesc = make_smem_desc(smem_u32(sB + stage * L::kBHalfBytes), 16, 1024, kSwizzle128B);
#pragma unroll
          for (int k4 = 0; k4 < kBK / 32; ++k4)
            umma_i8_pair(d_tmem, adesc + 2 * k4, bdesc + 2 * k4, idesc, (kb > 0 || k4 > 0) ? 1u : 0u);
          umma_commit_pair(map_to_cta(smem_u32(&empty[stage]), 0));   // stage free in this CTA ...
          umma_commit_pair(map_to_cta(smem_u32(&empty[stage]), 1));   // ... and in the peer
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit_pair(map_to_cta(smem_u32(&tfull[buf]), 0));
        umma_commit_pair(map_to_cta(smem_u32(&tfull[buf]), 1));
        if (++buf == 2) { buf = 0; tphase ^= 1; }
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue (both CTAs, own 128 rows)
    const int et = threadIdx.x - 64;
    const int quad = warp & 3;
    const int row_in_tile = quad * 32 + lane;
    int buf = 0;
    uint32_t tphase = 0;
    uint32_t chunk = 0;
    if constexpr (EPI == 2) {
      if (et == 0)
        for (int d = 0; d <= e.n_dest; ++d) prefetch_tensormap(&om.m[d]);
    }
    for (int u = pair; u < s.units; u += npairs) {
      const int ta = u % s.tiles_a, tb = u / s.tiles_a;
      named_barrier_sync(1, kEpiThreads);
      stage_channel_params<BN>(e, (int64_t)tb * BN, et, col_f0, col_f1, col_f2, col_i);
      named_barrier_sync(1, kEpiThreads);
      if (!epilogue_all(mbar_wait(&tfull[buf], tphase, abort_flag, kDevTimeoutEpilogue))) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + buf * BN;
      if constexpr (EPI == 2) {
        store_token_rows_tma<BN>(e, om, taddr, (int64_t)ta * 256 + rank * 128, quad, lane, et == 0, (int64_t)tb * BN, col_f0,
                                 col_f1, col_f2, col_i, smem_u32(smem + L::kPushOff), chunk);
      } else if constexpr (EPI == 1) {
        store_token_rows_push<BN>(e, taddr, (int64_t)ta * 256 + rank * 128 + quad * 32, lane, (int64_t)tb * BN, col_f0,
                                  col_f1, col_f2, col_i, smem_u32(smem + L::kPushOff) + (warp - 2) * kPushStageBytes);
      } else {
        store_token_rows<BN, CH>(e, taddr, (int64_t)ta * 256 + rank * 128 + row_in_tile, (int64_t)tb * BN, col_f0, col_f1,
                                 col_f2, col_i);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tempty[buf]), 0));
      if (++buf == 2) { buf = 0; tphase ^= 1; }
    }
    if constexpr (EPI == 2) {
      if (et == 0) bulk_wait_group<0>();                   // every store of this CTA has been performed
    }
  }

  // Teardown: neither CTA may leave while the other can still signal its barriers or read its operands.
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

// ---------------------------------------------------------------------------------------------
// Decode shapes (M <= 128) in one launch: swapped operands as above (weight rows on the 128-row MMA axis,
// tokens padded to BN), and K split across the CTAs of a thread-block cluster instead of across
// independent CTAs.  Each CTA of a cluster accumulates its K range of the same 128-channel tile in its
// own TMEM and parks the int32 partial tile in its shared memory; then every CTA finishes its share of the
// token columns: it adds all CTAs' partial tiles for those columns through distributed shared memory
// (coalesced ld.shared::cluster, lanes = channels) and runs the dequantising epilogue, so reduction and
// epilogue are spread over the cluster.  No scratch in global memory, no atomics, no second kernel.
// Clusters are persistent and stride over the channel tiles.
template <int BN, int STAGES>
struct DecodeLayout {
  static constexpr int kBTileBytes = BN * kBK;
  static constexpr int kStageBytes = kATileBytes + kBTileBytes;
  static constexpr int kTiles = STAGES * kStageBytes;
  static constexpr int kRedOff = kTiles;                            // [BN][128] int32: this CTA's partial tile
  static constexpr int kBarOff = kRedOff + BN * 128 * 4;            // full[S], empty[S], tfull[2], tempty[2], red_ready, red_free
  static constexpr int kMiscOff = kBarOff + (2 * STAGES + 6) * 8;   // tmem base, abort flag
  static constexpr int kColOff = kMiscOff + 16;                     // pertoken[BN]
  static constexpr int kTotal = kColOff + BN * 4;
  static constexpr int kDynamic = kTotal + 1024;
};

template <int BN, int STAGES>
__global__ void __launch_bounds__(kThreads, 1)
w8a8_decode_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const Epi e,
                   const Sched s) {
  using L = DecodeLayout<BN, STAGES>;
  constexpr int CH = BN < 32 ? 16 : 32;
  constexpr uint32_t kTmemCols = (2 * BN < 32) ? 32 : 2 * BN;
  static_assert(L::kDynamic > 116 * 1024 && L::kDynamic <= 227 * 1024, "one CTA per SM; shared memory budget");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * kATileBytes;
  int32_t* red = reinterpret_cast<int32_t*>(smem + L::kRedOff);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* empty = full + STAGES;
  uint64_t* tfull = empty + STAGES;
  uint64_t* tempty = tfull + 2;
  uint64_t* red_ready = tempty + 2;     // every CTA of the cluster has parked its partial tile
  uint64_t* red_free = red_ready + 1;   // every CTA of the cluster has finished reading this CTA's partial tile
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(smem + L::kMiscOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kMiscOff + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t crank = cluster_ctarank(), csize = cluster_nctarank();
  const int cluster = (int)cluster_id_x(), nclusters = (int)nclusters_x();
  // This CTA's K range (the same for every tile).
  const int kb0 = (int)crank * s.kb_per_split, kb1 = min(s.kblocks, kb0 + s.kb_per_split);

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull[i], 1);
      mbar_init(&tempty[i], kEpiThreads / 32);
    }
    mbar_init(red_ready, csize);       // one arrival per CTA of the cluster, this one included
    mbar_init(red_free, csize);
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tensormap(&tmA);
    prefetch_tensormap(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  if (csize > 1) cluster_sync_all();     // the peers' barriers exist before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      const uint64_t pol_w = policy_evict_first();      // weights are streamed once
      for (int u = cluster; u < s.units && ok; u += nclusters) {
        const int ta = u % s.tiles_a, tb = u / s.tiles_a;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag, kDevTimeoutProducer)) { ok = false; break; }
          mbar_arrive_expect_tx(&full[stage], L::kStageBytes);
          tma_load_2d_hint(sA + stage * kATileBytes, &tmA, &full[stage], kb * kBK, ta * kTileA, pol_w);
          tma_load_2d(sB + stage * L::kBTileBytes, &tmB, &full[stage], kb * kBK, tb * BN);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok)
        for (int i = 0; i < 200; ++i) __nanosleep(1000);
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(2 /*s32*/, 1 /*s8*/, 1 /*s8*/, 0, 0, kTileA, BN);
      int stage = 0, buf = 0;
      uint32_t phase = 0, tphase = 0;
      bool ok = true;
      for (int u = cluster; u < s.units && ok; u += nclusters) {
        if (!mbar_wait(&tempty[buf], tphase ^ 1, abort_flag, kDevTimeoutMma)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full[stage], phase, abort_flag, kDevTimeoutMma)) { ok = false; break; }
          tc_fence_after();
          const uint64_t adesc = make_smem_desc(smem_u32(sA + stage * kATileBytes), 16, 1024, kSwizzle128B);
          const uint64_t bdesc = make_smem_desc(smem_u32(sB + stage * L::kBTileBytes), 16, 1024, kSwizzle128B);
#pragma unroll
          for (int k4 = 0; k4 < kBK / 32; ++k4)
            umma_i8(d_tmem, adesc + 2 * k4, bdesc + 2 * k4, idesc, (kb > kb0 || k4 > 0) ? 1u : 0u);
          umma_commit(&empty[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&tfull[buf]);
        if (++buf == 2) { buf = 0; tphase ^= 1; }
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue / cluster reduction
    const int et = threadIdx.x - 64;
    const int quad = warp & 3;
    const int row_in_tile = quad * 32 + lane;          // channel row of the tile owned by this thread
    int buf = 0;
    uint32_t tphase = 0, rphase = 0;
    for (int u = cluster; u < s.units; u += nclusters) {
      const int ta = u % s.tiles_a, tb = u / s.tiles_a;
      const int64_t n = (int64_t)ta * kTileA + row_in_tile;
      const bool nv = n < e.n;
      const float sc = nv ? load_scale(e, n) : 0.0f, off = nv ? load_offset(e, n) : 0.0f;
      const float fb = nv ? load_float_bias(e, n) : 0.0f;
      const int ib = nv ? load_int_bias(e, n) : 0;
      if (!epilogue_all(mbar_wait(&tfull[buf], tphase, abort_flag, kDevTimeoutEpilogue))) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + buf * BN;
      if (csize == 1) {
        // No split: accumulator -> epilogue.
#pragma unroll 1
        for (int c = 0; c < BN / CH; ++c) {
          uint32_t r[CH];
          __syncwarp();
          tmem_ld_chunk<CH>(taddr + c * CH, r);
          tmem_ld_wait();
          if (nv) {
#pragma unroll
            for (int j = 0; j < CH; ++j) {
              const int64_t mm = (int64_t)tb * BN + c * CH + j;
              if (mm < e.m) {
                const int acc = (int)r[j];
                const float pt = (e.flags & kHasPt) ? __ldg(e.pertoken + mm) : 1.0f;
                store_one(e, mm * e.ldo + n, acc, ib, dequant(acc, ib, sc, pt, fb, off, e.flags));
              }
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty[buf]);
      } else {
        // Every CTA parks its partial tile (red[col][row], lanes write consecutive words) once all CTAs have
        // finished with the previous one, frees its accumulator, and tells every CTA of the cluster.
        if (!epilogue_all(mbar_wait_cluster(red_free, rphase ^ 1, abort_flag, kDevTimeoutEpilogue))) break;
#pragma unroll 1
        for (int c = 0; c < BN / CH; ++c) {
          uint32_t r[CH];
          __syncwarp();
          tmem_ld_chunk<CH>(taddr + c * CH, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < CH; ++j) red[(c * CH + j) * 128 + row_in_tile] = (int32_t)r[j];
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty[buf]);
        fence_acq_rel_cluster();
        named_barrier_sync(1, kEpiThreads);
        if (et < (int)csize) mbar_arrive_cluster(map_to_cta(smem_u32(red_ready), (uint32_t)et));
        if (!epilogue_all(mbar_wait_cluster(red_ready, rphase, abort_flag, kDevTimeoutEpilogue))) break;
        // This CTA finishes the token columns [crank * per, (crank + 1) * per): the sum over all CTAs' partial
        // tiles through distributed shared memory (coalesced: lanes = channels), then the epilogue.
        const int per = BN / (int)csize;
        const uint32_t red_addr = smem_u32(red) + row_in_tile * 4;
#pragma unroll 1
        for (int j0 = 0; j0 < per; j0 += 8) {
          uint32_t v[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) v[j] = 0;
          for (uint32_t p = 0; p < csize; ++p) {
            const uint32_t base = map_to_cta(red_addr + (uint32_t)((int)crank * per + j0) * 512u, p);
#pragma unroll
            for (int j = 0; j < 8; ++j)
              if (j0 + j < per) v[j] += ld_shared_cluster_u32(base + j * 512);
          }
          if (nv) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const int64_t mm = (int64_t)tb * BN + (int)crank * per + j0 + j;
              if (j0 + j < per && mm < e.m) {
                const int acc = (int)v[j];
                const float pt = (e.flags & kHasPt) ? __ldg(e.pertoken + mm) : 1.0f;
                store_one(e, mm * e.ldo + n, acc, ib, dequant(acc, ib, sc, pt, fb, off, e.flags));
              }
            }
          }
        }
        named_barrier_sync(1, kEpiThreads);             // every thread of this CTA has finished reading
        if (et < (int)csize) mbar_arrive_cluster(map_to_cta(smem_u32(red_free), (uint32_t)et));
        rphase ^= 1;
      }
      if (++buf == 2) { buf = 0; tphase ^= 1; }
    }
  }

  // Teardown: no CTA leaves while a peer may still read its partial tile or signal its barriers.
  tc_fence_before();
  __syncthreads();
  if (csize > 1) cluster_sync_all();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// Applies the epilogue to split-K accumulators: one thread per output element.
__global__ void splitk_finalize_kernel(const int32_t* __restrict__ acc, const Epi e) {
  const int64_t total = e.m * e.n;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t mm = i / e.n, n = i - mm * e.n;
    const int a = acc[i], ib = load_int_bias(e, n);
    const float pt = (e.flags & kHasPt) ? __ldg(e.pertoken + mm) : 1.0f;
    store_one(e, mm * e.ldo + n, a, ib, dequant(a, ib, load_scale(e, n), pt, load_float_bias(e, n), load_offset(e, n), e.flags));
  }
}

// Any shape, any strides: one thread per output element.  Used for operands that do not meet
// the TMA alignment rules (K not a multiple of 16, odd pointers) and for K == 0.
__global__ void w8a8_simt_kernel(const int8_t* __restrict__ x1, const int8_t* __restrict__ x2, int64_t k,
                                 int64_t sk, int64_t sn, const Epi e) {
  const int64_t n = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  const int64_t mm = blockIdx.y * (int64_t)blockDim.y + threadIdx.y;
  if (n >= e.n || mm >= e.m) return;
  int acc = 0;
  const int8_t* a = x1 + mm * k;
  const int8_t* b = x2 + n * sn;
  for (int64_t i = 0; i < k; ++i) acc += (int)a[i] * (int)b[i * sk];
  const int ib = load_int_bias(e, n);
  const float pt = (e.flags & kHasPt) ? __ldg(e.pertoken + mm) : 1.0f;
  store_one(e, mm * e.ldo + n, acc, ib,
            dequant(acc, ib, load_scale(e, n), pt, load_float_bias(e, n), load_offset(e, n), e.flags));
}

// One or two tokens (the kernel itself takes up to four): no tensor cores, no pipeline to fill.  A warp streams the K-major weight rows of MT
// consecutive output channels with 128-bit loads (L1 bypassed, eight loads in flight per lane) against the
// tokens held in shared memory; a token chunk read from shared memory is used for all MT channels, so the
// shared-memory traffic per weight byte does not grow with the token count.  Four dp4a per 16 bytes, token
// and channel, a shuffle reduction, and the lanes 0..MT-1 run the same dequantising epilogue.  The call is
// one launch whose fixed cost is a plain kernel's, which is what matters when the whole weight streams in a
// few microseconds.
template <int MT>
__global__ void __launch_bounds__(256) w8a8_gemv_kernel(const int8_t* __restrict__ x1, const int8_t* __restrict__ w,
                                                        int64_t k, int64_t w_pitch, const Epi e) {
  constexpr int R = MT;                                        // channels per warp and trip
  constexpr int U = 8 / R;                                     // chunks in flight per channel
  extern __shared__ __align__(16) uint8_t gemv_x[];           // [MT][k]
  const int chunks = (int)(k >> 4);                            // 16-byte chunks per row
  for (int i = threadIdx.x; i < MT * chunks; i += blockDim.x) {
    const int t = i / chunks, c = i - t * chunks;
    reinterpret_cast<uint4*>(gemv_x)[i] =
        t < e.m ? __ldg(reinterpret_cast<const uint4*>(x1 + (int64_t)t * k) + c) : make_uint4(0, 0, 0, 0);
  }
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int64_t nwarps = (int64_t)gridDim.x * (blockDim.x >> 5);
  for (int64_t n0 = warp * R; n0 < e.n; n0 += nwarps * R) {
    int acc[R][MT];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int t = 0; t < MT; ++t) acc[r][t] = 0;
    for (int c0 = lane; c0 < chunks; c0 += 32 * U) {
      uint4 v[R][U];
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const int64_t n = n0 + r < e.n ? n0 + r : e.n - 1;    // past the end: re-read the last row, result unused
        const uint4* wr = reinterpret_cast<const uint4*>(w + n * w_pitch);
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int c = c0 + 32 * u;
          v[r][u] = make_uint4(0, 0, 0, 0);
          if (c < chunks)
            asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                         : "=r"(v[r][u].x), "=r"(v[r][u].y), "=r"(v[r][u].z), "=r"(v[r][u].w) : "l"(wr + c));
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int c = c0 + 32 * u;
        if (c < chunks) {
#pragma unroll
          for (int t = 0; t < MT; ++t) {
            const uint4 xv = reinterpret_cast<const uint4*>(gemv_x)[t * chunks + c];
#pragma unroll
            for (int r = 0; r < R; ++r) {
              acc[r][t] = __dp4a((int)v[r][u].x, (int)xv.x, acc[r][t]);
              acc[r][t] = __dp4a((int)v[r][u].y, (int)xv.y, acc[r][t]);
              acc[r][t] = __dp4a((int)v[r][u].z, (int)xv.z, acc[r][t]);
              acc[r][t] = __dp4a((int)v[r][u].w, (int)xv.w, acc[r][t]);
            }
          }
        }
      }
    }
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int t = 0; t < MT; ++t) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc[r][t] += __shfl_xor_sync(0xffffffffu, acc[r][t], o);
      }
    // lane r finishes channel n0 + r
#pragma unroll
    for (int r = 0; r < R; ++r) {
      if (lane == r && n0 + r < e.n) {
        const int64_t n = n0 + r;
        const float sc = load_scale(e, n), off = load_offset(e, n), fb = load_float_bias(e, n);
        const int ib = load_int_bias(e, n);
#pragma unroll
        for (int t = 0; t < MT; ++t) {
          if (t < e.m) {
            const float pt = (e.flags & kHasPt) ? __ldg(e.pertoken + t) : 1.0f;
            store_one(e, (int64_t)t * e.ldo + n, acc[r][t], ib, dequant(acc[r][t], ib, sc, pt, fb, off, e.flags));
          }
        }
      }
    }
  }
}

// Three to sixteen tokens: still bound by the weight stream and too short to fill a tcgen05 pipeline, so the
// warp-level int8 MMA does the arithmetic (mma.sync m16n8k32: 16 channels x 8 tokens x 32 k per instruction).
// A CTA of eight warps owns 16 output channels; warp w takes the 64-byte K blocks w, w+8, w+16, ... of those
// 16 weight rows (so the eight warps together read 512 contiguous bytes of every row), eight or sixteen 128-bit
// weight loads in flight per lane (the deeper variant, which costs a resident CTA per SM, where there are
// few CTAs per SM anyway), the tokens' bytes through L1 (the whole activation is a few tens of KB).  Lane
// (g, q) loads 16 consecutive k of weight rows g and g+8 and of token g: those 16 bytes feed two MMAs whose k
// slots are a fixed permutation of the 64-wide block, the same permutation for both operands, so no shuffling
// is needed.  The eight warps' partial sums meet in shared memory and each thread finishes one output element
// with the common epilogue.  One launch, no scratch.
__device__ __forceinline__ void mma_s8_16x8x32(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int NG, int U>   // NG groups of eight tokens: 1 (m <= 8) or 2 (m <= 16); 2 * U weight loads in flight per lane
__global__ void __launch_bounds__(256) w8a8_small_m_kernel(const int8_t* __restrict__ x1, const int8_t* __restrict__ w,
                                                           int64_t k, int64_t w_pitch, const Epi e) {
  __shared__ int red[8][NG * 4][32];
  const int lane = threadIdx.x & 31, wi = threadIdx.x >> 5;
  const int g = lane >> 2, q = lane & 3;
  const int64_t n0 = (int64_t)blockIdx.x * 16;
  const int64_t r0 = n0 + g < e.n ? n0 + g : e.n - 1, r1 = n0 + g + 8 < e.n ? n0 + g + 8 : e.n - 1;   // clamped: unused results
  const int8_t* w0p = w + r0 * w_pitch + q * 16;
  const int8_t* w1p = w + r1 * w_pitch + q * 16;
  const int8_t* xp[NG];
  bool xv[NG];
#pragma unroll
  for (int t = 0; t < NG; ++t) {
    xv[t] = t * 8 + g < e.m;
    xp[t] = x1 + (int64_t)(xv[t] ? t * 8 + g : 0) * k + q * 16;
  }
  int acc[NG][4];
#pragma unroll
  for (int t = 0; t < NG; ++t)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[t][i] = 0;
  const int steps = (int)((k + 63) >> 6);
  for (int s0 = wi; s0 < steps; s0 += 8 * U) {
    uint4 a[U], b[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t kp = (int64_t)(s0 + 8 * u) * 64;
      a[u] = b[u] = make_uint4(0, 0, 0, 0);
      if (kp + q * 16 < k) {
        asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                     : "=r"(a[u].x), "=r"(a[u].y), "=r"(a[u].z), "=r"(a[u].w) : "l"(w0p + kp));
        asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                     : "=r"(b[u].x), "=r"(b[u].y), "=r"(b[u].z), "=r"(b[u].w) : "l"(w1p + kp));
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t kp = (int64_t)(s0 + 8 * u) * 64;
      if (kp < k) {                                       // same decision in every lane: the MMA is warp-wide
#pragma unroll
        for (int t = 0; t < NG; ++t) {
          uint4 xr = make_uint4(0, 0, 0, 0);
          if (xv[t] && kp + q * 16 < k) xr = __ldg(reinterpret_cast<const uint4*>(xp[t] + kp));
          mma_s8_16x8x32(acc[t], a[u].x, b[u].x, a[u].y, b[u].y, xr.x, xr.y);
          mma_s8_16x8x32(acc[t], a[u].z, b[u].z, a[u].w, b[u].w, xr.z, xr.w);
        }
      }
    }
  }
#pragma unroll
  for (int t = 0; t < NG; ++t)
#pragma unroll
    for (int i = 0; i < 4; ++i) red[wi][t * 4 + i][lane] = acc[t][i];
  __syncthreads();
  // Thread (reg, lane) finishes one output: accumulator register reg = 4 * token group + i of lane (g, q) is
  // channel n0 + g + 8 * (i >> 1), token 8 * group + 2 * q + (i & 1).
  for (int idx = threadIdx.x; idx < NG * 4 * 32; idx += blockDim.x) {
    const int reg = idx >> 5, ln = idx & 31;
    int sum = 0;
#pragma unroll
    for (int v = 0; v < 8; ++v) sum += red[v][reg][ln];
    const int i = reg & 3, t = reg >> 2;
    const int64_t n = n0 + (ln >> 2) + 8 * (i >> 1);
    const int64_t mm = t * 8 + 2 * (ln & 3) + (i & 1);
    if (n < e.n && mm < e.m) {
      const int ib = load_int_bias(e, n);
      const float pt = (e.flags & kHasPt) ? __ldg(e.pertoken + mm) : 1.0f;
      store_one(e, mm * e.ldo + n, sum, ib,
                dequant(sum, ib, load_scale(e, n), pt, load_float_bias(e, n), load_offset(e, n), e.flags));
    }
  }
}

// int8 [k,n] row-major -> [n,k] row-major through a 64x64 shared tile (k, n multiples of 16).
__global__ void __launch_bounds__(256) transpose_i8_kernel(const int8_t* __restrict__ src, int8_t* __restrict__ dst,
                                                          int64_t k, int64_t n) {
  __shared__ __align__(16) uint8_t tile[64][80];
  const int64_t k0 = (int64_t)blockIdx.y * 64, n0 = (int64_t)blockIdx.x * 64;
  const int r = threadIdx.x >> 2, seg = threadIdx.x & 3;
  uint4 v = make_uint4(0, 0, 0, 0);
  if (k0 + r < k && n0 + seg * 16 < n) v = *reinterpret_cast<const uint4*>(src + (k0 + r) * n + n0 + seg * 16);
  *reinterpret_cast<uint4*>(&tile[r][seg * 16]) = v;
  __syncthreads();
  if (n0 + r < n && k0 + seg * 16 < k) {
    uint32_t w[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      uint32_t x = 0;
#pragma unroll
      for (int b = 0; b < 4; ++b) x |= (uint32_t)tile[seg * 16 + q * 4 + b][r] << (8 * b);
      w[q] = x;
    }
    *reinterpret_cast<uint4*>(dst + (n0 + r) * k + k0 + seg * 16) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

template <int BN, int STAGES, bool SWAP, bool PUSH = false>
int launch_umma(const CUtensorMap& tmA, const CUtensorMap& tmB, const Epi& e, const Sched& s, cudaStream_t st) {
  using L = SmemLayout<BN, STAGES, PUSH>;
  static_assert(L::kDynamic <= 227 * 1024, "shared memory budget");
  constexpr auto kern = w8a8_umma_kernel<BN, STAGES, SWAP, PUSH>;
  if (int rc = ensure_dynamic_smem<kern>(L::kDynamic, "quant_matmul")) return rc;
  const int grid = s.units < sm_count() ? s.units : sm_count();
  kern<<<grid, kThreads, L::kDynamic, st>>>(tmA, tmB, e, s);
  return check_launch("quant_matmul (tcgen05)");
}

// Number of clusters of `csize` CTAs of `kern` that can be resident at once (cached per device and size).
template <auto Kern>
int resident_clusters(int csize, int dynamic_smem) {
  static std::mutex mu;
  static int cached[64][9] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64 || csize < 1 || csize > 8) return sm_count() / (csize > 0 ? csize : 1);
  std::lock_guard<std::mutex> lock(mu);
  if (cached[dev][csize] == 0) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(csize * (sm_count() / csize));
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = dynamic_smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = csize;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, Kern, &cfg) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      n = sm_count() / csize;
    }
    cached[dev][csize] = n < sm_count() / csize ? n : sm_count() / csize;
  }
  return cached[dev][csize];
}

template <int STAGES, int EPI>
int launch_umma_pair(const CUtensorMap& tmA, const CUtensorMap& tmB, const Epi& e, const Sched& s, cudaStream_t st,
                     const OutMaps* om = nullptr) {
  using L = PairLayout<STAGES, EPI>;
  constexpr auto kern = w8a8_umma_pair_kernel<STAGES, EPI>;
  if (int rc = ensure_dynamic_smem<kern>(L::kDynamic, "quant_matmul")) return rc;
  // Pairs that can be resident at once (cluster scheduling may leave an SM of a GPC unused).
  int pairs = resident_clusters<kern>(2, L::kDynamic);
  if (s.units < pairs) pairs = s.units;
  // cluster dims (2,1,1) are a kernel attribute
  if constexpr (EPI == 2) kern<<<2 * pairs, kThreads, L::kDynamic, st>>>(tmA, tmB, e, s, *om);
  else kern<<<2 * pairs, kThreads, L::kDynamic, st>>>(tmA, tmB, e, s, NoOutMaps{});
  return check_launch("quant_matmul (tcgen05, CTA pairs)");
}

template <int BN, int STAGES>
int launch_decode(const CUtensorMap& tmA, const CUtensorMap& tmB, const Epi& e, const Sched& s, int csize, cudaStream_t st) {
  using L = DecodeLayout<BN, STAGES>;
  constexpr auto kern = w8a8_decode_kernel<BN, STAGES>;
  if (int rc = ensure_dynamic_smem<kern>(L::kDynamic, "quant_matmul")) return rc;
  int clusters = resident_clusters<kern>(csize, L::kDynamic);
  if (s.units < clusters) clusters = s.units;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(csize * clusters);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = L::kDynamic;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = csize;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t err = cudaLaunchKernelEx(&cfg, kern, tmA, tmB, e, s);
  if (err != cudaSuccess) return fail(B200Q_ERR_LAUNCH, "quant_matmul (tcgen05, cluster split-K): %s", cudaGetErrorString(err));
  return check_launch("quant_matmul (tcgen05, cluster split-K)");
}

size_t align256(size_t v) { return (v + 255) & ~size_t(255); }

// Layout decision shared by the workspace query and the launch.
struct Plan {
  bool tensor_path;     // tcgen05 path usable
  bool transpose;       // contiguous [k,n] weight must be re-laid out as [n,k] first
  bool swap;            // M <= 128: weight rows on the MMA's 128-row axis
  bool decode;          // swapped, K split across the CTAs of a cluster (one launch, no scratch)
  bool gemv;            // one or two tokens: a warp per channel, dp4a, no tensor cores (one launch, no scratch)
  bool small_m;         // 3..16 tokens: warp-level int8 MMA on a streamed weight (one launch, no scratch)
  bool pair;            // CTA-pair kernel (256 x 256 tiles)
  int bn;               // B-operand tile rows
  int splits;           // swapped without clusters: K split across independent CTAs (int32 scratch + atomics)
  int csize;            // decode: CTAs per cluster = K splits
  size_t ws_transpose, ws_acc;
};

// `multi_gpu`: the epilogue also stores to peers (or routes rows); only the token-row epilogue can.
Plan make_plan(int64_t m, int64_t k, int64_t n, int64_t sk, int64_t sn, const void* x1, const void* x2,
               bool multi_gpu = false) {
  Plan p{};
  const bool kmajor = (sk == 1 || k == 1) && (sn >= k) && (sn % 16 == 0);
  const bool nmajor = (sn == 1 || n == 1) && (sk == n) && (n % 16 == 0);
  p.tensor_path = k >= 16 && k % 16 == 0 && (kmajor || nmajor) && m > 0 && n > 0 &&
                  (x1 == nullptr || aligned(x1, 16)) && (x2 == nullptr || aligned(x2, 16)) &&
                  k <= (1LL << 31) && m < (1LL << 31) && n < (1LL << 31);
  if (!p.tensor_path) return p;
  p.transpose = !kmajor;
  p.ws_transpose = p.transpose ? align256((size_t)n * k) : 0;
  p.swap = m <= 128 && !multi_gpu;
  p.splits = 1;
  p.csize = 1;
  const int sms = sm_count();
  if (p.swap && m <= 2 && k * 2 <= 200 * 1024) {
    const char* env = getenv("B200Q_W8A8_GEMV");
    p.gemv = env ? (env[0] != '0') : true;
  }
  if (p.gemv) return p;
  if (p.swap && m <= 16) {
    const char* env = getenv("B200Q_W8A8_SMALL_M");
    p.small_m = env ? (env[0] != '0') : true;
  }
  if (p.small_m) return p;
  if (p.swap) {
    p.bn = m <= 16 ? 16 : m <= 32 ? 32 : m <= 64 ? 64 : 128;
    const int64_t tiles = ceil_div(n, kTileA), kblocks = ceil_div(k, kBK);
    // Cluster split-K: rounds of resident clusters times the K blocks each CTA streams, plus a tail that
    // grows with the number of partial tiles the leader has to add.
    double best = 1e300;
    for (int c = 1; c <= 8 && c <= kblocks; c *= 2) {
      const int64_t per = ceil_div(kblocks, c);
      if (ceil_div(kblocks, per) != c) continue;          // every CTA of the cluster must own at least one K block
      const int64_t clusters = sms / c;
      const double cost = (double)ceil_div(tiles, clusters) * (double)per + 0.5 * c;
      if (cost < best) { best = cost; p.csize = c; }
    }
    // Measured: the cluster kernel wins where one round of resident clusters covers all channel tiles (the
    // synchronisation across the cluster at the end of every tile is not hidden when a cluster runs several).
    p.decode = tiles <= sms / p.csize && tiles * p.csize * 2 >= sms;
    const char* env = getenv("B200Q_W8A8_DECODE");
    if (env) p.decode = env[0] != '0';
    if (!p.decode) {
      // Few channel tiles and a long K: split K over independent CTAs so that all SMs stream weights;
      // cost = (weight bytes + atomic traffic) / SM utilisation.
      p.csize = 1;
      double bestc = 1e300;
      for (int sp = 1; sp <= 32 && sp <= kblocks; ++sp) {
        const int64_t per = ceil_div(kblocks, sp), eff_sp = ceil_div(kblocks, per);
        if (eff_sp != sp) continue;
        const int64_t units = tiles * sp;
        const double util = (double)units / (double)(ceil_div(units, sms) * sms);
        const double bytes = (double)k * n + (sp > 1 ? (double)sp * m * n * 8.0 : 0.0);
        const double cost = bytes / util;
        if (cost < bestc * 0.98) { bestc = cost; p.splits = sp; }
      }
      p.ws_acc = p.splits > 1 ? align256((size_t)m * n * 4) : 0;
    }
  } else {
    p.bn = n <= 128 ? 128 : 256;
    // CTA pairs (256 x 256 tiles, one per two SMs) against single CTAs (128 x BN tiles): both give an SM
    // the same work per tile, the pair streams a third less into shared memory and runs about a tenth
    // faster, so it wins whenever it does not need more rounds.  (A stream-K schedule for tile counts that
    // do not fill the last round - equal K-block ranges per pair, int32 partial tiles through scratch - was
    // built and measured 25-65 % SLOWER on every such shape: the pairs then sit at different K offsets, and
    // the kernel depends on concurrently running pairs fetching the same operand tiles at the same time.)
    const char* env = getenv("B200Q_W8A8_PAIR");
    const bool allow = env ? (env[0] != '0') : true;
    const int64_t t_pair = ceil_div(m, 256) * ceil_div(n, 256), t_one = ceil_div(m, kTileA) * ceil_div(n, p.bn);
    const double cost_pair = (double)ceil_div(t_pair, sms / 2), cost_one = 1.1 * (double)ceil_div(t_one, sms);
    p.pair = allow && m > 128 && n >= 256 && cost_pair <= cost_one;
  }
  return p;
}

}  // namespace
}  // namespace b200q

extern "C" size_t b200q_quant_matmul_workspace_bytes(int64_t m, int64_t k, int64_t n, int64_t x2_stride_k,
                                                     int64_t x2_stride_n) {
  using namespace b200q;
  if (m <= 0 || k <= 0 || n <= 0) return 0;
  Plan p = make_plan(m, k, n, x2_stride_k, x2_stride_n, nullptr, nullptr);
  return p.tensor_path ? p.ws_transpose + p.ws_acc : 0;
}

extern "C" int b200q_quant_matmul(const b200q_quant_matmul_args* a, void* stream) {
  using namespace b200q;
  clear_error();
  B200Q_REQUIRE(a != nullptr, B200Q_ERR_BAD_ARG, "quant_matmul: args is NULL");
  B200Q_REQUIRE(a->m >= 0 && a->k >= 0 && a->n >= 0, B200Q_ERR_BAD_ARG, "quant_matmul: negative size");
  if (a->m == 0 || a->n == 0) return B200Q_OK;
  const bool routed = a->route_rows > 0;
  const bool multi_gpu = routed || a->n_peer_out > 0;
  B200Q_REQUIRE((a->out != nullptr || routed) && a->scale != nullptr, B200Q_ERR_BAD_ARG, "quant_matmul: out or scale is NULL");
  B200Q_REQUIRE(a->k == 0 || (a->x1 != nullptr && a->x2 != nullptr), B200Q_ERR_BAD_ARG, "quant_matmul: x1 or x2 is NULL");
  B200Q_REQUIRE(a->out_dtype == B200Q_I8 || a->out_dtype == B200Q_F16 || a->out_dtype == B200Q_BF16 ||
                    a->out_dtype == B200Q_I32 || a->out_dtype == B200Q_F32,
                B200Q_ERR_UNSUPPORTED, "quant_matmul: output dtype enum %d is not int8/f16/bf16/int32/f32", a->out_dtype);
  B200Q_REQUIRE(a->scale_dtype == B200Q_F32 || a->scale_dtype == B200Q_BF16 || a->scale_dtype == B200Q_I64,
                B200Q_ERR_UNSUPPORTED, "quant_matmul: scale must be f32, bf16 or i64 (dtype enum %d)", a->scale_dtype);
  B200Q_REQUIRE(a->scale_len == 1 || a->scale_len == a->n, B200Q_ERR_BAD_ARG,
                "quant_matmul: scale has %lld elements, expected 1 or n=%lld", (long long)a->scale_len, (long long)a->n);
  B200Q_REQUIRE(a->offset == nullptr || a->offset_len == 1 || a->offset_len == a->n, B200Q_ERR_BAD_ARG,
                "quant_matmul: offset has %lld elements, expected 1 or n=%lld", (long long)a->offset_len, (long long)a->n);
  B200Q_REQUIRE(a->bias == nullptr || a->bias_dtype == B200Q_I32 || a->bias_dtype == B200Q_BF16 ||
                    a->bias_dtype == B200Q_F16 || a->bias_dtype == B200Q_F32,
                B200Q_ERR_UNSUPPORTED, "quant_matmul: bias must be i32, bf16, f16 or f32");
  B200Q_REQUIRE(a->out_row_stride == 0 || a->out_row_stride >= a->n, B200Q_ERR_BAD_ARG,
                "quant_matmul: out_row_stride (%lld) is smaller than n (%lld)", (long long)a->out_row_stride, (long long)a->n);
  B200Q_REQUIRE(!(a->out_dtype == B200Q_I32 && a->bias != nullptr && a->bias_dtype != B200Q_I32), B200Q_ERR_UNSUPPORTED,
                "quant_matmul: int32 output takes an int32 bias only");

  cudaStream_t st = static_cast<cudaStream_t>(stream);
  Epi e{};
  e.scale = a->scale; e.offset = a->offset; e.pertoken = a->pertoken_scale; e.bias = a->bias; e.out = a->out;
  e.acc_ws = nullptr; e.m = a->m; e.n = a->n;
  e.ldo = a->out_row_stride > 0 ? a->out_row_stride : a->n;
  e.scale_dtype = a->scale_dtype; e.scale_bcast = a->scale_len == 1; e.offset_bcast = a->offset_len == 1;
  e.bias_dtype = a->bias ? a->bias_dtype : B200Q_NONE; e.out_dtype = a->out_dtype;
  e.flags = (a->pertoken_scale ? kHasPt : 0u) | (a->offset ? kHasOff : 0u) |
            (a->bias ? (a->bias_dtype == B200Q_I32 ? kHasIntBias : kHasFloatBias) : 0u);
  const int64_t ob = a->out_dtype == B200Q_I8 ? 1 : (a->out_dtype == B200Q_I32 || a->out_dtype == B200Q_F32) ? 4 : 2;
  if ((a->out == nullptr || aligned(a->out, 16)) && (e.ldo * ob) % 16 == 0) e.flags |= kOutVec;

  Plan p = make_plan(a->m, a->k, a->n, a->x2_stride_k, a->x2_stride_n, a->x1, a->x2, multi_gpu);
  if (multi_gpu) {
    // Peer destinations are written by the token-row epilogue of the tcgen05 kernels, 128 bytes of a row at a time.
    const int n_dest = routed ? (int)ceil_div(a->m, a->route_rows) : a->n_peer_out;
    B200Q_REQUIRE(a->peer_out != nullptr && n_dest >= 1 && n_dest <= kMaxDest, B200Q_ERR_BAD_ARG,
                  "quant_matmul: %d peer destinations (1..%d allowed, with a non-NULL table)", n_dest, kMaxDest);
    B200Q_REQUIRE(p.tensor_path, B200Q_ERR_UNSUPPORTED,
                  "quant_matmul: peer destinations need operands that meet the TMA rules (k %% 16 == 0, 16-byte aligned)");
    B200Q_REQUIRE(ob != 1 && (a->n * ob) % 128 == 0 && (e.flags & kOutVec), B200Q_ERR_UNSUPPORTED,
                  "quant_matmul: peer destinations need a 16- or 32-bit output type, n*size a multiple of 128 bytes "
                  "and 16-byte aligned rows");
    for (int i = 0; i < n_dest; ++i) {
      B200Q_REQUIRE(a->peer_out[i] != nullptr && aligned(a->peer_out[i], 16), B200Q_ERR_BAD_ARG,
                    "quant_matmul: peer destination %d is NULL or misaligned", i);
      e.dest[i] = a->peer_out[i];
    }
    e.n_dest = n_dest;
    e.route_rows = routed ? a->route_rows : 0;
  }
  if (!p.tensor_path) {
    dim3 block(32, 8), grid((unsigned)ceil_div(a->n, 32), (unsigned)ceil_div(a->m, 8));
    B200Q_REQUIRE(grid.y <= 65535, B200Q_ERR_UNSUPPORTED,
                  "quant_matmul: operands that miss the 16-byte alignment rules are limited to m <= 524280");
    w8a8_simt_kernel<<<grid, block, 0, st>>>(a->x1, a->x2, a->k, a->x2_stride_k, a->x2_stride_n, e);
    return check_launch("quant_matmul (simt)");
  }
  const size_t need = p.ws_transpose + p.ws_acc;
  B200Q_REQUIRE(need == 0 || (a->workspace != nullptr && a->workspace_bytes >= need && aligned(a->workspace, 256)),
                B200Q_ERR_WORKSPACE, "quant_matmul: needs %zu bytes of 256-byte aligned workspace, got %zu", need,
                a->workspace_bytes);

  const int8_t* w_nk = a->x2;
  int64_t w_pitch = a->x2_stride_n;
  uint8_t* ws = static_cast<uint8_t*>(a->workspace);
  if (p.transpose) {
    int8_t* wt = reinterpret_cast<int8_t*>(ws);
    dim3 grid((unsigned)ceil_div(a->n, 64), (unsigned)ceil_div(a->k, 64));
    transpose_i8_kernel<<<grid, 256, 0, st>>>(a->x2, wt, a->k, a->n);
    if (int rc = check_launch("quant_matmul (weight re-layout)")) return rc;
    w_nk = wt;
    w_pitch = a->k;
  }
  if (p.ws_acc) {
    e.acc_ws = reinterpret_cast<int32_t*>(ws + p.ws_transpose);
    cudaError_t err = cudaMemsetAsync(e.acc_ws, 0, (size_t)a->m * a->n * 4, st);
    if (err != cudaSuccess) return fail(B200Q_ERR_LAUNCH, "quant_matmul: memset: %s", cudaGetErrorString(err));
  }

  if (p.gemv) {
    const int mt = a->m <= 1 ? 1 : a->m <= 2 ? 2 : 4;
    const int smem = (int)(mt * a->k);
    const int64_t want = ceil_div(a->n, 8 * mt);                // 8 warps per CTA, mt channels each per trip
    const int grid = (int)(want < (int64_t)sm_count() * 8 ? want : (int64_t)sm_count() * 8);
    int rc = B200Q_OK;
    switch (mt) {
      case 1:
        if ((rc = ensure_dynamic_smem<w8a8_gemv_kernel<1>>(200 * 1024, "quant_matmul"))) return rc;
        w8a8_gemv_kernel<1><<<grid, 256, smem, st>>>(a->x1, w_nk, a->k, w_pitch, e);
        break;
      case 2:
        if ((rc = ensure_dynamic_smem<w8a8_gemv_kernel<2>>(200 * 1024, "quant_matmul"))) return rc;
        w8a8_gemv_kernel<2><<<grid, 256, smem, st>>>(a->x1, w_nk, a->k, w_pitch, e);
        break;
      default:
        if ((rc = ensure_dynamic_smem<w8a8_gemv_kernel<4>>(200 * 1024, "quant_matmul"))) return rc;
        w8a8_gemv_kernel<4><<<grid, 256, smem, st>>>(a->x1, w_nk, a->k, w_pitch, e);
        break;
    }
    return check_launch("quant_matmul (gemv)");
  }

  if (p.small_m) {
    const unsigned grid = (unsigned)ceil_div(a->n, 16);
    const bool deep = (int64_t)grid <= 2 * (int64_t)sm_count();      // measured: 16 loads in flight win below ~2 CTAs per SM
    if (a->m <= 8) {
      if (deep) w8a8_small_m_kernel<1, 8><<<grid, 256, 0, st>>>(a->x1, w_nk, a->k, w_pitch, e);
      else w8a8_small_m_kernel<1, 4><<<grid, 256, 0, st>>>(a->x1, w_nk, a->k, w_pitch, e);
    } else {
      if (deep) w8a8_small_m_kernel<2, 8><<<grid, 256, 0, st>>>(a->x1, w_nk, a->k, w_pitch, e);
      else w8a8_small_m_kernel<2, 4><<<grid, 256, 0, st>>>(a->x1, w_nk, a->k, w_pitch, e);
    }
    return check_launch("quant_matmul (warp MMA, few tokens)");
  }

  // A operand fills the 128-row MMA axis: tokens normally, channels when swapped.
  const int8_t* a_ptr = p.swap ? w_nk : a->x1;
  const int64_t a_rows = p.swap ? a->n : a->m, a_pitch = p.swap ? w_pitch : a->k;
  const int8_t* b_ptr = p.swap ? a->x1 : w_nk;
  const int64_t b_rows = p.swap ? a->m : a->n, b_pitch = p.swap ? a->k : w_pitch;
  CUtensorMap tmA, tmB;
  if (int rc = make_tmap_2d_cached(&tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a_ptr, a->k, a_rows, a_pitch, kBK, kTileA,
                                   CU_TENSOR_MAP_SWIZZLE_128B, "quant_matmul (A operand)"))
    return rc;
  if (int rc = make_tmap_2d_cached(&tmB, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, b_ptr, a->k, b_rows, b_pitch, kBK,
                                   p.pair ? 128 : p.bn, CU_TENSOR_MAP_SWIZZLE_128B, "quant_matmul (B operand)"))
    return rc;
  if (p.pair) {
    Sched sp{};
    sp.tiles_a = (int)ceil_div(a->m, 256);
    sp.tiles_b = (int)ceil_div(a->n, 256);
    sp.kblocks = (int)ceil_div(a->k, kBK);
    sp.kb_per_split = sp.kblocks;
    sp.splits = 1;
    sp.units = sp.tiles_a * sp.tiles_b;
    if (e.n_dest > 0) {
      const bool two_byte = e.out_dtype == B200Q_BF16 || e.out_dtype == B200Q_F16;
      bool tma_stores = two_byte && e.route_rows == 0 && e.ldo % 8 == 0;
      if (const char* env = getenv("B200Q_W8A8_TMA_STORE")) tma_stores = tma_stores && env[0] != '0';   // tuning override
      if (tma_stores) {
        OutMaps om;
        for (int d = 0; d <= e.n_dest; ++d) {
          void* base = d == 0 ? e.out : e.dest[d - 1];
          if (int rc = make_tmap_2d_cached(&om.m[d], CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, base, (uint64_t)e.n, (uint64_t)e.m,
                                           (uint64_t)e.ldo * 2, 64, 128, CU_TENSOR_MAP_SWIZZLE_128B,
                                           "quant_matmul (output, TMA store)"))
            return rc;
        }
        return launch_umma_pair<5, 2>(tmA, tmB, e, sp, st, &om);
      }
      return launch_umma_pair<6, 1>(tmA, tmB, e, sp, st);
    }
    return launch_umma_pair<6, 0>(tmA, tmB, e, sp, st);
  }

  Sched s{};
  s.tiles_a = (int)ceil_div(a_rows, kTileA);
  s.tiles_b = (int)ceil_div(b_rows, p.bn);
  s.kblocks = (int)ceil_div(a->k, kBK);
  if (p.decode) {
    s.kb_per_split = (int)ceil_div(s.kblocks, p.csize);
    s.splits = p.csize;
    s.units = s.tiles_a * s.tiles_b;
    switch (p.bn) {
      case 16: return launch_decode<16, 8>(tmA, tmB, e, s, p.csize, st);
      case 32: return launch_decode<32, 8>(tmA, tmB, e, s, p.csize, st);
      case 64: return launch_decode<64, 6>(tmA, tmB, e, s, p.csize, st);
      default: return launch_decode<128, 4>(tmA, tmB, e, s, p.csize, st);
    }
  }
  s.kb_per_split = (int)ceil_div(s.kblocks, p.splits);
  s.splits = (int)ceil_div(s.kblocks, s.kb_per_split);
  const int64_t units = (int64_t)s.tiles_a * s.tiles_b * s.splits;
  B200Q_REQUIRE(units < (1LL << 31), B200Q_ERR_UNSUPPORTED, "quant_matmul: too many tiles");
  s.units = (int)units;

  int rc;
  if (p.swap) {
    switch (p.bn) {
      case 16: rc = launch_umma<16, 8, true>(tmA, tmB, e, s, st); break;
      case 32: rc = launch_umma<32, 8, true>(tmA, tmB, e, s, st); break;
      case 64: rc = launch_umma<64, 8, true>(tmA, tmB, e, s, st); break;
      default: rc = launch_umma<128, 6, true>(tmA, tmB, e, s, st); break;
    }
  } else {
    if (e.n_dest > 0)
      rc = (p.bn == 128) ? launch_umma<128, 6, false, true>(tmA, tmB, e, s, st) : launch_umma<256, 4, false, true>(tmA, tmB, e, s, st);
    else
      rc = (p.bn == 128) ? launch_umma<128, 6, false>(tmA, tmB, e, s, st) : launch_umma<256, 4, false>(tmA, tmB, e, s, st);
  }
  if (rc) return rc;
  if (e.acc_ws) {
    Epi f = e;
    f.acc_ws = nullptr;
    const int64_t total = a->m * a->n;
    const int blocks = (int)(ceil_div(total, 256) < (int64_t)sm_count() * 8 ? ceil_div(total, 256) : (int64_t)sm_count() * 8);
    splitk_finalize_kernel<<<blocks, 256, 0, st>>>(e.acc_ws, f);
    return check_launch("quant_matmul (split-K epilogue)");
  }
  return B200Q_OK;
}

// ---------------------------------------------------------------------------------------------
// Entry point for callers that cannot allocate device memory.
//
// Some hosts of this library never get to call cudaMalloc (or torch's allocator) at the moment a
// matmul is needed: an inference server that has already handed all free device memory to its
// KV-cache pool, a plugin that runs inside another framework's memory plan, code on a path where
// an allocation (which may synchronise the device) is forbidden.  b200q_quant_matmul asks such a
// caller for workspace it has no way to provide.  This variant takes the scratch for the split-K
// accumulators and for the [k,n] -> [n,k] weight re-layout from a fixed array that lives in the
// library's device image instead; every GPU that loads the library holds those 16 MiB until the
// process exits.
namespace b200q {
namespace {

constexpr size_t kStaticScratchBytes = size_t(16) << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// In host code the array's name is only a handle for the runtime, not a device address; the address
// is looked up once per device (with that device current) and cached.
int static_scratch_address(void** out) {
  static std::mutex mu;
  static void* cached[64] = {};
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64)
    return fail(B200Q_ERR_LAUNCH, "quant_matmul_static_scratch: no current CUDA device (%s)",
                e != cudaSuccess ? cudaGetErrorString(e) : "device index out of range");
  std::lock_guard<std::mutex> lock(mu);
  if (cached[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess || p == nullptr)
      return fail(B200Q_ERR_LAUNCH, "quant_matmul_static_scratch: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
    cached[dev] = p;
  }
  *out = cached[dev];
  return B200Q_OK;
}

}  // namespace
}  // namespace b200q

extern "C" size_t b200q_static_scratch_bytes(void) { return b200q::kStaticScratchBytes; }

extern "C" int b200q_quant_matmul_static_scratch(const b200q_quant_matmul_args* a, void* stream) {
  using namespace b200q;
  clear_error();
  B200Q_REQUIRE(a != nullptr, B200Q_ERR_BAD_ARG, "quant_matmul_static_scratch: args is NULL");
  const size_t need = b200q_quant_matmul_workspace_bytes(a->m, a->k, a->n, a->x2_stride_k, a->x2_stride_n);
  B200Q_REQUIRE(need <= kStaticScratchBytes, B200Q_ERR_WORKSPACE,
                "quant_matmul_static_scratch: this shape needs %zu bytes of scratch, the built-in array holds %zu; "
                "use b200q_quant_matmul with caller-provided workspace",
                need, kStaticScratchBytes);
  b200q_quant_matmul_args with_scratch = *a;
  with_scratch.workspace = nullptr;
  with_scratch.workspace_bytes = 0;
  if (need != 0) {
    void* scratch = nullptr;
    if (int rc = static_scratch_address(&scratch)) return rc;
    with_scratch.workspace = scratch;
    with_scratch.workspace_bytes = kStaticScratchBytes;
  }
  // The accumulator region is cleared on the stream by the matmul itself before every use, so
  // whatever an earlier call left in the array cannot leak into this one.
  return b200q_quant_matmul(&with_scratch, stream);
}
