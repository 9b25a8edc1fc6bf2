// npu_weight_quant_batchmatmul: weight-only quantised matmul (int4-packed W4A16, int8 W8A16)
// fused into one tcgen05 kernel.
//
// The packed weight is read from HBM exactly once.  Tokens sit on the M axis of the MMA (M = 64
// for up to 64 tokens, else 128 per chunk), 256 output channels on the N axis, so one
// tcgen05.mma.kind::f16 (K = 16) covers 256 channels and the fixed issue cost of an MMA is spread
// over 4096 weights.  Per 64-deep K block of a 256-channel tile:
//   warp 0       TMA: packed weight tile (8 KB int4 / 16 KB int8) and the activation tile
//                [M tokens x 64 k] (128B swizzle) into a ring of load stages
//   warps 2-17   two groups of eight warps, each owning every second K block: dequantise the packed
//                tile in registers, (w + offset) * scale, and write it as the bf16/fp16 B operand in
//                shared memory (canonical 128B-swizzled UMMA layout; MN-major when the weight is
//                n-contiguous, K-major when it is k-contiguous), fence.proxy.async, signal
//   warp 1       tcgen05.mma (fp32 accumulators in TMEM); one tcgen05.commit per K block frees
//                the load stage and the operand slot
// Work is split stream-K style when there are few tiles: the (tile, K block) space is cut into
// equal contiguous ranges, one per CTA, so all SMs stream weights.  A CTA that covers a tile's whole
// K range writes the output itself; otherwise it stores an fp32 partial tile into caller workspace
// (slot = its position among the CTAs sharing the tile) and wq_finalize_kernel adds the partials
// in a fixed order: the result does not depend on timing.
// The dequantising warps also run the epilogue (tcgen05.ld, bias, cast, 64-byte row segments).
// int4 values are expanded with the exponent-bias trick (nibble placed in the mantissa of
// 128.0 / 1024.0, then one exact subtract); w + offset and the product with scale are packed 16-bit
// operations, rounded exactly as the reference's golden does.
// All mbarrier waits are bounded (see ptx.cuh).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <stdlib.h>

#include <type_traits>

#include "common.cuh"
#include "ptx.cuh"
#include "tensormap.cuh"

namespace b200q {
namespace {

constexpr int kWqBK = 64;                   // K elements per stage (one 128-byte swizzle row of bf16)
constexpr int kWqTileN = 256;               // output channels per tile = UMMA N
constexpr int kWqDeqWarps = 16;
constexpr int kWqGroups = 2;                // groups of dequantising warps
constexpr int kWqGroupThreads = kWqDeqWarps / kWqGroups * 32;
constexpr int kWqDeqThreads = kWqDeqWarps * 32;
constexpr int kWqProducers = 1;                   // warps issuing TMA loads, one lane each
constexpr int kWqMmaWarp = kWqProducers;
constexpr int kWqThreads = (kWqProducers + 1) * 32 + kWqDeqThreads;
constexpr int kWqBBytes = kWqTileN * kWqBK * 2;   // one dequantised operand tile

enum WqLayout { kW4N = 0, kW8N = 1, kW8K = 2 };   // int4 [k,n/8]; int8 n-contiguous; int8 k-contiguous

struct WqParams {
  const void* scale;     // [groups, n]
  const void* offset;    // [groups, n] or null
  const void* bias;      // [n] or null
  void* out;             // [m, n]
  float* parts;          // stream-K partial tiles [max_parts][m][n] fp32, or null
  int64_t m, n, k;
  int64_t group_size;    // 0: per channel
  int64_t total_items;   // units * kblocks
  int tiles_n, m_chunks, kblocks, units;
  int stream_k;          // 1: contiguous item ranges per CTA; 0: whole units round-robin
  int ctas;              // grid size the partition was planned for
};

// Which K blocks of which unit a CTA works on, in order.  Every role of the CTA walks the same
// sequence.  stream-K: CTA c owns items [c*T/G, (c+1)*T/G) of the linearised (unit, K block) space.
struct WqWalk {
  int64_t i, end;
  int u, units, step, kblocks;
  bool stream_k;
  __device__ WqWalk(const WqParams& p, int cta, int grid) {
    stream_k = p.stream_k != 0;
    kblocks = p.kblocks;
    units = p.units;
    if (stream_k) {
      i = (int64_t)cta * p.total_items / grid;
      end = (int64_t)(cta + 1) * p.total_items / grid;
    } else {
      i = 0; end = 0;
    }
    u = cta;
    step = grid;
  }
  // Next segment: unit, first and one-past-last K block.  Returns false when the CTA is done.
  __device__ bool next(int& unit, int& kb0, int& kb1) {
    if (stream_k) {
      if (i >= end) return false;
      unit = (int)(i / kblocks);
      kb0 = (int)(i - (int64_t)unit * kblocks);
      const int64_t left = end - i;
      kb1 = (left < kblocks - kb0) ? kb0 + (int)left : kblocks;
      i += kb1 - kb0;
      return true;
    }
    if (u >= units) return false;
    unit = u; kb0 = 0; kb1 = kblocks;
    u += step;
    return true;
  }
};

// stream-K: the CTA whose range contains `item`.
__host__ __device__ inline int wq_cta_of_item(int64_t item, int64_t total, int grid) {
  int c = (int)((item * grid) / total);
  while (c + 1 < grid && (int64_t)(c + 1) * total / grid <= item) ++c;
  while (c > 0 && (int64_t)c * total / grid > item) --c;
  return c;
}

template <typename XT>
struct X2;
template <>
struct X2<__nv_bfloat16> {
  using type = __nv_bfloat162;
  static constexpr uint32_t kMagic = 0x43084308u;   // bf16 136.0 twice: 128 + (nibble ^ 8) == 136 + w
  static __device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_float(float v) { return __float2bfloat16_rn(v); }
  static __device__ __forceinline__ uint32_t pack(float a, float b) {
    __nv_bfloat162 r = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&r);
  }
};
template <>
struct X2<__half> {
  using type = __half2;
  static constexpr uint32_t kMagic = 0x64086408u;   // fp16 1032.0 twice: 1024 + (nibble ^ 8) == 1032 + w
  static __device__ __forceinline__ float to_float(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_float(float v) { return __float2half_rn(v); }
  static __device__ __forceinline__ uint32_t pack(float a, float b) {
    __half2 r = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&r);
  }
};

// The dequantisation repeats the reference golden's arithmetic in the activation dtype
// (test/contrib/test_linear_weight_quant.py:21-26): w + offset rounded to 16 bits, then the product
// with scale rounded again.  Integer weights are exact in fp16 and bf16.
template <typename XT, bool HAS_OFF>
__device__ __forceinline__ uint32_t add_mul2(uint32_t w2, uint32_t of2, uint32_t sc2) {
  using V = typename X2<XT>::type;
  V w = *reinterpret_cast<const V*>(&w2);
  if (HAS_OFF) w = __hadd2(w, *reinterpret_cast<const V*>(&of2));
  V r = __hmul2(w, *reinterpret_cast<const V*>(&sc2));
  return *reinterpret_cast<uint32_t*>(&r);
}
// Two int4 values sitting in bits [0,4) and [16,20) of t -> exact 16-bit floats (exponent-bias trick).
template <typename XT>
__device__ __forceinline__ uint32_t nibbles_to_x2(uint32_t t) {
  using V = typename X2<XT>::type;
  const uint32_t magic = X2<XT>::kMagic;
  uint32_t biased;                                   // (t & 0x000F000F) ^ magic as one three-input logic operation
  asm("lop3.b32 %0, %1, 0x000F000F, %2, 0x6A;" : "=r"(biased) : "r"(t), "r"(magic));
  V w = __hsub2(*reinterpret_cast<const V*>(&biased), *reinterpret_cast<const V*>(&magic));
  return *reinterpret_cast<uint32_t*>(&w);
}

// Two int8 values, bytes ba and bb of a word whose bytes were biased by 128 (w ^ 0x80808080), as exact 16-bit
// floats without the integer-to-float converter (a quarter-rate unit): each byte goes into the mantissa of
// 2^23 by one byte-permute, one packed fp32 subtraction removes 2^23 + 128 exactly, one packed conversion
// rounds to the 16-bit type (exact: |value| <= 128).
template <typename XT>
__device__ __forceinline__ uint32_t bytes_to_x2(uint32_t w_biased, int ba, int bb) {
  const float2 raw = make_float2(__uint_as_float(__byte_perm(w_biased, 0x4B000000u, 0x7440 | ba)),
                                 __uint_as_float(__byte_perm(w_biased, 0x4B000000u, 0x7440 | bb)));
  const float2 v = __fadd2_rn(raw, make_float2(-8388736.0f, -8388736.0f));
  return X2<XT>::pack(v.x, v.y);
}

// Fetches this thread's eight per-channel scale and offset values of group g (raw 16-bit values;
// channels beyond n read as zero).  Kept separate from pair_params8 so that the loads for the next
// K block can be in flight while the current one is dequantised.
template <typename XT>
__device__ __forceinline__ void fetch_params8(const WqParams& p, int64_t g, int64_t n0, uint4& s, uint4& o) {
  s = make_uint4(0, 0, 0, 0);
  o = make_uint4(0, 0, 0, 0);
  if (n0 + 8 <= p.n) {
    s = __ldg(reinterpret_cast<const uint4*>(static_cast<const XT*>(p.scale) + g * p.n + n0));
    if (p.offset) o = __ldg(reinterpret_cast<const uint4*>(static_cast<const XT*>(p.offset) + g * p.n + n0));
  } else {
    unsigned short* sv = reinterpret_cast<unsigned short*>(&s);
    unsigned short* ov = reinterpret_cast<unsigned short*>(&o);
    for (int j = 0; j < 8; ++j) {
      if (n0 + j < p.n) {
        sv[j] = static_cast<const unsigned short*>(p.scale)[g * p.n + n0 + j];
        if (p.offset) ov[j] = static_cast<const unsigned short*>(p.offset)[g * p.n + n0 + j];
      }
    }
  }
}
// Arranges the fetched values as four 16-bit pairs each: (j, j+4) for int4 tiles, (2j, 2j+1) for int8.
template <int LAYOUT>
__device__ __forceinline__ void pair_params8(const uint4& s, const uint4& o, uint32_t (&sc2)[4], uint32_t (&of2)[4]) {
  if (LAYOUT == kW4N) {
    sc2[0] = __byte_perm(s.x, s.z, 0x5410); sc2[1] = __byte_perm(s.x, s.z, 0x7632);
    sc2[2] = __byte_perm(s.y, s.w, 0x5410); sc2[3] = __byte_perm(s.y, s.w, 0x7632);
    of2[0] = __byte_perm(o.x, o.z, 0x5410); of2[1] = __byte_perm(o.x, o.z, 0x7632);
    of2[2] = __byte_perm(o.y, o.w, 0x5410); of2[3] = __byte_perm(o.y, o.w, 0x7632);
  } else {
    sc2[0] = s.x; sc2[1] = s.y; sc2[2] = s.z; sc2[3] = s.w;
    of2[0] = o.x; of2[1] = o.y; of2[2] = o.z; of2[3] = o.w;
  }
}

// int4 tiles keep the nibble pairs (j, j+4) of a word together, so operand row (= accumulator
// column) 8q+i carries channel 8q + perm(i), perm = (0,4,1,5,2,6,3,7); column of channel 8q+o is
// 8q + inv(o) with inv(o) = ((o & 3) << 1) | (o >> 2).
__host__ __device__ constexpr int w4_channel_to_column(int o) { return (o & ~7) + (((o & 3) << 1) | ((o & 7) >> 2)); }

// Shared-memory plan: AS operand slots (32 KB each) and LS load stages (packed weight tile +
// activation tile).  LS > AS so that a group never waits on a barrier a whole phase behind.
template <int LAYOUT, int MM, int NCH>
struct WqCfg {
  static constexpr int kRawBytes = LAYOUT == kW4N ? kWqBK * 128 : kWqBK * 256;
  static constexpr int kXBytes = NCH * MM * 128;            // NCH token chunks of MM rows share one weight tile
  static constexpr int kLoadBytes = kRawBytes + kXBytes;
  static constexpr int kBudget = 212 * 1024;
  static constexpr int kLS3 = (kBudget - 3 * kWqBBytes) / kLoadBytes;
  static constexpr int kASlots = kLS3 > 3 ? 3 : 2;
  static constexpr int kLoadWanted = (kBudget - kASlots * kWqBBytes) / kLoadBytes;
  static constexpr int kLoadStages = kLoadWanted > 12 ? 12 : kLoadWanted;
  static constexpr int kBOff = 0;
  static constexpr int kXOff = kASlots * kWqBBytes;
  static constexpr int kRawOff = kXOff + kLoadStages * kXBytes;
  static constexpr int kBarOff = kRawOff + kLoadStages * kRawBytes;   // full[L], done[L], aready[A], tfull, tempty
  static constexpr int kMiscOff = kBarOff + (2 * kLoadStages + kASlots + 2) * 8;
  static constexpr int kTotal = kMiscOff + 16;
  static constexpr int kDynamic = kTotal + 1024;
  static constexpr uint32_t kTmemCols = NCH * kWqTileN;
  static_assert(kLoadStages > kASlots && kLoadStages > kWqGroups, "ring depths");
  // A producer moves from K block it to it + kWqProducers; the stage of the second one must have been
  // used last by a K block no later than it, or its wait could pass a whole phase early.
  static_assert(kLoadStages >= kWqProducers, "more producers than load stages");
  static_assert(kDynamic <= 227 * 1024 && kDynamic > 116 * 1024, "shared memory budget; one CTA per SM");
};

__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint2 lds_u64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}
__device__ __forceinline__ void sts_u128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// Dequantises one packed [64 k x 256 n] tile into the UMMA B-operand tile with the GT threads of a
// warp group (thread index lg).  raw and b_tile are shared-memory addresses.  Packed words are
// fetched in batches before any arithmetic so that shared-memory latency and the dependent 16-bit
// operations of different items overlap.  Every address is a per-thread constant plus a
// compile-time offset.
template <int LAYOUT, typename XT, int GT, bool HAS_OFF>
__device__ __forceinline__ void dequant_tile(uint32_t raw, uint32_t b_tile, int lg, const uint32_t (&sc2)[4],
                                             const uint32_t (&of2)[4], const WqParams& p, int64_t g, int64_t n_tile0) {
  constexpr int ITEMS = (kWqBK * (kWqTileN / 8)) / GT;      // 8-value items per thread (2048 per tile)
  constexpr int BATCH = ITEMS < 8 ? ITEMS : 8;
  if constexpr (LAYOUT != kW8K) {
    static_assert(GT == 256, "a thread's items are 8 k rows apart: one 1024-byte operand group per item");
    constexpr uint32_t kWord = LAYOUT == kW4N ? 4 : 8;      // packed bytes per 8 channels
    const uint32_t wc = lg & 31;                             // 8-channel group inside the tile
    const uint32_t r = (lg >> 5) & 7;                        // k row inside every 8-row group
    const uint32_t ng = wc >> 3, c = wc & 7;                 // 64-channel block, 16-byte chunk in its 128-byte row
    const uint32_t src = raw + (r * 32 + wc) * kWord;        // item i: k row r + 8 i
    // MN-major operand: [64-channel block][8-k group][k row of 128 B][16-byte chunk ^ row]
    const uint32_t dst = b_tile + ng * 8192 + r * 128 + ((c ^ r) << 4);
#pragma unroll
    for (int b0 = 0; b0 < ITEMS; b0 += BATCH) {
      uint2 v[BATCH];
#pragma unroll
      for (int i = 0; i < BATCH; ++i) {
        if constexpr (LAYOUT == kW4N) v[i] = make_uint2(lds_u32(src + (b0 + i) * 8 * 32 * kWord), 0u);
        else v[i] = lds_u64(src + (b0 + i) * 8 * 32 * kWord);
      }
#pragma unroll
      for (int i = 0; i < BATCH; ++i) {
        uint32_t o[4];
        if constexpr (LAYOUT == kW4N) {
          // halves of o[j]: values j and j+4 -> stored in the order (v0,v4,v1,v5,v2,v6,v3,v7)
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            o[j] = add_mul2<XT, HAS_OFF>(nibbles_to_x2<XT>(v[i].x >> (4 * j)), of2[j], sc2[j]);
          }
        } else {
          const uint32_t w2[2] = {v[i].x ^ 0x80808080u, v[i].y ^ 0x80808080u};
#pragma unroll
          for (int j = 0; j < 8; j += 2)
            o[j >> 1] = add_mul2<XT, HAS_OFF>(bytes_to_x2<XT>(w2[j >> 2], j & 3, (j + 1) & 3), of2[j >> 1], sc2[j >> 1]);
        }
        sts_u128(dst + (b0 + i) * 1024, o[0], o[1], o[2], o[3]);
      }
    }
  } else {
    static_assert(GT == 256, "a thread's items are 32 channel rows apart: four 1024-byte operand groups per item");
    const uint32_t c = lg & 7;                               // 8-wide k chunk inside the 64-deep block
    const uint32_t nr0 = (uint32_t)lg >> 3;                  // channel row of item 0; item i: nr0 + 32 i
    const uint32_t r = nr0 & 7;
    const uint32_t src = raw + (nr0 * 8 + c) * 8;
    // K-major operand: [8-channel group][channel row of 128 B][16-byte chunk ^ row]
    const uint32_t dst = b_tile + (nr0 >> 3) * 1024 + r * 128 + ((c ^ r) << 4);
    const XT* sc_row = static_cast<const XT*>(p.scale) + g * p.n + n_tile0 + nr0;
    const XT* of_row = HAS_OFF ? static_cast<const XT*>(p.offset) + g * p.n + n_tile0 + nr0 : nullptr;
    const int64_t n_left = p.n - n_tile0 - nr0;              // channels from this thread's first row to the end
#pragma unroll
    for (int b0 = 0; b0 < ITEMS; b0 += BATCH) {
      uint2 v[BATCH];
      uint32_t s2[BATCH], o2[BATCH];
#pragma unroll
      for (int i = 0; i < BATCH; ++i) {
        const bool nv = 32 * (b0 + i) < n_left;
        const float scv = nv ? X2<XT>::to_float(sc_row[32 * (b0 + i)]) : 0.0f;
        const float ofv = (nv && HAS_OFF) ? X2<XT>::to_float(of_row[32 * (b0 + i)]) : 0.0f;
        s2[i] = X2<XT>::pack(scv, scv);
        o2[i] = X2<XT>::pack(ofv, ofv);
        v[i] = lds_u64(src + (b0 + i) * 32 * 8 * 8);
      }
#pragma unroll
      for (int i = 0; i < BATCH; ++i) {
        const uint32_t w2[2] = {v[i].x ^ 0x80808080u, v[i].y ^ 0x80808080u};
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 8; j += 2)
          o[j >> 1] = add_mul2<XT, HAS_OFF>(bytes_to_x2<XT>(w2[j >> 2], j & 3, (j + 1) & 3), o2[i], s2[i]);
        sts_u128(dst + (b0 + i) * 4 * 1024, o[0], o[1], o[2], o[3]);
      }
    }
  }
}

template <int LAYOUT, typename XT, int MM, int NCH, bool HAS_OFF>
__global__ void __launch_bounds__(kWqThreads, 1)
wq_umma_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, const WqParams p) {
  using C = WqCfg<LAYOUT, MM, NCH>;
  constexpr int LS = C::kLoadStages, AS = C::kASlots;
  constexpr bool B_MN = LAYOUT != kW8K;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sB = smem + C::kBOff;
  uint8_t* sX = smem + C::kXOff;
  uint8_t* sRaw = smem + C::kRawOff;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + C::kBarOff);
  uint64_t* done = full + LS;
  uint64_t* aready = done + LS;
  uint64_t* tfull = aready + AS;
  uint64_t* tempty = tfull + 1;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(smem + C::kMiscOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + C::kMiscOff + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int i = 0; i < LS; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&done[i], 1);
    }
    for (int i = 0; i < AS; ++i) mbar_init(&aready[i], kWqDeqWarps / kWqGroups);
    mbar_init(tfull, 1);
    mbar_init(tempty, kWqDeqWarps);
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tensormap(&tmW);
    prefetch_tensormap(&tmX);
  }
  if (warp == kWqMmaWarp) {
    tmem_alloc(tmem_holder, C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp < kWqProducers) {
    // ----------------------------------------------------------- TMA producers
    // K block `it` of this CTA's sequence is loaded by producer it % kWqProducers.  (Loads issued by one
    // thread are served a few at a time, so a pure copy streams faster from several issuing warps; this
    // kernel is bound by shared-memory bandwidth and the tensor pipe instead and runs best with one.)
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      WqWalk walk(p, blockIdx.x, gridDim.x);
      int unit, kb0, kb1;
      auto weight_coords = [&](int tn, int kb, int& c0, int& c1) {
        if (LAYOUT == kW4N) { c0 = tn * 128; c1 = kb * kWqBK; }            // bytes of packed nibbles: 128 bytes = 256 channels per row of k
        else if (LAYOUT == kW8N) { c0 = tn * kWqTileN; c1 = kb * kWqBK; }
        else { c0 = kb * kWqBK; c1 = tn * kWqTileN; }                      // k-contiguous: rows are channels
      };
      while (ok && walk.next(unit, kb0, kb1)) {
        const int tn = unit % p.tiles_n, mc = unit / p.tiles_n;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          if (it % kWqProducers != warp) continue;
          const int stage = it % LS;
          if (!mbar_wait(&done[stage], (uint32_t)((it / LS) & 1) ^ 1u, abort_flag, kDevTimeoutProducer)) { ok = false; break; }
          mbar_arrive_expect_tx(&full[stage], C::kRawBytes + C::kXBytes);
          int c0, c1;
          weight_coords(tn, kb, c0, c1);
          tma_load_2d(sRaw + stage * C::kRawBytes, &tmW, &full[stage], c0, c1);
#pragma unroll
          for (int ch = 0; ch < NCH; ++ch)
            tma_load_2d(sX + stage * C::kXBytes + ch * MM * 128, &tmX, &full[stage], kb * kWqBK, (mc * NCH + ch) * MM);
        }
      }
      if (!ok)
        for (int i = 0; i < 200; ++i) __nanosleep(1000);   // let copies in flight land before smem is released
    }
  } else if (warp == kWqMmaWarp) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t fmt = std::is_same<XT, __nv_bfloat16>::value ? 1u : 0u;
      constexpr uint32_t idesc = make_idesc(1 /*f32*/, fmt, fmt, 0, B_MN ? 1 : 0, MM, kWqTileN);
      int it = 0;
      uint32_t tphase = 0;
      bool ok = true;
      WqWalk walk(p, blockIdx.x, gridDim.x);
      int unit, kb0, kb1;
      while (ok && walk.next(unit, kb0, kb1)) {
        if (!mbar_wait(tempty, tphase ^ 1, abort_flag, kDevTimeoutMma)) { ok = false; break; }
        tc_fence_after();
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int stage = it % LS, slot = it % AS;
          if (!mbar_wait(&aready[slot], (uint32_t)(it / AS) & 1u, abort_flag, kDevTimeoutMma) ||
              !mbar_wait(&full[stage], (uint32_t)(it / LS) & 1u, abort_flag, kDevTimeoutMma)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(sX + stage * C::kXBytes), b_addr = smem_u32(sB + slot * kWqBBytes);
#pragma unroll
          for (int k16 = 0; k16 < kWqBK / 16; ++k16) {
            // K-major A / B: 16 k = 32 bytes inside the 128-byte swizzle row; 8-row groups 1024 B apart.
            // MN-major B: 16 k = two 8-row groups of 1024 B; 64-channel blocks 8192 B apart.
            const uint64_t bdesc = B_MN ? make_smem_desc(b_addr + k16 * 2048, 8192, 1024, kSwizzle128B)
                                        : make_smem_desc(b_addr + k16 * 32, 16, 1024, kSwizzle128B);
#pragma unroll
            for (int ch = 0; ch < NCH; ++ch) {
              const uint64_t adesc = make_smem_desc(a_addr + ch * MM * 128 + k16 * 32, 16, 1024, kSwizzle128B);
              umma_f16(tmem_base + ch * kWqTileN, adesc, bdesc, idesc, (kb > kb0 || k16 > 0) ? 1u : 0u);
            }
          }
          umma_commit(&done[stage]);                     // load stage and operand slot are free once these MMAs retire
        }
        if (!ok) break;
        umma_commit(tfull);
        tphase ^= 1;
      }
    }
  } else {
    // ------------------------------------------- dequantise, then epilogue
    constexpr int GT = kWqGroupThreads;
    const int dw = warp - (kWqProducers + 1);          // 0..15
    const int group = dw / (kWqDeqWarps / kWqGroups);
    const int lg = (dw % (kWqDeqWarps / kWqGroups)) * 32 + lane;   // thread index inside the group
    const int quad = warp & 3;                         // TMEM lane quadrant of this warp
    // Quantisation groups are whole K blocks (checked on the host); 0 = one group per channel.
    const uint32_t gs_blocks = p.group_size > 0 ? (uint32_t)(p.group_size / kWqBK) : 0u;
    const uint32_t sRaw_u32 = smem_u32(sRaw), sB_u32 = smem_u32(sB);
    int it_base = 0;                                   // K blocks this CTA has been through before this segment
    uint32_t tphase = 0;
    bool ok = true;
    WqWalk walk(p, blockIdx.x, gridDim.x);
    int unit, kb0, kb1;
    while (ok && walk.next(unit, kb0, kb1)) {
      const int tn = unit % p.tiles_n, mc = unit / p.tiles_n;
      const int64_t n_tile0 = (int64_t)tn * kWqTileN;
      int64_t cur_group = -1;
      uint32_t sc2[4], of2[4];   // this thread's 8 channels as 16-bit pairs: kW4N (j, j+4), kW8N (2j, 2j+1)
      uint4 ns, no;              // parameters fetched ahead for the next K block of this group
      const int64_t n_oct0 = n_tile0 + (lg & 31) * 8;
      int kb = kb0 + ((group - it_base % kWqGroups + kWqGroups) % kWqGroups);   // first K block owned by the group
      // Group of the K block ahead, kept by counting (no division in the loop).
      uint32_t g_next = gs_blocks ? (uint32_t)kb / gs_blocks : 0u;
      uint32_t g_rem = gs_blocks ? (uint32_t)kb % gs_blocks : 0u;
      if (LAYOUT != kW8K && kb < kb1) fetch_params8<XT>(p, g_next, n_oct0, ns, no);
      for (; kb < kb1; kb += kWqGroups) {
        const int it = it_base + (kb - kb0);
        const int stage = it % LS, slot = it % AS;
        const int64_t g = g_next;
        if (LAYOUT != kW8K && g != cur_group) {
          cur_group = g;
          pair_params8<LAYOUT>(ns, no, sc2, of2);
        }
        if (gs_blocks && kb + kWqGroups < kb1) {       // loads for the group's next K block fly during this one
          g_rem += kWqGroups;
          while (g_rem >= gs_blocks) { g_rem -= gs_blocks; ++g_next; }
          if (LAYOUT != kW8K && (int64_t)g_next != g) fetch_params8<XT>(p, g_next, n_oct0, ns, no);
        }
        // The tile must have landed, and the MMAs that read this operand slot AS tiles ago must have retired.
        bool got = mbar_wait(&full[stage], (uint32_t)(it / LS) & 1u, abort_flag, kDevTimeoutEpilogue);
        if (got && it >= AS)
          got = mbar_wait(&done[(it - AS) % LS], (uint32_t)((it - AS) / LS) & 1u, abort_flag, kDevTimeoutEpilogue);
        if (!__all_sync(0xffffffffu, got)) { ok = false; break; }   // warp-uniform, the warp stays converged
        dequant_tile<LAYOUT, XT, GT, HAS_OFF>(sRaw_u32 + stage * C::kRawBytes, sB_u32 + slot * kWqBBytes, lg, sc2, of2,
                                              p, g, n_tile0);
        fence_proxy_async_smem();                      // generic-proxy stores -> visible to the MMA (async proxy)
        __syncwarp();
        if (lane == 0) mbar_arrive(&aready[slot]);
      }
      it_base += kb1 - kb0;
      // The stop decision is taken by all dequantising warps together (named barrier 2).
      {
        bool got = ok && mbar_wait(tfull, tphase, abort_flag, kDevTimeoutEpilogue);
        uint32_t all;
        asm volatile(
            "{\n\t.reg .pred p, q;\n\t"
            "setp.ne.u32 p, %1, 0;\n\t"
            "bar.red.and.pred q, 2, %2, p;\n\t"
            "selp.u32 %0, 1, 0, q;\n\t}"
            : "=r"(all) : "r"((uint32_t)got), "r"(kWqDeqThreads) : "memory");
        if (!all) { ok = false; break; }
      }
      tc_fence_after();
      tphase ^= 1;
      // -------- epilogue: accumulator rows are tokens, columns are channels; four warps share a lane quadrant.
      // With M = 64 the rows sit in lanes 0-15 of each quadrant.
      {
        const int share = dw >> 2;                     // this warp's slot among the four of its quadrant
        const int row = MM == 128 ? quad * 32 + lane : quad * 16 + lane;
        const bool row_ok = MM == 128 || lane < 16;
        const bool whole = (kb0 == 0 && kb1 == p.kblocks);
        const int first = whole ? 0 : wq_cta_of_item((int64_t)unit * p.kblocks, p.total_items, (int)gridDim.x);
#pragma unroll 1
        for (int cc = share; cc < NCH * (kWqTileN / 32); cc += 4) {
          const int ch = cc / (kWqTileN / 32), c = cc % (kWqTileN / 32);
          const int64_t token = ((int64_t)mc * NCH + ch) * MM + row;
          const bool tv = row_ok && token < p.m;
          float* part = whole ? nullptr : p.parts + ((int64_t)((int)blockIdx.x - first) * p.m + token) * p.n;
          const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + ch * kWqTileN;
          uint32_t r[32];
          __syncwarp();
          tmem_ld_x32(taddr + c * 32, r);
          tmem_ld_wait();
          const int64_t n0 = n_tile0 + c * 32;
          if (!tv || n0 >= p.n) continue;
          const bool vec = n0 + 32 <= p.n;
          if (!whole) {
            // fp32 partial tile, channel order restored
            if (vec) {
              float4* dst = reinterpret_cast<float4*>(part + n0);
#pragma unroll
              for (int q = 0; q < 8; ++q) {
                float v[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const int o = 4 * q + j;
                  v[j] = __uint_as_float(r[LAYOUT == kW4N ? w4_channel_to_column(o) : o]);
                }
                dst[q] = make_float4(v[0], v[1], v[2], v[3]);
              }
            } else {
#pragma unroll
              for (int o = 0; o < 32; ++o)
                if (n0 + o < p.n) part[n0 + o] = __uint_as_float(r[LAYOUT == kW4N ? w4_channel_to_column(o) : o]);
            }
          } else {
            XT* dst = static_cast<XT*>(p.out) + token * p.n + n0;
            if (vec) {
              uint32_t packed[16];
#pragma unroll
              for (int o = 0; o < 32; o += 2) {
                float v0 = __uint_as_float(r[LAYOUT == kW4N ? w4_channel_to_column(o) : o]);
                float v1 = __uint_as_float(r[LAYOUT == kW4N ? w4_channel_to_column(o + 1) : o + 1]);
                if (p.bias) {
                  v0 = __fadd_rn(v0, X2<XT>::to_float(static_cast<const XT*>(p.bias)[n0 + o]));
                  v1 = __fadd_rn(v1, X2<XT>::to_float(static_cast<const XT*>(p.bias)[n0 + o + 1]));
                }
                packed[o >> 1] = X2<XT>::pack(v0, v1);
              }
#pragma unroll
              for (int q = 0; q < 4; ++q)
                reinterpret_cast<uint4*>(dst)[q] =
                    make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
            } else {
#pragma unroll
              for (int o = 0; o < 32; ++o) {
                if (n0 + o < p.n) {
                  float v = __uint_as_float(r[LAYOUT == kW4N ? w4_channel_to_column(o) : o]);
                  if (p.bias) v = __fadd_rn(v, X2<XT>::to_float(static_cast<const XT*>(p.bias)[n0 + o]));
                  dst[o] = X2<XT>::from_float(v);
                }
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty);
    }
    if (dw == 0 && lane == 0) {
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kWqMmaWarp) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

// stream-K: adds the fp32 partial tiles of every unit that was shared by several CTAs, in CTA
// order, then bias and cast.  Units computed whole by one CTA were written by that CTA.  One CTA
// (256 threads = 4 rows x 64 four-channel vectors) per 16-row slice of a unit.
template <typename XT>
__global__ void __launch_bounds__(256) wq_finalize_kernel(const WqParams p, int mm_rows) {
  __shared__ int s_first, s_last;
  const int slices = mm_rows / 16;
  const int c4 = threadIdx.x & 63, rsub = threadIdx.x >> 6;
  for (int64_t w = blockIdx.x; w < (int64_t)p.units * slices; w += gridDim.x) {
    const int unit = (int)(w / slices), sl = (int)(w - (int64_t)unit * slices);
    const int tn = unit % p.tiles_n, mc = unit / p.tiles_n;
    const int64_t row0 = (int64_t)mc * mm_rows + sl * 16;
    if (row0 >= p.m) continue;                               // block-uniform
    __syncthreads();                                         // the previous slice's readers are done
    if (threadIdx.x == 0) {
      s_first = wq_cta_of_item((int64_t)unit * p.kblocks, p.total_items, p.ctas);
      s_last = wq_cta_of_item((int64_t)(unit + 1) * p.kblocks - 1, p.total_items, p.ctas);
    }
    __syncthreads();
    const int parts = s_last - s_first + 1;
    if (parts <= 1) continue;
    const int64_t n = (int64_t)tn * kWqTileN + c4 * 4;
    if (n >= p.n) continue;
    float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
    if (p.bias) {
      const XT* bp = static_cast<const XT*>(p.bias) + n;
      b = make_float4(X2<XT>::to_float(bp[0]), X2<XT>::to_float(bp[1]), X2<XT>::to_float(bp[2]), X2<XT>::to_float(bp[3]));
    }
#pragma unroll
    for (int rr = 0; rr < 4; ++rr) {
      const int64_t token = row0 + rr * 4 + rsub;
      if (token >= p.m) break;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int c = 0; c < parts; ++c) {
        const float4 t = __ldcs(reinterpret_cast<const float4*>(p.parts + ((int64_t)c * p.m + token) * p.n + n));
        v.x = __fadd_rn(v.x, t.x); v.y = __fadd_rn(v.y, t.y); v.z = __fadd_rn(v.z, t.z); v.w = __fadd_rn(v.w, t.w);
      }
      if (p.bias) { v.x = __fadd_rn(v.x, b.x); v.y = __fadd_rn(v.y, b.y); v.z = __fadd_rn(v.z, b.z); v.w = __fadd_rn(v.w, b.w); }
      *reinterpret_cast<uint2*>(static_cast<XT*>(p.out) + token * p.n + n) =
          make_uint2(X2<XT>::pack(v.x, v.y), X2<XT>::pack(v.z, v.w));
    }
  }
}

// Any shape, any strides: one thread per output element, fp32 dequantisation and accumulation.
template <typename XT>
__global__ void wq_simt_kernel(const XT* __restrict__ x, const void* __restrict__ w, int bits, int64_t sk, int64_t sn,
                               const WqParams p) {
  const int64_t n = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  const int64_t mm = blockIdx.y * (int64_t)blockDim.y + threadIdx.y;
  if (n >= p.n || mm >= p.m) return;
  float acc = 0.0f;
  for (int64_t kk = 0; kk < p.k; ++kk) {
    const int64_t g = p.group_size > 0 ? kk / p.group_size : 0;
    float wv;
    if (bits == 4) {
      const uint32_t word = static_cast<const uint32_t*>(w)[kk * (p.n / 8) + n / 8];
      const int nib = (word >> (4 * (n & 7))) & 0xF;
      wv = (float)(nib > 7 ? nib - 16 : nib);
    } else {
      wv = (float)static_cast<const int8_t*>(w)[kk * sk + n * sn];
    }
    const float sc = X2<XT>::to_float(static_cast<const XT*>(p.scale)[g * p.n + n]);
    const float of = p.offset ? X2<XT>::to_float(static_cast<const XT*>(p.offset)[g * p.n + n]) : 0.0f;
    float wd = wv;                                    // two roundings in the activation dtype, as above
    if (p.offset) wd = X2<XT>::to_float(X2<XT>::from_float(__fadd_rn(wd, of)));
    wd = X2<XT>::to_float(X2<XT>::from_float(__fmul_rn(wd, sc)));
    acc = fmaf(X2<XT>::to_float(x[mm * p.k + kk]), wd, acc);
  }
  if (p.bias) acc += X2<XT>::to_float(static_cast<const XT*>(p.bias)[n]);
  static_cast<XT*>(p.out)[mm * p.n + n] = X2<XT>::from_float(acc);
}

}  // namespace
}  // namespace b200q
#include "w4a16_stream.cuh"
namespace b200q {
namespace {

// Few tokens, int4: the streaming warp-MMA kernel (one launch, no workspace) instead of the tcgen05 one.
bool wq_use_stream(int64_t m, int64_t k, int64_t n, int bits) {
  if (const char* env = getenv("B200Q_WQ_STREAM")) {                  // tuning override
    if (env[0] == '0') return false;
  }
  return bits == 4 && m <= kWsMaxTokens && n % 32 == 0 && k >= kWsKBlock && k % kWsKBlock == 0;
}

struct WqPlan {
  int mm;            // tokens per unit: 64 (M = 64 MMAs), 128, or 256 (two M = 128 chunks sharing each weight tile)
  int tiles_n, m_chunks, kblocks, units, ctas, stream_k, max_parts;
  int64_t total_items;
  size_t ws_bytes;
};

// Tiling and work split; shared by the workspace query and the launch.
WqPlan wq_plan(int64_t m, int64_t k, int64_t n) {
  WqPlan pl{};
  pl.mm = m <= 64 ? 64 : m <= 128 ? 128 : 256;
  pl.tiles_n = (int)ceil_div(n, kWqTileN);
  pl.m_chunks = (int)ceil_div(m, pl.mm);
  pl.kblocks = (int)ceil_div(k, kWqBK);
  const int64_t units = (int64_t)pl.tiles_n * pl.m_chunks;
  pl.units = (int)units;
  pl.total_items = units * pl.kblocks;
  const int sms = sm_count();
  // Splitting K costs an fp32 partial tile per (CTA, tile) pair.  It pays when whole tiles would leave
  // SMs idle in the last round (less than 90 % of the SM-rounds used) and the partials stay small next
  // to the weight stream, or when most SMs would have no tile at all.
  const int64_t rounds = ceil_div(units, (int64_t)sms);
  const bool uneven = units * 10 < rounds * sms * 9;
  pl.stream_k = (pl.kblocks >= 2 && ((uneven && 128 * m <= k && units < 4LL * sms) || 2 * units < sms)) ? 1 : 0;
  if (const char* env = getenv("B200Q_WQ_STREAMK")) pl.stream_k = (env[0] != '0' && pl.kblocks >= 2) ? 1 : 0;   // tuning override
  pl.ctas = (int)(pl.stream_k ? (pl.total_items < sms ? pl.total_items : sms) : (units < sms ? units : sms));
  pl.max_parts = 0;
  if (pl.stream_k) {
    for (int64_t u = 0; u < units; ++u) {
      const int first = wq_cta_of_item(u * pl.kblocks, pl.total_items, pl.ctas);
      const int last = wq_cta_of_item((u + 1) * pl.kblocks - 1, pl.total_items, pl.ctas);
      if (last > first && last - first + 1 > pl.max_parts) pl.max_parts = last - first + 1;
    }
  }
  pl.ws_bytes = (size_t)pl.max_parts * (size_t)m * (size_t)n * sizeof(float);
  return pl;
}

template <int LAYOUT, typename XT, int MM, int NCH, bool HAS_OFF>
int launch_wq(const CUtensorMap& tmW, const CUtensorMap& tmX, const WqParams& p, cudaStream_t st) {
  using C = WqCfg<LAYOUT, MM, NCH>;
  constexpr auto kern = wq_umma_kernel<LAYOUT, XT, MM, NCH, HAS_OFF>;
  if (int rc = ensure_dynamic_smem<kern>(C::kDynamic, "weight_quant_matmul")) return rc;
  kern<<<p.ctas, kWqThreads, C::kDynamic, st>>>(tmW, tmX, p);
  if (int rc = check_launch("weight_quant_matmul (tcgen05)")) return rc;
  if (p.parts) {
    const int64_t want = (int64_t)p.units * (MM * NCH / 16);
    const int blocks = (int)(want < (int64_t)sm_count() * 8 ? want : (int64_t)sm_count() * 8);
    wq_finalize_kernel<XT><<<blocks, 256, 0, st>>>(p, MM * NCH);
    return check_launch("weight_quant_matmul (stream-K sum)");
  }
  return B200Q_OK;
}

template <int LAYOUT, typename XT, bool HAS_OFF>
int dispatch_mm(int mm, const CUtensorMap& tmW, const CUtensorMap& tmX, const WqParams& p, cudaStream_t st) {
  if (mm == 64) return launch_wq<LAYOUT, XT, 64, 1, HAS_OFF>(tmW, tmX, p, st);
  if (mm == 128) return launch_wq<LAYOUT, XT, 128, 1, HAS_OFF>(tmW, tmX, p, st);
  return launch_wq<LAYOUT, XT, 128, 2, HAS_OFF>(tmW, tmX, p, st);   // mm == 256: two 128-token chunks per weight tile
}
template <int LAYOUT, typename XT>
int dispatch_off(int mm, const CUtensorMap& tmW, const CUtensorMap& tmX, const WqParams& p, cudaStream_t st) {
  return p.offset ? dispatch_mm<LAYOUT, XT, true>(mm, tmW, tmX, p, st) : dispatch_mm<LAYOUT, XT, false>(mm, tmW, tmX, p, st);
}

template <typename XT>
int dispatch_layout(int layout, int mm, const CUtensorMap& tmW, const CUtensorMap& tmX, const WqParams& p,
                    cudaStream_t st) {
  switch (layout) {
    case kW4N: return dispatch_off<kW4N, XT>(mm, tmW, tmX, p, st);
    case kW8N: return dispatch_off<kW8N, XT>(mm, tmW, tmX, p, st);
    default: return dispatch_off<kW8K, XT>(mm, tmW, tmX, p, st);
  }
}

}  // namespace
}  // namespace b200q

extern "C" size_t b200q_weight_quant_matmul_workspace_bytes(int64_t m, int64_t k, int64_t n, int weight_bits) {
  if (m <= 0 || k <= 0 || n <= 0) return 0;
  if (b200q::wq_use_stream(m, k, n, weight_bits)) return 0;
  return b200q::wq_plan(m, k, n).ws_bytes;
}

extern "C" int b200q_weight_quant_matmul(const b200q_weight_quant_matmul_args* a, void* stream) {
  using namespace b200q;
  clear_error();
  B200Q_REQUIRE(a != nullptr, B200Q_ERR_BAD_ARG, "weight_quant_matmul: args is NULL");
  B200Q_REQUIRE(a->m >= 0 && a->k >= 0 && a->n >= 0 && a->group_size >= 0, B200Q_ERR_BAD_ARG,
                "weight_quant_matmul: negative size");
  B200Q_REQUIRE(a->x_dtype == B200Q_BF16 || a->x_dtype == B200Q_F16, B200Q_ERR_UNSUPPORTED,
                "weight_quant_matmul: x must be bf16 or f16 (dtype enum %d)", a->x_dtype);
  B200Q_REQUIRE(a->weight_bits == 4 || a->weight_bits == 8, B200Q_ERR_UNSUPPORTED,
                "weight_quant_matmul: weight_bits must be 4 or 8, got %d", a->weight_bits);
  B200Q_REQUIRE(a->weight_bits == 8 || a->n % 8 == 0, B200Q_ERR_BAD_ARG,
                "weight_quant_matmul: int4 weights need n to be a multiple of 8");
  if (a->m == 0 || a->n == 0) return B200Q_OK;
  B200Q_REQUIRE(a->out != nullptr && a->antiquant_scale != nullptr, B200Q_ERR_BAD_ARG,
                "weight_quant_matmul: out or antiquant_scale is NULL");
  B200Q_REQUIRE(a->k == 0 || (a->x != nullptr && a->weight != nullptr), B200Q_ERR_BAD_ARG,
                "weight_quant_matmul: x or weight is NULL");
  cudaStream_t st = static_cast<cudaStream_t>(stream);

  WqParams p{};
  p.scale = a->antiquant_scale; p.offset = a->antiquant_offset; p.bias = a->bias; p.out = a->out;
  p.m = a->m; p.n = a->n; p.k = a->k; p.group_size = a->group_size;

  int layout = -1;
  if (a->weight_bits == 4) {
    if (a->n % 32 == 0) layout = kW4N;
  } else if (a->w_stride_n == 1 && a->w_stride_k >= a->n && a->w_stride_k % 16 == 0) {
    layout = kW8N;
  } else if (a->w_stride_k == 1 && a->w_stride_n >= a->k && a->w_stride_n % 16 == 0) {
    layout = kW8K;
  }
  const bool fused = layout >= 0 && a->k >= 8 && a->k % 8 == 0 && a->n % 8 == 0 && aligned(a->x, 16) &&
                     aligned(a->weight, 16) && aligned(a->antiquant_scale, 16) && aligned(a->out, 16) &&
                     (a->antiquant_offset == nullptr || aligned(a->antiquant_offset, 16)) &&
                     (a->group_size == 0 || a->group_size % kWqBK == 0) && a->k < (1LL << 31) && a->n < (1LL << 31) &&
                     a->m < (1LL << 31);
  if (!fused) {
    dim3 block(32, 8), grid((unsigned)ceil_div(a->n, 32), (unsigned)ceil_div(a->m, 8));
    B200Q_REQUIRE(grid.y <= 65535, B200Q_ERR_UNSUPPORTED,
                  "weight_quant_matmul: operands that miss the alignment rules are limited to m <= 524280");
    if (a->x_dtype == B200Q_BF16)
      wq_simt_kernel<__nv_bfloat16><<<grid, block, 0, st>>>(static_cast<const __nv_bfloat16*>(a->x), a->weight,
                                                            a->weight_bits, a->w_stride_k, a->w_stride_n, p);
    else
      wq_simt_kernel<__half><<<grid, block, 0, st>>>(static_cast<const __half*>(a->x), a->weight, a->weight_bits,
                                                     a->w_stride_k, a->w_stride_n, p);
    return check_launch("weight_quant_matmul (simt)");
  }

  if (layout == kW4N && wq_use_stream(a->m, a->k, a->n, 4) && (a->bias == nullptr || aligned(a->bias, 16)) &&
      (a->group_size == 0 || a->group_size % kWsKBlock == 0)) {
    if (a->x_dtype == B200Q_BF16) return dispatch_wq_stream<__nv_bfloat16>(a->x, a->weight, p, st);
    return dispatch_wq_stream<__half>(a->x, a->weight, p, st);
  }

  const WqPlan pl = wq_plan(a->m, a->k, a->n);
  B200Q_REQUIRE(pl.total_items < (1LL << 40) && (int64_t)pl.tiles_n * pl.m_chunks < (1LL << 31), B200Q_ERR_UNSUPPORTED,
                "weight_quant_matmul: too many tiles");
  p.tiles_n = pl.tiles_n; p.m_chunks = pl.m_chunks; p.kblocks = pl.kblocks; p.units = pl.units;
  p.total_items = pl.total_items; p.stream_k = pl.stream_k; p.ctas = pl.ctas;
  p.parts = nullptr;
  if (pl.ws_bytes) {
    B200Q_REQUIRE(a->workspace != nullptr && a->workspace_bytes >= pl.ws_bytes && aligned(a->workspace, 256),
                  B200Q_ERR_WORKSPACE, "weight_quant_matmul: needs %zu bytes of 256-byte aligned workspace, got %zu",
                  pl.ws_bytes, a->workspace_bytes);
    p.parts = static_cast<float*>(a->workspace);
  }

  CUtensorMap tmW, tmX;
  int rc;
  if (layout == kW4N)
    rc = make_tmap_2d(&tmW, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a->weight, a->n / 2, a->k, a->n / 2, 128, kWqBK,
                      CU_TENSOR_MAP_SWIZZLE_NONE, "weight_quant_matmul (int4 weight)");
  else if (layout == kW8N)
    rc = make_tmap_2d(&tmW, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a->weight, a->n, a->k, a->w_stride_k, kWqTileN, kWqBK,
                      CU_TENSOR_MAP_SWIZZLE_NONE, "weight_quant_matmul (int8 weight)");
  else
    rc = make_tmap_2d(&tmW, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a->weight, a->k, a->n, a->w_stride_n, kWqBK, kWqTileN,
                      CU_TENSOR_MAP_SWIZZLE_NONE, "weight_quant_matmul (int8 weight)");
  if (rc) return rc;
  rc = make_tmap_2d(&tmX, a->x_dtype == B200Q_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                    2, a->x, a->k, a->m, a->k * 2, kWqBK, pl.mm == 64 ? 64 : 128, CU_TENSOR_MAP_SWIZZLE_128B,
                    "weight_quant_matmul (activations)");
  if (rc) return rc;
  if (a->x_dtype == B200Q_BF16) return dispatch_layout<__nv_bfloat16>(layout, pl.mm, tmW, tmX, p, st);
  return dispatch_layout<__half>(layout, pl.mm, tmW, tmX, p, st);
}
