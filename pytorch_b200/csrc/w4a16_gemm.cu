// npu_weight_quant_batchmatmul: weight-only quantised matmul (int4-packed W4A16, int8 W8A16)
// fused into one tcgen05 kernel.
//
// The quantised weight is the dominant traffic, so it takes the 128-row axis of the MMA
// (A operand, 128 output channels per CTA tile) and is read from HBM exactly once, still
// packed.  Per 64-deep K block:
//   warp 0       TMA: packed weight tile (4 KB int4 / 8 KB int8) and the activation tile
//                [BNX tokens x 64 k] (128B swizzle) into a deep ring of load stages (up to 16, so
//                that enough bytes are in flight from HBM)
//   warps 2-17   in G groups, each owning every G-th K block (so G stages are in work at once):
//                dequantise the packed tile in registers, (w + offset) * scale, and write it as
//                a bf16/fp16 UMMA operand tile in shared memory (canonical 128B-swizzled layout;
//                MN-major when the weight is n-contiguous, K-major when it is k-contiguous),
//                fence.proxy.async, signal
//   warp 1       tcgen05.mma.kind::f16 (M=128 channels, N=BNX tokens, K=16), fp32 accumulators
//                in TMEM; tcgen05.commit frees the operand slot and the load stage
// After the last K block the dequantising warps turn into the epilogue: tcgen05.ld, bias,
// cast, coalesced stores along n.  int4 values are expanded with the exponent-bias trick
// (nibble placed in the mantissa of 128.0 / 1024.0, then one exact subtract); w + offset and the
// product with scale are packed 16-bit operations, rounded exactly as the reference's golden does.
// All mbarrier waits are bounded (see ptx.cuh).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <type_traits>

#include "common.cuh"
#include "ptx.cuh"
#include "tensormap.cuh"

namespace b200q {
namespace {

constexpr int kWqBK = 64;                   // K elements per stage (one 128-byte swizzle row of bf16)
constexpr int kWqTileN = 128;               // output channels per tile = UMMA M
constexpr int kWqDeqWarps = 16;
constexpr int kWqDeqThreads = kWqDeqWarps * 32;
constexpr int kWqThreads = 64 + kWqDeqThreads;
constexpr int kWqABytes = kWqTileN * kWqBK * 2;

enum WqLayout { kW4N = 0, kW8N = 1, kW8K = 2 };   // int4 [k,n/8]; int8 n-contiguous; int8 k-contiguous

// int4 tiles keep the nibble pairs (j, j+4) of a word together, so operand row 8q+i carries channel
// 8q + perm(i) with perm = (0,4,1,5,2,6,3,7), i.e. perm(i) = (i >> 1) + 4 * (i & 1).
__device__ __forceinline__ int w4_row_to_channel(int row) { return (row & ~7) + ((row & 7) >> 1) + 4 * (row & 1); }

struct WqParams {
  const void* scale;     // [groups, n]
  const void* offset;    // [groups, n] or null
  const void* bias;      // [n] or null
  void* out;             // [m, n]
  int64_t m, n, k;
  int64_t group_size;    // 0: per channel
  int tiles_n, m_chunks, kblocks, units;
};

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
template <typename XT>
__device__ __forceinline__ uint32_t add_mul2(uint32_t w2, uint32_t of2, uint32_t sc2, bool has_offset) {
  using V = typename X2<XT>::type;
  V w = *reinterpret_cast<const V*>(&w2);
  if (has_offset) w = __hadd2(w, *reinterpret_cast<const V*>(&of2));
  V r = __hmul2(w, *reinterpret_cast<const V*>(&sc2));
  return *reinterpret_cast<uint32_t*>(&r);
}
// Two int4 values sitting in bits [0,4) and [16,20) of t -> exact 16-bit floats (exponent-bias trick).
template <typename XT>
__device__ __forceinline__ uint32_t nibbles_to_x2(uint32_t t) {
  using V = typename X2<XT>::type;
  const uint32_t magic = X2<XT>::kMagic;
  const uint32_t biased = (t & 0x000F000Fu) ^ magic;
  V w = __hsub2(*reinterpret_cast<const V*>(&biased), *reinterpret_cast<const V*>(&magic));
  return *reinterpret_cast<uint32_t*>(&w);
}

// Shared-memory plan.  Two rings: a deep one of load stages (packed weight tile + activation tile,
// filled by TMA; its depth sets how many bytes are in flight from HBM) and a short one of operand
// slots (dequantised weight tiles, 16 KB each, one per group of dequantising warps).
template <int LAYOUT, int BNX>
struct WqCfg {
  static constexpr int kRawBytes = LAYOUT == kW4N ? kWqBK * 64 : kWqBK * 128;
  static constexpr int kXBytes = BNX * 128;
  static constexpr int kLoadBytes = kRawBytes + kXBytes;
  static constexpr int kASlots = 4;
  static constexpr int kLoadWanted = (200 * 1024 - kASlots * kWqABytes) / kLoadBytes;
  static constexpr int kLoadStages = kLoadWanted > 16 ? 16 : kLoadWanted;
  static constexpr int kAOff = 0;
  static constexpr int kXOff = kASlots * kWqABytes;
  static constexpr int kRawOff = kXOff + kLoadStages * kXBytes;
  static constexpr int kBarOff = kRawOff + kLoadStages * kRawBytes;   // full[L], lfree[L], aready[A], afree[A], tfull, tempty
  static constexpr int kMiscOff = kBarOff + (2 * kLoadStages + 2 * kASlots + 2) * 8;
  static constexpr int kTotal = kMiscOff + 16;
  static constexpr int kDynamic = kTotal + 1024;
  static constexpr uint32_t kTmemCols = BNX < 32 ? 32 : BNX;
  static_assert(kLoadStages >= 2, "pipeline needs at least two load stages");
  static_assert(kDynamic <= 227 * 1024, "shared memory budget");
  static_assert(kDynamic > 116 * 1024 || kTmemCols <= 256, "TMEM budget with two resident CTAs");
};

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

// Dequantises one packed [64 k x 128 n] tile into the UMMA operand tile, using the GT threads of a
// warp group (thread index lg).  Packed words are fetched in batches of eight before any arithmetic
// so that the shared-memory latency and the dependent 16-bit operations of different items overlap.
template <int LAYOUT, typename XT, int GT>
__device__ __forceinline__ void dequant_tile(const uint8_t* __restrict__ raw, uint8_t* __restrict__ a_tile, int lg,
                                             const uint32_t (&sc2)[4], const uint32_t (&of2)[4], bool has_off,
                                             const WqParams& p, int64_t g, int64_t n_tile0) {
  constexpr int ITEMS = (kWqBK * 16) / GT;             // 8-value items per thread (1024 per tile)
  constexpr int BATCH = ITEMS < 8 ? ITEMS : 8;
  if constexpr (LAYOUT == kW4N) {
    const int wc = lg & 15;                            // 8-channel group inside the tile
    const uint32_t ng = wc >> 3, c = wc & 7;
    const uint32_t* raw32 = reinterpret_cast<const uint32_t*>(raw);
#pragma unroll
    for (int b0 = 0; b0 < ITEMS; b0 += BATCH) {
      uint32_t v[BATCH];
#pragma unroll
      for (int i = 0; i < BATCH; ++i) v[i] = raw32[((lg >> 4) + (GT / 16) * (b0 + i)) * 16 + wc];
#pragma unroll
      for (int i = 0; i < BATCH; ++i) {
        const int kr = (lg >> 4) + (GT / 16) * (b0 + i);
        uint32_t pr[4];
#pragma unroll
        for (int j = 0; j < 4; ++j)                    // halves of pr[j]: values j and j+4
          pr[j] = add_mul2<XT>(nibbles_to_x2<XT>(v[i] >> (4 * j)), of2[j], sc2[j], has_off);
        // Stored in the order (v0,v4,v1,v5,v2,v6,v3,v7): MMA row 8q+i of the tile holds channel
        // 8q + kW4RowPerm[i]; the epilogue undoes the permutation when it computes n.
        const uint32_t r = kr & 7;
        *reinterpret_cast<uint4*>(a_tile + ng * 8192 + (kr >> 3) * 1024 + r * 128 + ((c ^ r) << 4)) =
            make_uint4(pr[0], pr[1], pr[2], pr[3]);
      }
    }
  } else if constexpr (LAYOUT == kW8N) {
    const int wc = lg & 15;
    const uint32_t ng = wc >> 3, c = wc & 7;
    const uint2* raw64 = reinterpret_cast<const uint2*>(raw);
#pragma unroll
    for (int b0 = 0; b0 < ITEMS; b0 += BATCH) {
      uint2 v[BATCH];
#pragma unroll
      for (int i = 0; i < BATCH; ++i) v[i] = raw64[((lg >> 4) + (GT / 16) * (b0 + i)) * 16 + wc];
#pragma unroll
      for (int i = 0; i < BATCH; ++i) {
        const int kr = (lg >> 4) + (GT / 16) * (b0 + i);
        const uint32_t w2[2] = {v[i].x, v[i].y};
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 8; j += 2) {
          const float a = (float)(int8_t)(w2[j >> 2] >> (8 * (j & 3)));
          const float b = (float)(int8_t)(w2[j >> 2] >> (8 * ((j + 1) & 3)));
          o[j >> 1] = add_mul2<XT>(X2<XT>::pack(a, b), of2[j >> 1], sc2[j >> 1], has_off);
        }
        const uint32_t r = kr & 7;
        *reinterpret_cast<uint4*>(a_tile + ng * 8192 + (kr >> 3) * 1024 + r * 128 + ((c ^ r) << 4)) =
            make_uint4(o[0], o[1], o[2], o[3]);
      }
    }
  } else {
    const uint32_t c = lg & 7;                         // 8-wide k chunk inside the 64-deep block
    const uint2* raw64 = reinterpret_cast<const uint2*>(raw);
#pragma unroll
    for (int b0 = 0; b0 < ITEMS; b0 += BATCH) {
      uint2 v[BATCH];
      uint32_t s2[BATCH], o2[BATCH];
#pragma unroll
      for (int i = 0; i < BATCH; ++i) {
        const int nr = (lg >> 3) + (GT / 8) * (b0 + i);    // channel row inside the tile
        const int64_t n = n_tile0 + nr;
        const bool nv = n < p.n;
        const float scv = nv ? X2<XT>::to_float(static_cast<const XT*>(p.scale)[g * p.n + n]) : 0.0f;
        const float ofv = (nv && has_off) ? X2<XT>::to_float(static_cast<const XT*>(p.offset)[g * p.n + n]) : 0.0f;
        s2[i] = X2<XT>::pack(scv, scv);
        o2[i] = X2<XT>::pack(ofv, ofv);
        v[i] = raw64[nr * 8 + c];
      }
#pragma unroll
      for (int i = 0; i < BATCH; ++i) {
        const int nr = (lg >> 3) + (GT / 8) * (b0 + i);
        const uint32_t w2[2] = {v[i].x, v[i].y};
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 8; j += 2) {
          const float a = (float)(int8_t)(w2[j >> 2] >> (8 * (j & 3)));
          const float b = (float)(int8_t)(w2[j >> 2] >> (8 * ((j + 1) & 3)));
          o[j >> 1] = add_mul2<XT>(X2<XT>::pack(a, b), o2[i], s2[i], has_off);
        }
        const uint32_t r = nr & 7;
        *reinterpret_cast<uint4*>(a_tile + (nr >> 3) * 1024 + r * 128 + ((c ^ r) << 4)) =
            make_uint4(o[0], o[1], o[2], o[3]);
      }
    }
  }
}

template <int LAYOUT, typename XT, int BNX>
__global__ void __launch_bounds__(kWqThreads, 1)
wq_umma_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, const WqParams p) {
  using C = WqCfg<LAYOUT, BNX>;
  constexpr int LS = C::kLoadStages, AS = C::kASlots;
  constexpr bool A_MN = LAYOUT != kW8K;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem + C::kAOff;
  uint8_t* sX = smem + C::kXOff;
  uint8_t* sRaw = smem + C::kRawOff;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + C::kBarOff);
  uint64_t* lfree = full + LS;
  uint64_t* aready = lfree + LS;
  uint64_t* afree = aready + AS;
  uint64_t* tfull = afree + AS;
  uint64_t* tempty = tfull + 1;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(smem + C::kMiscOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + C::kMiscOff + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int i = 0; i < LS; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&lfree[i], 1);
    }
    for (int i = 0; i < AS; ++i) {
      mbar_init(&aready[i], kWqDeqWarps / (LS > AS ? AS : 2));
      mbar_init(&afree[i], 1);
    }
    mbar_init(tfull, 1);
    mbar_init(tempty, kWqDeqWarps);
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tensormap(&tmW);
    prefetch_tensormap(&tmX);
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, C::kTmemCols);
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
      for (int u = blockIdx.x; u < p.units && ok; u += gridDim.x) {
        const int tn = u % p.tiles_n, mc = u / p.tiles_n;
        for (int kb = 0; kb < p.kblocks; ++kb) {
          if (!mbar_wait(&lfree[stage], phase ^ 1, abort_flag, kDevTimeoutProducer)) { ok = false; break; }
          mbar_arrive_expect_tx(&full[stage], C::kRawBytes + C::kXBytes);
          if (LAYOUT == kW4N)        // bytes of packed nibbles: 64 bytes = 128 channels per row of k
            tma_load_2d(sRaw + stage * C::kRawBytes, &tmW, &full[stage], tn * 64, kb * kWqBK);
          else if (LAYOUT == kW8N)
            tma_load_2d(sRaw + stage * C::kRawBytes, &tmW, &full[stage], tn * kWqTileN, kb * kWqBK);
          else                       // k-contiguous: rows are channels
            tma_load_2d(sRaw + stage * C::kRawBytes, &tmW, &full[stage], kb * kWqBK, tn * kWqTileN);
          tma_load_2d(sX + stage * C::kXBytes, &tmX, &full[stage], kb * kWqBK, mc * BNX);
          if (++stage == LS) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok)
        for (int i = 0; i < 200; ++i) __nanosleep(1000);   // let copies in flight land before smem is released
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t fmt = sizeof(XT) == 2 && std::is_same<XT, __nv_bfloat16>::value ? 1u : 0u;
      constexpr uint32_t idesc = make_idesc(1 /*f32*/, fmt, fmt, A_MN ? 1 : 0, 0, kWqTileN, BNX);
      int stage = 0, slot = 0;
      uint32_t phase = 0, aphase = 0, tphase = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < p.units && ok; u += gridDim.x) {
        if (!mbar_wait(tempty, tphase ^ 1, abort_flag, kDevTimeoutMma)) { ok = false; break; }
        tc_fence_after();
        for (int kb = 0; kb < p.kblocks; ++kb) {
          if (!mbar_wait(&aready[slot], aphase, abort_flag, kDevTimeoutMma) ||
              !mbar_wait(&full[stage], phase, abort_flag, kDevTimeoutMma)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(sA + slot * kWqABytes), b_addr = smem_u32(sX + stage * C::kXBytes);
#pragma unroll
          for (int k16 = 0; k16 < kWqBK / 16; ++k16) {
            // MN-major A: 16 k = two 8-row groups of 1024 B; 64-channel groups 8192 B apart.
            // K-major A / B: 16 k = 32 bytes inside the 128-byte swizzle row; 8-row groups 1024 B apart.
            const uint64_t adesc = A_MN ? make_smem_desc(a_addr + k16 * 2048, 8192, 1024, kSwizzle128B)
                                        : make_smem_desc(a_addr + k16 * 32, 16, 1024, kSwizzle128B);
            const uint64_t bdesc = make_smem_desc(b_addr + k16 * 32, 16, 1024, kSwizzle128B);
#if !(defined(B200Q_DIAG) && (B200Q_DIAG & 2))
            umma_f16(tmem_base, adesc, bdesc, idesc, (kb > 0 || k16 > 0) ? 1u : 0u);
#endif
          }
          umma_commit(&afree[slot]);                     // operand slot may be overwritten ...
          umma_commit(&lfree[stage]);                    // ... and the load stage refilled
          if (++stage == LS) { stage = 0; phase ^= 1; }
          if (++slot == AS) { slot = 0; aphase ^= 1; }
        }
        if (!ok) break;
        umma_commit(tfull);
        tphase ^= 1;
      }
    }
  } else {
    // ------------------------------------------- dequantise, then epilogue
    // The sixteen warps form G groups; group g owns every G-th K block, so G tiles are being
    // dequantised at the same time and no warp waits for another inside a tile.  G stays below the
    // number of load stages: a group must never wait for a phase of a `full` barrier while that
    // barrier is still a whole phase behind (the parity test could not tell the two apart).
    constexpr int G = LS > AS ? AS : 2;
    constexpr int WG = kWqDeqWarps / G;                // warps per group
    constexpr int GT = WG * 32;                        // threads per group
    const int dw = warp - 2;                           // 0..15
    const int group = dw / WG;
    const int lg = (dw % WG) * 32 + lane;              // thread index inside the group
    const int quad = warp & 3;                         // TMEM lane quadrant of this warp
    const bool has_off = p.offset != nullptr;
    int it_base = 0;                                   // K blocks this CTA has been through before this tile
    uint32_t tphase = 0;
    bool ok = true;
    for (int u = blockIdx.x; u < p.units && ok; u += gridDim.x) {
      const int tn = u % p.tiles_n, mc = u / p.tiles_n;
      const int64_t n_tile0 = (int64_t)tn * kWqTileN;
      int64_t cur_group = -1;
      uint32_t sc2[4], of2[4];   // this thread's 8 channels as 16-bit pairs: kW4N (j, j+4), kW8N (2j, 2j+1)
      uint4 ns, no;              // parameters fetched ahead for the next K block of this group
      const int64_t n_oct0 = n_tile0 + (lg & 15) * 8;
      auto quant_group = [&](int kb) -> int64_t { return p.group_size > 0 ? ((int64_t)kb * kWqBK) / p.group_size : 0; };
      int kb = (group - it_base % G + G) % G;          // first K block of this tile owned by the group
      int64_t g_next = quant_group(kb);
      if (LAYOUT != kW8K && kb < p.kblocks) fetch_params8<XT>(p, g_next, n_oct0, ns, no);
      for (; kb < p.kblocks; kb += G) {
        const int it = it_base + kb;
        const int stage = it % LS;
        const uint32_t phase = (uint32_t)(it / LS) & 1u;
        const int slot = it % AS;
        const uint32_t aphase = (uint32_t)(it / AS) & 1u;
        const int64_t g = g_next;
        if (LAYOUT != kW8K) {
          if (g != cur_group) {
            cur_group = g;
            pair_params8<LAYOUT>(ns, no, sc2, of2);
          }
          if (kb + G < p.kblocks) {                    // loads for the group's next K block fly during this one
            g_next = quant_group(kb + G);
            if (g_next != g) fetch_params8<XT>(p, g_next, n_oct0, ns, no);
          }
        } else if (kb + G < p.kblocks) {
          g_next = quant_group(kb + G);
        }
        // warp-uniform decision, so that the warp stays converged for __syncwarp below
        const bool got = __all_sync(0xffffffffu, mbar_wait(&full[stage], phase, abort_flag, kDevTimeoutEpilogue) &&
                                                     mbar_wait(&afree[slot], aphase ^ 1, abort_flag, kDevTimeoutEpilogue));
        if (!got) { ok = false; break; }
#if !(defined(B200Q_DIAG) && (B200Q_DIAG & 1))
        dequant_tile<LAYOUT, XT, GT>(sRaw + stage * C::kRawBytes, sA + slot * kWqABytes, lg, sc2, of2, has_off, p, g,
                                     n_tile0);
#endif
        fence_proxy_async_smem();                      // generic-proxy stores -> visible to the MMA (async proxy)
        __syncwarp();
        if (lane == 0) mbar_arrive(&aready[slot]);
      }
      it_base += p.kblocks;
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
      // -------- epilogue: rows are channels, columns are tokens; four warps share a lane quadrant
      {
        constexpr int CH = BNX < 32 ? 16 : 32;
        constexpr int kChunks = BNX / CH;
        constexpr int kShare = kWqDeqWarps / 4;        // warps sharing one TMEM lane quadrant
        const int share = dw >> 2;                     // this warp's slot among them
        const int row = quad * 32 + lane;              // accumulator row = TMEM lane
        const int64_t n = n_tile0 + (LAYOUT == kW4N ? w4_row_to_channel(row) : row);
        const bool nv = n < p.n;
        const float bias = (nv && p.bias) ? X2<XT>::to_float(static_cast<const XT*>(p.bias)[n]) : 0.0f;
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
#pragma unroll 1
        for (int c = share; c < kChunks; c += kShare) {
          uint32_t r[CH];
          __syncwarp();
          if constexpr (CH == 32) tmem_ld_x32(taddr + c * CH, r);
          else tmem_ld_x16(taddr + c * CH, r);
          tmem_ld_wait();
          if (nv) {
#pragma unroll
            for (int j = 0; j < CH; ++j) {
              const int64_t mm = (int64_t)mc * BNX + c * CH + j;
              if (mm < p.m) {
                float v = __uint_as_float(r[j]);
                if (p.bias) v = __fadd_rn(v, bias);
                static_cast<XT*>(p.out)[mm * p.n + n] = X2<XT>::from_float(v);
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
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

template <int LAYOUT, typename XT, int BNX>
int launch_wq(const CUtensorMap& tmW, const CUtensorMap& tmX, const WqParams& p, cudaStream_t st) {
  using C = WqCfg<LAYOUT, BNX>;
  auto kern = wq_umma_kernel<LAYOUT, XT, BNX>;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kDynamic);
    if (err != cudaSuccess)
      return fail(B200Q_ERR_LAUNCH, "weight_quant_matmul: cudaFuncSetAttribute: %s", cudaGetErrorString(err));
    configured[dev] = true;
  }
  const int grid = p.units < sm_count() ? p.units : sm_count();
  kern<<<grid, kWqThreads, C::kDynamic, st>>>(tmW, tmX, p);
  return check_launch("weight_quant_matmul (tcgen05)");
}

template <int LAYOUT, typename XT>
int dispatch_bnx(int bnx, const CUtensorMap& tmW, const CUtensorMap& tmX, const WqParams& p, cudaStream_t st) {
  switch (bnx) {
    case 16: return launch_wq<LAYOUT, XT, 16>(tmW, tmX, p, st);
    case 32: return launch_wq<LAYOUT, XT, 32>(tmW, tmX, p, st);
    case 64: return launch_wq<LAYOUT, XT, 64>(tmW, tmX, p, st);
    case 128: return launch_wq<LAYOUT, XT, 128>(tmW, tmX, p, st);
    default: return launch_wq<LAYOUT, XT, 256>(tmW, tmX, p, st);
  }
}

template <typename XT>
int dispatch_layout(int layout, int bnx, const CUtensorMap& tmW, const CUtensorMap& tmX, const WqParams& p,
                    cudaStream_t st) {
  switch (layout) {
    case kW4N: return dispatch_bnx<kW4N, XT>(bnx, tmW, tmX, p, st);
    case kW8N: return dispatch_bnx<kW8N, XT>(bnx, tmW, tmX, p, st);
    default: return dispatch_bnx<kW8K, XT>(bnx, tmW, tmX, p, st);
  }
}

}  // namespace
}  // namespace b200q

extern "C" size_t b200q_weight_quant_matmul_workspace_bytes(int64_t, int64_t, int64_t, int) { return 0; }

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
                     aligned(a->weight, 16) && aligned(a->antiquant_scale, 16) &&
                     (a->antiquant_offset == nullptr || aligned(a->antiquant_offset, 16)) &&
                     (a->group_size == 0 || a->group_size % kWqBK == 0) && a->k < (1LL << 31) && a->n < (1LL << 31);
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

  const int bnx = a->m <= 16 ? 16 : a->m <= 32 ? 32 : a->m <= 64 ? 64 : a->m <= 128 ? 128 : 256;
  p.tiles_n = (int)ceil_div(a->n, kWqTileN);
  p.m_chunks = (int)ceil_div(a->m, bnx);
  p.kblocks = (int)ceil_div(a->k, kWqBK);
  const int64_t units = (int64_t)p.tiles_n * p.m_chunks;
  B200Q_REQUIRE(units < (1LL << 31), B200Q_ERR_UNSUPPORTED, "weight_quant_matmul: too many tiles");
  p.units = (int)units;

  CUtensorMap tmW, tmX;
  int rc;
  if (layout == kW4N)
    rc = make_tmap_2d(&tmW, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a->weight, a->n / 2, a->k, a->n / 2, 64, kWqBK,
                      CU_TENSOR_MAP_SWIZZLE_NONE, "weight_quant_matmul (int4 weight)");
  else if (layout == kW8N)
    rc = make_tmap_2d(&tmW, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a->weight, a->n, a->k, a->w_stride_k, kWqTileN, kWqBK,
                      CU_TENSOR_MAP_SWIZZLE_NONE, "weight_quant_matmul (int8 weight)");
  else
    rc = make_tmap_2d(&tmW, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a->weight, a->k, a->n, a->w_stride_n, kWqBK, kWqTileN,
                      CU_TENSOR_MAP_SWIZZLE_NONE, "weight_quant_matmul (int8 weight)");
  if (rc) return rc;
  rc = make_tmap_2d(&tmX, a->x_dtype == B200Q_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                    2, a->x, a->k, a->m, a->k * 2, kWqBK, bnx, CU_TENSOR_MAP_SWIZZLE_128B,
                    "weight_quant_matmul (activations)");
  if (rc) return rc;
  if (a->x_dtype == B200Q_BF16) return dispatch_layout<__nv_bfloat16>(layout, bnx, tmW, tmX, p, st);
  return dispatch_layout<__half>(layout, bnx, tmW, tmX, p, st);
}
