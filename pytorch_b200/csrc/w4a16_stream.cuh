// W4A16 for a few tokens (decode): the int4-packed weight streamed from HBM exactly once, in one
// launch, with no shared-memory staging of the weight and no pipeline hand-offs.
//
// Included by w4a16_gemm.cu after its dequantisation helpers (X2, nibbles_to_x2, add_mul2,
// fetch_params8, pair_params8) and WqParams.
//
// Every warp is on its own.  Per 32-deep K block it loads, per lane, eight k rows (k = 8 * tig + r)
// of two consecutive packed words (16 channels): eight lanes side by side read 64 contiguous bytes
// of a row, and one L2 prefetch per lane, a few blocks ahead, covers the warp's 32 rows.  A packed
// word holds eight channels at ONE k, and the 16-bit expansion of a word (mask, exponent-bias trick)
// yields registers that hold the channel pair (j, j+4) at one k, while a warp-level MMA operand
// register wants one channel at two consecutive k: one byte-permute per expanded register regroups
// them.  The dequantised values are bit-identical to the tcgen05 kernel's ((w + offset) * scale in
// the activation dtype, two roundings).  The MMA's k slots are a fixed permutation of the 32-deep
// block, the same for the weight and the token operand, so the activations are read with one
// 16-byte load per lane and token group.  Tokens sit on the N axis of mma.m16n8k16 (eight per MMA),
// channels on the M axis.
// K is split over the warps of a CTA and, when the column strips alone would leave SMs idle, over
// the CTAs of a cluster; partial sums meet in shared memory (distributed shared memory across the
// cluster) and are added in a fixed order: the result does not depend on timing.  The only
// inter-CTA synchronisation is the hardware cluster barrier.
//
// What bounds it: the expansion costs about five half-rate instructions per two weights (shift,
// three-input logic op, subtract, add offset, multiply by scale) and a byte-permute, so the kernel
// is bound by instruction issue, not by HBM.  Variants tried and measured no faster: keeping the
// expanded registers unpermuted and separating channel j from j+4 with two MMAs whose token operand
// has every second k slot zeroed; four packed words per lane (128-byte row pieces); a second K
// block in registers.
#pragma once

#include <mutex>

namespace b200q {
namespace {

constexpr int kWsWarps = 4;           // warps per CTA, each on its own K range
constexpr int kWsKBlock = 32;         // k rows per loop iteration

template <typename XT>
__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
  if constexpr (std::is_same<XT, __nv_bfloat16>::value) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  } else {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
}

template <int WL>
struct WsRow { uint32_t w[WL]; };

template <int WL>
__device__ __forceinline__ WsRow<WL> ws_load_row(const uint32_t* p) {
  static_assert(WL == 2, "two packed words per lane and row");
  WsRow<WL> r;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(r.w[0]), "=r"(r.w[1]) : "l"(p));
  return r;
}

// 64-bit pointer plus an unsigned 32-bit byte offset, as one wide multiply-add (off * 1 + p).
__device__ __forceinline__ const uint32_t* add_u32(const char* p, uint32_t off) {
  uint64_t r;
  asm("mad.wide.u32 %0, %1, 1, %2;" : "=l"(r) : "r"(off), "l"(reinterpret_cast<uint64_t>(p)));
  return reinterpret_cast<const uint32_t*>(r);
}

// Accumulator register of lane (gid, tig) that holds token tl of the CTA's token block and channel cl
// of its column strip.  The inverse of the operand arrangement described above.
template <int MT, int WL>
__device__ __forceinline__ void ws_locate(int tl, int cl, int& lane, int& reg) {
  const int gid = cl / (WL * 8), word = (cl % (WL * 8)) >> 3, nib = cl & 7;
  const int t = nib & 3, hi = nib >> 2, mt = tl >> 3, tig = (tl & 7) >> 1, odd = tl & 1;
  lane = gid * 4 + tig;
  reg = (((word * 4 + t) * MT + mt) * 4) + hi * 2 + odd;
}

template <typename XT, int MT, bool HAS_OFF>
struct WsCfg {
  static constexpr int kWords = 2;                                     // packed words per lane and k row
  static constexpr int kAcc = kWords * 16 * MT;                        // fp32 accumulators per lane
  static constexpr int kMinCtas = MT == 1 ? 5 : 4;                     // resident CTAs per SM the register budget aims at
  static constexpr int kRedBytes = kWsWarps * kAcc * 32 * 4;           // every warp's accumulators
  static constexpr int kFinBytes = kAcc * 32 * 4;                      // their sum (read by the cluster)
  static constexpr int kDynamic = kRedBytes + kFinBytes;
  static constexpr int kPrefetchAhead = 2;                             // K blocks ahead of the loads
};

template <typename XT, int MT, bool HAS_OFF>
__global__ void __launch_bounds__(kWsWarps * 32, WsCfg<XT, MT, HAS_OFF>::kMinCtas)
wq_stream_kernel(const XT* __restrict__ x, const uint32_t* __restrict__ w, const WqParams p, const int ksplit) {
  using C = WsCfg<XT, MT, HAS_OFF>;
  constexpr int WL = C::kWords;
  constexpr int AC = C::kAcc;
  extern __shared__ __align__(16) float ws_smem[];
  float* red = ws_smem;                        // [warp][reg][lane]
  float* fin = ws_smem + kWsWarps * AC * 32;   // [reg][lane]

  const int lane = threadIdx.x & 31, wi = threadIdx.x >> 5;
  const int gid = lane >> 2, tig = lane & 3;
  const int rank = ksplit > 1 ? (int)cluster_ctarank() : 0;
  const int strip = blockIdx.x / ksplit;
  const int wpr = (int)(p.n >> 3);                                   // packed words per k row
  // Lanes beyond the last channel read the last WL words of the row instead; their sums are never stored.
  const int wcol_true = strip * (WL * 8) + gid * WL;
  const int wcol = wcol_true + WL <= wpr ? wcol_true : wpr - WL;
  const int64_t nbase = (int64_t)wcol * 8;                           // first channel of this lane
  const int bpg = (int)((p.group_size > 0 ? p.group_size : p.k) / kWsKBlock);   // K blocks per scale group

  // K blocks of this warp: an equal contiguous share of the k / 32 blocks.
  const int nblocks = (int)(p.k / kWsKBlock);
  const int kw = rank * kWsWarps + wi, kparts = ksplit * kWsWarps;
  const int it0 = (int)((int64_t)kw * nblocks / kparts), it1 = (int)((int64_t)(kw + 1) * nblocks / kparts);

  const uint32_t row_bytes = (uint32_t)wpr * 4u;
  const char* wp = reinterpret_cast<const char*>(w + (int64_t)(8 * tig) * wpr + wcol) + (int64_t)it0 * kWsKBlock * row_bytes;
  uint32_t roff[8];                                                  // byte offsets of this lane's eight k rows
#pragma unroll
  for (int r = 0; r < 8; ++r) roff[r] = (uint32_t)r * row_bytes;
  // L2 prefetch: one line per lane covers the warp's 32 rows of a K block.
  const int pcol = strip * (WL * 8) + WL * 8 <= wpr ? strip * (WL * 8) : wpr - WL * 8 > 0 ? wpr - WL * 8 : 0;
  const char* pp = reinterpret_cast<const char*>(w + (int64_t)lane * wpr + pcol) +
                   (int64_t)(it0 + C::kPrefetchAhead) * kWsKBlock * row_bytes;
  // Tokens beyond m read token 0; their sums are never stored.
  const char* xp[MT];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
    xp[mt] = reinterpret_cast<const char*>(x + (int64_t)(mt * 8 + gid < p.m ? mt * 8 + gid : 0) * p.k + 8 * tig +
                                           (int64_t)it0 * kWsKBlock);

  float acc[AC / 4][4];
#pragma unroll
  for (int i = 0; i < AC / 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

  uint32_t sc2[WL][4], of2[WL][4];
#pragma unroll
  for (int q = 0; q < WL; ++q)
#pragma unroll
    for (int t = 0; t < 4; ++t) { sc2[q][t] = 0u; of2[q][t] = 0u; }
  int g = it0 / bpg;                          // scale group of the block about to be computed
  int g_left = 0;                             // blocks left before the next group's parameters are due

  WsRow<WL> cur[8];
  uint4 xcur[MT];
  // Loads the block wp / xp point at.
  auto load_block = [&](WsRow<WL> (&rows)[8], uint4 (&xs)[MT]) {
#pragma unroll
    for (int r = 0; r < 8; ++r) rows[r] = ws_load_row<WL>(add_u32(wp, roff[r]));
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) xs[mt] = __ldg(reinterpret_cast<const uint4*>(xp[mt]));
  };
  // Prefetches the block kPrefetchAhead after block `it`, if this warp will read it.
  auto prefetch_block = [&](int it) {
    if (it + C::kPrefetchAhead < it1) prefetch_l2(pp);
  };
  auto advance = [&]() {
    wp += (int64_t)kWsKBlock * row_bytes;
    pp += (int64_t)kWsKBlock * row_bytes;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) xp[mt] += kWsKBlock * 2;
  };
  // One expanded register: channels (t, t+4) of packed word `word` at one k, dequantised.
  auto expand = [&](uint32_t word, int q, int t) -> uint32_t {
    return add_mul2<XT, HAS_OFF>(nibbles_to_x2<XT>(word >> (4 * t)), of2[q][t], sc2[q][t]);
  };
  auto compute_block = [&](const WsRow<WL> (&rows)[8], const uint4 (&xs)[MT]) {
    if (g_left == 0) {                                                 // warp-uniform
#pragma unroll
      for (int q = 0; q < WL; ++q) {
        uint4 s, o;
        fetch_params8<XT>(p, g, nbase + q * 8, s, o);
        pair_params8<kW4N>(s, o, sc2[q], of2[q]);
      }
      g_left = bpg;
      ++g;
    }
    --g_left;
#pragma unroll
    for (int s = 0; s < 2; ++s) {                                      // k rows 4s .. 4s+3 of this lane
      uint32_t b0[MT], b1[MT];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        b0[mt] = s == 0 ? xs[mt].x : xs[mt].z;
        b1[mt] = s == 0 ? xs[mt].y : xs[mt].w;
      }
#pragma unroll
      for (int q = 0; q < WL; ++q)
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const uint32_t c0 = expand(rows[4 * s].w[q], q, t), c1 = expand(rows[4 * s + 1].w[q], q, t);
          const uint32_t c2 = expand(rows[4 * s + 2].w[q], q, t), c3 = expand(rows[4 * s + 3].w[q], q, t);
          // rows of A: channel t (rows 0-7 of the MMA), channel t+4 (rows 8-15); columns: (k, k+1) pairs
          const uint32_t a0 = __byte_perm(c0, c1, 0x5410), a1 = __byte_perm(c0, c1, 0x7632);
          const uint32_t a2 = __byte_perm(c2, c3, 0x5410), a3 = __byte_perm(c2, c3, 0x7632);
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) mma_16816<XT>(acc[(q * 4 + t) * MT + mt], a0, a1, a2, a3, b0[mt], b1[mt]);
        }
    }
  };

  if (it0 < it1) {
    // The first block of a warp may start inside a scale group.
    g_left = 0;
    const int into = it0 - g * bpg;                                    // blocks of group g already behind it0
    // Blocks it0 .. it0 + kPrefetchAhead - 1 are fetched by the plain loads' own misses.
    bool first = true;
    for (int it = it0; it < it1; ++it) {
      prefetch_block(it);
      load_block(cur, xcur);
      compute_block(cur, xcur);
      if (first) { g_left = bpg - into - 1; first = false; }
      advance();
    }
  }
  // The warps' partial sums, then the CTA's, then the cluster's: always in index order.
#pragma unroll
  for (int i = 0; i < AC / 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) red[(wi * AC + i * 4 + j) * 32 + lane] = acc[i][j];
  __syncthreads();
  for (int idx = threadIdx.x; idx < AC * 32; idx += kWsWarps * 32) {
    float s = red[idx];
#pragma unroll
    for (int v = 1; v < kWsWarps; ++v) s = __fadd_rn(s, red[v * AC * 32 + idx]);
    fin[idx] = s;
  }
  if (ksplit > 1) cluster_sync_all(); else __syncthreads();

  // Items of eight consecutive channels of one token; the CTAs of a cluster share them out.
  constexpr int kItems = MT * 8 * WL * 8;
  const uint32_t fin_addr = smem_u32(fin);
  for (int item = threadIdx.x * ksplit + rank; item < kItems; item += kWsWarps * 32 * ksplit) {
    const int tl = item / (WL * 8), c8 = item % (WL * 8);
    const int64_t n0 = (int64_t)strip * (WL * 64) + c8 * 8;
    if (tl < p.m && n0 < p.n) {
      float v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        int ln, rg;
        ws_locate<MT, WL>(tl, c8 * 8 + j, ln, rg);
        const uint32_t off = (uint32_t)(rg * 32 + ln) * 4u;
        if (ksplit > 1) {
          float s = __uint_as_float(ld_shared_cluster_u32(map_to_cta(fin_addr + off, 0)));
          for (int r = 1; r < ksplit; ++r)
            s = __fadd_rn(s, __uint_as_float(ld_shared_cluster_u32(map_to_cta(fin_addr + off, (uint32_t)r))));
          v[j] = s;
        } else {
          v[j] = fin[rg * 32 + ln];
        }
      }
      if (p.bias) {
        const uint4 b = __ldg(reinterpret_cast<const uint4*>(static_cast<const XT*>(p.bias) + n0));
        const XT* bv = reinterpret_cast<const XT*>(&b);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = __fadd_rn(v[j], X2<XT>::to_float(bv[j]));
      }
      *reinterpret_cast<uint4*>(static_cast<XT*>(p.out) + (int64_t)tl * p.n + n0) =
          make_uint4(X2<XT>::pack(v[0], v[1]), X2<XT>::pack(v[2], v[3]), X2<XT>::pack(v[4], v[5]),
                     X2<XT>::pack(v[6], v[7]));
    }
  }
  if (ksplit > 1) cluster_sync_all();                                  // nobody leaves while its sums are being read
}

// CTAs of this kernel that fit on the device at once (per-device cache).
template <auto Kern>
int ws_resident_ctas(int dynamic_smem) {
  static std::mutex mu;
  static int cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return sm_count();
  std::lock_guard<std::mutex> lock(mu);
  if (cached[dev] == 0) {
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, Kern, kWsWarps * 32, dynamic_smem) != cudaSuccess || per_sm <= 0) {
      cudaGetLastError();
      per_sm = 1;
    }
    cached[dev] = per_sm * sm_count();
  }
  return cached[dev];
}

// Cluster size along K (1..8): the one whose CTAs fill the resident slots best, counting whole rounds;
// ties go to the smaller cluster.  A warp keeps at least two K blocks.
inline int ws_pick_ksplit(int strips, int nblocks, int slots) {
  int best = 1;
  double best_eff = 0.0;
  for (int ks = 1; ks <= 8; ++ks) {
    if (ks > 1 && nblocks < kWsWarps * ks * 2) break;
    const int64_t ctas = (int64_t)strips * ks;
    const int64_t rounds = (ctas + slots - 1) / slots;
    const double eff = (double)ctas / (double)(rounds * slots);
    if (eff > best_eff + 0.02) { best_eff = eff; best = ks; }
  }
  return best;
}

template <typename XT, int MT, bool HAS_OFF>
int launch_wq_stream(const void* x, const void* w, const WqParams& p, cudaStream_t st) {
  using C = WsCfg<XT, MT, HAS_OFF>;
  constexpr auto kern = wq_stream_kernel<XT, MT, HAS_OFF>;
  if (int rc = ensure_dynamic_smem<kern>(C::kDynamic, "weight_quant_matmul")) return rc;
  const int strips = (int)ceil_div(p.n, (int64_t)C::kWords * 64);
  const int nblocks = (int)(p.k / kWsKBlock);
  int ksplit = ws_pick_ksplit(strips, nblocks, ws_resident_ctas<kern>(C::kDynamic));
  if (const char* env = getenv("B200Q_WQ_KSPLIT")) {                  // tuning override
    const int v = atoi(env);
    if (v >= 1 && v <= 8) ksplit = v;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(strips * ksplit));
  cfg.blockDim = dim3(kWsWarps * 32);
  cfg.dynamicSmemBytes = C::kDynamic;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)ksplit;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t err = cudaLaunchKernelEx(&cfg, kern, static_cast<const XT*>(x), static_cast<const uint32_t*>(w), p, ksplit);
  if (err != cudaSuccess) return fail(B200Q_ERR_LAUNCH, "weight_quant_matmul (streaming): %s", cudaGetErrorString(err));
  return check_launch("weight_quant_matmul (streaming)");
}

constexpr int kWsMaxTokens = 16;

// One or two token groups of eight.
template <typename XT>
int dispatch_wq_stream(const void* x, const void* w, const WqParams& p, cudaStream_t st) {
  if (p.m <= 8) return p.offset ? launch_wq_stream<XT, 1, true>(x, w, p, st) : launch_wq_stream<XT, 1, false>(x, w, p, st);
  return p.offset ? launch_wq_stream<XT, 2, true>(x, w, p, st) : launch_wq_stream<XT, 2, false>(x, w, p, st);
}

}  // namespace
}  // namespace b200q
