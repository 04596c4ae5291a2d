// NVFP4 GEMM for sm_100a on CTA pairs: out[m,n] = epilogue(alpha * sum_k A[m,k] * W[n,k]).
//
// Same contract as the 1-CTA kernel in gemm_nvfp4.cu; this is the large-M path. Two CTAs of a
// (2,1,1) cluster compute one 256x256 output tile with tcgen05.mma.cta_group::2: each CTA
// loads its own 128 rows of A and its own 128-row half of the W tile, the leader CTA issues
// the MMAs, and each CTA ends up with its 128x256 slice of the accumulator in its own TMEM.
// Against the 1-CTA tile this cuts the shared-memory fill per SM and K tile from 54 KB to
// 38 KB, which is what lets five stages cover the load latency. No TMA multicast is used:
// the only cluster-wide operations are tcgen05.commit arrivals and remote mbarrier arrivals.
//
// Per CTA, 320 threads:
//   warp 0     TMA producer (tensor-map loads of A, W-half, the CTA's scale atoms of A and the
//              scale atoms of the whole W tile; bytes are counted on the LEADER's stage barrier)
//   warp 1     TMEM owner; in the leader one lane issues scale copies smem->TMEM and MMAs for
//              both CTAs, frees stages in both CTAs with a multicast commit
//   warps 2-9  epilogue: TMEM -> registers -> alpha/bias/GELU/gated residual -> bf16 -> swizzled
//              shared staging -> TMA store (one store per destination: local output and peers)
// TMEM (512 columns): two 256-column accumulators at columns 0 and 192 that overlap in
// [192,256); the epilogue reads the overlapping 64 columns first and then releases the next
// tile's MMA, so the drain of tile i runs under the main loop of tile i+1. Scale factors sit
// in columns [448,496).
// Every mbarrier wait is bounded (see ptx.cuh); a wait that gives up raises the CTA's abort
// flag, every role falls through to the tear-down, and the host reads the status word.
#include <cuda_bf16.h>
#include <cstdint>
#include <cstdlib>

#include "epilogue.cuh"
#include "internal.h"
#include "ptx.cuh"
#include "quant_dev.cuh"

namespace tnf {

namespace pair {
constexpr int kThreads = 320;  // producer warp, MMA warp, 8 epilogue warps
// Which warps take which role. The epilogue warp with index e reads TMEM lane quarter (warp id & 3).
#ifdef TNF_ROLES_LAST  // experiment: producer and MMA issuer in the last two warps instead of the first two
constexpr int kProducerWarp = 8, kMmaWarp = 9, kFirstEpilogueWarp = 0;
#else
constexpr int kProducerWarp = 0, kMmaWarp = 1, kFirstEpilogueWarp = 2;
#endif
constexpr int kStagingBytes = 8 * 4096;  // 8 epilogue warps x (32 rows x 128 B)
constexpr int kBiasBytes = 8 * 256;      // 8 epilogue warps x 64 f32 bias values (the column group being processed)
constexpr int kLutBytes = 512;           // 1/(scale*g) per E4M3 code for the quantising epilogue
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kAccStride = 192;  // accumulator b starts at column b * 192
constexpr uint32_t kSfaCol = 448, kSfbCol = 464;
}  // namespace pair

// KB = 64-element K blocks (one MMA each) per pipeline stage. 4 is what the library uses: five 38 KB stages of
// 256 K elements (128-byte swizzled rows). Ten 19 KB stages of 128 K elements (KB = 2) hold the same bytes
// but were measured 45 % slower on B200 (98 against 67 us on 4352 x 3072 x 9216): the fixed cost per stage
// (barrier round trip, twelve scale copies, commit) does not shrink with the stage.
template <int KB>
struct PairCfg {
  static constexpr int kStages = KB == 4 ? 5 : 10;
  static constexpr int kRowBytes = KB * 32;             // packed E2M1 bytes per operand row and stage
  static constexpr int kABytes = 128 * kRowBytes;       // this CTA's 128 rows of A
  static constexpr int kBBytes = 128 * kRowBytes;       // this CTA's half of the 256-row W tile
  static constexpr int kSfaBytes = 512 * KB;            // KB atoms: 128 rows x 4 blocks each
  static constexpr int kSfbBytes = 2 * 512 * KB;        // two 128-row groups
  static constexpr int kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;
  static constexpr int kSmemBytes = kStages * kStageBytes + pair::kStagingBytes + pair::kBiasBytes + pair::kLutBytes + 1024 + 256;
  static constexpr int kSfSlots = KB == 4 ? 1 : 2;      // scale-factor slots in TMEM
  static_assert(kSmemBytes <= 227 * 1024, "shared memory overflow");
};
template <int KB>
__device__ __forceinline__ uint64_t make_desc_operand(uint32_t saddr) {
  // K-major rows of KB*32 bytes, swizzle = row width; SBO = 8 rows
  constexpr uint64_t kLayout = KB == 4 ? 2 : 4;  // SWIZZLE_128B : SWIZZLE_64B
  return uint64_t((saddr & 0x3FFFFu) >> 4) | (uint64_t(1) << 16) | (uint64_t((8 * KB * 32) >> 4) << 32) | (uint64_t(1) << 46) |
         (kLayout << 61);
}

__device__ __forceinline__ uint64_t desc64(uint32_t lo, uint32_t hi) { return (uint64_t(hi) << 32) | lo; }

struct PairOutMaps {
  CUtensorMap m[kMaxPeers];
};

// One warp's 32 rows x 64 columns: accumulator registers -> bf16 rows in the swizzled staging
// buffer (128 bytes per row; 16-byte chunk j of row `lane` lands at chunk j ^ (lane & 7)).
template <bool kGelu, bool kChain, bool kGate, bool kQuant>
__device__ __forceinline__ void epilogue_pair_math(const uint32_t (&r)[64], const GemmParams& p, uint32_t row, uint32_t ncol0,
                                                   uint8_t* buf_gen, const float* bias_smem, const float* lut, int lane,
                                                   uint8_t* stage_q, uint32_t gq) {
  const bool row_ok = row < p.m;
  const float alpha = (kGelu && !kChain) ? 0.5f * p.alpha : p.alpha;  // the fused GELU works on x/2
  // NVFP4 copy of this row's 64 columns: 32 code bytes + 4 scale bytes. Each 16-byte group of codes
  // is stored as soon as it is complete, so only four code words are live beside the accumulators
  // (holding all eight spilled, and the spill reloads, not the math, cost ~30 us on the MLP-up shape).
  const bool q_on = kQuant && row_ok && ncol0 < p.n;  // n % 64 == 0: the whole group is in range
  const uint32_t qcol = p.n_offset + ncol0;  // the copy is an [m, ldo] operand; this launch fills n_offset .. n_offset + n
  uint32_t cw[4], sw = 0;
  uint4 prev = make_uint4(0, 0, 0, 0);
#pragma unroll
  for (int sub = 0; sub < 2; ++sub) {
    uint4 g4[4], s4[4];
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) {  // global loads first so that their latencies overlap
      const uint32_t nc = ncol0 + (sub * 4 + jj) * 8;
      g4[jj] = s4[jj] = make_uint4(0, 0, 0, 0);
      if (kGate && nc < p.n) {
        g4[jj] = __ldg(reinterpret_cast<const uint4*>(p.gate + nc));
        if (row_ok) s4[jj] = __ldg(reinterpret_cast<const uint4*>(p.residual + uint64_t(row) * p.n + nc));
      }
    }
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) {
      const int j = sub * 4 + jj;
      const uint4 o = epilogue8<kGelu, kChain, kGate>(&r[j * 8], alpha, bias_smem + j * 8, g4[jj], s4[jj]);  // broadcast reads
      if (!kQuant || p.store_bf16)  // with only the NVFP4 copy wanted, the bf16 rows are never staged
        *reinterpret_cast<uint4*>(buf_gen + lane * 128 + ((j ^ (lane & 7)) << 4)) = o;
      if (kQuant) {  // quantise the bf16-ROUNDED values, 16 columns at a time
        if (jj & 1) {
          const uint32_t w[8] = {prev.x, prev.y, prev.z, prev.w, o.x, o.y, o.z, o.w};
          uint32_t lo, hi;
          const uint32_t sc = quant_block16_bf16(w, lut, p.q_inv_t, lo, hi);
          cw[jj - 1] = lo;
          cw[jj] = hi;
          sw |= sc << (8 * (j >> 1));
        } else {
          prev = o;
        }
      }
    }
    if (kQuant && stage_q) {
      // multicast output: this row's 16 code bytes go to the CTA's staging tile (128 rows x 128 bytes, 16-byte
      // chunks XOR-swizzled by the row) and leave later as whole 128-byte row segments
      const uint32_t lr = row & 127u, c = gq * 2u + uint32_t(sub);
      *reinterpret_cast<uint4*>(stage_q + lr * 128u + ((c ^ (lr & 7u)) << 4)) = make_uint4(cw[0], cw[1], cw[2], cw[3]);
    } else if (q_on && !(kDiag && (p.diag & 128u))) {
      const uint64_t off = uint64_t(row) * (p.ldo >> 1) + (qcol >> 1) + sub * 16;
      const uint4 v = make_uint4(cw[0], cw[1], cw[2], cw[3]);
      if (p.q_codes_mc) multimem_st_v4(p.q_codes_mc + off, v);  // every rank's copy of the operand, this one included
      else *reinterpret_cast<uint4*>(p.q_codes + off) = v;
    }
  }
  if (kQuant && stage_q) {
    // the scale word into the staged copy of this 64-column group's 512-byte atom; rows past m hold zero scales
    const uint32_t lr = row & 127u;
    *reinterpret_cast<uint32_t*>(stage_q + 16384u + gq * 512u + (lr & 31u) * 16u + (lr >> 5) * 4u) = row_ok ? sw : 0u;
  } else if (q_on && !(kDiag && (p.diag & 128u))) {
    const uint64_t off = sf_device_offset(row, qcol >> 4, p.q_k_atoms);
    if (p.q_scales_mc) multimem_st_b32(p.q_scales_mc + off, sw);
    else *reinterpret_cast<uint32_t*>(p.q_scales + off) = sw;
  }
}

// SwiGLU pairwise gating (thinfer-core/src/ops/silu_mul.rs: out = silu(a) * b, silu(v) = v / (1 + exp(-v))) on a
// GEMM over the row-interleaved weight [W1 row 0, W3 row 0, W1 row 1, ...]: accumulator columns 2j and 2j+1 are
// a[j] and b[j], one output column. One warp's 32 rows x 64 accumulator columns -> 32 bf16 per row, staged as
// dense 64-byte rows (no swizzle) for a 32-column TMA store. Chain mode rounds a and b to bf16 first, as the
// reference's two matmul dispatches do.
template <bool kChain>
__device__ __forceinline__ void epilogue_pair_swiglu(const uint32_t (&r)[64], const GemmParams& p, uint8_t* buf_gen,
                                                     const float* bias_smem, int lane) {
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float4 bl = *reinterpret_cast<const float4*>(bias_smem + j * 8), bh = *reinterpret_cast<const float4*>(bias_smem + j * 8 + 4);
    const float bv[8] = {bl.x, bl.y, bl.z, bl.w, bh.x, bh.y, bh.z, bh.w};
    float o[4];
#pragma unroll
    for (int h = 0; h < 4; ++h) {
      float a, b;
      if (kChain) {
        a = bf16r(bf16r(__uint_as_float(r[j * 8 + 2 * h]) * p.alpha) + bv[2 * h]);
        b = bf16r(bf16r(__uint_as_float(r[j * 8 + 2 * h + 1]) * p.alpha) + bv[2 * h + 1]);
      } else {
        unpack2(fma2(pack2u(r[j * 8 + 2 * h], r[j * 8 + 2 * h + 1]), pack2(p.alpha, p.alpha), pack2(bv[2 * h], bv[2 * h + 1])), a, b);
      }
      o[h] = __fdividef(a, 1.0f + __expf(-a)) * b;
    }
    __nv_bfloat162 p0 = __floats2bfloat162_rn(o[0], o[1]), p1 = __floats2bfloat162_rn(o[2], o[3]);
    *reinterpret_cast<uint2*>(buf_gen + lane * 64 + j * 8) = make_uint2(*reinterpret_cast<uint32_t*>(&p0), *reinterpret_cast<uint32_t*>(&p1));
  }
}

__device__ __forceinline__ void epilogue_pair_dispatch(uint32_t mode, const uint32_t (&r)[64], const GemmParams& p,
                                                       uint32_t row, uint32_t ncol0, uint8_t* buf_gen, const float* bias_smem,
                                                       const float* lut, int lane, uint8_t* stage_q, uint32_t gq) {
  switch (mode) {
    case 0: epilogue_pair_math<false, false, false, false>(r, p, row, ncol0, buf_gen, bias_smem, lut, lane, stage_q, gq); break;
    case 1: epilogue_pair_math<true, false, false, false>(r, p, row, ncol0, buf_gen, bias_smem, lut, lane, stage_q, gq); break;
    case 2: epilogue_pair_math<false, true, false, false>(r, p, row, ncol0, buf_gen, bias_smem, lut, lane, stage_q, gq); break;
    case 3: epilogue_pair_math<true, true, false, false>(r, p, row, ncol0, buf_gen, bias_smem, lut, lane, stage_q, gq); break;
    case 4: epilogue_pair_math<false, false, true, false>(r, p, row, ncol0, buf_gen, bias_smem, lut, lane, stage_q, gq); break;
    case 5: epilogue_pair_math<true, false, true, false>(r, p, row, ncol0, buf_gen, bias_smem, lut, lane, stage_q, gq); break;
    case 6: epilogue_pair_math<false, true, true, false>(r, p, row, ncol0, buf_gen, bias_smem, lut, lane, stage_q, gq); break;
    case 7: epilogue_pair_math<true, true, true, false>(r, p, row, ncol0, buf_gen, bias_smem, lut, lane, stage_q, gq); break;
    // with an NVFP4 copy of the output (the host refuses the combination with a gated residual)
    case 8: epilogue_pair_math<false, false, false, true>(r, p, row, ncol0, buf_gen, bias_smem, lut, lane, stage_q, gq); break;
    case 9: epilogue_pair_math<true, false, false, true>(r, p, row, ncol0, buf_gen, bias_smem, lut, lane, stage_q, gq); break;
    case 10: epilogue_pair_math<false, true, false, true>(r, p, row, ncol0, buf_gen, bias_smem, lut, lane, stage_q, gq); break;
    case 12: epilogue_pair_swiglu<false>(r, p, buf_gen, bias_smem, lane); break;
    case 13: epilogue_pair_swiglu<true>(r, p, buf_gen, bias_smem, lane); break;
    default: epilogue_pair_math<true, true, false, true>(r, p, row, ncol0, buf_gen, bias_smem, lut, lane, stage_q, gq); break;
  }
}

// Work item w of the persistent loop -> row tile, first column and MMA width. Tiles [0, full_tiles) run whole
// (256 columns, fewer on a ragged last column tile: n_eff is a multiple of 16). The tiles of the last, partly filled
// wave are split into two 128-column halves when that lets every pair take part in it: the tail then costs half a
// tile time instead of a whole one (4352 x 9216: 612 tiles on 74 pairs = 8 waves + 20 tiles -> 40 halves).
__device__ __forceinline__ void decode_item(const GemmParams& p, uint32_t tiles_m2, uint32_t w, uint32_t& tm2, uint32_t& n0,
                                            uint32_t& n_eff) {
  uint32_t tile = w, sub = 0u, width = 256u;
  if (w >= p.full_tiles) {
    const uint32_t t = w - p.full_tiles;
    tile = p.full_tiles + (t >> 1);
    sub = t & 1u;
    width = 128u;
  }
  tm2 = tile % tiles_m2;
  n0 = (tile / tiles_m2) * 256u + sub * 128u;
  n_eff = min(width, (p.n - n0 + 15u) & ~15u);
}

// kDense: the dense-activation arm of the same kernel. A is bf16 [m,k] (not quantised), W the exact bf16 image of
// code x block scale [n,k] made once per weight; a stage holds 64 K elements of each (the same 128-byte swizzled
// rows), there are no scale factors, and the MMAs are kind::f16 with K = 16. Pipeline and epilogue are shared.
template <int KB, bool kDense>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(pair::kThreads, 1)
    nvfp4_gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                           const __grid_constant__ CUtensorMap map_sfa, const __grid_constant__ CUtensorMap map_sfb,
                           const __grid_constant__ PairOutMaps out_maps, const GemmParams p) {
  using namespace pair;
  using Cfg = PairCfg<KB>;
  constexpr int S = Cfg::kStages;
  constexpr int kABytes = Cfg::kABytes, kBBytes = Cfg::kBBytes, kSfaBytes = Cfg::kSfaBytes, kSfbBytes = Cfg::kSfbBytes;
  constexpr int kStageBytes = Cfg::kStageBytes;
  constexpr uint32_t kStageK = kDense ? KB * 16 : KB * 64;  // K elements per stage: 128 bytes of bf16 or of packed E2M1
  constexpr uint32_t kStageX = kDense ? kStageK : uint32_t(Cfg::kRowBytes);  // stage step along dim 0 of the operand maps
  constexpr uint32_t kLoadBytes = kDense ? uint32_t(kABytes + kBBytes) : uint32_t(kStageBytes);
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t sA = smem_base;
  const uint32_t sB = sA + S * kABytes;
  const uint32_t sSfa = sB + S * kBBytes;
  const uint32_t sSfb = sSfa + S * kSfaBytes;
  const uint32_t sStaging = sSfb + S * kSfbBytes;  // 1024-aligned: every size above is a multiple of 1024
  const uint32_t sBias = sStaging + kStagingBytes;
  const uint32_t sLut = sBias + kBiasBytes;
  const uint32_t sBar = sLut + kLutBytes;
  float* lut_gen = reinterpret_cast<float*>(smem_gen + (sLut - smem_base));
  const uint32_t bar_full = sBar;               // S barriers, used in the leader only
  const uint32_t bar_empty = bar_full + 8 * S;  // S
  const uint32_t bar_acc_full = bar_empty + 8 * S;
  const uint32_t bar_acc_free = bar_acc_full + 8;  // used in the leader only
  const uint32_t tmem_holder = bar_acc_free + 8;
  volatile uint32_t* tmem_holder_gen = reinterpret_cast<volatile uint32_t*>(smem_gen + (tmem_holder - smem_base));
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem_gen + (tmem_holder + 8 - smem_base));
  // staged NVFP4 multicast output: the CTA's eight epilogue warps meet on these ("tile staged" / "staging free")
  const uint32_t bar_qs_full = tmem_holder + 16, bar_qs_free = tmem_holder + 24;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  const bool ktr = kDiag && (p.diag & 16u) && blockIdx.x == 0 && threadIdx.x == 0;
  if (ktr) p.trace[1200] = clock64();
  const uint32_t pair_id = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const uint32_t tiles_m2 = p.tiles_m;  // tiles_m counts 256-row pair tiles here
  const uint32_t num_tiles = p.full_tiles + (p.tiles_m * p.tiles_n - p.full_tiles) * 2u;  // work items (see decode_item)
  const uint32_t num_k_tiles = (p.k + kStageK - 1u) / kStageK;
  const long long wait_limit = p.wait_limit > 0 ? p.wait_limit : kDefaultWaitLimitCycles;

  if (threadIdx.x == 0) {
    for (int i = 0; i < S; ++i) {
      mbar_init(bar_full + 8 * i, 1);
      mbar_init(bar_empty + 8 * i, 1);
    }
    mbar_init(bar_acc_full, 1);
    mbar_init(bar_acc_free, 16);  // every epilogue warp of both CTAs arrives once per tile
    mbar_init(bar_qs_full, 8);
    mbar_init(bar_qs_free, 8);
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&map_a);
    prefetch_tensormap(&map_w);
    prefetch_tensormap(&map_sfa);
    prefetch_tensormap(&map_sfb);
    prefetch_tensormap(&out_maps.m[0]);
  }
  if (p.q_codes) fill_inv_scale_lut(lut_gen, p.q_global, threadIdx.x, blockDim.x);
  if (warp == kMmaWarp) {
    tmem_alloc_pair(tmem_holder, kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_arrive();
  cluster_wait();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder_gen;
  pdl_launch_dependents();  // the next kernel's CTAs may be scheduled as ours retire
  pdl_wait();               // operands written by the previous kernel are complete and visible
  if (ktr) p.trace[1201] = clock64();

  if (warp == kProducerWarp) {
    // ---------------- TMA producer (both CTAs): the whole warp runs the loop, one lane issues ----------------
    {
      uint32_t stage = 0, phase = 0, titer = 0;
      bool ok = true;
      for (uint32_t tile = pair_id; tile < num_tiles && ok; tile += num_pairs) {
        // A narrower item (ragged last column tile, half tile of the tail) runs a narrower MMA of n_eff columns: the
        // pair's two halves of the W tile are then rows [n0, n0 + n_eff/2) and [n0 + n_eff/2, n0 + n_eff), so that
        // accumulator column j is still output column n0 + j.
        uint32_t tm2, n0u, n_eff;
        decode_item(p, tiles_m2, tile, tm2, n0u, n_eff);
        const int32_t m0 = int32_t(tm2 * 256u + rank * 128u), n0 = int32_t(n0u);
        const int32_t sfa_row0 = int32_t((tm2 * 2u + rank) * p.k_atoms * 4u);
        const int32_t sfb_row0 = int32_t((uint32_t(n0) >> 7) * p.k_atoms * 4u);
        for (uint32_t kt = 0; kt < num_k_tiles; ++kt) {
          if (!mbar_wait_warp(bar_empty + 8 * stage, phase ^ 1u, abort_flag, kStatusProducerTimeout, wait_limit)) {
            ok = false;
            break;
          }
          const bool tr = kDiag && (p.diag & 16u) && rank == 0 && pair_id == 0 && titer < 256u;
          const bool skip_ab = kDiag && (p.diag & 8u) != 0u;
          const uint32_t full = mapa_cluster(bar_full + 8 * stage, 0);  // the leader's barrier counts both CTAs' bytes
          // p.stall (wait self-test): nothing is loaded and no bytes are expected, so the MMA warp's first wait on a
          // loaded stage runs out, raises the abort flag and every role leaves through the tear-down
          if (!p.stall && elect_one()) {
            if (tr) p.trace[titer * 4 + 0] = clock64();
            const bool skip_a = kDiag && (p.diag & 32u) != 0u;
            if (rank == 0)
              mbar_arrive_expect_tx(bar_full + 8 * stage, skip_ab ? 2u * (kSfaBytes + kSfbBytes) : 2u * (kLoadBytes - (skip_a ? kABytes : 0)));
            if (!skip_ab) {
              if (!skip_a) tma_load_2d_pair(sA + stage * kABytes, &map_a, full, int32_t(kt * kStageX), m0);
              tma_load_2d_pair(sB + stage * kBBytes, &map_w, full, int32_t(kt * kStageX), n0 + int32_t(rank * (n_eff >> 1)));
            }
            if (!kDense) {
              tma_load_2d_pair(sSfa + stage * kSfaBytes, &map_sfa, full, 0, sfa_row0 + int32_t(kt * (KB * 4u)));
              tma_load_2d_pair(sSfb + stage * kSfbBytes, &map_sfb, full, 0, sfb_row0 + int32_t(kt * (KB * 4u)));
              tma_load_2d_pair(sSfb + stage * kSfbBytes + 512 * KB, &map_sfb, full, 0,
                               sfb_row0 + int32_t(p.k_atoms * 4u + kt * (KB * 4u)));
            }
            if (tr) p.trace[titer * 4 + 1] = clock64();
          }
          __syncwarp();
          ++titer;
          if (++stage == S) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == kMmaWarp) {
    // ---------------- MMA issuer (leader CTA only) ----------------
    if (rank == 0) {  // whole warp runs the loop; one elected lane issues the tcgen05 instructions

      // descriptor words of stage 0, K block 0 (see make_desc_operand / make_desc_sf); the loop only adds to the low word
      const uint64_t op0 = make_desc_operand<KB>(sA), sf0 = make_desc_sf(sSfa);
      const uint32_t op_hi = uint32_t(op0 >> 32), sf_hi = uint32_t(sf0 >> 32);
      const uint32_t a_lo0 = uint32_t(op0), b_lo0 = uint32_t(make_desc_operand<KB>(sB));
      const uint32_t sfa_lo0 = uint32_t(sf0), sfb_lo0 = uint32_t(make_desc_sf(sSfb));
      uint32_t stage = 0, phase = 0, it = 0, titer = 0;
      bool ok = true, ready = false;
      for (uint32_t tile = pair_id; tile < num_tiles && ok; tile += num_pairs, ++it) {
        const bool ttr = kDiag && (p.diag & 16u) && pair_id == 0 && it < 16u && lane == 0;
        if (ttr) p.trace[1024 + it * 8 + 0] = clock64();
        if (it > 0) {  // the previous tile's epilogues (both CTAs) have read the overlapping columns
          if (!mbar_wait_warp(bar_acc_free, (it - 1u) & 1u, abort_flag, kStatusAccEmptyTimeout, wait_limit)) {
            ok = false;
            break;
          }
          tc_fence_after();
        }
        if (ttr) p.trace[1024 + it * 8 + 1] = clock64();
        const uint32_t d_tmem = tmem_base + (it & 1u) * kAccStride;
        uint32_t tm2_, n0_, n_eff;
        decode_item(p, tiles_m2, tile, tm2_, n0_, n_eff);  // as in the producer
        const uint32_t idesc = kDense ? make_idesc_bf16(256, n_eff) : make_idesc_nvfp4(256, n_eff);
        for (uint32_t kt = 0; kt < num_k_tiles; ++kt) {
          if (kDiag && (p.diag & 16u) && pair_id == 0 && titer < 256u && lane == 0) p.trace[1300 + titer] = clock64();
          // `ready`: the probe issued one stage ago already saw this stage loaded (the usual case once the loads
          // run ahead), so the warp goes straight to issuing; otherwise it waits here
          if (!ready && !mbar_wait_warp(bar_full + 8 * stage, phase, abort_flag, kStatusMmaTimeout, wait_limit)) {
            ok = false;
            break;
          }
          tc_fence_after();
          // probe the NEXT stage now: the answer arrives while this stage's instructions are being issued
          const uint32_t nstage = stage + 1u == uint32_t(S) ? 0u : stage + 1u;
          const bool probe = mbar_test_wait(bar_full + 8 * nstage, nstage == 0u ? phase ^ 1u : phase);
          const bool tr = kDiag && (p.diag & 16u) && pair_id == 0 && titer < 256u;
          if (elect_one()) {
          if (tr) p.trace[titer * 4 + 2] = clock64();
          // Descriptors of this stage: the constant high words were built before the loop, a stage only moves the
          // 14-bit start-address field (shared addresses are below 256 KB, so the add never carries out of it).
          const uint32_t a_lo = a_lo0 + stage * uint32_t(kABytes >> 4), b_lo = b_lo0 + stage * uint32_t(kBBytes >> 4);
          const uint32_t sfa_lo = sfa_lo0 + stage * uint32_t(kSfaBytes >> 4), sfb_lo = sfb_lo0 + stage * uint32_t(kSfbBytes >> 4);
          // scale factors of this stage: slot (kt & 1) when two slots exist, so that these copies
          // do not wait for the previous stage's MMAs to finish reading theirs
          const uint32_t sf_slot = Cfg::kSfSlots == 2 ? (kt & 1u) : 0u;
          const uint32_t t_sfa = tmem_base + kSfaCol + sf_slot * (KB * 4), t_sfb = tmem_base + kSfbCol + sf_slot * (KB * 8);
          const bool do_cp = !(kDiag && (p.diag & 2u)) || kt == 0, do_mma = !(kDiag && (p.diag & 4u));
          if (kDense) {
#pragma unroll
            for (int kb = 0; kb < KB; ++kb)
              tc_mma_bf16_pair(d_tmem, desc64(a_lo + kb * 2, op_hi), desc64(b_lo + kb * 2, op_hi), idesc, (kt | uint32_t(kb)) != 0u);
          } else if (kDiag && (p.diag & 64u)) {  // diagnostic order: each K block's scale copies right before its MMA
#pragma unroll
            for (int kb = 0; kb < KB; ++kb) {
              if (do_cp) {
                tc_cp_32x128b_warpx4_pair(t_sfa + kb * 4, desc64(sfa_lo + kb * 32, sf_hi));
                tc_cp_32x128b_warpx4_pair(t_sfb + kb * 8, desc64(sfb_lo + kb * 32, sf_hi));
                tc_cp_32x128b_warpx4_pair(t_sfb + kb * 8 + 4, desc64(sfb_lo + 32 * KB + kb * 32, sf_hi));
              }
              if (do_mma)
                tc_mma_nvfp4_pair(d_tmem, desc64(a_lo + kb * 2, op_hi), desc64(b_lo + kb * 2, op_hi), idesc, t_sfa + kb * 4,
                                  t_sfb + kb * 8, (kt | uint32_t(kb)) != 0u);
            }
          } else {
            if (do_cp)
#pragma unroll
              for (int kb = 0; kb < KB; ++kb) {
                tc_cp_32x128b_warpx4_pair(t_sfa + kb * 4, desc64(sfa_lo + kb * 32, sf_hi));
                tc_cp_32x128b_warpx4_pair(t_sfb + kb * 8, desc64(sfb_lo + kb * 32, sf_hi));
                tc_cp_32x128b_warpx4_pair(t_sfb + kb * 8 + 4, desc64(sfb_lo + 32 * KB + kb * 32, sf_hi));
              }
            if (do_mma)
#pragma unroll
              for (int kb = 0; kb < KB; ++kb)
                tc_mma_nvfp4_pair(d_tmem, desc64(a_lo + kb * 2, op_hi), desc64(b_lo + kb * 2, op_hi), idesc, t_sfa + kb * 4,
                                  t_sfb + kb * 8, (kt | uint32_t(kb)) != 0u);
          }
          tc_commit_pair_mc(bar_empty + 8 * stage, 3);  // frees the stage in both CTAs
          if (tr) p.trace[titer * 4 + 3] = clock64();
          }
          ready = __all_sync(0xFFFFFFFFu, probe) != 0;
          ++titer;
          if (++stage == S) { stage = 0; phase ^= 1u; }
        }
        if (ok && elect_one()) tc_commit_pair_mc(bar_acc_full, 3);  // accumulator ready in both CTAs
        __syncwarp();
        if (ttr) p.trace[1024 + it * 8 + 2] = clock64();
      }
    }
  } else {
    // ---------------- epilogue (warps 2..9, both CTAs) ----------------
    // Warp w reads TMEM lanes [32*(w%4), +32). Two warps share a lane quarter: the one with
    // h == 0 takes the first two 64-column groups in drain order (the first of which overlaps the
    // other accumulator), h == 1 the last two.
    const uint32_t ew = uint32_t(warp - kFirstEpilogueWarp);  // 0..7
    const uint32_t q = warp & 3, h = ew >> 2;
    const uint32_t buf = sStaging + ew * 4096u;
    uint8_t* buf_gen = smem_gen + (buf - smem_base);
    float* bias_gen = reinterpret_cast<float*>(smem_gen + (sBias - smem_base) + ew * 256u);  // 64 f32: the current group's bias
    const float bias_mul = (p.act == 1u && !p.chain) ? 0.5f : 1.0f;                          // the fused GELU works on x/2
    const uint32_t acc_free_leader = mapa_cluster(bar_acc_free, 0);
    uint32_t it = 0;
    bool ok = true;
    const uint32_t mode = p.swiglu ? (p.chain ? 13u : 12u)
                                   : (p.act == 1u ? 1u : 0u) | (p.chain ? 2u : 0u) | (p.q_codes ? 8u : (p.gate ? 4u : 0u));
    // NVFP4 output through the multicast alias with no bf16 store: the (then idle) bf16 staging area collects the
    // CTA's whole tile of codes and scale atoms, and all eight warps write it out in 128-byte row segments and whole
    // 16-byte atom rows. Scattered 16- and 4-byte multimem stores straight from the registers ran at a fifth of the link rate.
    uint8_t* stage_q = (p.q_codes_mc && !p.store_bf16) ? smem_gen + (sStaging - smem_base) : nullptr;
    for (uint32_t tile = pair_id; tile < num_tiles && ok; tile += num_pairs, ++it) {
      uint32_t tm2, n0, n_eff;
      decode_item(p, tiles_m2, tile, tm2, n0, n_eff);
      const uint32_t row0 = tm2 * 256u + rank * 128u + q * 32u;
      const uint32_t b = it & 1u;
      const uint32_t first = b ? 0u : 3u;  // 64-column group that overlaps the other accumulator
      const uint32_t g0 = (2u * h + first) & 3u, g1 = (2u * h + 1u + first) & 3u;
      // this warp's 2 x 64 bias values: every lane fetches two columns of each group now, while the main loop
      // is still running; they go to shared memory as f32 right before the group's arithmetic
      uint32_t bq0 = 0u, bq1 = 0u;
      if (p.bias) {
        const uint32_t nc0 = n0 + g0 * 64u + uint32_t(lane) * 2u, nc1 = n0 + g1 * 64u + uint32_t(lane) * 2u;
        if (nc0 < p.n) bq0 = __ldg(reinterpret_cast<const uint32_t*>(p.bias + nc0));
        if (nc1 < p.n) bq1 = __ldg(reinterpret_cast<const uint32_t*>(p.bias + nc1));
      }
      if (lane == 0 && p.gate) {
        if (n0 + g0 * 64u < p.n) asm volatile("prefetch.global.L1 [%0];" ::"l"(p.gate + n0 + g0 * 64u));
        if (n0 + g1 * 64u < p.n) asm volatile("prefetch.global.L1 [%0];" ::"l"(p.gate + n0 + g1 * 64u));
      }
      const bool ttr = kDiag && (p.diag & 16u) && pair_id == 0 && rank == 0 && it < 16u && lane == 0 && warp == kFirstEpilogueWarp;
      if (ttr) p.trace[1024 + it * 8 + 3] = clock64();
      if (!mbar_wait_bounded(bar_acc_full, it & 1u, abort_flag, kStatusEpilogueTimeout, wait_limit)) {
        ok = false;
        break;
      }
      tc_fence_after();
      if (ttr) p.trace[1024 + it * 8 + 4] = clock64();
      // The next tile's MMA overwrites the accumulator of tile it-1 and this tile's overlapping
      // columns. h == 0 warps arrive once those columns are in registers (below); h == 1 warps never
      // touch them and arrive here: having passed this wait they are done reading tile it-1.
      if (h == 1) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(acc_free_leader);
      }
      const uint32_t t_addr = tmem_base + b * kAccStride + ((q * 32u) << 16);
      uint32_t r[64];
      tmem_ld_32x32b_x32(t_addr + g0 * 64u, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
      tmem_ld_32x32b_x32(t_addr + g0 * 64u + 32u, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
      tmem_ld_wait();
      if (ttr) p.trace[1024 + it * 8 + 7] = clock64();
      if (h == 0) {  // the overlapping columns are in registers: the next tile's MMA may start
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(acc_free_leader);
        if (ttr) p.trace[1024 + it * 8 + 5] = clock64();
      }
      const uint32_t row = row0 + lane;
      if (stage_q && it > 0u &&  // the previous tile's write-out has finished reading the staging area
          !mbar_wait_bounded(bar_qs_free, (it - 1u) & 1u, abort_flag, kStatusEpilogueTimeout, wait_limit)) {
        ok = false;
        break;
      }
#pragma unroll 1
      for (uint32_t half = 0; half < 2; ++half) {
        const uint32_t g = half ? g1 : g0;
        if (half) {
          tmem_ld_32x32b_x32(t_addr + g * 64u, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
          tmem_ld_32x32b_x32(t_addr + g * 64u + 32u, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
          tmem_ld_wait();
        }
        const uint32_t ncol0 = n0 + g * 64u;
        // warp-uniform; with a staged output a warp whose rows are all past m still stages their (zero) scale words
        if (g * 64u >= n_eff || ncol0 >= p.n || (row0 >= p.m && !stage_q)) continue;
        if (kDiag && (p.diag & 256u)) continue;      // diagnostic: drain the accumulator only
        if (lane == 0) bulk_wait_group_read<0>();  // the previous store has finished reading the staging buffer
        __syncwarp();                              // ... and every lane its reads of the previous group's bias
        const uint32_t bq = half ? bq1 : bq0;
        *reinterpret_cast<float2*>(bias_gen + lane * 2) = make_float2(bf16_lo(bq) * bias_mul, bf16_hi(bq) * bias_mul);
        __syncwarp();
        epilogue_pair_dispatch(mode, r, p, row, ncol0, buf_gen, bias_gen, lut_gen, lane, stage_q, g);
        fence_proxy_async();  // generic-proxy writes to smem -> visible to the TMA store
        __syncwarp();
        if (lane == 0) {
          // SwiGLU halves the columns: the 64 accumulator columns of this group are output columns ncol0/2 .. +32
          if (!(kDiag && (p.diag & 1u)) && p.store_bf16 && !p.out_mc)
            tma_store_2d(&out_maps.m[0], buf, int32_t(p.swiglu ? ncol0 >> 1 : ncol0), int32_t(row0));
          bulk_commit_group();
        }
        // Multicast output: the staging rows leave as 16-byte multimem stores (8 lanes cover one 128-byte row
        // segment, a warp instruction writes 4 rows); the switch delivers them to every rank's copy of the output,
        // this rank's included, so there is no separate local store and no gather pass afterwards.
        if (p.out_mc && p.store_bf16) {
          const uint32_t chunk = lane & 7u, col = ncol0 + chunk * 8u;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const uint32_t rr = uint32_t(i) * 4u + (lane >> 3);
            const uint4 v = *reinterpret_cast<const uint4*>(buf_gen + rr * 128u + ((chunk ^ (rr & 7u)) << 4));
            if (row0 + rr < p.m && col < p.n) multimem_st_v4(p.out_mc + uint64_t(row0 + rr) * p.ldo + p.n_offset + col, v);
          }
        }
        // Peer windows: coalesced 16-byte stores straight from the staging rows (8 lanes cover one
        // 128-byte row segment, a warp instruction writes 4 rows). TMA stores to peer memory reached
        // only ~160 GB/s per GPU with three peers; plain vector stores are what NVLink packs well.
        if (p.n_out > 1u && !(kDiag && (p.diag & 1u))) {
          const uint32_t chunk = lane & 7u, col = ncol0 + chunk * 8u;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const uint32_t rr = uint32_t(i) * 4u + (lane >> 3);
            const uint4 v = *reinterpret_cast<const uint4*>(buf_gen + rr * 128u + ((chunk ^ (rr & 7u)) << 4));
            if (row0 + rr < p.m && col < p.n) {
              const uint64_t off = uint64_t(row0 + rr) * p.ldo + p.n_offset + col;
              for (uint32_t d = 1; d < p.n_out; ++d) *reinterpret_cast<uint4*>(p.out[d] + off) = v;
            }
          }
        }
      }
      if (stage_q && ok) {
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_qs_full);  // release: this warp's part of the tile is staged
        if (!mbar_wait_bounded(bar_qs_full, it & 1u, abort_flag, kStatusEpilogueTimeout, wait_limit)) {
          ok = false;
          break;
        }
        const uint32_t t = ew * 32u + uint32_t(lane);
        const uint32_t trow0 = tm2 * 256u + rank * 128u, qcol0 = p.n_offset + n0;
#pragma unroll
        for (uint32_t pass = 0; pass < 4u; ++pass) {  // 8 lanes cover a row's 128 code bytes, 32 rows per pass
          const uint32_t lr = pass * 32u + (t >> 3), c = t & 7u, grow = trow0 + lr;
          if (grow < p.m && (c >> 1) * 64u < n_eff && n0 + (c >> 1) * 64u < p.n)
            multimem_st_v4(p.q_codes_mc + uint64_t(grow) * (p.ldo >> 1) + (qcol0 >> 1) + c * 16u,
                           *reinterpret_cast<const uint4*>(stage_q + lr * 128u + ((c ^ (lr & 7u)) << 4)));
        }
        if (t < 128u && trow0 < p.m && (t >> 5) * 64u < n_eff && n0 + (t >> 5) * 64u < p.n)  // four 512-byte scale atoms, 16 bytes per thread
          multimem_st_v4(p.q_scales_mc + sf_device_offset(trow0, (qcol0 >> 4) + (t >> 5) * 4u, p.q_k_atoms) + (t & 31u) * 16u,
                         *reinterpret_cast<const uint4*>(stage_q + 16384u + (t >> 5) * 512u + (t & 31u) * 16u));
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_qs_free);
      }
      if (ttr) p.trace[1024 + it * 8 + 6] = clock64();
    }
    if (lane == 0) bulk_wait_group_read<0>();
    if (p.out_mc || p.q_codes_mc) __threadfence_system();  // multicast stores are performed before the kernel ends
  }

  // ---------------- tear-down ----------------
  tc_fence_before();
  __syncthreads();
  if (ktr) p.trace[1202] = clock64();
  if (*abort_flag != 0u) {
    if (threadIdx.x == 0) atomicCAS(p.status, 0u, *abort_flag);
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);  // let copies and MMAs in flight retire
  }
  cluster_arrive();
  cluster_wait();
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
  if (ktr) p.trace[1203] = clock64();
}

static uint32_t env_u32_pair(const char* name, uint32_t dflt) {
  if (!kDiag) return dflt;  // the default build reads no environment variable
  const char* v = getenv(name);
  return v ? uint32_t(strtoul(v, nullptr, 0)) : dflt;
}

bool gemm_use_pair(uint32_t m, uint32_t n, uint32_t k) {
  (void)k;
  static uint32_t force = env_u32_pair("TNF_GEMM_KERNEL", 0);  // diagnostic builds: 1 = always 1-CTA, 2 = always pair
  if (force == 1) return false;
  if (force == 2) return true;
  // a pair works on a 256x256 tile; with few tiles (skinny M) the 1-CTA kernel's 128x128 tiles fill more SMs
  return m > 128 && uint64_t((m + 255u) / 256u) * ((n + 255u) / 256u) >= 32u;
}

uint32_t gemm_pair_kblocks() { return 4u; }

template <int KB, bool kDense>
static cudaError_t launch_pair_kb(const CUtensorMap& map_a, const CUtensorMap& map_w, const CUtensorMap& map_sfa,
                                  const CUtensorMap& map_sfb, const CUtensorMap* out_maps, const GemmParams& p_in,
                                  int sm_count, cudaStream_t s) {
  using Cfg = PairCfg<KB>;
  static PerDeviceOnce once;
  static int max_pairs[kMaxDevices] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= kMaxDevices) dev = 0;
  if (once.first_use() >= 0) {  // the shared-memory opt-in is a per-device attribute of the function
    cudaError_t e = cudaFuncSetAttribute(nvfp4_gemm_pair_kernel<KB, kDense>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (e != cudaSuccess) return e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(unsigned(sm_count & ~1), 1, 1);
    cfg.blockDim = dim3(pair::kThreads, 1, 1);
    cfg.dynamicSmemBytes = Cfg::kSmemBytes;
    int clusters = 0;
    e = cudaOccupancyMaxActiveClusters(&clusters, nvfp4_gemm_pair_kernel<KB, kDense>, &cfg);
    if (e != cudaSuccess || clusters <= 0) {
      cudaGetLastError();
      clusters = sm_count / 2;
    }
    max_pairs[dev] = std::min(clusters, sm_count / 2);
  }
  GemmParams p = p_in;
  static uint32_t diag = env_u32_pair("TNF_GEMM_DIAG", 0);
  p.diag = diag;
  p.tiles_m = (p.m + 255u) / 256u;
  p.tiles_n = (p.n + 255u) / 256u;
  const uint32_t tiles = p.tiles_m * p.tiles_n;
  if (tiles == 0) return cudaSuccess;
  const uint32_t avail = uint32_t(max_pairs[dev] > 0 ? max_pairs[dev] : sm_count / 2);
  const uint32_t tail = tiles % avail;
  // split the last wave's tiles into halves when every half then finds a pair of its own (and no half is empty)
  p.full_tiles = (tiles > avail && tail > 0 && 2u * tail <= avail && p.n % 256u == 0u && !(kDiag && (diag & 2048u))) ? tiles - tail : tiles;
  const uint32_t items = p.full_tiles + (tiles - p.full_tiles) * 2u;
  const uint32_t pairs = std::min<uint32_t>(items, avail);
  PairOutMaps om;
  for (int i = 0; i < kMaxPeers; ++i) om.m[i] = out_maps[i];
  return launch_pdl(nvfp4_gemm_pair_kernel<KB, kDense>, dim3(pairs * 2), dim3(pair::kThreads), Cfg::kSmemBytes, s, map_a, map_w, map_sfa,
                    map_sfb, om, p);
}

cudaError_t launch_gemm_nvfp4_pair(const CUtensorMap& map_a, const CUtensorMap& map_w, const CUtensorMap& map_sfa,
                                   const CUtensorMap& map_sfb, const CUtensorMap* out_maps, const GemmParams& p,
                                   int sm_count, cudaStream_t s) {
  return p.dense ? launch_pair_kb<4, true>(map_a, map_w, map_sfa, map_sfb, out_maps, p, sm_count, s)
                 : launch_pair_kb<4, false>(map_a, map_w, map_sfa, map_sfb, out_maps, p, sm_count, s);
}

}  // namespace tnf
