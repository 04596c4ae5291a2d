// NVFP4 GEMM for sm_100a: out[m,n] = epilogue(alpha * sum_k A[m,k] * W[n,k]) with E2M1
// operands and one UE4M3 scale per 16 K-elements on both sides.
//
// Replaces the reference's dequant + matmul / matmul_i8 dispatches and the bias / GELU /
// gated-residual dispatches after them (thinfer-core/src/ops/matmul.rs:150-749,
// matmul_i8.rs:196-393, bcast_add.rs, gelu.rs:21-31, bcast_fma.rs) with one kernel.
//
// Structure (one persistent CTA per SM, 192 threads):
//   warp 0     TMA producer: per 256-element K tile, one 2-D tensor-map load each for the A
//              and W code tiles (128-byte rows, 128-byte swizzle) and untiled bulk copies of
//              the matching 512-byte scale atoms, all completing on the stage's mbarrier.
//   warp 1     owns TMEM; one lane copies the scale atoms shared->TMEM (tcgen05.cp) and issues
//              tcgen05.mma kind::mxf4nvf4 block16, four K=64 steps per stage; tcgen05.commit
//              frees the stage and, after the last K tile, publishes the accumulator.
//   warps 2-5  epilogue: tcgen05.ld the accumulator (each warp its own 32-lane quarter),
//              alpha, bias, tanh-GELU, gated residual, bf16 RNE, 16-byte stores to the local
//              output and to any peer windows.
// Every mbarrier wait is bounded; a wait that gives up raises a CTA-wide abort flag, records
// a status code for the host and every role falls through to the common tear-down, which
// frees TMEM.
#include <cuda_bf16.h>
#include <cstdint>
#include <cstdlib>

#include "epilogue.cuh"
#include "internal.h"
#include "ptx.cuh"

namespace tnf {

constexpr int kBlockM = 128;
constexpr int kBlockKBytes = 128;  // 256 E2M1 elements
constexpr int kBlockK = 256;
constexpr int kThreads = 192;
constexpr uint32_t kTmemCols = 512;

template <int BN>
struct TileCfg {
  // 128-row scale blocks a tile touches: tiles that divide 128 never straddle a block
  static constexpr int kSfbAtoms = (BN % 128 == 0) ? BN / 128 : (128 % BN == 0 ? 1 : (BN + 96 + 127) / 128);
  // scale factors in TMEM: two slots used by alternate K tiles, so that a tile's copies do not wait for the
  // previous tile's MMAs to finish reading theirs
  static constexpr int kSfSlotCols = 16 + 16 * kSfbAtoms;
  static constexpr int kAccStages = (2 * BN + 2 * kSfSlotCols <= 512) ? 2 : 1;
  static constexpr int kABytes = kBlockM * kBlockKBytes;
  static constexpr int kBBytes = BN * kBlockKBytes;
  static constexpr int kSfaBytes = 2048;
  static constexpr int kSfbBytes = 2048 * kSfbAtoms;
  static constexpr int kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;
  static constexpr int kStages = (BN >= 224) ? 4 : (BN >= 192 ? 5 : (BN >= 128 ? 6 : 7));
  static constexpr int kEpiVecBytes = 4 * 1536;  // per epilogue warp: the tile's bias as f32 (1 KB) and gate as bf16 (512 B)
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*align slack*/ + 256 /*barriers*/ + kEpiVecBytes;
  static constexpr uint32_t kAccCol0 = 0;
  static constexpr uint32_t kSfaCol = kAccStages * BN;
  static constexpr uint32_t kSfbCol = kSfaCol + 16;  // within a slot: 16 columns of A scales, then W's
  static_assert(kSfaCol + 2 * kSfSlotCols <= 512, "TMEM overflow");
  static_assert(kSmemBytes <= 227 * 1024, "shared memory overflow");
};

__device__ __forceinline__ float bf16_bits_to_f32(uint32_t h) { return __uint_as_float(h << 16); }

// One epilogue warp's 32 rows of a tile, 32 columns at a time; each lane holds its own row. The arithmetic is the
// pair kernel's (epilogue8), chosen once per tile instead of per element: with one warp per scheduler every
// branch and every dependent instruction is paid in full. Each lane then trades half of its four 16-byte vectors with its
// neighbour so that a lane pair stores whole 32-byte sectors of one row per instruction.
template <int BN, bool kGelu, bool kChain, bool kGate>
__device__ __forceinline__ void epilogue_tile(const GemmParams& p, uint32_t t_addr, uint32_t row, uint32_t n0, int lane,
                                              float alpha, const float* bias_smem, const uint4* gate_smem, bool skip_stores) {
  constexpr int NC = BN / 32;
  const bool odd = (lane & 1) != 0;
  const uint32_t row_even = row & ~1u, c8 = odd ? 8u : 0u;
  // even lane: columns [0,8) and [16,24) of both rows of the pair; odd lane: columns [8,16) and [24,32)
  const uint64_t base_off = uint64_t(row_even) * p.ldo + p.n_offset + n0 + c8;
  uint16_t* const out0 = p.out[0] + base_off;
  const bool row_ok[2] = {row_even < p.m, row_even + 1u < p.m};
  // one 32-column chunk out of `rc`; the read of the next chunk goes into `rn` meanwhile
#pragma unroll 1
  for (int c = 0; c < NC; ++c) {
    const uint32_t nc = n0 + c * 32;
    if (nc >= p.n) break;                       // warp-uniform
    const uint32_t ncols = min(32u, p.n - nc);  // multiple of 8
    uint32_t rc[32];
    tmem_ld_32x32b_x32(t_addr + c * 32, rc);
    // the residual row's four vectors are requested together, before the accumulator read is waited for
    uint4 res[4] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
    if (kGate && row < p.m) {
      const uint16_t* res_row = p.residual + uint64_t(row) * p.n + nc;
#pragma unroll
      for (int v8 = 0; v8 < 4; ++v8)
        if (uint32_t(v8 * 8) < ncols) res[v8] = __ldg(reinterpret_cast<const uint4*>(res_row + v8 * 8));
    }
    tmem_ld_wait();
    uint4 v[4];
#pragma unroll
    for (int v8 = 0; v8 < 4; ++v8)
      v[v8] = epilogue8<kGelu, kChain, kGate>(rc + v8 * 8, alpha, bias_smem + c * 32 + v8 * 8,
                                             kGate ? gate_smem[c * 4 + v8] : make_uint4(0, 0, 0, 0), res[v8]);
    uint4 mine[2], theirs[2];  // vectors of this lane's row it still stores / of the neighbour's row it stores for it
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const uint4 give = odd ? v[2 * j] : v[2 * j + 1];
      mine[j] = odd ? v[2 * j + 1] : v[2 * j];
      theirs[j].x = __shfl_xor_sync(0xFFFFFFFFu, give.x, 1);
      theirs[j].y = __shfl_xor_sync(0xFFFFFFFFu, give.y, 1);
      theirs[j].z = __shfl_xor_sync(0xFFFFFFFFu, give.z, 1);
      theirs[j].w = __shfl_xor_sync(0xFFFFFFFFu, give.w, 1);
    }
    if (skip_stores) continue;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      if (c8 + 16u * j >= ncols) break;
#pragma unroll
      for (int rr = 0; rr < 2; ++rr) {
        if (!row_ok[rr]) continue;
        const uint4 o4 = (odd == (rr == 1)) ? mine[j] : theirs[j];
        const uint64_t off = uint64_t(rr) * p.ldo + uint32_t(c * 32 + 16 * j);
        *reinterpret_cast<uint4*>(out0 + off) = o4;
        for (uint32_t d = 1; d < p.n_out; ++d) *reinterpret_cast<uint4*>(p.out[d] + base_off + off) = o4;
      }
    }
  }
}

template <int BN>
__global__ void __launch_bounds__(kThreads, 1)
    nvfp4_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                      const GemmParams p) {
  using Cfg = TileCfg<BN>;
  constexpr int S = Cfg::kStages;
  constexpr int AS = Cfg::kAccStages;
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment for the 128-byte swizzle atoms
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t sA = smem_base;
  const uint32_t sB = sA + S * Cfg::kABytes;
  const uint32_t sSfa = sB + S * Cfg::kBBytes;
  const uint32_t sSfb = sSfa + S * Cfg::kSfaBytes;
  const uint32_t sBar = sSfb + S * Cfg::kSfbBytes;  // 8-byte aligned (all sizes are multiples of 512)
  const uint32_t bar_full = sBar;                   // S barriers
  const uint32_t bar_empty = bar_full + 8 * S;      // S
  const uint32_t bar_acc_full = bar_empty + 8 * S;  // AS
  const uint32_t bar_acc_empty = bar_acc_full + 8 * AS;
  const uint32_t tmem_holder = bar_acc_empty + 8 * AS;
  volatile uint32_t* abort_flag =
      reinterpret_cast<volatile uint32_t*>(smem_gen + (tmem_holder + 8 - smem_base));
  volatile uint32_t* tmem_holder_gen = reinterpret_cast<volatile uint32_t*>(smem_gen + (tmem_holder - smem_base));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t num_tiles = p.tiles_m * p.tiles_n;
  const bool ktr = kDiag && (p.diag & 16u) && blockIdx.x == 0;

  const uint32_t num_k_tiles = (p.k + kBlockK - 1) / kBlockK;
  const long long wait_limit = p.wait_limit > 0 ? p.wait_limit : kDefaultWaitLimitCycles;

  if (threadIdx.x == 0) {
    for (int i = 0; i < S; ++i) {
      mbar_init(bar_full + 8 * i, 1);
      mbar_init(bar_empty + 8 * i, 1);
    }
    for (int i = 0; i < AS; ++i) {
      mbar_init(bar_acc_full + 8 * i, 1);
      mbar_init(bar_acc_empty + 8 * i, 4);
    }
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&map_a);
    prefetch_tensormap(&map_w);
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder_gen;
  pdl_launch_dependents();
  pdl_wait();  // before any access to global memory
  if (ktr && threadIdx.x == 0) p.trace[1201] = clock64();

  if (warp == 0) {
    // ---------------- TMA producer: the whole warp runs the loop (uniform addresses), one lane issues ----------------
    {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (uint32_t tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const uint32_t tm = tile % p.tiles_m, tn = tile / p.tiles_m;
        const uint32_t m0 = tm * kBlockM, n0 = tn * BN;
        const uint8_t* sfa_src = p.sfa + uint64_t(tm) * p.k_atoms * 512u;
        const uint8_t* sfb_src = p.sfb + uint64_t(n0 >> 7) * p.k_atoms * 512u;
        for (uint32_t kt = 0; kt < num_k_tiles; ++kt) {
          if (!mbar_wait_warp(bar_empty + 8 * stage, phase ^ 1u, abort_flag, kStatusProducerTimeout, wait_limit)) {
            ok = false;
            break;
          }
          const uint32_t full = bar_full + 8 * stage;
          if (ktr && kt < 16 && lane == 0) p.trace[1240 + kt] = clock64();
          if (elect_one()) {
          if (kDiag && (p.diag & 8u)) {
            mbar_arrive_expect_tx(full, Cfg::kSfaBytes + Cfg::kSfbBytes);
          } else {
            mbar_arrive_expect_tx(full, Cfg::kStageBytes);
            tma_load_2d(sA + stage * Cfg::kABytes, &map_a, full, int32_t(kt * kBlockKBytes), int32_t(m0));
            tma_load_2d(sB + stage * Cfg::kBBytes, &map_w, full, int32_t(kt * kBlockKBytes), int32_t(n0));
          }
          bulk_load_1d(sSfa + stage * Cfg::kSfaBytes, sfa_src + uint64_t(kt) * 2048u, 2048u, full);
#pragma unroll
          for (int j = 0; j < Cfg::kSfbAtoms; ++j)
            bulk_load_1d(sSfb + stage * Cfg::kSfbBytes + j * 2048, sfb_src + (uint64_t(j) * p.k_atoms + kt * 4u) * 512u,
                         2048u, full);
          }
          __syncwarp();
          if (++stage == S) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer: whole warp runs the loop, one elected lane issues ----------------
    {
      constexpr uint32_t idesc = make_idesc_nvfp4(kBlockM, BN);
      // descriptor words of stage 0, K block 0; the loop only moves the 14-bit start-address field of the low
      // word (shared addresses are below 256 KB, so the add never carries out of it)
      const uint64_t op0 = make_desc_sw128(sA), sf0 = make_desc_sf(sSfa);
      const uint32_t op_hi = uint32_t(op0 >> 32), sf_hi = uint32_t(sf0 >> 32);
      const uint32_t a_lo0 = uint32_t(op0), b_lo0 = uint32_t(make_desc_sw128(sB));
      const uint32_t sfa_lo0 = uint32_t(sf0), sfb_lo0 = uint32_t(make_desc_sf(sSfb));
      auto d64 = [](uint32_t lo, uint32_t hi) { return (uint64_t(hi) << 32) | lo; };
      uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0, titer = 0;
      bool ok = true, ready = false;
      for (uint32_t tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const uint32_t n0 = (tile / p.tiles_m) * BN;
        const uint32_t sfb_shift = (n0 & 127u) >> 5;  // TMEM column shift when the tile starts inside a 128-row scale block
        if (!mbar_wait_warp(bar_acc_empty + 8 * acc, acc_phase ^ 1u, abort_flag, kStatusAccEmptyTimeout, wait_limit)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + Cfg::kAccCol0 + acc * BN;
        for (uint32_t kt = 0; kt < num_k_tiles; ++kt, ++titer) {
          // `ready`: the probe issued one stage ago already saw this stage loaded; otherwise the warp waits here
          if (!ready && !mbar_wait_warp(bar_full + 8 * stage, phase, abort_flag, kStatusMmaTimeout, wait_limit)) {
            ok = false;
            break;
          }
          tc_fence_after();
          // probe the next stage now: the answer arrives while this stage's instructions are being issued
          const uint32_t nstage = stage + 1u == uint32_t(S) ? 0u : stage + 1u;
          const bool probe = mbar_test_wait(bar_full + 8 * nstage, nstage == 0u ? phase ^ 1u : phase);
          if (ktr && kt == 0 && lane == 0) p.trace[1204] = clock64();
          if (ktr && kt < 16 && lane == 0) p.trace[1220 + kt] = clock64();
          if (elect_one()) {
          const uint32_t a_lo = a_lo0 + stage * uint32_t(Cfg::kABytes >> 4), b_lo = b_lo0 + stage * uint32_t(Cfg::kBBytes >> 4);
          const uint32_t sfa_lo = sfa_lo0 + stage * uint32_t(Cfg::kSfaBytes >> 4), sfb_lo = sfb_lo0 + stage * uint32_t(Cfg::kSfbBytes >> 4);
          const uint32_t slot = tmem_base + (titer & 1u) * uint32_t(Cfg::kSfSlotCols);
          const uint32_t t_sfa = slot + Cfg::kSfaCol, t_sfb = slot + Cfg::kSfbCol;
          if (!(kDiag && (p.diag & 2u)) || kt == 0)
#pragma unroll
          for (int kb = 0; kb < 4; ++kb) {
            tc_cp_32x128b_warpx4(t_sfa + kb * 4, d64(sfa_lo + kb * 32, sf_hi));
#pragma unroll
            for (int j = 0; j < Cfg::kSfbAtoms; ++j)
              tc_cp_32x128b_warpx4(t_sfb + kb * (4 * Cfg::kSfbAtoms) + j * 4, d64(sfb_lo + j * 128 + kb * 32, sf_hi));
          }
          if (!(kDiag && (p.diag & 4u)))
#pragma unroll
          for (int kb = 0; kb < 4; ++kb) {
            tc_mma_nvfp4(d_tmem, d64(a_lo + kb * 2, op_hi), d64(b_lo + kb * 2, op_hi), idesc, t_sfa + kb * 4,
                         t_sfb + kb * (4 * Cfg::kSfbAtoms) + sfb_shift, (kt | kb) != 0u);
          }
          tc_commit(bar_empty + 8 * stage);
          }
          ready = __all_sync(0xFFFFFFFFu, probe) != 0;
          if (++stage == S) { stage = 0; phase ^= 1u; }
        }
        if (ktr && lane == 0) p.trace[1205] = clock64();
        if (ok && elect_one()) tc_commit(bar_acc_full + 8 * acc);
        __syncwarp();
        if (++acc == AS) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else {
    // ---------------- epilogue (warps 2..5) ----------------
    const uint32_t quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter+32) belong to this warp
    // this warp's copy of the tile's bias (as f32, halved for the fused GELU) and gate columns: fetched while the
    // main loop runs, so that their latency is not paid after the accumulator is ready (with few tiles per SM
    // nothing else would hide it)
    float* bias_smem = reinterpret_cast<float*>(smem_gen + (sBar + 256 - smem_base)) + quarter * 384;
    uint4* gate_smem = reinterpret_cast<uint4*>(bias_smem + 256);
    const float bias_mul = (p.act == 1u && !p.chain) ? 0.5f : 1.0f;  // the fused GELU works on x/2
    const float alpha = p.alpha * bias_mul;
    const uint32_t mode = (p.act == 1u ? 1u : 0u) | (p.chain ? 2u : 0u) | (p.gate ? 4u : 0u);
    uint32_t acc = 0, acc_phase = 0;
    bool ok = true;
    for (uint32_t tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      const uint32_t tm = tile % p.tiles_m, tn = tile / p.tiles_m;
      const uint32_t row = tm * kBlockM + quarter * 32 + lane;
      const uint32_t n0 = tn * BN;
      {
        const uint32_t col = n0 + lane * 8;
        const bool live = lane * 8 < uint32_t(BN) && col < p.n;  // n is a multiple of 8
        uint4 b4 = make_uint4(0, 0, 0, 0);
        if (p.bias && live) b4 = __ldg(reinterpret_cast<const uint4*>(p.bias + col));
        if (lane * 8 < uint32_t(BN)) {
          *reinterpret_cast<float4*>(bias_smem + lane * 8) =
              make_float4(bf16_lo(b4.x) * bias_mul, bf16_hi(b4.x) * bias_mul, bf16_lo(b4.y) * bias_mul, bf16_hi(b4.y) * bias_mul);
          *reinterpret_cast<float4*>(bias_smem + lane * 8 + 4) =
              make_float4(bf16_lo(b4.z) * bias_mul, bf16_hi(b4.z) * bias_mul, bf16_lo(b4.w) * bias_mul, bf16_hi(b4.w) * bias_mul);
        }
        if (p.gate) gate_smem[lane] = live ? __ldg(reinterpret_cast<const uint4*>(p.gate + col)) : make_uint4(0, 0, 0, 0);
        __syncwarp();
      }
      if (!mbar_wait_bounded(bar_acc_full + 8 * acc, acc_phase, abort_flag, kStatusEpilogueTimeout, wait_limit)) {
        ok = false;
        break;
      }
      tc_fence_after();
      if (ktr && warp == 2 && lane == 0) p.trace[1206] = clock64();
      const uint32_t t_addr = tmem_base + Cfg::kAccCol0 + acc * BN + ((quarter * 32u) << 16);
      {
        const bool skip = kDiag && (p.diag & 1u);
        switch (mode) {  // warp-uniform
          case 0: epilogue_tile<BN, false, false, false>(p, t_addr, row, n0, lane, alpha, bias_smem, gate_smem, skip); break;
          case 1: epilogue_tile<BN, true, false, false>(p, t_addr, row, n0, lane, alpha, bias_smem, gate_smem, skip); break;
          case 2: epilogue_tile<BN, false, true, false>(p, t_addr, row, n0, lane, alpha, bias_smem, gate_smem, skip); break;
          case 3: epilogue_tile<BN, true, true, false>(p, t_addr, row, n0, lane, alpha, bias_smem, gate_smem, skip); break;
          case 4: epilogue_tile<BN, false, false, true>(p, t_addr, row, n0, lane, alpha, bias_smem, gate_smem, skip); break;
          case 5: epilogue_tile<BN, true, false, true>(p, t_addr, row, n0, lane, alpha, bias_smem, gate_smem, skip); break;
          case 6: epilogue_tile<BN, false, true, true>(p, t_addr, row, n0, lane, alpha, bias_smem, gate_smem, skip); break;
          default: epilogue_tile<BN, true, true, true>(p, t_addr, row, n0, lane, alpha, bias_smem, gate_smem, skip); break;
        }
      }
      tc_fence_before();
      __syncwarp();
      if (ktr && warp == 2 && lane == 0) p.trace[1207] = clock64();
      if (lane == 0) mbar_arrive(bar_acc_empty + 8 * acc);
      if (++acc == AS) { acc = 0; acc_phase ^= 1u; }
    }
  }

  // ---------------- tear-down ----------------
  tc_fence_before();
  __syncthreads();
  if (ktr && threadIdx.x == 0) p.trace[1202] = clock64();
  if (threadIdx.x == 0 && *abort_flag != 0u) atomicCAS(p.status, 0u, *abort_flag);
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

static uint32_t env_u32(const char* name, uint32_t dflt) {
  if (!kDiag) return dflt;  // the default build reads no environment variable
  const char* v = getenv(name);
  return v ? uint32_t(strtoul(v, nullptr, 0)) : dflt;
}

uint32_t gemm_tile_n(uint32_t m, uint32_t n) {
  static uint32_t forced = env_u32("TNF_GEMM_TILE_N", 0);  // tuning knob: 64, 128 or 256
  if (forced == 64 || forced == 128 || forced == 256) return forced;
  // 256-wide tiles only when they still fill the SMs; 128-wide tiles also double-buffer the accumulator; with so
  // few tiles that half the SMs would idle, 64-wide ones: a CTA's time is what it has to pull in (its A tile
  // and its share of W) and what it writes out, and both shrink with the tile
  const uint64_t tm = (m + 127u) / 128u;
  if (tm * ((n + 255u) / 256u) >= 148u) return 256u;
  return tm * ((n + 127u) / 128u) * 2u <= 148u ? 64u : 128u;
}

template <int BN>
static cudaError_t launch_bn(const CUtensorMap& map_a, const CUtensorMap& map_w, GemmParams p, int sm_count,
                             cudaStream_t s) {
  using Cfg = TileCfg<BN>;
  static PerDeviceOnce once;
  if (once.first_use() >= 0) {  // the shared-memory opt-in is a per-device attribute of the function
    cudaError_t e = cudaFuncSetAttribute(nvfp4_gemm_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (e != cudaSuccess) return e;
  }
  static uint32_t diag = env_u32("TNF_GEMM_DIAG", 0);
  p.diag = diag;
  p.tiles_m = (p.m + kBlockM - 1) / kBlockM;
  p.tiles_n = (p.n + BN - 1) / BN;
  uint32_t tiles = p.tiles_m * p.tiles_n;
  if (tiles == 0) return cudaSuccess;
  uint32_t grid = std::min<uint32_t>(tiles, uint32_t(sm_count));
  return launch_pdl(nvfp4_gemm_kernel<BN>, dim3(grid), dim3(kThreads), Cfg::kSmemBytes, s, map_a, map_w, p);
}

cudaError_t launch_gemm_nvfp4(const CUtensorMap& map_a, const CUtensorMap& map_w, const GemmParams& p, int sm_count,
                              cudaStream_t s) {
  switch (gemm_tile_n(p.m, p.n)) {
    case 64: return launch_bn<64>(map_a, map_w, p, sm_count, s);
    case 128: return launch_bn<128>(map_a, map_w, p, sm_count, s);
    default: return launch_bn<256>(map_a, map_w, p, sm_count, s);
  }
}

}  // namespace tnf
