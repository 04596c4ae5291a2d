// Skinny-M NVFP4 linear on the tensor cores with the operands swapped (M <= 16 rows: the M = 1 modulation
// linears of every block, thinfer-models/src/qwen_image/dit.rs:484-707): ONE launch computes
// out = epilogue(alpha * quant(A) W^T) as D[128 W rows, 16] = W_tile . quant(A)^T.
//
// With a handful of rows the work is reading W once (0.5625 B per weight): HBM-bound. Widening the codes on the CUDA
// cores costs about 1.4 instructions per weight whatever the trick (hardware cvt + packed f16, or byte permutes +
// dp4a, both measured), which caps that route near 2 TB/s. The block-scaled MMA takes the packed codes and the scale
// bytes as they lie in memory, so here the weight is the M-side operand:
//   * a CTA owns 128 consecutive output columns = 128 rows of W = one row block of W's device scale layout. Its
//     K tiles (128 rows x 256 elements: 16 KB of codes by one tiled TMA load, 2 KB of scales by one bulk copy) go
//     into a ring that holds as many stages as shared memory allows -- 9 of the 12 tiles at K = 3072 -- and all of
//     them are requested before anything else happens, so HBM streams at its own rate from the first microsecond;
//   * the activation quantiser IS the prologue (A is a few KB and every CTA re-quantises it: the one place where
//     fusing the quantiser into the GEMM costs nothing): every thread quantises some 16-element blocks exactly as
//     the stand-alone quantiser does (same operations, same table) and writes the codes straight into the
//     128-byte-swizzled K-major layout the MMA reads (16 rows per K tile, rows >= m zero) and the scale bytes into
//     512-byte scale atoms; A's loads are issued before the weight's so that they do not queue behind them;
//   * one elected thread copies the scale atoms to TMEM and issues tcgen05.mma kind::mxf4nvf4 with M = 128, N = 16
//     (four per K tile); the accumulator is 16 TMEM columns;
//   * four warps read the accumulator (lane = W row = output column, register i = activation row i) and apply the
//     usual epilogue (alpha, bias, tanh-GELU, gated residual, bf16 RNE); consecutive lanes store consecutive
//     output columns.
// Every mbarrier wait is bounded; a wait that gives up sets the context's status word and the kernel returns.
#include <cuda.h>
#include <cuda_bf16.h>

#include <algorithm>
#include <cstdint>

#include "epilogue.cuh"
#include "internal.h"
#include "ptx.cuh"
#include "quant_dev.cuh"

namespace tnf {

namespace sk {
constexpr int kThreads = 256;           // warp 0 loads, warp 1 issues MMAs, warps 4-7 read the accumulator; all quantise A
constexpr uint32_t kMaxM = 16;          // the MMA's N
constexpr uint32_t kTileK = 256;        // elements per K tile: 128 bytes of codes per row, four scale atoms
constexpr uint32_t kWBytes = 128 * 128; // W codes of one stage
constexpr uint32_t kSfBytes = 2048;     // four 512-byte scale atoms
constexpr uint32_t kStageBytes = kWBytes + kSfBytes;
constexpr uint32_t kABytes = kMaxM * 128;  // A codes of one K tile
constexpr uint32_t kTmemCols = 64;
constexpr uint32_t kAccCol = 0, kSfwCol = 16, kSfaCol = 32;  // accumulator | W scales (M side) | A scales (N side)
constexpr uint32_t kSmemMax = 227u * 1024u;
constexpr uint32_t kSmemTail = 1024u /* alignment slack */ + 2048u /* barriers, holder, flag | quantiser table */;
}  // namespace sk

struct SkinnyParams {
  const uint16_t* a;   // bf16 [m, k]
  const uint8_t* sfw;  // W scales, device layout
  const uint16_t* bias;
  const uint16_t* gate;
  const uint16_t* residual;
  uint16_t* out;
  uint32_t* status;
  long long wait_limit;
  uint32_t m, n, k, k_atoms, ldo, n_offset, act, chain, stages;
  float a_global, inv_t, alpha;
};

__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

__global__ void __launch_bounds__(sk::kThreads, 1)
    nvfp4_skinny_tc_kernel(const __grid_constant__ CUtensorMap map_w, const SkinnyParams p) {
  using namespace sk;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;  // the 128-byte swizzle atoms want 1024
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t S = p.stages;
  const uint32_t nkt = (p.k + kTileK - 1u) / kTileK;
  const uint32_t nb = p.k >> 4;
  const uint32_t sW = smem_base;                // [S][128 rows][128 B], swizzled by the TMA
  const uint32_t sSfw = sW + S * kWBytes;       // [S][4 atoms]
  const uint32_t sA = sSfw + S * kSfBytes;      // [nkt][16 rows][128 B], swizzled by the prologue
  const uint32_t sSfa = sA + nkt * kABytes;     // [nkt][4 atoms]
  const uint32_t sBar = sSfa + nkt * kSfBytes;
  const uint32_t bar_full = sBar, bar_empty = bar_full + 8u * S, bar_acc = bar_empty + 8u * S;
  const uint32_t tmem_holder = bar_acc + 8u;
  volatile uint32_t* tmem_holder_gen = reinterpret_cast<volatile uint32_t*>(smem_gen + (tmem_holder - smem_base));
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem_gen + (tmem_holder + 8u - smem_base));
  uint8_t* a_gen = smem_gen + (sA - smem_base);
  uint8_t* sfa_gen = smem_gen + (sSfa - smem_base);
  float* inv_d_lut = reinterpret_cast<float*>(smem_gen + (sBar + 1024u - smem_base));  // the barriers take < 1 KB
  const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
  const uint32_t row0 = blockIdx.x * 128u;  // first W row (output column) of this CTA
  const long long wait_limit = p.wait_limit > 0 ? p.wait_limit : kDefaultWaitLimitCycles;

  if (tid == 0) {
    for (uint32_t i = 0; i < S; ++i) {
      mbar_init(bar_full + 8u * i, 1);
      mbar_init(bar_empty + 8u * i, 1);
    }
    mbar_init(bar_acc, 1);
    *abort_flag = 0;
    fence_barrier_init();
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
  pdl_wait();  // before any access to global memory: A may be the previous kernel's output

  // ---- A's first blocks are requested before the weight, so that they do not wait behind it ----
  const uint32_t total = p.m * nb;  // 16-element blocks of A
  uint4 v0 = make_uint4(0, 0, 0, 0), v1 = v0;
  if (tid < total) {
    const uint32_t row = tid / nb, b = tid - row * nb;
    const uint4* src = reinterpret_cast<const uint4*>(p.a + uint64_t(row) * p.k + b * 16u);
    v0 = __ldg(src);
    v1 = __ldg(src + 1);
  }
  // ---- every stage of the ring is requested now ----
  const uint8_t* sfw_src = p.sfw + uint64_t(blockIdx.x) * p.k_atoms * 512u;
  auto load_tile = [&](uint32_t kt, uint32_t stage) {  // one elected lane
    const uint32_t full = bar_full + 8u * stage;
    mbar_arrive_expect_tx(full, kStageBytes);
    tma_load_2d(sW + stage * kWBytes, &map_w, full, int32_t(kt * 128u), int32_t(row0));
    bulk_load_1d(sSfw + stage * kSfBytes, sfw_src + uint64_t(kt) * kSfBytes, kSfBytes, full);
  };
  if (warp == 0 && elect_one())
    for (uint32_t kt = 0; kt < min(S, nkt); ++kt) load_tile(kt, kt);
  // ---- prologue: zero A's tiles and scale atoms, then quantise the real rows into them ----
  {
    uint4* z = reinterpret_cast<uint4*>(a_gen);  // sA and sSfa are adjacent
    const uint32_t n16 = nkt * (kABytes + kSfBytes) / 16u;
    for (uint32_t i = tid; i < n16; i += kThreads) z[i] = make_uint4(0, 0, 0, 0);
  }
  fill_inv_scale_lut(inv_d_lut, p.a_global, tid, kThreads);
  __syncthreads();
  for (uint32_t i = tid; i < total; i += kThreads) {
    const uint32_t row = i / nb, b = i - row * nb;
    if (i != tid) {
      const uint4* src = reinterpret_cast<const uint4*>(p.a + uint64_t(row) * p.k + b * 16u);
      v0 = __ldg(src);
      v1 = __ldg(src + 1);
    }
    const uint32_t w[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
    uint32_t lo, hi;
    const uint32_t sc = quant_block16_bf16(w, inv_d_lut, p.inv_t, lo, hi);
    // block b: K tile b/16; its 8 code bytes are half (b & 1) of 16-byte chunk (b % 16) / 2 of the row's 128 bytes;
    // the 128-byte swizzle stores chunk c of row r at chunk position c ^ (r % 8)
    const uint32_t kt = b >> 4, c = (b & 15u) >> 1;
    *reinterpret_cast<uint2*>(a_gen + kt * kABytes + row * 128u + ((c ^ (row & 7u)) << 4) + (b & 1u) * 8u) = make_uint2(lo, hi);
    // scale atom b/4: row r (< 32) has its four bytes at r*16, block b at byte b % 4
    sfa_gen[(b >> 2) * 512u + row * 16u + (b & 3u)] = uint8_t(sc);
  }
  fence_proxy_async();  // the MMA and the scale copies read what the threads above wrote
  __syncthreads();

  if (warp == 0) {
    // ---------------- loader: the tiles that did not fit the ring at the start ----------------
    uint32_t stage = 0, phase = 0;
    for (uint32_t kt = S; kt < nkt; ++kt) {
      if (!mbar_wait_warp(bar_empty + 8u * stage, phase, abort_flag, kStatusProducerTimeout, wait_limit)) break;
      if (elect_one()) load_tile(kt, stage);
      __syncwarp();
      if (++stage == S) {
        stage = 0;
        phase ^= 1u;
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    constexpr uint32_t idesc = make_idesc_nvfp4(128, kMaxM);
    uint32_t stage = 0, phase = 0;
    bool ok = true;
    for (uint32_t kt = 0; kt < nkt; ++kt) {
      if (!mbar_wait_warp(bar_full + 8u * stage, phase, abort_flag, kStatusMmaTimeout, wait_limit)) {
        ok = false;
        break;
      }
      tc_fence_after();
      if (elect_one()) {
        const uint32_t w_addr = sW + stage * kWBytes, a_addr = sA + kt * kABytes;
        const uint32_t sfw_addr = sSfw + stage * kSfBytes, sfa_addr = sSfa + kt * kSfBytes;
#pragma unroll
        for (uint32_t kb = 0; kb < 4; ++kb) {
          tc_cp_32x128b_warpx4(tmem_base + kSfwCol + kb * 4u, make_desc_sf(sfw_addr + kb * 512u));
          tc_cp_32x128b_warpx4(tmem_base + kSfaCol + kb * 4u, make_desc_sf(sfa_addr + kb * 512u));
        }
#pragma unroll
        for (uint32_t kb = 0; kb < 4; ++kb)
          tc_mma_nvfp4(tmem_base + kAccCol, make_desc_sw128(w_addr + kb * 32u), make_desc_sw128(a_addr + kb * 32u), idesc,
                       tmem_base + kSfwCol + kb * 4u, tmem_base + kSfaCol + kb * 4u, (kt | kb) != 0u);
        tc_commit(bar_empty + 8u * stage);
      }
      __syncwarp();
      if (++stage == S) {
        stage = 0;
        phase ^= 1u;
      }
    }
    if (ok && elect_one()) tc_commit(bar_acc);
    __syncwarp();
  } else if (warp >= 4) {
    // ---------------- epilogue: lane = W row = output column; register i = activation row i ----------------
    const uint32_t quarter = warp & 3u;
    const uint32_t n = row0 + quarter * 32u + lane;
    // the column's bias and gate are requested before the wait: their latency runs under the main loop
    const float bias = (p.bias && n < p.n) ? bf16_lo(uint32_t(__ldg(p.bias + n))) : 0.0f;
    const float gate = (p.gate && n < p.n) ? bf16_lo(uint32_t(__ldg(p.gate + n))) : 0.0f;
    if (mbar_wait_bounded(bar_acc, 0, abort_flag, kStatusEpilogueTimeout, wait_limit)) {
      tc_fence_after();
      uint32_t r[16];
      tmem_ld_32x32b_x16(tmem_base + ((quarter * 32u) << 16) + kAccCol, r);
      tmem_ld_wait();
      if (n < p.n) {
#pragma unroll
        for (uint32_t i = 0; i < kMaxM; ++i) {
          if (i < p.m) {
            float x = __uint_as_float(r[i]) * p.alpha;
            if (p.chain) x = bf16r(x);
            if (p.bias) {
              x += bias;
              if (p.chain) x = bf16r(x);
            }
            if (p.act == 1u) {
              x = p.chain ? gelu_tanh_exact(x) : gelu_tanh_fast(x);
              if (p.chain) x = bf16r(x);
            }
            if (p.gate) x = fmaf(gate, x, bf16_lo(uint32_t(p.residual[uint64_t(i) * p.n + n])));
            p.out[uint64_t(i) * p.ldo + p.n_offset + n] = __bfloat16_as_ushort(__float2bfloat16_rn(x));
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
  if (tid == 0 && *abort_flag != 0u) atomicCAS(p.status, 0u, *abort_flag);
}

// Ring depth for a K: what is left of shared memory beside A's tiles and scale atoms, at most one stage per K tile.
static uint32_t skinny_stages(uint32_t k) {
  const uint32_t nkt = (k + sk::kTileK - 1u) / sk::kTileK;
  const uint64_t fixed = uint64_t(nkt) * (sk::kABytes + sk::kSfBytes) + sk::kSmemTail;
  if (fixed >= sk::kSmemMax) return 0;
  return uint32_t(std::min<uint64_t>((sk::kSmemMax - fixed) / sk::kStageBytes, nkt));
}

bool skinny_tc_capable(uint32_t m, uint32_t n, uint32_t k) {
  return m >= 1 && m <= sk::kMaxM && k % 32 == 0 && n % 8 == 0 && skinny_stages(k) >= std::min(4u, (k + 255u) / 256u);
}

// Every CTA quantises all of A in its prologue, so the kernel's time grows with m * k (0.4 us per row at K = 3072,
// 0.9 at K = 9216) while quantiser + GEMM does not depend on m at these sizes. Measured back to back on rotating
// weights, the one launch wins up to m * k = 12288 (m = 4 at K = 3072: 7.5 against 7.8 us at N = 3072) and, where the
// other path has many tiles to get through, up to 24576 (m = 8 at N = 18432: 11.8 against 12.9 us).
bool skinny_tc_applies(uint32_t m, uint32_t n, uint32_t k) {
  return skinny_tc_capable(m, n, k) && uint64_t(m) * k <= (n >= 12288u ? 24576u : 12288u);
}

cudaError_t launch_skinny_tc(const CUtensorMap& map_w, const void* a_bf16, float a_global, const GemmParams& g, cudaStream_t s) {
  SkinnyParams p{};
  p.a = static_cast<const uint16_t*>(a_bf16);
  p.sfw = g.sfb;
  p.bias = g.bias;
  p.gate = g.gate;
  p.residual = g.residual;
  p.out = g.out[0];
  p.status = g.status;
  p.wait_limit = g.wait_limit;
  p.m = g.m; p.n = g.n; p.k = g.k;
  p.k_atoms = g.k_atoms;
  p.ldo = g.ldo;
  p.n_offset = g.n_offset;
  p.act = g.act;
  p.chain = g.chain;
  p.stages = skinny_stages(g.k);
  p.a_global = a_global;
  p.inv_t = 1.0f / (6.0f * a_global);
  p.alpha = g.alpha;
  if (p.stages == 0) return cudaErrorInvalidValue;
  const uint32_t nkt = (g.k + sk::kTileK - 1u) / sk::kTileK;
  const size_t smem = size_t(p.stages) * sk::kStageBytes + size_t(nkt) * (sk::kABytes + sk::kSfBytes) + sk::kSmemTail;
  static PerDeviceOnce once;
  if (once.first_use() >= 0) {
    cudaError_t e = cudaFuncSetAttribute(nvfp4_skinny_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(sk::kSmemMax));
    if (e != cudaSuccess) return e;
  }
  return launch_pdl(nvfp4_skinny_tc_kernel, dim3((g.n + 127u) / 128u), dim3(sk::kThreads), smem, s, map_w, p);
}

}  // namespace tnf
