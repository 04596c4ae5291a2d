// Joint scaled-dot-product attention between the linears of a DiT block (op_sdpa, thinfer-core/src/ops/sdpa.rs:10-47;
// call site thinfer-models/src/qwen_image/dit.rs:618-655: full attention over [txt ++ img], has_mask = 0, D = 128):
// out = softmax(Q K^T * scale) V per (batch, head), bf16 in and out, f32 softmax statistics and accumulation.
//
// One CTA per (128 query rows, head, batch); flash-attention tiling over 128-key tiles, both products on the tensor
// cores (tcgen05.mma kind::f16); scores, probabilities and the running output live in TMEM:
//   columns   0-127  S: the score buffer (f32); a thread takes its row into registers at once, so one buffer serves
//                    both softmax groups in turn
//           128-255  P_0, P_1: the groups' probability buffers (bf16 pairs, 64 columns each)
//           256-319  Q (bf16 pairs), copied from shared memory once
//           384-511  O: the one running output (f32) both groups' products accumulate into
//   Both products read their A operand (Q, P) from tensor memory: neither costs shared-memory bandwidth in the loop.
//   warps 0, 10 TMA: the Q tile once, then K tiles (warp 0) and V tiles (warp 10) into two-stage rings ([128 rows x
//               64 bf16] boxes with 128-byte swizzle straight out of the [B, S, H, D] tensors: a head is a 256-byte
//               column window);
//   warp 1      one elected thread issues S = Q K_j^T (K the K-major B operand, 8 MMAs of K = 16) as soon as the previous
//               tile's score rows have been taken into registers, and O += P_g V_j in tile order, with V as it lies in
//               memory (keys x d: an MN-major B operand, no transpose pass);
//   warps 2-9   two softmax groups of four warps, one query row per thread (TMEM lane = row); the key tiles alternate
//               between them, so that one group's exponentials run under the other's TMEM traffic and waits. The
//               reference maximum m of a row is ONE chain through all tiles: the thread of tile j takes m_{j-1} from
//               the other group's thread of the same row (shared memory, an mbarrier per lane quarter and tile
//               parity), decides m_j -- it only moves when the tile's row maximum exceeds it by more than 8 in the
//               exp2 domain, so probabilities stay below 256 -- and publishes it before its expensive part. Only when m
//               moves is O rescaled (tcgen05.ld / mul / tcgen05.st by the thread that moved it, once the previous
//               product has completed); both threads of the row scale their partial sums. Then
//               p = exp2(s * scale * log2e - m), summed in f32, goes as bf16 pairs into P_g with tcgen05.st. At the
//               end the two partial sums are joined and each group writes half of the columns of O / l.
// Why this shape: a 128 x 128 x 16 MMA with both operands in shared memory reads 8 KB in its 64 cycles, all of an SM's
// 128 B/clk (measured: 119 cycles), and the TMA's writes of K and V come on top. With Q and P in tensor memory a key
// tile moves 128 KB through shared memory instead of 224 KB; with one O and one S instead of one per group there are
// TMEM columns for them.
// The reference's kernel is the same recurrence one key at a time in f32 (m' = max(m, s); o = o * exp(m - m') +
// exp(s - m') v; l likewise); here it runs a tile at a time, p is rounded to bf16 for the tensor cores, and exp is
// exp2 with the scale folded in: the result agrees with the f32 recurrence to bf16 rounding (tests: relative
// Frobenius error <= 4e-3 against the restated reference).
// Keys past s_k in the last tile get p = 0; query rows past s_q are computed and not stored. Every mbarrier wait is
// bounded; a wait that gives up sets the context's status word and the kernel returns.
#include <cuda.h>
#include <cuda_bf16.h>

#include <cstdint>

#include "../../include/thinfer_nvfp4.h"
#include "context.h"
#include "epilogue.cuh"
#include "internal.h"
#include "ptx.cuh"
#include "quant_dev.cuh"

namespace tnf {

namespace at {
constexpr int kThreads = 352;          // Q/K loader, MMA issuer, two softmax groups of four warps, V loader
constexpr uint32_t kD = 128;           // head dimension
constexpr uint32_t kRows = 128;        // query rows per CTA, keys per tile
constexpr uint32_t kSub = 128 * 128;   // one [128 rows x 64 bf16] swizzled box: 16 KB
constexpr uint32_t kTile = 2 * kSub;   // [128 x 128] bf16
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kSCol = 0;          // the score buffer (f32, 128 columns): a thread takes its row to registers at once, so one
                                       // buffer serves both groups in turn
constexpr uint32_t kPCol = 128;        // the groups' probability buffers (bf16 pairs) at columns 128 and 192
constexpr uint32_t kQCol = 256;        // the Q tile (bf16 pairs, 64 columns): the A operand of every score MMA
constexpr uint32_t kOCol = 384;        // the running output
constexpr float kLazy = 8.0f;          // the reference maximum moves only when the row maximum exceeds it by this much
constexpr uint32_t kSmemBytes = 1024 + 5 * kTile + 512 + 512 + 2048;  // Q | K x 2 | V x 2 | barriers | quantiser table | row statistics
}  // namespace at

struct SdpaParams {
  uint16_t* out;        // bf16 [b, s_q, h_q, 128], or null when only the NVFP4 copy is wanted
  uint8_t* q_codes;     // NVFP4 copy of the output as an [b * s_q, h_q * 128] operand: codes ...
  uint8_t* q_scales;    // ... and DEVICE-layout scales; null when not asked for
  float q_global, q_inv_t;
  uint32_t q_k_atoms;
  uint32_t* status;
  long long wait_limit;
  uint32_t s_q, s_k, h_q, h_kv;
  float scale_log2;  // scale * log2(e)
};

// MN-major operand, 128-byte swizzle: rows of 128 bytes hold 64 consecutive MN elements of one K index, 8-row (K)
// groups are 1024 bytes apart (SBO), the next 64 MN elements start `lbo_bytes` further (LBO).
__device__ __forceinline__ uint64_t make_desc_mn_sw128(uint32_t saddr, uint32_t lbo_bytes) {
  return uint64_t((saddr & 0x3FFFFu) >> 4) | (uint64_t(lbo_bytes >> 4) << 16) | (uint64_t(1024 >> 4) << 32) | (uint64_t(1) << 46) |
         (uint64_t(2) << 61);
}
__device__ __forceinline__ void tc_mma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_st_32x32b_x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
      "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
      "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]),
      "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_ld_32x32b_x8(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tmem_st_32x32b_x8(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr), "r"(r[0]), "r"(r[1]),
               "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}
__device__ __forceinline__ void tmem_st_32x32b_x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
      "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]: the A operand (bf16, two K elements per 32-bit column, lane = row) comes from tensor memory.
__device__ __forceinline__ void tc_mma_bf16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Two non-negative finite f32 -> bf16 pair by integer arithmetic (add half an ulp of bf16, keep the high halves: round
// to nearest, ties up): the hardware conversion shares the special-function pipe with exp2, which is this kernel's
// bottleneck, and a tie is one value in 65536.
__device__ __forceinline__ uint32_t pack_bf16x2_pos(float lo, float hi) {
  return __byte_perm(__float_as_uint(lo) + 0x8000u, __float_as_uint(hi) + 0x8000u, 0x7632);
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t d;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  return d;
}

__global__ void __launch_bounds__(at::kThreads, 1)
    sdpa_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                const __grid_constant__ CUtensorMap map_v, const SdpaParams p) {
  using namespace at;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t sQ = smem_base, sK = sQ + kTile, sV = sK + 2 * kTile, sBar = sV + 2 * kTile;
  const uint32_t q_full = sBar, k_full = sBar + 8, k_empty = sBar + 24, v_full = sBar + 40, v_empty = sBar + 56;
  const uint32_t s_full = sBar + 72, p_full = sBar + 88, pv_done = sBar + 104, s_free = sBar + 120;
  const uint32_t chain_bar = sBar + 136;  // [4 lane quarters][2 tile parities]: "m of tile j is published", 32 arrivals
  const uint32_t q_ready = sBar + 200;    // Q has been copied to tensor memory (128 arrivals)
  const uint32_t tmem_holder = sBar + 208;
  volatile uint32_t* tmem_holder_gen = reinterpret_cast<volatile uint32_t*>(smem_gen + (tmem_holder - smem_base));
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem_gen + (tmem_holder + 8u - smem_base));
  float* inv_d_lut = reinterpret_cast<float*>(smem_gen + (sBar + 512u - smem_base));  // the activation quantiser's table
  float* m_chain = reinterpret_cast<float*>(smem_gen + (sBar + 1024u - smem_base));   // [2 tile parities][128 rows]
  float* l_part = m_chain + 256;                                                       // [2 groups][128 rows]

  const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
  const uint32_t qt = blockIdx.x, hq = blockIdx.y, bb = blockIdx.z;
  const uint32_t hkv = (hq * p.h_kv) / p.h_q;
  const uint32_t q_row0 = bb * p.s_q + qt * kRows, k_row0 = bb * p.s_k;
  const uint32_t tiles = (p.s_k + kRows - 1u) / kRows;
  const long long wait_limit = p.wait_limit > 0 ? p.wait_limit : kDefaultWaitLimitCycles;

  if (tid == 0) {
    mbar_init(q_full, 1);
    for (uint32_t i = 0; i < 2; ++i) {
      mbar_init(k_full + 8 * i, 1);
      mbar_init(k_empty + 8 * i, 1);
      mbar_init(v_full + 8 * i, 1);
      mbar_init(v_empty + 8 * i, 1);
      mbar_init(s_full + 8 * i, 1);
      mbar_init(p_full + 8 * i, 128);
      mbar_init(pv_done + 8 * i, 1);
      mbar_init(s_free + 8 * i, 128);
    }
    for (uint32_t i = 0; i < 8; ++i) mbar_init(chain_bar + 8 * i, 32);
    mbar_init(q_ready, 128);
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&map_q);
    prefetch_tensormap(&map_k);
    prefetch_tensormap(&map_v);
  }
  if (p.q_codes) fill_inv_scale_lut(inv_d_lut, p.q_global, tid, kThreads);
  if (warp == 1) {
    tmem_alloc(tmem_holder, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder_gen;
  pdl_launch_dependents();
  pdl_wait();  // Q, K and V are the previous kernels' outputs

  // Key tile j belongs to group g = j % 2 and is the group's use = j / 2; it travels through ring stage g, score
  // buffer g, probability tile g and output g.
  if (warp == 0) {
    // ---------------- Q and K loader ----------------
    if (elect_one()) {
      mbar_arrive_expect_tx(q_full, kTile);
      tma_load_2d(sQ, &map_q, q_full, int32_t(hq * kD), int32_t(q_row0));
      tma_load_2d(sQ + kSub, &map_q, q_full, int32_t(hq * kD + 64), int32_t(q_row0));
    }
    __syncwarp();
    for (uint32_t j = 0; j < tiles; ++j) {
      const uint32_t g = j & 1u, use = j >> 1;
      if (use > 0 && !mbar_wait_warp(k_empty + 8 * g, (use - 1u) & 1u, abort_flag, kStatusProducerTimeout, wait_limit)) break;
      if (elect_one()) {
        mbar_arrive_expect_tx(k_full + 8 * g, kTile);
        tma_load_2d(sK + g * kTile, &map_k, k_full + 8 * g, int32_t(hkv * kD), int32_t(k_row0 + j * kRows));
        tma_load_2d(sK + g * kTile + kSub, &map_k, k_full + 8 * g, int32_t(hkv * kD + 64), int32_t(k_row0 + j * kRows));
      }
      __syncwarp();
    }
  } else if (warp == 10) {
    // ---------------- V loader (its ring frees later than K's: a warp of its own, so that K never waits behind V) ----------------
    for (uint32_t j = 0; j < tiles; ++j) {
      const uint32_t g = j & 1u, use = j >> 1;
      if (use > 0 && !mbar_wait_warp(v_empty + 8 * g, (use - 1u) & 1u, abort_flag, kStatusProducerTimeout, wait_limit)) break;
      if (elect_one()) {
        mbar_arrive_expect_tx(v_full + 8 * g, kTile);
        tma_load_2d(sV + g * kTile, &map_v, v_full + 8 * g, int32_t(hkv * kD), int32_t(k_row0 + j * kRows));
        tma_load_2d(sV + g * kTile + kSub, &map_v, v_full + 8 * g, int32_t(hkv * kD + 64), int32_t(k_row0 + j * kRows));
      }
      __syncwarp();
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    constexpr uint32_t idesc_qk = make_idesc_bf16(kRows, kRows);               // A and B K-major
    constexpr uint32_t idesc_pv = make_idesc_bf16(kRows, kD) | (1u << 16);     // B (V) MN-major
    bool ok = mbar_wait_warp(q_ready, 0, abort_flag, kStatusMmaTimeout, wait_limit);
    // S = Q K_j^T into the ONE score buffer, Q from tensor memory: with Q and K both in shared memory a 128 x 128 x 16
    // MMA needs 8 KB per 64 cycles, all of the SM's shared-memory bandwidth, and measured 119 cycles. Issued as soon as
    // the previous tile's scores have been taken into registers (that tile belongs to the other group) and K_j has
    // landed; the barriers alternate by tile parity although the buffer does not, so that no wait ever looks at a barrier
    // two phases behind.
    auto issue_s = [&](uint32_t j) -> bool {
      const uint32_t g = j & 1u, use = j >> 1;
      if (!mbar_wait_warp(k_full + 8 * g, use & 1u, abort_flag, kStatusMmaTimeout, wait_limit)) return false;
      if (j > 0 && !mbar_wait_warp(s_free + 8 * ((j - 1u) & 1u), ((j - 1u) >> 1) & 1u, abort_flag, kStatusAccEmptyTimeout, wait_limit)) return false;
      tc_fence_after();
      if (elect_one()) {
#pragma unroll
        for (uint32_t kk = 0; kk < 8; ++kk) {
          const uint32_t off = (kk >> 2) * kSub + (kk & 3u) * 32u;
          tc_mma_bf16_ts(tmem_base + kSCol, tmem_base + kQCol + kk * 8u, make_desc_sw128(sK + g * kTile + off), idesc_qk, kk != 0u);
        }
        tc_commit(s_full + 8 * g);
        tc_commit(k_empty + 8 * g);
      }
      __syncwarp();
      return true;
    };
    if (ok) ok = issue_s(0);
    if (ok && tiles > 1) ok = issue_s(1);
    for (uint32_t j = 0; j < tiles && ok; ++j) {
      const uint32_t g = j & 1u, use = j >> 1;
      if (j + 2 < tiles && !issue_s(j + 2)) break;
      if (!mbar_wait_warp(p_full + 8 * g, use & 1u, abort_flag, kStatusMmaTimeout, wait_limit)) break;
      if (!mbar_wait_warp(v_full + 8 * g, use & 1u, abort_flag, kStatusMmaTimeout, wait_limit)) break;
      tc_fence_after();
      if (elect_one()) {
#pragma unroll
        for (uint32_t kk = 0; kk < 8; ++kk)  // 16 keys each: P's packed columns 8kk.. in TMEM, V rows 16kk..
          tc_mma_bf16_ts(tmem_base + kOCol, tmem_base + kPCol + g * 64u + kk * 8u, make_desc_mn_sw128(sV + g * kTile + kk * 2048u, kSub),
                         idesc_pv, (j | kk) != 0u);
        tc_commit(pv_done + 8 * g);
        tc_commit(v_empty + 8 * g);
      }
      __syncwarp();
    }
  } else {
    // ---------------- softmax: two groups, one query row per thread ----------------
    const uint32_t g = (warp - 2u) >> 2, quarter = warp & 3u, row = quarter * 32u + lane;
    const uint32_t lane_addr = tmem_base + ((quarter * 32u) << 16);
    const uint32_t s_addr = lane_addr + kSCol, p_addr = lane_addr + kPCol + g * 64u, o_addr = lane_addr + kOCol;
    float m_known = -INFINITY, l = 0.0f;  // l is this group's partial row sum, relative to m_known
    bool ok = true;
    uint32_t s0[32], s1[32], s2[32], s3[32];
    uint32_t use = 0;
    if (g == 0) {
      // Q goes from shared to tensor memory once: as the A operand of the score MMAs it then costs no shared-memory
      // bandwidth. A thread undoes the 128-byte swizzle of its row: chunk c sits at position c ^ (row % 8).
      ok = mbar_wait_warp(q_full, 0, abort_flag, kStatusEpilogueTimeout, wait_limit);
      if (ok) {
        const uint8_t* qrow = smem_gen + (sQ - smem_base) + row * 128u;
#pragma unroll
        for (uint32_t c = 0; c < 8; ++c) {
          const uint4 a = *reinterpret_cast<const uint4*>(qrow + ((c ^ (row & 7u)) << 4));
          const uint4 b = *reinterpret_cast<const uint4*>(qrow + kSub + ((c ^ (row & 7u)) << 4));
          s0[c * 4] = a.x; s0[c * 4 + 1] = a.y; s0[c * 4 + 2] = a.z; s0[c * 4 + 3] = a.w;
          s1[c * 4] = b.x; s1[c * 4 + 1] = b.y; s1[c * 4 + 2] = b.z; s1[c * 4 + 3] = b.w;
        }
        tmem_st_32x32b_x32(lane_addr + kQCol, s0);
        tmem_st_32x32b_x32(lane_addr + kQCol + 32u, s1);
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive(q_ready);
      }
    }
    // m_{j}: published by the thread of tile j for the thread of tile j + 1 (the same row, the other group)
    auto chain_wait = [&](uint32_t j) -> bool {
      return mbar_wait_warp(chain_bar + 8 * (quarter * 2u + (j & 1u)), (j >> 1) & 1u, abort_flag, kStatusEpilogueTimeout, wait_limit);
    };
    auto adopt = [&](float m_new) {  // bring the partial sum to a new reference maximum
      if (m_new != m_known) {
        l *= ex2(m_known - m_new);  // m_known = -inf only while l = 0: ex2(-inf) = 0
        m_known = m_new;
      }
    };
    for (uint32_t j = g; j < tiles && ok; j += 2, ++use) {
      const uint32_t valid = min(kRows, p.s_k - j * kRows);  // keys of this tile that exist
      if (!mbar_wait_warp(s_full + 8 * g, use & 1u, abort_flag, kStatusEpilogueTimeout, wait_limit)) {
        ok = false;
        break;
      }
      tc_fence_after();
      // the whole score row goes to registers in one round trip (four loads in flight, one wait)
      tmem_ld_32x32b_x32(s_addr, s0);
      tmem_ld_32x32b_x32(s_addr + 32u, s1);
      tmem_ld_32x32b_x32(s_addr + 64u, s2);
      tmem_ld_32x32b_x32(s_addr + 96u, s3);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(s_free + 8 * g);  // the score buffer can take the group's next tile
      float mx = -INFINITY;
      auto row_max = [&](const uint32_t(&c)[32], uint32_t c4) {
        if (valid >= (c4 + 1u) * 32u) {
          float a = -INFINITY, b = -INFINITY, d = -INFINITY, e = -INFINITY;
#pragma unroll
          for (int i = 0; i < 32; i += 8) {  // three-input maxima: 16 instructions for 32 values
            a = max3(a, __uint_as_float(c[i]), __uint_as_float(c[i + 1]));
            b = max3(b, __uint_as_float(c[i + 2]), __uint_as_float(c[i + 3]));
            d = max3(d, __uint_as_float(c[i + 4]), __uint_as_float(c[i + 5]));
            e = max3(e, __uint_as_float(c[i + 6]), __uint_as_float(c[i + 7]));
          }
          mx = fmaxf(mx, fmaxf(fmaxf(a, b), fmaxf(d, e)));
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (c4 * 32u + uint32_t(i) < valid) mx = fmaxf(mx, __uint_as_float(c[i]));
        }
      };
      row_max(s0, 0);
      row_max(s1, 1);
      row_max(s2, 2);
      row_max(s3, 3);
      mx *= p.scale_log2;  // scale > 0: the maximum commutes with it
      // the chain: take m_{j-1}, decide m_j, publish it at once (the other group's next tile waits for nothing else)
      float alpha = 1.0f;
      if (j == 0) {
        m_known = mx;
      } else {
        if (!chain_wait(j - 1u)) {
          ok = false;
          break;
        }
        adopt(m_chain[((j - 1u) & 1u) * 128u + row]);
        if (mx > m_known + kLazy) {
          alpha = ex2(m_known - mx);
          l *= alpha;
          m_known = mx;
        }
      }
      m_chain[(j & 1u) * 128u + row] = m_known;
      mbar_arrive(chain_bar + 8 * (quarter * 2u + (j & 1u)));
      // A parity wait is only meaningful on a barrier that is at most one phase behind the awaited one. The group's own
      // previous product (tile j-2) is therefore awaited first -- it also frees the probability buffer --: its completion
      // implies tile j-3's, which puts the other group's barrier one phase before tile j-1's, awaited below.
      if (use > 0) {
        if (!mbar_wait_warp(pv_done + 8 * g, (use - 1u) & 1u, abort_flag, kStatusEpilogueTimeout, wait_limit)) {
          ok = false;
          break;
        }
      }
      if (j > 0 && __any_sync(0xFFFFFFFFu, alpha != 1.0f)) {
        // rare (the maximum jumped by more than 2^8): O is rescaled once every earlier product has completed (the pipe
        // runs them in order, so tile j-1's completion covers them all). This tile's product is issued only after this
        // thread's arrival below, and the next tile's after it.
        const uint32_t pj = j - 1u;
        if (!mbar_wait_warp(pv_done + 8 * (pj & 1u), (pj >> 1) & 1u, abort_flag, kStatusEpilogueTimeout, wait_limit)) {
          ok = false;
          break;
        }
        tc_fence_after();
        uint32_t o8[8];
#pragma unroll 1
        for (uint32_t c = 0; c < kD; c += 8u) {
          tmem_ld_32x32b_x8(o_addr + c, o8);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 8; ++i) o8[i] = __float_as_uint(__uint_as_float(o8[i]) * alpha);
          tmem_st_32x32b_x8(o_addr + c, o8);
        }
      }
      // p = exp2(s * scale_log2 - m), row sum in f32, P as bf16 pairs into the group's probability buffer
      const float neg_m = -m_known;
      const uint64_t sc2 = pack2(p.scale_log2, p.scale_log2), nm2 = pack2(neg_m, neg_m);
      uint64_t l01 = pack2(0.0f, 0.0f), l23 = l01;
      auto emit = [&](uint32_t(&c)[32], uint32_t c4) {
#pragma unroll
        for (int i = 0; i < 32; i += 2) {  // the scale and the shift for two scores in one packed FMA
          float x0, x1;
          unpack2(fma2(pack2u(c[i], c[i + 1]), sc2, nm2), x0, x1);
          c[i] = __float_as_uint(ex2(x0));
          c[i + 1] = __float_as_uint(ex2(x1));
        }
        if (valid < (c4 + 1u) * 32u) {  // only the last tile of a ragged s_k: keys that do not exist weigh nothing
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (c4 * 32u + uint32_t(i) >= valid) c[i] = 0u;
        }
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          l01 = add2(l01, pack2u(c[i], c[i + 1]));
          l23 = add2(l23, pack2u(c[i + 2], c[i + 3]));
        }
        uint32_t w[16];  // two probabilities per 32-bit column, key 2i in the low half
#pragma unroll
        for (int i = 0; i < 16; ++i) w[i] = pack_bf16x2_pos(__uint_as_float(c[2 * i]), __uint_as_float(c[2 * i + 1]));
        tmem_st_32x32b_x16(p_addr + c4 * 16u, w);
      };
      emit(s0, 0);
      emit(s1, 1);
      emit(s2, 2);
      emit(s3, 3);
      {
        float l0, l1, l2, l3;
        unpack2(l01, l0, l1);
        unpack2(l23, l2, l3);
        l += (l0 + l1) + (l2 + l3);
      }
      tmem_st_wait();
      tc_fence_before();  // this thread's TMEM reads and writes are ordered before the arrival below
      mbar_arrive(p_full + 8 * g);
    }
    // ---------------- O / (l_0 + l_1) -> global: each group half of the columns ----------------
    const uint32_t last = tiles - 1u;
    if (ok && (last & 1u) != g) {  // the last tile was the other group's: its m is the final one
      ok = chain_wait(last);
      if (ok) adopt(m_chain[(last & 1u) * 128u + row]);
    }
    // the group's own last product first (one phase ahead of what it has seen), then the very last one if it is the
    // other group's: the same rule about parity waits
    if (ok && use > 0) ok = mbar_wait_warp(pv_done + 8 * g, (use - 1u) & 1u, abort_flag, kStatusEpilogueTimeout, wait_limit);
    if (ok && (last & 1u) != g) ok = mbar_wait_warp(pv_done + 8 * (last & 1u), (last >> 1) & 1u, abort_flag, kStatusEpilogueTimeout, wait_limit);
    l_part[g * 128u + row] = l;
    asm volatile("bar.sync 1, 256;" ::: "memory");  // the eight softmax warps; every one of them gets here, whatever happened
    tc_fence_after();
    if (ok && __all_sync(0xFFFFFFFFu, *abort_flag == 0u)) {
      const float inv = 1.0f / (l + l_part[(g ^ 1u) * 128u + row]);
      const bool store = qt * kRows + row < p.s_q;
      const uint64_t grow = uint64_t(q_row0) + row;  // row of the [b * s_q, h_q * 128] matrix
      uint16_t* dst = p.out ? p.out + (grow * p.h_q + hq) * kD + g * 64u : nullptr;  // group g writes columns 64g .. 64g+63
      uint32_t sc4 = 0;  // the four block scales of this thread's 64 columns: one word of the scale layout
#pragma unroll 1
      for (uint32_t c2 = 0; c2 < 2; ++c2) {
        tmem_ld_32x32b_x32(o_addr + g * 64u + c2 * 32u, s0);
        tmem_ld_wait();
        if (store) {
          uint32_t w[16];  // 32 columns as bf16 pairs
#pragma unroll
          for (int i = 0; i < 16; ++i) w[i] = pack_bf16x2(__uint_as_float(s0[2 * i]) * inv, __uint_as_float(s0[2 * i + 1]) * inv);
          if (dst) {
#pragma unroll
            for (uint32_t q = 0; q < 4; ++q)
              *reinterpret_cast<uint4*>(dst + c2 * 32u + q * 8u) = make_uint4(w[q * 4], w[q * 4 + 1], w[q * 4 + 2], w[q * 4 + 3]);
          }
          if (p.q_codes) {
            // the out-projection's activation quantiser, on the bf16-rounded values: two 16-column blocks per 32 columns,
            // 8 code bytes each; the same bits tnf_quantize_act makes of the bf16 output
            uint32_t codes[4];
#pragma unroll
            for (uint32_t blk = 0; blk < 2; ++blk) {
              const uint32_t w8[8] = {w[blk * 8], w[blk * 8 + 1], w[blk * 8 + 2], w[blk * 8 + 3], w[blk * 8 + 4], w[blk * 8 + 5], w[blk * 8 + 6], w[blk * 8 + 7]};
              const uint32_t sc = quant_block16_bf16(w8, inv_d_lut, p.q_inv_t, codes[blk * 2], codes[blk * 2 + 1]);
              sc4 |= sc << (8u * (c2 * 2u + blk));
            }
            *reinterpret_cast<uint4*>(p.q_codes + grow * (uint64_t(p.h_q) * 64u) + hq * 64u + g * 32u + c2 * 16u) =
                make_uint4(codes[0], codes[1], codes[2], codes[3]);
          }
        }
      }
      if (p.q_scales && store) {
        // blocks hq*8 + g*4 .. +3 of the row: one 4-byte word of atom hq*2 + g (the launcher has cleared the padding)
        *reinterpret_cast<uint32_t*>(p.q_scales + ((grow >> 7) * p.q_k_atoms + hq * 2u + g) * 512u + (grow & 31u) * 16u + ((grow & 127u) >> 5) * 4u) = sc4;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
  if (tid == 0 && *abort_flag != 0u) atomicCAS(p.status, 0u, *abort_flag);
}

}  // namespace tnf

using namespace tnf;

extern "C" int32_t tnf_sdpa(tnf_ctx* ctx, const tnf_sdpa_args* a) {
  if (!ctx || !a) {
    set_error("tnf_sdpa: null context or args");
    return TNF_ERR_INVALID_ARGUMENT;
  }
  if (a->b == 0 || a->s_q == 0 || a->s_k == 0 || a->h_q == 0 || a->h_kv == 0 || a->d != at::kD || a->h_q % a->h_kv != 0 ||
      !(a->scale > 0.0f) || a->mask_mode != 0 || (a->flags & ~uint32_t(TNF_SDPA_OUT_NVFP4 | TNF_SDPA_NO_BF16_OUT)) ||
      ((a->flags & TNF_SDPA_NO_BF16_OUT) && !(a->flags & TNF_SDPA_OUT_NVFP4)) || ((a->flags & TNF_SDPA_OUT_NVFP4) && !(a->out_global > 0.0f))) {
    set_error("tnf_sdpa: b=%u s_q=%u s_k=%u h_q=%u h_kv=%u d=%u scale=%g mask_mode=%u (d must be 128, h_kv must divide h_q, "
              "scale > 0, mask_mode 0; flags 0x%x: NO_BF16_OUT needs OUT_NVFP4, which needs out_global > 0)", a->b, a->s_q, a->s_k, a->h_q, a->h_kv,
              a->d, a->scale, a->mask_mode, a->flags);
    return TNF_ERR_INVALID_ARGUMENT;
  }
  const uint64_t q_rows = uint64_t(a->b) * a->s_q, k_rows = uint64_t(a->b) * a->s_k;
  if (q_rows >= (1ull << 31) || k_rows >= (1ull << 31) || uint64_t(a->s_q + 127u) / 128u > 0x7FFFFFFFull || a->h_q > 65535u || a->b > 65535u) {
    set_error("tnf_sdpa: problem too large for the grid (b*s < 2^31, h_q and b <= 65535)");
    return TNF_ERR_INVALID_ARGUMENT;
  }
  int32_t st = TNF_OK;
  const uint64_t q_cols = uint64_t(a->h_q) * at::kD, kv_cols = uint64_t(a->h_kv) * at::kD;
  // leading dimensions in elements: q, k and v may be column windows of one wider matrix (the fused QKV output)
  const uint64_t q_ld = a->q_ld ? a->q_ld : q_cols, kv_ld = a->kv_ld ? a->kv_ld : kv_cols;
  if (q_ld < q_cols || kv_ld < kv_cols || q_ld % 8 != 0 || kv_ld % 8 != 0) {
    set_error("tnf_sdpa: q_ld %llu / kv_ld %llu must cover the heads (%llu / %llu elements) and be multiples of 8",
              (unsigned long long)q_ld, (unsigned long long)kv_ld, (unsigned long long)q_cols, (unsigned long long)kv_cols);
    return TNF_ERR_INVALID_ARGUMENT;
  }
  uint8_t* q = resolve(ctx, a->q, ((q_rows - 1) * q_ld + q_cols) * 2, "q", &st);
  if (!q) return st;
  uint8_t* k = resolve(ctx, a->k, ((k_rows - 1) * kv_ld + kv_cols) * 2, "k", &st);
  if (!k) return st;
  uint8_t* v = resolve(ctx, a->v, ((k_rows - 1) * kv_ld + kv_cols) * 2, "v", &st);
  if (!v) return st;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v)) & 15u) {
    set_error("tnf_sdpa: q, k and v must start on 16-byte boundaries");
    return TNF_ERR_INVALID_ARGUMENT;
  }
  uint8_t* out = nullptr;
  if (!(a->flags & TNF_SDPA_NO_BF16_OUT)) {
    out = resolve(ctx, a->out, q_rows * q_cols * 2, "out", &st);
    if (!out) return st;
  }
  uint8_t *q_codes = nullptr, *q_scales = nullptr;
  if (a->flags & TNF_SDPA_OUT_NVFP4) {  // the out-projection's A operand: [b * s_q, h_q * 128] codes + DEVICE scales
    q_codes = resolve(ctx, a->out_codes, q_rows * (q_cols / 2), "out_codes", &st);
    if (!q_codes) return st;
    q_scales = resolve(ctx, a->out_scales, sf_device_bytes(uint32_t(q_rows), uint32_t(q_cols)), "out_scales", &st);
    if (!q_scales) return st;
  }
  if (cudaSetDevice(ctx->device) != cudaSuccess) return cuda_fail(cudaGetLastError(), "cudaSetDevice");
  CUtensorMap mq, mk, mv;  // [rows, heads * 128] bf16, boxes of 64 columns x 128 rows, 128-byte swizzle
  if (!get_map(ctx, MapSpec{q, 2, q_cols, q_rows, q_ld * 2, 64, 128, 128}, &mq) ||
      !get_map(ctx, MapSpec{k, 2, kv_cols, k_rows, kv_ld * 2, 64, 128, 128}, &mk) ||
      !get_map(ctx, MapSpec{v, 2, kv_cols, k_rows, kv_ld * 2, 64, 128, 128}, &mv))
    return TNF_ERR_INVALID_ARGUMENT;
  SdpaParams p{};
  p.out = reinterpret_cast<uint16_t*>(out);
  if (q_codes) {
    p.q_codes = q_codes;
    p.q_scales = q_scales;
    p.q_global = a->out_global;
    p.q_inv_t = 1.0f / (6.0f * a->out_global);
    p.q_k_atoms = sf_k_atoms(uint32_t(q_cols));
    // benign (zero) scales where the kernel writes none: the K-padding atoms of every row block, and the rows of the
    // last 128-row block past the matrix
    const uint32_t used_atoms = uint32_t(q_cols / 64), row_blocks = uint32_t((q_rows + 127u) / 128u);
    if (used_atoms < p.q_k_atoms) {
      cudaError_t e = cudaMemset2DAsync(q_scales + uint64_t(used_atoms) * 512u, uint64_t(p.q_k_atoms) * 512u, 0,
                                        uint64_t(p.q_k_atoms - used_atoms) * 512u, row_blocks, ctx->compute);
      if (e != cudaSuccess) return cuda_fail(e, "out_scales padding clear");
    }
    if (q_rows % 128u != 0) {
      cudaError_t e = cudaMemsetAsync(q_scales + uint64_t(row_blocks - 1u) * p.q_k_atoms * 512u, 0, uint64_t(p.q_k_atoms) * 512u, ctx->compute);
      if (e != cudaSuccess) return cuda_fail(e, "out_scales last block clear");
    }
  }
  p.status = ctx->dwords;
  p.wait_limit = ctx->wait_limit_cycles;
  p.s_q = a->s_q; p.s_k = a->s_k; p.h_q = a->h_q; p.h_kv = a->h_kv;
  p.scale_log2 = a->scale * 1.4426950408889634f;
  static PerDeviceOnce once;
  if (once.first_use() >= 0) {
    cudaError_t e = cudaFuncSetAttribute(sdpa_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(at::kSmemBytes));
    if (e != cudaSuccess) return cuda_fail(e, "sdpa kernel attribute");
  }
  cudaError_t e = launch_pdl(sdpa_kernel, dim3((a->s_q + 127u) / 128u, a->h_q, a->b), dim3(at::kThreads), at::kSmemBytes, ctx->compute,
                             mq, mk, mv, p);
  if (e != cudaSuccess) return cuda_fail(e, "sdpa launch");
  return TNF_OK;
}
