// Skinny-M NVFP4 linear (M <= 8 rows: the M = 1 modulation linears of every block,
// thinfer-models/src/qwen_image/dit.rs:484-707): out = epilogue(alpha * quant(A) W^T) in ONE launch.
//
// With a handful of rows the work is reading W once (0.5625 B per weight): HBM-bound. A 128-row MMA tile wastes
// 127/128 of the tensor pipe and its launch chain (quantiser kernel, then GEMM kernel) costs more than the
// transfer. Here the activation quantiser IS the prologue (A is a few KB and every CTA re-quantises it: the one
// place where fusing the quantiser into the GEMM costs nothing) and W is streamed by the CUDA cores:
//   * a CTA owns 64 consecutive output columns (half of a 128-row block of W's device scale layout) and stages
//     that half's scale bytes in shared memory, row-major; a warp has four rows, two of them in flight at any time
//     (128 rows per CTA, eight per warp one after the other, was latency-bound: 14 us for a 5 MB weight);
//   * every thread quantises some 16-element blocks of A exactly as the stand-alone quantiser does (same
//     operations, same table), and leaves the E2M1 values in shared memory as f16 pairs (exact) with the decoded
//     block scales beside them;
//   * a warp takes one W row at a time, its lanes covering 512 contiguous bytes of codes per step (32 elements
//     = two 16-blocks per lane); the codes are widened by the hardware (cvt.rn.f16x2.e2m1x2), the products of a
//     half block are summed in packed f16 (at most 8 x 36 in steps of 1/4: exact), the block sum is scaled by
//     a_scale * w_scale and accumulated in f32: the block-scaled dot product the tensor-core path computes;
//   * a shuffle reduction per row, then the usual epilogue (alpha, bias, tanh-GELU, gated residual, bf16 RNE).
// Operands are the buffers the tensor-core kernels read (codes row-major, device-layout scales).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cstdint>

#include "epilogue.cuh"
#include "internal.h"
#include "ptx.cuh"
#include "quant_dev.cuh"

namespace tnf {

namespace gemv {
constexpr int kMaxM = 8;
constexpr int kRows = 64;      // output columns per CTA: half of a 128-row block of W's scale layout
constexpr int kThreads = 512;  // 16 warps, 4 W rows each, two of them in flight; two CTAs share an SM, so the 288 CTAs
                               // of an 18432-column weight are one wave on 148 SMs
}  // namespace gemv

// two E2M1 codes of one byte -> f16x2 (element 2i in the low half), exact
__device__ __forceinline__ void e2m1x8_to_f16x2(uint32_t w, uint32_t (&h)[4]) {
  asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
      "mov.b32 {b0, b1, b2, b3}, %4;\n\t"
      "cvt.rn.f16x2.e2m1x2 %0, b0;\n\t"
      "cvt.rn.f16x2.e2m1x2 %1, b1;\n\t"
      "cvt.rn.f16x2.e2m1x2 %2, b2;\n\t"
      "cvt.rn.f16x2.e2m1x2 %3, b3;\n\t}"
      : "=r"(h[0]), "=r"(h[1]), "=r"(h[2]), "=r"(h[3])
      : "r"(w));
}

struct GemvParams {
  const uint16_t* a;  // bf16 [m, k]
  const uint8_t* w_codes;
  const uint8_t* w_scales;  // device layout
  const uint16_t* bias;
  const uint16_t* gate;
  const uint16_t* residual;
  uint16_t* out;
  uint32_t m, n, k, k_atoms, ldo, n_offset, act, chain;
  float a_global, inv_t, alpha;
};

template <int M>
__global__ void __launch_bounds__(gemv::kThreads, M <= 2 ? 2 : 1) nvfp4_gemv_kernel(const GemvParams p) {
  using namespace gemv;
  extern __shared__ __align__(16) uint8_t smem[];
  const uint32_t nb = p.k >> 4;                     // 16-element blocks per row
  const uint32_t kp = (p.k + 1023u) & ~1023u;       // A rows are padded to whole warp steps of 1024 elements
  const uint32_t nbp = p.k_atoms * 4u;              // blocks per row of the scale layout (padded to whole atoms)
  // [M][kp/2] E2M1 values of A as f16 pairs, permuted so that the 32 lanes of a warp step read consecutive 16-byte
  // pieces: the piece of lane l, quarter j of warp step c sits at ((c*4 + j)*32 + l) * 16 bytes
  __half2* a_h = reinterpret_cast<__half2*>(smem);
  float* a_s = reinterpret_cast<float*>(smem + size_t(M) * kp * 2);    // [M][nb] decoded block scales of A
  uint8_t* w_sf = reinterpret_cast<uint8_t*>(a_s + size_t(M) * nb);    // this CTA's W scales, row-major [64][nbp]
  __shared__ float inv_d_lut[128];
  __shared__ float e4m3_lut[128];
  const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
  pdl_launch_dependents();
  pdl_wait();  // A may be the previous kernel's output (and so may W be, right after a weight quantiser)
  // ---- the W rows of this warp go on their way first: 4096 elements (four 512-byte warp loads) per pass, one W row
  // per warp at a time; their HBM latency runs under the prologue below ----
  const uint32_t passes = (p.k + 4095u) >> 12;
  const uint32_t rows_here = min(uint32_t(kRows), p.n - min(p.n, blockIdx.x * kRows));
  const uint32_t my_rows = warp < rows_here ? (rows_here - warp + (kThreads / 32) - 1u) / (kThreads / 32) : 0u;
  const uint32_t iters = my_rows * passes;
  uint4 cur[4], nxt[4];
  auto fetch = [&](uint32_t it, uint4(&dst)[4]) {
    const uint32_t rr = warp + (it / passes) * (kThreads / 32), ps = it % passes;
    const uint8_t* wrow = p.w_codes + uint64_t(blockIdx.x * kRows + rr) * (p.k >> 1);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const uint32_t e0 = ((ps * 4u + uint32_t(c)) * 32u + lane) * 32u;
      dst[c] = e0 < p.k ? __ldg(reinterpret_cast<const uint4*>(wrow + (e0 >> 1))) : make_uint4(0, 0, 0, 0);
    }
  };
  if (iters) fetch(0, cur);
  if (iters > 1) fetch(1, nxt);
  {  // this CTA's half h of row block rb: in every atom, row r's scale bytes of quarters 2h and 2h+1 sit at r*16 + h*8
    const uint32_t rb = blockIdx.x >> 1, h = blockIdx.x & 1u;
    const uint8_t* src = p.w_scales + uint64_t(rb) * p.k_atoms * 512u + h * 8u;
    for (uint32_t i = tid; i < p.k_atoms * 32u; i += kThreads) {
      const uint32_t atom = i >> 5, r = i & 31u;
      const uint2 v = __ldg(reinterpret_cast<const uint2*>(src + atom * 512u + r * 16u));
      *reinterpret_cast<uint32_t*>(w_sf + r * nbp + atom * 4u) = v.x;
      *reinterpret_cast<uint32_t*>(w_sf + (32u + r) * nbp + atom * 4u) = v.y;
    }
  }
  fill_inv_scale_lut(inv_d_lut, p.a_global, tid, kThreads);
  for (uint32_t c = tid; c < 128u; c += kThreads) e4m3_lut[c] = e4m3_decode_dev(c);
  __syncthreads();
  // ---- prologue: quantise A (every CTA, the same bits as the stand-alone quantiser) ----
  for (uint32_t i = tid; i < uint32_t(M) * nb; i += kThreads) {
    const uint32_t row = i / nb, b = i - row * nb;
    uint32_t lo = 0, hi = 0, sc = 0;
    if (row < p.m) {
      const uint4* src = reinterpret_cast<const uint4*>(p.a + uint64_t(row) * p.k + b * 16u);
      const uint4 v0 = __ldg(src), v1 = __ldg(src + 1);
      const uint32_t w[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
      sc = quant_block16_bf16(w, inv_d_lut, p.inv_t, lo, hi);
    }
    uint32_t h[4];
    // block b is half of lane-chunk L = b/2 (warp step c = L/32, lane l = L%32): quarters j = 2*(b&1), 2*(b&1)+1
    const uint32_t L = b >> 1, j0 = (b & 1u) * 2u;
    uint4* dst = reinterpret_cast<uint4*>(a_h + (size_t(row) * kp >> 1)) + ((L >> 5) * 4u + j0) * 32u + (L & 31u);
    e2m1x8_to_f16x2(lo, h);
    dst[0] = make_uint4(h[0], h[1], h[2], h[3]);
    e2m1x8_to_f16x2(hi, h);
    dst[32] = make_uint4(h[0], h[1], h[2], h[3]);
    a_s[i] = e4m3_lut[sc];
  }
  __syncthreads();

  // ---- main loop ----
  float acc[M];
#pragma unroll
  for (int i = 0; i < M; ++i) acc[i] = 0.0f;
  for (uint32_t it = 0; it < iters; ++it) {
    const uint32_t rr = warp + (it / passes) * (kThreads / 32), ps = it % passes;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const uint32_t e0 = ((ps * 4u + uint32_t(c)) * 32u + lane) * 32u;  // first element of this lane's 32
      if (e0 < p.k) {
        const uint32_t wcw[4] = {cur[c].x, cur[c].y, cur[c].z, cur[c].w};
        const uint32_t b0 = e0 >> 4;  // two blocks: b0, b0 + 1 (same scale word of the atom)
        const uint32_t sf2 = *reinterpret_cast<const uint16_t*>(w_sf + rr * nbp + b0);  // consecutive lanes, consecutive pairs
        const float sw[2] = {e4m3_lut[sf2 & 0x7Fu], e4m3_lut[(sf2 >> 8) & 0x7Fu]};
        uint32_t wh[16];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint32_t t4[4];
          e2m1x8_to_f16x2(wcw[q], t4);
          wh[q * 4] = t4[0]; wh[q * 4 + 1] = t4[1]; wh[q * 4 + 2] = t4[2]; wh[q * 4 + 3] = t4[3];
        }
#pragma unroll
        for (int i = 0; i < M; ++i) {
          const uint4* ap = reinterpret_cast<const uint4*>(a_h + (size_t(i) * kp >> 1)) + (ps * 4u + uint32_t(c)) * 128u + lane;
          const float2 as2 = *reinterpret_cast<const float2*>(a_s + size_t(i) * nb + b0);
#pragma unroll
          for (int blk = 0; blk < 2; ++blk) {
            const uint4 a0 = ap[blk * 64], a1 = ap[blk * 64 + 32];
            const uint32_t av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            __half2 sacc = __float2half2_rn(0.0f);
#pragma unroll
            for (int j = 0; j < 8; ++j)
              sacc = __hfma2(*reinterpret_cast<const __half2*>(&av[j]), *reinterpret_cast<const __half2*>(&wh[blk * 8 + j]), sacc);
            const float bs = __low2float(sacc) + __high2float(sacc);  // each half: 8 products <= 36 in steps of 1/4, exact in f16
            acc[i] = fmaf(bs, (blk ? as2.y : as2.x) * sw[blk], acc[i]);
          }
        }
      }
    }
    if (ps + 1 == passes) {  // the row is complete: reduce over the lanes, epilogue, store
      const uint32_t n = blockIdx.x * kRows + rr;
#pragma unroll
      for (int i = 0; i < M; ++i) {
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) acc[i] += __shfl_xor_sync(0xFFFFFFFFu, acc[i], off);
      }
      if (lane < p.m) {
        float x = 0.0f;
#pragma unroll
        for (int i = 0; i < M; ++i)
          if (lane == uint32_t(i)) x = acc[i];
        x *= p.alpha;
        if (p.chain) x = bf16r(x);
        if (p.bias) {
          x += bf16_lo(uint32_t(p.bias[n]));
          if (p.chain) x = bf16r(x);
        }
        if (p.act == 1u) {
          x = p.chain ? gelu_tanh_exact(x) : gelu_tanh_fast(x);
          if (p.chain) x = bf16r(x);
        }
        if (p.gate) x = fmaf(bf16_lo(uint32_t(p.gate[n])), x, bf16_lo(uint32_t(p.residual[uint64_t(lane) * p.n + n])));
        p.out[uint64_t(lane) * p.ldo + p.n_offset + n] = __bfloat16_as_ushort(__float2bfloat16_rn(x));
      }
#pragma unroll
      for (int i = 0; i < M; ++i) acc[i] = 0.0f;
    }
#pragma unroll
    for (int c = 0; c < 4; ++c) cur[c] = nxt[c];
    if (it + 2 < iters) fetch(it + 2, nxt);  // two passes (both rows of a warp at K <= 4096) are always in flight
  }
}

static uint64_t gemv_smem_bytes(uint32_t m_pad, uint32_t k) {
  const uint64_t kp = (uint64_t(k) + 1023u) & ~uint64_t(1023);
  return uint64_t(m_pad) * kp * 2 + uint64_t(m_pad) * (k >> 4) * 4 + uint64_t(sf_k_atoms(k)) * 256;
}
static uint32_t gemv_m_pad(uint32_t m) { return m <= 1 ? 1u : (m <= 2 ? 2u : (m <= 4 ? 4u : 8u)); }

bool gemv_applies(uint32_t m, uint32_t n, uint32_t k) {
  // the quantised A (f16 pairs + scales) and the CTA's W scales must fit in shared memory with at least two CTAs to an SM
  return m >= 1 && m <= uint32_t(gemv::kMaxM) && k % 32 == 0 && n % 8 == 0 && gemv_smem_bytes(gemv_m_pad(m), k) <= 96u * 1024u;
}

template <int M>
static cudaError_t launch_gemv_m(const GemvParams& p, cudaStream_t s) {
  const size_t smem = gemv_smem_bytes(M, p.k);
  static PerDeviceOnce once;
  if (once.first_use() >= 0) {
    cudaError_t e = cudaFuncSetAttribute(nvfp4_gemv_kernel<M>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
    if (e != cudaSuccess) return e;
  }
  const unsigned blocks = (p.n + gemv::kRows - 1) / gemv::kRows;
  return launch_pdl(nvfp4_gemv_kernel<M>, dim3(blocks), dim3(gemv::kThreads), smem, s, p);
}

cudaError_t launch_gemv_nvfp4(const void* a_bf16, float a_global, const uint8_t* w_codes, const GemmParams& g, cudaStream_t s) {
  GemvParams p{};
  p.a = static_cast<const uint16_t*>(a_bf16);
  p.w_codes = w_codes;
  p.w_scales = g.sfb;
  p.bias = g.bias;
  p.gate = g.gate;
  p.residual = g.residual;
  p.out = g.out[0];
  p.m = g.m; p.n = g.n; p.k = g.k;
  p.k_atoms = g.k_atoms;
  p.ldo = g.ldo;
  p.n_offset = g.n_offset;
  p.act = g.act;
  p.chain = g.chain;
  p.a_global = a_global;
  p.inv_t = 1.0f / (6.0f * a_global);
  p.alpha = g.alpha;
  if (g.m <= 1) return launch_gemv_m<1>(p, s);
  if (g.m <= 2) return launch_gemv_m<2>(p, s);
  if (g.m <= 4) return launch_gemv_m<4>(p, s);
  return launch_gemv_m<8>(p, s);
}

}  // namespace tnf
