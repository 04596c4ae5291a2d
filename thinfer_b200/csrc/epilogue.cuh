// Epilogue arithmetic shared by the two GEMM kernels, so that a linear gives the same bits whichever
// kernel the shape selects.
#pragma once
#include <cuda_bf16.h>
#include <cstdint>

namespace tnf {

// tanh-GELU, 0.5*x*(1+tanh(u)) with u = sqrt(2/pi)*(x + 0.044715 x^3)
// (thinfer-core/src/ops/gelu.rs:21-31). Fused mode: hardware tanh.approx (relative error ~2^-11,
// below the bf16 rounding of the result).
__device__ __forceinline__ float gelu_tanh_fast(float x) {
  float u = x * (0.7978845608028654f + 0.035677408136300125f * x * x);
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(u));
  float hx = 0.5f * x;
  return fmaf(hx, t, hx);
}
// Chain mode (parity_mode = 1) exists to be compared with the reference's op chain, so it evaluates the
// formula as written there, one separately rounded operation at a time, with the accurate tanhf.
__device__ __forceinline__ float gelu_tanh_exact(float x) {
  const float x3 = __fmul_rn(__fmul_rn(__fmul_rn(0.044715f, x), x), x);
  const float inner = __fmul_rn(0.7978845608028654f, __fadd_rn(x, x3));
  return __fmul_rn(__fmul_rn(0.5f, x), __fadd_rn(1.0f, tanhf(inner)));
}
template <bool kChain>
__device__ __forceinline__ float gelu_tanh(float x) {
  return kChain ? gelu_tanh_exact(x) : gelu_tanh_fast(x);
}

// ---- packed f32x2 arithmetic (sm_100): one instruction for two elements ------------------------------
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ uint64_t pack2u(uint32_t lo, uint32_t hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
// Fused tanh-GELU of two elements given y = x/2 (the caller folds the 1/2 into its alpha and bias):
// u = x (c0 + c1 x^2) = y (2 c0 + 8 c1 y^2), result = y + y tanh(u). Four packed operations and two tanh.approx.
__device__ __forceinline__ uint64_t gelu_tanh_fast2_half(uint64_t y2) {
  const uint64_t sq = mul2(y2, y2);
  const uint64_t pp = fma2(sq, pack2(8.0f * 0.035677408136300125f, 8.0f * 0.035677408136300125f),
                           pack2(2.0f * 0.7978845608028654f, 2.0f * 0.7978845608028654f));
  const uint64_t u2 = mul2(y2, pp);
  float u0, u1, t0, t1;
  unpack2(u2, u0, u1);
  asm("tanh.approx.f32 %0, %1;" : "=f"(t0) : "f"(u0));
  asm("tanh.approx.f32 %0, %1;" : "=f"(t1) : "f"(u1));
  return fma2(y2, pack2(t0, t1), y2);
}

__device__ __forceinline__ float bf16r(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }

// 8 accumulator columns -> 8 bf16 (one 16-byte vector of an output row). `b8` points at the 8 bias values
// in shared memory as f32 (zero without a bias); in the fused GELU variant alpha and the bias arrive halved.
// The fused variants work on packed pairs (fma.rn.f32x2): one FMA applies alpha and the bias to two columns.
template <bool kGelu, bool kChain, bool kGate>
__device__ __forceinline__ uint4 epilogue8(const uint32_t* r, float alpha, const float* b8, uint4 g4, uint4 s4) {
  const uint32_t gw[4] = {g4.x, g4.y, g4.z, g4.w}, sw[4] = {s4.x, s4.y, s4.z, s4.w};
  const float4 bl = *reinterpret_cast<const float4*>(b8), bh = *reinterpret_cast<const float4*>(b8 + 4);
  const float bv[8] = {bl.x, bl.y, bl.z, bl.w, bh.x, bh.y, bh.z, bh.w};
  uint32_t o[4];
#pragma unroll
  for (int h = 0; h < 4; ++h) {
    float v0, v1;
    if (kChain) {  // the reference's op chain: every step rounded to bf16, accurate tanh
      float v[2];
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        float x = bf16r(__uint_as_float(r[2 * h + e]) * alpha);
        x = bf16r(x + bv[2 * h + e]);  // adding the zero of "no bias" changes nothing
        if (kGelu) x = bf16r(gelu_tanh_exact(x));
        v[e] = x;
      }
      v0 = v[0];
      v1 = v[1];
    } else {
      uint64_t y2 = fma2(pack2u(r[2 * h], r[2 * h + 1]), pack2(alpha, alpha), pack2(bv[2 * h], bv[2 * h + 1]));
      if (kGelu) y2 = gelu_tanh_fast2_half(y2);
      unpack2(y2, v0, v1);
    }
    if (kGate) {
      v0 = fmaf(bf16_lo(gw[h]), v0, bf16_lo(sw[h]));
      v1 = fmaf(bf16_hi(gw[h]), v1, bf16_hi(sw[h]));
    }
    __nv_bfloat162 pk = __floats2bfloat162_rn(v0, v1);
    o[h] = *reinterpret_cast<uint32_t*>(&pk);
  }
  return make_uint4(o[0], o[1], o[2], o[3]);
}

}  // namespace tnf
