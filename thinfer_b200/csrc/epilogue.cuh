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

}  // namespace tnf
