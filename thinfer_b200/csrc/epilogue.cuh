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

__device__ __forceinline__ float bf16r(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }

}  // namespace tnf
