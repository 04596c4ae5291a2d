// Device-side NVFP4 block quantiser shared by the standalone quantisers and the GEMM epilogue.
// Explicitly rounded IEEE f32 operations and the hardware cvt.rn.satfinite narrowing: bit-exact
// with the CPU oracle (see quant.cu).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp4.h>
#include <cuda_fp8.h>
#include <cstdint>

namespace tnf {

__device__ __forceinline__ float e4m3_decode_dev(uint32_t c) {
  uint32_t e = (c >> 3) & 0xFu, m = c & 7u;
  return e == 0 ? float(m) * 0.001953125f : __uint_as_float(((e + 120u) << 23) | (m << 20));
}

// Table of 1/(decode(sc) * g) for every E4M3 scale code, filled once per kernel (g is fixed for a
// launch) with the same two IEEE operations the per-block form used, so the codes do not change;
// it takes the division out of the per-block path. `lut` holds 128 floats; threads tid..tid+stride.
__device__ __forceinline__ void fill_inv_scale_lut(float* lut, float g, uint32_t tid, uint32_t stride) {
  for (uint32_t sc = tid; sc < 128u; sc += stride)
    lut[sc] = (sc == 0u || sc == 127u) ? 0.0f : __fdiv_rn(1.0f, __fmul_rn(e4m3_decode_dev(sc), g));
}

// 8 f32 values -> 4 code bytes in one word (value 0 in the low nibble of byte 0): four hardware
// conversions and one byte pack, instead of a shift and an OR per byte.
__device__ __forceinline__ uint32_t e2m1x8(float x0, float x1, float x2, float x3, float x4, float x5, float x6, float x7) {
  uint32_t out;
  asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n\t"
      "mov.b32 %0, {b0, b1, b2, b3};\n\t}"
      : "=r"(out)
      : "f"(x0), "f"(x1), "f"(x2), "f"(x3), "f"(x4), "f"(x5), "f"(x6), "f"(x7));
  return out;
}

// 16 f32 values -> 8 code bytes (returned as two u32) + the E4M3 scale byte.
__device__ __forceinline__ uint32_t quant_block16(const float (&x)[16], const float* inv_d_lut, float inv_t, uint32_t& lo,
                                                  uint32_t& hi) {
  float bmax = 0.0f;
#pragma unroll
  for (int i = 0; i < 16; ++i) bmax = fmaxf(bmax, fabsf(x[i]));
  float s_raw = __fmul_rn(bmax, inv_t);
  uint32_t sc = (uint32_t)__nv_cvt_float_to_fp8(s_raw, __NV_SATFINITE, __NV_E4M3) & 0xFFu;
  if (sc == 0x7Fu || sc == 0xFFu) sc = 0;  // NaN scale -> treated as a zero block
  sc &= 0x7Fu;
  lo = 0;
  hi = 0;
  if (sc != 0) {
    const float inv_d = inv_d_lut[sc];
    float y[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) y[i] = __fmul_rn(x[i], inv_d);
    lo = e2m1x8(y[0], y[1], y[2], y[3], y[4], y[5], y[6], y[7]);
    hi = e2m1x8(y[8], y[9], y[10], y[11], y[12], y[13], y[14], y[15]);
  }
  return sc;
}

// The same block from 8 packed bf16 pairs (element 2i in the low half of w[i]): the block maximum is
// taken on the packed values (exact: a maximum of bf16 magnitudes, NaNs dropped like fmaxf drops
// them), which halves the instructions and the live registers of the f32 form. Same bits out.
// kDirect: no table, 1/(decode(sc) * g) is computed for this one block with the table's two operations
// (a kernel whose threads quantise a single block each gains nothing from filling a table).
template <bool kDirect>
__device__ __forceinline__ uint32_t quant_block16_bf16_impl(const uint32_t (&w)[8], const float* inv_d_lut, float g, float inv_t,
                                                            uint32_t& lo, uint32_t& hi) {
  __nv_bfloat162 m2[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    m2[i] = __habs2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
  }
#pragma unroll
  for (int s = 4; s >= 1; s >>= 1)
#pragma unroll
    for (int i = 0; i < s; ++i) m2[i] = __hmax2(m2[i], m2[i + s]);
  const uint32_t mm = *reinterpret_cast<const uint32_t*>(&m2[0]);
  const float bmax = fmaxf(fmaxf(0.0f, __uint_as_float(mm << 16)), __uint_as_float(mm & 0xFFFF0000u));
  float s_raw = __fmul_rn(bmax, inv_t);
  uint32_t sc = (uint32_t)__nv_cvt_float_to_fp8(s_raw, __NV_SATFINITE, __NV_E4M3) & 0xFFu;
  if (sc == 0x7Fu || sc == 0xFFu) sc = 0;  // NaN scale -> treated as a zero block
  sc &= 0x7Fu;
  lo = 0;
  hi = 0;
  if (sc != 0) {
    const float inv_d = kDirect ? __fdiv_rn(1.0f, __fmul_rn(e4m3_decode_dev(sc), g)) : inv_d_lut[sc];
    float y[16];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      y[2 * i] = __fmul_rn(__uint_as_float(w[i] << 16), inv_d);
      y[2 * i + 1] = __fmul_rn(__uint_as_float(w[i] & 0xFFFF0000u), inv_d);
    }
    lo = e2m1x8(y[0], y[1], y[2], y[3], y[4], y[5], y[6], y[7]);
    hi = e2m1x8(y[8], y[9], y[10], y[11], y[12], y[13], y[14], y[15]);
  }
  return sc;
}

__device__ __forceinline__ uint32_t quant_block16_bf16(const uint32_t (&w)[8], const float* inv_d_lut, float inv_t,
                                                       uint32_t& lo, uint32_t& hi) {
  return quant_block16_bf16_impl<false>(w, inv_d_lut, 0.0f, inv_t, lo, hi);
}
__device__ __forceinline__ uint32_t quant_block16_bf16_direct(const uint32_t (&w)[8], float g, float inv_t, uint32_t& lo,
                                                              uint32_t& hi) {
  return quant_block16_bf16_impl<true>(w, nullptr, g, inv_t, lo, hi);
}

__device__ __forceinline__ uint64_t sf_device_offset(uint32_t r, uint32_t b, uint32_t k_atoms) {
  uint64_t atom = uint64_t(r >> 7) * k_atoms + (b >> 2);
  return atom * 512u + (r & 31u) * 16u + ((r & 127u) >> 5) * 4u + (b & 3u);
}


}  // namespace tnf
