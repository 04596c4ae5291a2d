// NVFP4 quantisers for sm_100a: absolute maximum, weight and activation block quantisers,
// scale-layout conversion. Every f32 operation is an explicitly rounded IEEE operation
// (__fmul_rn / __fdiv_rn) so that the packed codes and scales match the CPU oracle bit for
// bit; the E4M3 / E2M1 narrowing uses the hardware cvt.rn.satfinite conversions.
//
// Stand in for the reference's act_quant (thinfer-core/src/ops/act_quant.rs:58-191) and its
// upload-time weight prep (thinfer-core/src/ops/weight_prep.rs:86-163). As there, the block
// parameter is narrowed to its storage type first and the codes are computed against the
// stored value; an all-zero block gets a zero scale and zero codes.
#include <cuda_bf16.h>
#include <cuda_fp4.h>
#include <cuda_fp8.h>
#include <cstdint>

#include "internal.h"

namespace tnf {

__device__ __forceinline__ float e4m3_decode_dev(uint32_t c) {
  uint32_t e = (c >> 3) & 0xFu, m = c & 7u;
  return e == 0 ? float(m) * 0.001953125f : __uint_as_float(((e + 120u) << 23) | (m << 20));
}

// 16 f32 values -> 8 code bytes (returned as two u32) + the E4M3 scale byte.
__device__ __forceinline__ uint32_t quant_block16(const float (&x)[16], float g, uint32_t& lo, uint32_t& hi) {
  float bmax = 0.0f;
#pragma unroll
  for (int i = 0; i < 16; ++i) bmax = fmaxf(bmax, fabsf(x[i]));
  float t = __fmul_rn(6.0f, g);
  float inv_t = __fdiv_rn(1.0f, t);
  float s_raw = __fmul_rn(bmax, inv_t);
  uint32_t sc = (uint32_t)__nv_cvt_float_to_fp8(s_raw, __NV_SATFINITE, __NV_E4M3) & 0xFFu;
  if (sc == 0x7Fu || sc == 0xFFu) sc = 0;  // NaN scale -> treated as a zero block
  sc &= 0x7Fu;
  lo = 0;
  hi = 0;
  if (sc != 0) {
    float d = __fmul_rn(e4m3_decode_dev(sc), g);
    float inv_d = __fdiv_rn(1.0f, d);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float2 v = make_float2(__fmul_rn(x[2 * i], inv_d), __fmul_rn(x[2 * i + 1], inv_d));
      uint32_t b = (uint32_t)__nv_cvt_float2_to_fp4x2(v, __NV_E2M1, cudaRoundNearest) & 0xFFu;
      if (i < 4) lo |= b << (8 * i);
      else hi |= b << (8 * (i - 4));
    }
  }
  return sc;
}

__device__ __forceinline__ uint64_t sf_device_offset(uint32_t r, uint32_t b, uint32_t k_atoms) {
  uint64_t atom = uint64_t(r >> 7) * k_atoms + (b >> 2);
  return atom * 512u + (r & 31u) * 16u + ((r & 127u) >> 5) * 4u + (b & 3u);
}

// ---- absolute maximum -----------------------------------------------------------------------
template <typename T>
__global__ void amax_kernel(const T* __restrict__ x, uint64_t n, uint32_t* __restrict__ out_bits) {
  float m = 0.0f;
  uint64_t stride = uint64_t(gridDim.x) * blockDim.x;
  for (uint64_t i = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    float v;
    if constexpr (sizeof(T) == 2) v = __bfloat162float(x[i]);
    else v = x[i];
    m = fmaxf(m, fabsf(v));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
  if ((threadIdx.x & 31) == 0) atomicMax(out_bits, __float_as_uint(m));  // non-negative floats order as uints
}

// amax bits -> per-tensor scale amax/(6*448), 1.0 for an all-zero tensor.
__global__ void global_scale_kernel(const uint32_t* amax_bits, float* g) {
  float a = __uint_as_float(*amax_bits);
  *g = a > 0.0f ? __fdiv_rn(a, 2688.0f) : 1.0f;
}

// ---- block quantiser --------------------------------------------------------------------------
// One thread per 16-element block over the PADDED block grid (rows up to a multiple of 128,
// blocks up to k_atoms*4) when the scales go to the device layout, so that padding bytes are
// written as zero. g_ptr (device) wins over g_val when not null.
template <typename T, bool kDeviceLayout>
__global__ void quantize_kernel(const T* __restrict__ src, uint32_t rows, uint32_t k, const float* __restrict__ g_ptr,
                                float g_val, uint8_t* __restrict__ codes, uint8_t* __restrict__ scales,
                                uint32_t k_atoms) {
  const uint32_t nb = k >> 4;
  const uint32_t nb_grid = kDeviceLayout ? k_atoms * 4u : nb;
  const uint32_t rows_grid = kDeviceLayout ? ((rows + 127u) & ~127u) : rows;
  uint64_t t = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t >= uint64_t(rows_grid) * nb_grid) return;
  uint32_t r = uint32_t(t / nb_grid), b = uint32_t(t % nb_grid);
  if (r >= rows || b >= nb) {
    if (kDeviceLayout) scales[sf_device_offset(r, b, k_atoms)] = 0;
    return;
  }
  const float g = g_ptr ? *g_ptr : g_val;
  float x[16];
  const T* p = src + uint64_t(r) * k + uint64_t(b) * 16u;
  if constexpr (sizeof(T) == 2) {
    const uint4* p4 = reinterpret_cast<const uint4*>(p);
    uint4 v0 = __ldg(p4), v1 = __ldg(p4 + 1);
    uint32_t w[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      x[2 * i] = __uint_as_float(w[i] << 16);
      x[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    }
  } else {
    const float4* p4 = reinterpret_cast<const float4*>(p);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float4 v = __ldg(p4 + i);
      x[4 * i] = v.x; x[4 * i + 1] = v.y; x[4 * i + 2] = v.z; x[4 * i + 3] = v.w;
    }
  }
  uint32_t lo, hi;
  uint32_t sc = quant_block16(x, g, lo, hi);
  *reinterpret_cast<uint2*>(codes + uint64_t(r) * (k >> 1) + uint64_t(b) * 8u) = make_uint2(lo, hi);
  if (kDeviceLayout) scales[sf_device_offset(r, b, k_atoms)] = uint8_t(sc);
  else scales[uint64_t(r) * nb + b] = uint8_t(sc);
}

// canonical [rows, k/16] -> device layout, padding written as zero
__global__ void scales_to_device_kernel(const uint8_t* __restrict__ in, uint32_t rows, uint32_t nb, uint32_t k_atoms,
                                        uint8_t* __restrict__ out) {
  const uint32_t nb_grid = k_atoms * 4u, rows_grid = (rows + 127u) & ~127u;
  uint64_t t = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t >= uint64_t(rows_grid) * nb_grid) return;
  uint32_t r = uint32_t(t / nb_grid), b = uint32_t(t % nb_grid);
  out[sf_device_offset(r, b, k_atoms)] = (r < rows && b < nb) ? in[uint64_t(r) * nb + b] : uint8_t(0);
}

// ---- launchers ----------------------------------------------------------------------------------
cudaError_t launch_amax(const void* x, int dtype, uint64_t n, uint32_t* amax_bits, cudaStream_t s) {
  cudaError_t e = cudaMemsetAsync(amax_bits, 0, 4, s);
  if (e != cudaSuccess) return e;
  int blocks = int(std::min<uint64_t>((n + 1023) / 1024, 148ull * 8));
  if (blocks < 1) blocks = 1;
  if (dtype == 1) amax_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>((const __nv_bfloat16*)x, n, amax_bits);
  else amax_kernel<float><<<blocks, 256, 0, s>>>((const float*)x, n, amax_bits);
  return cudaGetLastError();
}

cudaError_t launch_global_scale(const uint32_t* amax_bits, float* g, cudaStream_t s) {
  global_scale_kernel<<<1, 1, 0, s>>>(amax_bits, g);
  return cudaGetLastError();
}

cudaError_t launch_quantize(const void* src, int dtype, uint32_t rows, uint32_t k, const float* g_ptr, float g_val,
                            uint8_t* codes, uint8_t* scales, bool device_layout, cudaStream_t s) {
  const uint32_t k_atoms = sf_k_atoms(k);
  uint64_t threads = device_layout ? uint64_t((rows + 127u) & ~127u) * (k_atoms * 4u) : uint64_t(rows) * (k >> 4);
  if (threads == 0) return cudaSuccess;
  unsigned blocks = unsigned((threads + 255) / 256);
  if (dtype == 1) {
    auto* p = (const __nv_bfloat16*)src;
    if (device_layout) quantize_kernel<__nv_bfloat16, true><<<blocks, 256, 0, s>>>(p, rows, k, g_ptr, g_val, codes, scales, k_atoms);
    else quantize_kernel<__nv_bfloat16, false><<<blocks, 256, 0, s>>>(p, rows, k, g_ptr, g_val, codes, scales, k_atoms);
  } else {
    auto* p = (const float*)src;
    if (device_layout) quantize_kernel<float, true><<<blocks, 256, 0, s>>>(p, rows, k, g_ptr, g_val, codes, scales, k_atoms);
    else quantize_kernel<float, false><<<blocks, 256, 0, s>>>(p, rows, k, g_ptr, g_val, codes, scales, k_atoms);
  }
  return cudaGetLastError();
}

cudaError_t launch_scales_to_device(const uint8_t* in, uint32_t rows, uint32_t k, uint8_t* out, cudaStream_t s) {
  const uint32_t k_atoms = sf_k_atoms(k);
  uint64_t threads = uint64_t((rows + 127u) & ~127u) * (k_atoms * 4u);
  if (threads == 0) return cudaSuccess;
  scales_to_device_kernel<<<unsigned((threads + 255) / 256), 256, 0, s>>>(in, rows, k >> 4, k_atoms, out);
  return cudaGetLastError();
}

}  // namespace tnf
