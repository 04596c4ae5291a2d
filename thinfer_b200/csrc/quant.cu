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
#include "quant_dev.cuh"

namespace tnf {

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
  float gv = a > 0.0f ? __fdiv_rn(a, 2688.0f) : 1.0f;
  g[0] = gv;
  g[1] = __fdiv_rn(1.0f, __fmul_rn(6.0f, gv));  // 1/(6g), shared by every block
}

// ---- block quantiser --------------------------------------------------------------------------
// One 16-element block per (thread, round): in a round a warp takes 32 consecutive blocks of the
// block grid (1 KB of bf16). The grid is persistent (at most 6 CTAs of 8 warps per SM, 40
// registers): warp w handles rounds w, w + W, w + 2W, ... and issues the loads of its next round
// before the arithmetic of the current one, so a thread always has 64-128 bytes in flight and
// there is no half-empty last wave. With the device scale layout the block grid is PADDED (rows up
// to a multiple of 128, blocks up to k_atoms*4), each aligned group of 4 lanes owns one 4-byte
// scale word (row r, blocks 4i..4i+3), assembled with shuffles; padding words are written as zero.
// g_ptr (device: {g, 1/(6g)}) wins over g_val when not null. The launcher guarantees
// rows_grid*nb_grid < 2^32.
template <typename T, bool kDeviceLayout>
__global__ void __launch_bounds__(256, 6)
    quantize_kernel(const T* __restrict__ src, uint32_t rows, uint32_t k, const float* __restrict__ g_ptr, float g_val,
                    float inv_t_val, uint8_t* __restrict__ codes, uint8_t* __restrict__ scales, uint32_t k_atoms) {
  constexpr int kVec = sizeof(T) == 2 ? 2 : 4;  // 16-byte loads per block
  const uint32_t nb = k >> 4;
  const uint32_t nb_grid = kDeviceLayout ? k_atoms * 4u : nb;
  const uint32_t rows_grid = kDeviceLayout ? ((rows + 127u) & ~127u) : rows;
  const uint32_t total = rows_grid * nb_grid;
  const uint32_t n_rounds = (total + 31u) >> 5;  // the padded grid is a multiple of 32 blocks
  const uint32_t warps_total = gridDim.x * (blockDim.x >> 5);
  const uint32_t lane = threadIdx.x & 31u;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");  // launched with programmatic dependent launch: see internal.h
  const float g = g_ptr ? g_ptr[0] : g_val;
  const float inv_t = g_ptr ? g_ptr[1] : inv_t_val;
  __shared__ float inv_d_lut[128];
  fill_inv_scale_lut(inv_d_lut, g, threadIdx.x, blockDim.x);
  __syncthreads();

  uint32_t wr = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  // (row, block) of this lane in round wr; later rounds step by a fixed (rows, blocks) stride, so
  // the loop needs no division
  const uint32_t stride = warps_total * 32u;
  const uint32_t step_r = stride / nb_grid, step_b = stride - step_r * nb_grid;
  uint32_t t_n = wr * 32u + lane;
  uint32_t r_n = t_n / nb_grid, b_n = t_n - r_n * nb_grid;
  uint32_t r = 0, b = 0;
  bool valid = false;
  uint4 cur[kVec];
  auto fetch = [&](uint32_t& rr, uint32_t& bb, bool& ok, uint4(&raw)[kVec]) {  // loads round (t_n, r_n, b_n), then steps it
    rr = r_n;
    bb = b_n;
    ok = t_n < total && r_n < rows && b_n < nb;
    if (ok) {
      const uint4* p4 = reinterpret_cast<const uint4*>(src + uint64_t(r_n) * k + uint64_t(b_n) * 16u);
#pragma unroll
      for (int i = 0; i < kVec; ++i) raw[i] = __ldg(p4 + i);
    }
    t_n = (t_n < total) ? t_n + stride : total;  // saturates: no wrap-around past the last round
    r_n += step_r;
    b_n += step_b;
    if (b_n >= nb_grid) {
      b_n -= nb_grid;
      ++r_n;
    }
  };
  if (wr < n_rounds) fetch(r, b, valid, cur);
  while (wr < n_rounds) {  // warp-uniform
    uint32_t r_x = 0, b_x = 0;
    bool valid_n = false;
    uint4 nxt[kVec];
    fetch(r_x, b_x, valid_n, nxt);
    uint32_t sc = 0;
    if (valid) {
      uint32_t lo, hi;
      if constexpr (sizeof(T) == 2) {
        const uint32_t w[8] = {cur[0].x, cur[0].y, cur[0].z, cur[0].w, cur[1].x, cur[1].y, cur[1].z, cur[1].w};
        sc = quant_block16_bf16(w, inv_d_lut, inv_t, lo, hi);
      } else {
        float x[16];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          x[4 * i] = __uint_as_float(cur[i].x);
          x[4 * i + 1] = __uint_as_float(cur[i].y);
          x[4 * i + 2] = __uint_as_float(cur[i].z);
          x[4 * i + 3] = __uint_as_float(cur[i].w);
        }
        sc = quant_block16(x, inv_d_lut, inv_t, lo, hi);
      }
      *reinterpret_cast<uint2*>(codes + uint64_t(r) * (k >> 1) + uint64_t(b) * 8u) = make_uint2(lo, hi);
    }
    if (kDeviceLayout) {  // every lane of a round of the padded grid is in range: the shuffles are warp-wide
      uint32_t w = sc << (8u * (b & 3u));
      w |= __shfl_xor_sync(0xFFFFFFFFu, w, 1);
      w |= __shfl_xor_sync(0xFFFFFFFFu, w, 2);
      if ((b & 3u) == 0u) *reinterpret_cast<uint32_t*>(scales + sf_device_offset(r, b, k_atoms)) = w;
    } else if (valid) {
      scales[uint64_t(r) * nb + b] = uint8_t(sc);
    }
    wr += warps_total;
    r = r_x;
    b = b_x;
    valid = valid_n;
#pragma unroll
    for (int i = 0; i < kVec; ++i) cur[i] = nxt[i];
  }
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

// NVFP4 weight -> the dense bf16 image the dense-activation arm multiplies with: code x block scale WITHOUT the
// per-tensor scale, which the GEMM epilogue applies. E2M1 has two significant bits and E4M3 four, so every
// product is exact in bf16 (and below 6 * 448): the image loses nothing. One thread per 16-element block.
__device__ __forceinline__ float e2m1_decode_dev(uint32_t c) {
  const uint32_t m = c & 7u;
  const float v = m < 2u ? 0.5f * float(m) : __uint_as_float(((126u + (m >> 1)) << 23) | ((m & 1u) << 22));  // 0, .5, 1, 1.5, 2, 3, 4, 6
  return (c & 8u) ? -v : v;
}
__global__ void dequant_dense_kernel(const uint8_t* __restrict__ codes, const uint8_t* __restrict__ scales_device, uint32_t n,
                                     uint32_t nb, uint32_t k_atoms, uint16_t* __restrict__ out) {
  uint64_t t = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t >= uint64_t(n) * nb) return;
  const uint32_t r = uint32_t(t / nb), b = uint32_t(t % nb);
  const float d = e4m3_decode_dev(scales_device[sf_device_offset(r, b, k_atoms)] & 0x7Fu);
  const uint2 cw = *reinterpret_cast<const uint2*>(codes + (uint64_t(r) * nb + b) * 8u);
  const uint32_t w[2] = {cw.x, cw.y};
  uint32_t o[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint32_t by = (w[i >> 2] >> (8 * (i & 3))) & 0xFFu;
    __nv_bfloat162 pk = __floats2bfloat162_rn(e2m1_decode_dev(by & 0xFu) * d, e2m1_decode_dev(by >> 4) * d);
    o[i] = *reinterpret_cast<uint32_t*>(&pk);
  }
  uint4* dst = reinterpret_cast<uint4*>(out + (uint64_t(r) * nb + b) * 16u);
  dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
  dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
}

// ---- launchers ----------------------------------------------------------------------------------
cudaError_t launch_dequant_dense(const uint8_t* codes, const uint8_t* scales_device, uint32_t n, uint32_t k, uint16_t* out_bf16,
                                 cudaStream_t s) {
  const uint64_t threads = uint64_t(n) * (k >> 4);
  if (threads == 0) return cudaSuccess;
  dequant_dense_kernel<<<unsigned((threads + 255) / 256), 256, 0, s>>>(codes, scales_device, n, k >> 4, sf_k_atoms(k), out_bf16);
  return cudaGetLastError();
}

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
  const float inv_t_val = 1.0f / (6.0f * g_val);  // same f32 operations as the device and the oracle
  uint64_t threads = device_layout ? uint64_t((rows + 127u) & ~127u) * (k_atoms * 4u) : uint64_t(rows) * (k >> 4);
  if (threads == 0) return cudaSuccess;
  if (threads >= (uint64_t(1) << 32) - (uint64_t(1) << 20)) return cudaErrorInvalidValue;  // the kernel indexes blocks with 32 bits (one stride of headroom)
  static int sms_of[kMaxDevices] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= kMaxDevices) dev = 0;
  if (sms_of[dev] == 0 && (cudaDeviceGetAttribute(&sms_of[dev], cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms_of[dev] <= 0))
    sms_of[dev] = 148;
  const int sms = sms_of[dev];
  // persistent: 8 warps per CTA, one 32-block round per warp and iteration, at most 6 CTAs per SM
  unsigned blocks = unsigned(std::min<uint64_t>((threads + 255) / 256, uint64_t(sms) * 6));
  // Keep the SMs in the same L1/shared-memory split as the GEMMs that run before and after (they take
  // the whole 227 KB as shared memory): a kernel that prefers L1 makes every following GEMM launch wait
  // for the split to be switched back.
  static PerDeviceOnce carveout;
  if (carveout.first_use() >= 0) {  // a per-device attribute of each function
    cudaFuncSetAttribute(quantize_kernel<__nv_bfloat16, true>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    cudaFuncSetAttribute(quantize_kernel<__nv_bfloat16, false>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    cudaFuncSetAttribute(quantize_kernel<float, true>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    cudaFuncSetAttribute(quantize_kernel<float, false>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
  }
  if (dtype == 1) {
    auto* p = (const __nv_bfloat16*)src;
    if (device_layout) return launch_pdl(quantize_kernel<__nv_bfloat16, true>, dim3(blocks), dim3(256), 0, s, p, rows, k, g_ptr, g_val, inv_t_val, codes, scales, k_atoms);
    return launch_pdl(quantize_kernel<__nv_bfloat16, false>, dim3(blocks), dim3(256), 0, s, p, rows, k, g_ptr, g_val, inv_t_val, codes, scales, k_atoms);
  } else {
    auto* p = (const float*)src;
    if (device_layout) return launch_pdl(quantize_kernel<float, true>, dim3(blocks), dim3(256), 0, s, p, rows, k, g_ptr, g_val, inv_t_val, codes, scales, k_atoms);
    return launch_pdl(quantize_kernel<float, false>, dim3(blocks), dim3(256), 0, s, p, rows, k, g_ptr, g_val, inv_t_val, codes, scales, k_atoms);
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
