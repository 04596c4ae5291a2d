// tnf_norm_modulate_quantize: LayerNorm (no affine) + AdaLN modulation + NVFP4 activation
// quantiser in one pass over the rows.
//
// In front of every block linear the reference runs two dispatches, each with its own bf16 round
// trip of the [rows, dim] activation: op_layernorm (thinfer-core/src/ops/layernorm.rs:95-125,
// called at thinfer-models/src/qwen_image/dit.rs:521,757) and op_modulate = x * (1 + scale) + shift
// (thinfer-core/src/ops/bcast_modulate.rs:93-102, dit.rs:523-532,759-768); the NVFP4 path then adds
// the activation quantiser. Here a CTA works on one row at a time: a thread holds one 16-element block in
// registers, the row statistics are two block reductions (mean first, then the squared deviations,
// like the reference's two loops), the modulated value is rounded to bf16 exactly once (twice in
// chain mode, which keeps the reference's rounding between its two dispatches) and quantised from
// those bf16 bits -- so codes and scales equal what tnf_quantize_act makes of the bf16 output.
//
// Reductions add in a fixed tree order, not the reference's sequential order: the bf16 output is
// compared with the CPU restatement under a tolerance, the NVFP4 copy bit for bit against the
// quantiser applied to this kernel's own bf16 output.
#include <cuda_runtime.h>

#include <algorithm>

#include "context.h"
#include "internal.h"
#include "quant_dev.cuh"

namespace tnf {

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
  return v;
}

// sum over the CTA, the same value in every thread; `red` holds one float per warp. One barrier per
// call: the caller alternates between buffers so that a buffer is rewritten only two calls later,
// after every thread has passed the barrier of the call in between.
__device__ __forceinline__ float block_sum(float v, float* red, uint32_t warp, uint32_t lane, uint32_t n_warps) {
  v = warp_sum(v);
  if (lane == 0) red[warp] = v;
  __syncthreads();
  return warp_sum(lane < n_warps ? red[lane] : 0.0f);  // fixed tree order
}

__device__ __forceinline__ float bf16_round_f32(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// blockDim.x = nb_grid rounded up to a warp; thread t owns block t of a row (blocks past dim/16
// are padding of the device scale layout and produce zero scale bytes). The grid is persistent:
// a CTA takes rows blockIdx.x, blockIdx.x + gridDim.x, ... and loads its next row before the
// reductions of the current one, so the load latency of a row hides under the previous row's work.
template <bool kChain>
__global__ void __launch_bounds__(1024, 1)
    norm_modulate_quant_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ scale,
                               const uint16_t* __restrict__ shift, float mod_bias, float eps, uint32_t rows, uint32_t dim,
                               uint32_t nb_grid, float g, float inv_t, uint16_t* __restrict__ out_bf16,
                               uint8_t* __restrict__ codes, uint8_t* __restrict__ scales, uint32_t k_atoms) {
  __shared__ float red[4][32];
  __shared__ float inv_d_lut[128];
  const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5, n_warps = blockDim.x >> 5;
  const uint32_t nb = dim >> 4;
  const bool active = tid < nb;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");  // launched with programmatic dependent launch: see internal.h
  fill_inv_scale_lut(inv_d_lut, g, tid, blockDim.x);  // once per CTA; the first block_sum barrier publishes it
  const float inv_dim = __fdiv_rn(1.0f, float(dim));
  uint32_t par = 0;
  uint4 nxt[2] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
  auto fetch = [&](uint32_t r) {
    if (active && r < rows) {
      const uint4* p4 = reinterpret_cast<const uint4*>(x + uint64_t(r) * dim + uint64_t(tid) * 16u);
      nxt[0] = __ldg(p4);
      nxt[1] = __ldg(p4 + 1);
    }
  };
  fetch(blockIdx.x);
  for (uint32_t row = blockIdx.x; row < rows; row += gridDim.x) {  // CTA-uniform
    const uint32_t xw[8] = {nxt[0].x, nxt[0].y, nxt[0].z, nxt[0].w, nxt[1].x, nxt[1].y, nxt[1].z, nxt[1].w};
    fetch(row + gridDim.x);
    float v[16];
#pragma unroll
    for (int i = 0; i < 8; ++i) {  // inactive threads hold zeros
      v[2 * i] = active ? __uint_as_float(xw[i] << 16) : 0.0f;
      v[2 * i + 1] = active ? __uint_as_float(xw[i] & 0xFFFF0000u) : 0.0f;
    }
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) s += v[i];
    const float mean = block_sum(s, red[par], warp, lane, n_warps) * inv_dim;
    float ss = 0.0f;
    if (active) {
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float d = __fsub_rn(v[i], mean);
        ss = __fmaf_rn(d, d, ss);
      }
    }
    const float var = block_sum(ss, red[par + 1], warp, lane, n_warps) * inv_dim;
    const float inv = __frsqrt_rn(var + eps);
    par ^= 2u;

    uint32_t sc = 0;
    if (active) {
      uint4 s4[2] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)}, t4[2] = {s4[0], s4[0]};
      if (scale) {  // 64 bytes per thread, the same for every row: L1 hits after the first
        const uint4* sp = reinterpret_cast<const uint4*>(scale + uint64_t(tid) * 16u);
        const uint4* tp = reinterpret_cast<const uint4*>(shift + uint64_t(tid) * 16u);
        s4[0] = __ldg(sp);
        s4[1] = __ldg(sp + 1);
        t4[0] = __ldg(tp);
        t4[1] = __ldg(tp + 1);
      }
      const uint32_t sw[8] = {s4[0].x, s4[0].y, s4[0].z, s4[0].w, s4[1].x, s4[1].y, s4[1].z, s4[1].w};
      const uint32_t tw[8] = {t4[0].x, t4[0].y, t4[0].z, t4[0].w, t4[1].x, t4[1].y, t4[1].z, t4[1].w};
      uint32_t w[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float y[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          float n = __fmul_rn(__fsub_rn(v[2 * i + e], mean), inv);
          if (kChain) n = bf16_round_f32(n);
          if (scale) {
            const float sv = __uint_as_float(e ? (sw[i] & 0xFFFF0000u) : (sw[i] << 16));
            const float tv = __uint_as_float(e ? (tw[i] & 0xFFFF0000u) : (tw[i] << 16));
            n = __fadd_rn(__fmul_rn(n, __fadd_rn(sv, mod_bias)), tv);  // x * (s + bias) + t, separately rounded
          }
          y[e] = n;
        }
        const __nv_bfloat162 pk = __floats2bfloat162_rn(y[0], y[1]);
        w[i] = *reinterpret_cast<const uint32_t*>(&pk);
      }
      if (out_bf16) {
        uint4* o4 = reinterpret_cast<uint4*>(out_bf16 + uint64_t(row) * dim + uint64_t(tid) * 16u);
        o4[0] = make_uint4(w[0], w[1], w[2], w[3]);
        o4[1] = make_uint4(w[4], w[5], w[6], w[7]);
      }
      uint32_t lo, hi;
      sc = quant_block16_bf16(w, inv_d_lut, inv_t, lo, hi);
      *reinterpret_cast<uint2*>(codes + uint64_t(row) * (dim >> 1) + uint64_t(tid) * 8u) = make_uint2(lo, hi);
    }
    if (tid < nb_grid) {  // nb_grid is a multiple of 4: whole quads of lanes get here together
      uint32_t wv = sc << (8u * (tid & 3u));
      const uint32_t quad = 0xFu << (lane & ~3u);
      wv |= __shfl_xor_sync(quad, wv, 1);
      wv |= __shfl_xor_sync(quad, wv, 2);
      if ((tid & 3u) == 0u) *reinterpret_cast<uint32_t*>(scales + sf_device_offset(row, tid, k_atoms)) = wv;
    }
  }
}

}  // namespace

}  // namespace tnf

using namespace tnf;

extern "C" int32_t tnf_norm_modulate_quantize(tnf_ctx* ctx, const tnf_norm_quant_args* a) {
  if (!ctx || !a) {
    set_error("tnf_norm_modulate_quantize: null argument");
    return TNF_ERR_INVALID_ARGUMENT;
  }
  cudaError_t e = cudaSetDevice(ctx->device);
  if (e != cudaSuccess) return cuda_fail(e, "cudaSetDevice");
  if (a->m == 0 || a->k == 0 || a->k % 16 != 0 || a->k > 16384 || !(a->out_global > 0.0f) || !(a->eps >= 0.0f) ||
      (a->scale_bf16.len == 0) != (a->shift_bf16.len == 0)) {
    set_error("tnf_norm_modulate_quantize: m %u, k %u (a multiple of 16, at most 16384), out_global %g > 0, eps %g >= 0, "
              "scale and shift given together", a->m, a->k, double(a->out_global), double(a->eps));
    return TNF_ERR_INVALID_ARGUMENT;
  }
  int32_t st = TNF_OK;
  const uint64_t elems = uint64_t(a->m) * a->k;
  const uint8_t* x = resolve(ctx, a->x_bf16, elems * 2, "x_bf16", &st);
  if (!x) return st;
  const uint8_t *sc = nullptr, *sh = nullptr;
  if (a->scale_bf16.len) {
    sc = resolve(ctx, a->scale_bf16, uint64_t(a->k) * 2, "scale_bf16", &st);
    if (!sc) return st;
    sh = resolve(ctx, a->shift_bf16, uint64_t(a->k) * 2, "shift_bf16", &st);
    if (!sh) return st;
  }
  uint8_t* out = nullptr;
  if (a->out_bf16.len) {
    out = resolve(ctx, a->out_bf16, elems * 2, "out_bf16", &st);
    if (!out) return st;
  }
  uint8_t* codes = resolve(ctx, a->out_codes, elems / 2, "out_codes", &st);
  if (!codes) return st;
  const uint64_t sbytes = sf_device_bytes(a->m, a->k);
  uint8_t* scales = resolve(ctx, a->out_scales, sbytes, "out_scales", &st);
  if (!scales) return st;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(sc) | reinterpret_cast<uintptr_t>(sh) |
       reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(codes) | reinterpret_cast<uintptr_t>(scales)) & 15u) {
    set_error("tnf_norm_modulate_quantize: views must start on 16-byte boundaries");
    return TNF_ERR_INVALID_ARGUMENT;
  }
  const uint32_t k_atoms = sf_k_atoms(a->k);
  const uint32_t nb_grid = k_atoms * 4u;
  // rows past m of the last 128-row group are never visited: their scale bytes must be benign
  if (a->m % 128u) {
    const uint64_t full = uint64_t(a->m / 128u) * k_atoms * 512u;
    e = cudaMemsetAsync(scales + full, 0, sbytes - full, ctx->compute);
    if (e != cudaSuccess) return cuda_fail(e, "out_scales clear");
  }
  const uint32_t threads = (nb_grid + 31u) & ~31u;
  // persistent grid: as many CTAs as stay resident (about 1024 threads per SM at this kernel's register count)
  const uint32_t per_sm = std::max(1u, 1024u / threads);
  const uint32_t blocks = std::min<uint64_t>(a->m, uint64_t(ctx->sm_count) * per_sm);
  const float inv_t = 1.0f / (6.0f * a->out_global);  // same f32 operations as the quantiser and the oracle
  auto launch = [&](auto kernel) {
    return launch_pdl(kernel, dim3(blocks), dim3(threads), 0, ctx->compute, reinterpret_cast<const uint16_t*>(x),
                      reinterpret_cast<const uint16_t*>(sc), reinterpret_cast<const uint16_t*>(sh), a->mod_bias, a->eps, a->m,
                      a->k, nb_grid, a->out_global, inv_t, reinterpret_cast<uint16_t*>(out), codes, scales, k_atoms);
  };
  e = a->parity_mode ? launch(norm_modulate_quant_kernel<true>) : launch(norm_modulate_quant_kernel<false>);
  if (e != cudaSuccess) return cuda_fail(e, "norm_modulate_quant launch");
  return TNF_OK;
}
