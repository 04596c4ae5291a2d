// tnf_linear_nvfp4_noalloc: the NVFP4 linear for callers that must not allocate device memory.
//
// tnf_linear_nvfp4 keeps the quantised copy of the activations (E2M1 codes + device-layout
// E4M3 scales) in scratch that the context grows on demand with cudaMalloc. A caller that runs
// under a fixed memory plan -- every byte of the device handed out up front by its own arena, a
// latency-critical serving thread that may not hit the driver's allocator, an embedding host
// that forbids allocation after start-up -- cannot take that path. This entry point runs the
// same two kernels (activation quantiser, then the tcgen05 GEMM with the fused epilogue) with
// the scratch in a fixed array that is part of the loaded library image.
//
// Limits and rules:
//   * the array is kScratchBytes (16 MiB) and every GPU that loads the library holds it until
//     the process exits; a linear needs m*k/2 bytes of codes plus the device-layout scales of an
//     [m,k] operand (tnf_device_scales_bytes); larger problems are refused with
//     TNF_ERR_INVALID_ARGUMENT and nothing is launched;
//   * the first call on a device looks the array's device address up (cudaGetSymbolAddress with
//     that device current). Make that first call before any stream capture;
//   * all calls share the one array and it keeps the previous call's contents. Nothing in it has
//     to start at zero: the quantiser rewrites every byte the GEMM will read, including the zero
//     padding of the scale layout, and rows past m are zero-filled by the TMA loads. Two calls
//     whose kernels overlap on the GPU (different streams, different contexts of one device)
//     race on the array: keep them stream-ordered;
//   * no cudaMalloc / cudaFree / allocating library routine is called; tensor maps are built on
//     the host stack and not cached.
#include <mutex>

#include "context.h"

namespace {

constexpr uint64_t kScratchBytes = 16ull << 20;
static __device__ __align__(256) uint8_t g_noalloc_scratch[kScratchBytes];

// In host code `g_noalloc_scratch` is only a stand-in for the symbol; the address a kernel can use
// comes from cudaGetSymbolAddress, per device.
constexpr int kMaxDevices = 64;
uint8_t* g_scratch_ptr[kMaxDevices] = {nullptr};
std::mutex g_scratch_mu;

int32_t scratch_for_device(int device, uint8_t** out) {
  if (device < 0 || device >= kMaxDevices) {
    tnf::set_error("tnf_linear_nvfp4_noalloc: device %d out of range", device);
    return TNF_ERR_INVALID_ARGUMENT;
  }
  std::lock_guard<std::mutex> lk(g_scratch_mu);
  if (!g_scratch_ptr[device]) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);  // the caller made `device` current
    if (e != cudaSuccess) return tnf::cuda_fail(e, "cudaGetSymbolAddress(no-alloc scratch)");
    g_scratch_ptr[device] = static_cast<uint8_t*>(p);
  }
  *out = g_scratch_ptr[device];
  return TNF_OK;
}

inline uint64_t align256(uint64_t x) { return (x + 255ull) & ~255ull; }

}  // namespace

using namespace tnf;

extern "C" {

uint64_t tnf_noalloc_scratch_bytes(void) { return kScratchBytes; }

int32_t tnf_linear_nvfp4_noalloc(tnf_ctx* ctx, const tnf_linear_args* a) {
  if (!ctx || !a) {
    set_error("tnf_linear_nvfp4_noalloc: null argument");
    return TNF_ERR_INVALID_ARGUMENT;
  }
  cudaError_t ce = cudaSetDevice(ctx->device);
  if (ce != cudaSuccess) return cuda_fail(ce, "cudaSetDevice");
  if (a->m == 0 || a->n == 0 || a->k == 0 || a->k % 32 || a->n % 8 || !(a->a_global > 0.0f) || !(a->w_global > 0.0f) ||
      a->act > 1 || a->parity_mode > 1) {
    set_error("tnf_linear_nvfp4_noalloc: bad problem m=%u n=%u k=%u (k %% 32, n %% 8), scales > 0, act <= 1", a->m, a->n, a->k);
    return TNF_ERR_INVALID_ARGUMENT;
  }
  if (a->flags != 0) {
    set_error("tnf_linear_nvfp4_noalloc: flags are not supported here (got 0x%x)", a->flags);
    return TNF_ERR_INVALID_ARGUMENT;
  }
  const uint64_t codes_bytes = align256(uint64_t(a->m) * (a->k / 2));
  const uint64_t scales_bytes = sf_device_bytes(a->m, a->k);
  if (codes_bytes + scales_bytes > kScratchBytes) {
    set_error("tnf_linear_nvfp4_noalloc: m=%u k=%u needs %llu bytes of scratch, the built-in array holds %llu; "
              "use tnf_linear_nvfp4 or split the rows",
              a->m, a->k, (unsigned long long)(codes_bytes + scales_bytes), (unsigned long long)kScratchBytes);
    return TNF_ERR_INVALID_ARGUMENT;
  }
  uint8_t* scratch = nullptr;
  int32_t st = scratch_for_device(ctx->device, &scratch);
  if (st != TNF_OK) return st;
  uint8_t* a_codes = scratch;
  uint8_t* a_scales = scratch + codes_bytes;

  const uint32_t ldo = a->ldo ? a->ldo : a->n;
  if (ldo % 8 || a->n_offset % 8 || a->n_offset + a->n > ldo) {
    set_error("tnf_linear_nvfp4_noalloc: bad output window (n_offset %u, n %u, ldo %u)", a->n_offset, a->n, ldo);
    return TNF_ERR_INVALID_ARGUMENT;
  }
  uint8_t* src = resolve(ctx, a->a_bf16, uint64_t(a->m) * a->k * 2, "a_bf16", &st);
  if (!src) return st;
  uint8_t* w_codes = resolve(ctx, a->w_codes, uint64_t(a->n) * (a->k / 2), "w_codes", &st);
  if (!w_codes) return st;
  uint8_t* w_scales = resolve(ctx, a->w_scales, sf_device_bytes(a->n, a->k), "w_scales", &st);
  if (!w_scales) return st;
  uint8_t* out = resolve(ctx, a->out_bf16, (uint64_t(a->m - 1) * ldo + a->n_offset + a->n) * 2, "out_bf16", &st);
  if (!out) return st;

  GemmParams p{};
  p.m = a->m; p.n = a->n; p.k = a->k;
  p.k_atoms = sf_k_atoms(a->k);
  p.alpha = a->a_global * a->w_global;
  p.sfa = a_scales;
  p.sfb = w_scales;
  if (a->bias_bf16.len) {
    p.bias = reinterpret_cast<const uint16_t*>(resolve(ctx, a->bias_bf16, uint64_t(a->n) * 2, "bias_bf16", &st));
    if (!p.bias) return st;
  }
  if (a->gate_bf16.len) {
    p.gate = reinterpret_cast<const uint16_t*>(resolve(ctx, a->gate_bf16, uint64_t(a->n) * 2, "gate_bf16", &st));
    if (!p.gate) return st;
    p.residual = reinterpret_cast<const uint16_t*>(resolve(ctx, a->residual_bf16, uint64_t(a->m) * a->n * 2, "residual_bf16", &st));
    if (!p.residual) return st;
  }
  p.out[0] = reinterpret_cast<uint16_t*>(out);
  p.n_out = 1;
  p.ldo = ldo;
  p.n_offset = a->n_offset;
  p.act = a->act;
  p.chain = a->parity_mode;
  p.store_bf16 = 1;
  p.status = ctx->dwords;
  p.wait_limit = ctx->wait_limit_cycles;
  p.trace = reinterpret_cast<unsigned long long*>(ctx->dwords + 64);

  ce = launch_quantize(src, TNF_DTYPE_BF16, a->m, a->k, nullptr, a->a_global, a_codes, a_scales, true, ctx->compute);
  if (ce != cudaSuccess) return cuda_fail(ce, "activation quantise launch");

  const bool pair = gemm_use_pair(a->m, a->n, a->k);
  CUtensorMap ma, mw;
  const uint32_t kb = gemm_pair_kblocks();
  const uint32_t box_bytes = pair ? kb * 32 : 128, swz = box_bytes;  // the pair kernel's stage width sets the box
  if (make_tensor_map(&ma, MapSpec{a_codes, 1, a->k / 2, a->m, a->k / 2, box_bytes, 128, swz}) != TNF_OK) return TNF_ERR_INVALID_ARGUMENT;
  if (make_tensor_map(&mw, MapSpec{w_codes, 1, a->k / 2, a->n, a->k / 2, box_bytes, pair ? 128u : gemm_tile_n(a->m, a->n), swz}) != TNF_OK)
    return TNF_ERR_INVALID_ARGUMENT;
  if (pair) {
    CUtensorMap msa, msb, outs[kMaxPeers];
    if (make_tensor_map(&msa, MapSpec{a_scales, 1, 128, scales_bytes / 128, 128, 128, kb * 4, 0}) != TNF_OK) return TNF_ERR_INVALID_ARGUMENT;
    if (make_tensor_map(&msb, MapSpec{w_scales, 1, 128, sf_device_bytes(a->n, a->k) / 128, 128, 128, kb * 4, 0}) != TNF_OK)
      return TNF_ERR_INVALID_ARGUMENT;
    if (make_tensor_map(&outs[0], MapSpec{p.out[0] + a->n_offset, 2, a->n, a->m, uint64_t(ldo) * 2, 64, 32, 1}) != TNF_OK)
      return TNF_ERR_INVALID_ARGUMENT;
    for (int d = 1; d < kMaxPeers; ++d) outs[d] = outs[0];
    ce = launch_gemm_nvfp4_pair(ma, mw, msa, msb, outs, p, ctx->sm_count, ctx->compute);
  } else {
    ce = launch_gemm_nvfp4(ma, mw, p, ctx->sm_count, ctx->compute);
  }
  if (ce != cudaSuccess) return cuda_fail(ce, "nvfp4 gemm launch");
  return TNF_OK;
}

}  // extern "C"
