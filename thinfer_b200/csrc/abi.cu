// C ABI of the NVFP4 linear path: context, buffers, quantisers, the linear, uploads.
// See include/thinfer_nvfp4.h for the reference interface each entry point replaces.
#include <algorithm>
#include <chrono>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <thread>

#include "context.h"

namespace tnf {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int32_t cuda_fail(cudaError_t e, const char* what) {
  set_error("%s: %s (%s)", what, cudaGetErrorName(e), cudaGetErrorString(e));
  return e == cudaErrorMemoryAllocation ? TNF_ERR_ALLOCATE_OOM : TNF_ERR_LAUNCH;
}

#define TNF_CUDA(call, what)                               \
  do {                                                     \
    cudaError_t _e = (call);                               \
    if (_e != cudaSuccess) return tnf::cuda_fail(_e, what); \
  } while (0)

#define TNF_CHECK_CTX(ctx)                          \
  do {                                              \
    if (!(ctx)) {                                   \
      tnf::set_error("null context");               \
      return TNF_ERR_INVALID_ARGUMENT;              \
    }                                               \
    cudaError_t _e = cudaSetDevice((ctx)->device);  \
    if (_e != cudaSuccess) return tnf::cuda_fail(_e, "cudaSetDevice"); \
  } while (0)

uint8_t* resolve(tnf_ctx* ctx, const tnf_buf& b, uint64_t need, const char* name, int32_t* status) {
  std::lock_guard<std::mutex> lk(ctx->mu);
  auto it = ctx->bufs.find(b.id);
  if (it == ctx->bufs.end()) {
    set_error("%s: unknown buffer id %llu", name, (unsigned long long)b.id);
    *status = TNF_ERR_UNKNOWN_BUFFER;
    return nullptr;
  }
  if (b.offset > it->second.bytes || b.len > it->second.bytes - b.offset || need > b.len) {
    set_error("%s: view {off %llu, len %llu} needs %llu bytes, buffer has %llu", name, (unsigned long long)b.offset,
              (unsigned long long)b.len, (unsigned long long)need, (unsigned long long)it->second.bytes);
    *status = TNF_ERR_INVALID_ARGUMENT;
    return nullptr;
  }
  if (b.offset % 16 != 0) {
    set_error("%s: view offset %llu is not 16-byte aligned", name, (unsigned long long)b.offset);
    *status = TNF_ERR_INVALID_ARGUMENT;
    return nullptr;
  }
  return static_cast<uint8_t*>(it->second.ptr) + b.offset;
}

uint8_t* resolve_multicast(tnf_ctx* ctx, const tnf_buf& b, const char* name, int32_t* status) {
  std::lock_guard<std::mutex> lk(ctx->mu);
  auto it = ctx->bufs.find(b.id);
  if (it == ctx->bufs.end() || !it->second.mc) {
    set_error("%s: TNF_LINEAR_MULTICAST_OUT needs a buffer registered with tnf_import_symmetric that has a multicast alias", name);
    *status = TNF_ERR_INVALID_ARGUMENT;
    return nullptr;
  }
  return static_cast<uint8_t*>(it->second.mc) + b.offset;
}

int32_t alloc_locked(tnf_ctx* ctx, uint64_t bytes, int category, uint64_t* id) {
  if (category < 0 || category > 2 || bytes == 0) {
    set_error("tnf_alloc: bad category %d or zero size", category);
    return TNF_ERR_INVALID_ARGUMENT;
  }
  uint64_t total = ctx->live[0] + ctx->live[1] + ctx->live[2];
  if (ctx->budget && total + bytes > ctx->budget && !ctx->in_reclaim) {
    // reclaim_until_fits (thinfer-core/src/arbiter.rs:129-160): ask the registered holders, in order, to give
    // memory back before refusing; a holder frees whole weight sets and streams them from then on
    ctx->in_reclaim = true;
    // the idle workspace pool is first in the chain (RECLAIM_IDLE_POOL, thinfer-core/src/arbiter.rs:37-38)
    ws_spill_locked(ctx, total + bytes - ctx->budget);
    for (auto& r : ctx->reclaimers) {
      total = ctx->live[0] + ctx->live[1] + ctx->live[2];
      if (total + bytes <= ctx->budget) break;
      ctx->reclaimed += r.fn(r.owner, total + bytes - ctx->budget);
    }
    ctx->in_reclaim = false;
    total = ctx->live[0] + ctx->live[1] + ctx->live[2];
  }
  if (ctx->budget && total + bytes > ctx->budget) {
    // refused on the host; the device is not touched
    set_error("budget exceeded: live %llu + request %llu > budget %llu", (unsigned long long)total,
              (unsigned long long)bytes, (unsigned long long)ctx->budget);
    return TNF_ERR_BUDGET_EXCEEDED;
  }
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return cuda_fail(e, "cudaMalloc");
  }
  uint64_t nid = ctx->next_id++;
  ctx->bufs[nid] = tnf_buffer_rec{p, bytes, category};
  ctx->live[category] += bytes;
  ctx->peak[category] = std::max(ctx->peak[category], ctx->live[category]);
  ctx->true_peak = std::max(ctx->true_peak, total + bytes);
  *id = nid;
  return TNF_OK;
}

int32_t free_locked(tnf_ctx* ctx, uint64_t id) {
  auto it = ctx->bufs.find(id);
  if (it == ctx->bufs.end()) {
    set_error("tnf_free: unknown buffer id %llu", (unsigned long long)id);
    return TNF_ERR_UNKNOWN_BUFFER;
  }
  // cudaFree waits for work that may still use the memory; an imported range is only forgotten
  cudaError_t e = it->second.owned ? cudaFree(it->second.ptr) : cudaSuccess;
  ctx->live[it->second.category] -= it->second.bytes;
  // tensor maps over the freed range are dropped (a later buffer may reuse the address)
  for (auto m = ctx->maps.begin(); m != ctx->maps.end();) {
    const uint8_t* b = static_cast<const uint8_t*>(m->first.base);
    const uint8_t* lo = static_cast<const uint8_t*>(it->second.ptr);
    if (b >= lo && b < lo + it->second.bytes) m = ctx->maps.erase(m);
    else ++m;
  }
  ctx->bufs.erase(it);
  // a pool buffer freed directly leaves the pool's books too
  auto rented = ctx->ws_rented.find(id);
  if (rented != ctx->ws_rented.end()) {
    ctx->ws_rented.erase(rented);
  } else {
    for (auto c = ctx->ws_free.begin(); c != ctx->ws_free.end(); ++c) {
      auto pos = std::find(c->second.begin(), c->second.end(), id);
      if (pos == c->second.end()) continue;
      c->second.erase(pos);
      ctx->ws_pool_bytes -= c->first;
      if (c->second.empty()) ctx->ws_free.erase(c);
      break;
    }
  }
  if (e != cudaSuccess) return cuda_fail(e, "cudaFree");
  return TNF_OK;
}

// spill_pool_locked (thinfer-core/src/workspace.rs:52-85): classes in ascending size, newest buffer of a class first.
uint64_t ws_spill_locked(tnf_ctx* ctx, uint64_t at_least) {
  uint64_t freed = 0;
  while (freed < at_least && !ctx->ws_free.empty()) {
    auto c = ctx->ws_free.begin();
    const uint64_t cls = c->first, id = c->second.back();
    c->second.pop_back();
    if (c->second.empty()) ctx->ws_free.erase(c);
    ctx->ws_pool_bytes -= cls;
    free_locked(ctx, id);
    freed += cls;
  }
  ctx->ws_spilled += freed;
  return freed;
}

typedef CUresult (*encode_tiled_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static encode_tiled_fn get_encode_fn() {
  static encode_tiled_fn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<encode_tiled_fn>(p);
  }
  return fn;
}

int make_tensor_map(CUtensorMap* out, const MapSpec& sp) {
  encode_tiled_fn fn = get_encode_fn();
  if (!fn) {
    set_error("cuTensorMapEncodeTiled is not available from this driver");
    return TNF_ERR_LAUNCH;
  }
  cuuint64_t gdim[2] = {sp.dim0, sp.dim1};
  cuuint64_t gstride[1] = {sp.stride1};
  cuuint32_t box[2] = {sp.box0, sp.box1};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, sp.elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 2,
                  const_cast<void*>(sp.base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  sp.swizzle128 == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : (sp.swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE),
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with CUresult %d (base %p dims %llu x %llu stride %llu box %u x %u)", int(r),
              sp.base, (unsigned long long)sp.dim0, (unsigned long long)sp.dim1, (unsigned long long)sp.stride1, sp.box0,
              sp.box1);
    return TNF_ERR_INVALID_ARGUMENT;
  }
  return TNF_OK;
}

// The map is copied out under the lock: a pointer into the cache could be invalidated by the next lookup's
// eviction or by another thread's tnf_free before the launch copies it.
bool get_map(tnf_ctx* ctx, const MapSpec& spec, CUtensorMap* out) {
  std::lock_guard<std::mutex> lk(ctx->mu);
  auto it = ctx->maps.find(spec);
  if (it != ctx->maps.end()) {
    *out = it->second;
    return true;
  }
  if (make_tensor_map(out, spec) != TNF_OK) return false;
  if (ctx->maps.size() >= 8192) ctx->maps.erase(ctx->maps.begin());  // bounded cache: drop one entry, never all
  ctx->maps[spec] = *out;
  return true;
}

// packed E2M1 codes viewed as bytes [rows, k/2]: box {128 bytes, box_rows}, 128-byte swizzle
static MapSpec codes_spec(const void* base, uint32_t rows, uint32_t k, uint32_t box_rows) {
  return MapSpec{base, 1, k / 2, rows, k / 2, 128, box_rows, 1};
}
// device-layout scales viewed as rows of 128 bytes: box = 16 rows = four 512-byte atoms
static MapSpec scales_spec(const void* base, uint32_t rows, uint32_t k, uint32_t atoms_per_box) {
  return MapSpec{base, 1, 128, sf_device_bytes(rows, k) / 128, 128, 128, atoms_per_box * 4, 0};
}
// codes for the pair kernel: box {kb*32 bytes, 128 rows}, swizzle = box width
static MapSpec pair_codes_spec(const void* base, uint32_t rows, uint32_t k, uint32_t kb) {
  return MapSpec{base, 1, k / 2, rows, k / 2, kb * 32, 128, kb * 32};
}
// bf16 output window [m, n] with leading dimension ldo: box {64 columns, 32 rows}, 128-byte swizzle
static MapSpec out_spec(const void* base, uint32_t m, uint32_t n, uint32_t ldo) {
  return MapSpec{base, 2, n, m, uint64_t(ldo) * 2, 64, 32, 1};
}

static int32_t ensure_scratch(tnf_ctx* ctx, uint32_t m, uint32_t k) {
  uint64_t need_codes = uint64_t(m) * (k / 2), need_scales = sf_device_bytes(m, k);
  std::lock_guard<std::mutex> lk(ctx->mu);
  if (need_codes > ctx->scratch_codes_bytes || need_scales > ctx->scratch_scales_bytes) ctx->scratch_m = ctx->scratch_k = 0;
  if (need_codes > ctx->scratch_codes_bytes) {
    if (ctx->scratch_codes_id) free_locked(ctx, ctx->scratch_codes_id);
    ctx->scratch_codes_id = 0;
    ctx->scratch_codes_bytes = 0;
    int32_t st = alloc_locked(ctx, need_codes, TNF_CAT_WORKSPACE, &ctx->scratch_codes_id);
    if (st != TNF_OK) return st;
    ctx->scratch_codes_bytes = need_codes;
  }
  if (need_scales > ctx->scratch_scales_bytes) {
    if (ctx->scratch_scales_id) free_locked(ctx, ctx->scratch_scales_id);
    ctx->scratch_scales_id = 0;
    ctx->scratch_scales_bytes = 0;
    int32_t st = alloc_locked(ctx, need_scales, TNF_CAT_WORKSPACE, &ctx->scratch_scales_id);
    if (st != TNF_OK) return st;
    ctx->scratch_scales_bytes = need_scales;
  }
  return TNF_OK;
}

// Workspace for the bf16 image of NVFP4 activations (the mixed arm: low-bit activations x a dense bf16 weight).
static int32_t ensure_wide(tnf_ctx* ctx, uint64_t bytes) {
  std::lock_guard<std::mutex> lk(ctx->mu);
  if (bytes <= ctx->wide_bytes) return TNF_OK;
  if (ctx->wide_id) free_locked(ctx, ctx->wide_id);
  ctx->wide_id = 0;
  ctx->wide_bytes = 0;
  int32_t st = alloc_locked(ctx, bytes, TNF_CAT_WORKSPACE, &ctx->wide_id);
  if (st != TNF_OK) return st;
  ctx->wide_bytes = bytes;
  return TNF_OK;
}

// Mixed arm: NVFP4 activations (codes + device scales) against a dense bf16 weight. The tensor cores have no
// FP4 x bf16 form, so the activations are widened to bf16 first -- exact: a code times its block scale has at
// most 6 significant bits -- and the bf16 GEMM applies a_global * w_global in its epilogue.
static int32_t run_gemm(tnf_ctx* ctx, const tnf_linear_args* a, const uint8_t* a_codes, const uint8_t* a_scales,
                        const uint8_t* a_raw, bool widened);
static int32_t run_mixed(tnf_ctx* ctx, const tnf_linear_args* a, const uint8_t* a_codes, const uint8_t* a_scales) {
  int32_t st = ensure_wide(ctx, uint64_t(a->m) * a->k * 2);
  if (st != TNF_OK) return st;
  uint8_t* wide = static_cast<uint8_t*>(ctx->bufs[ctx->wide_id].ptr);
  TNF_CUDA(launch_dequant_dense(a_codes, a_scales, a->m, a->k, reinterpret_cast<uint16_t*>(wide), ctx->compute),
           "activation widening launch");
  return run_gemm(ctx, a, wide, nullptr, nullptr, true);
}

static int32_t check_dims(uint32_t m, uint32_t n, uint32_t k) {
  if (m == 0 || n == 0 || k == 0) {
    set_error("empty problem m=%u n=%u k=%u", m, n, k);
    return TNF_ERR_INVALID_ARGUMENT;
  }
  if (k % 32 != 0) {
    set_error("k=%u must be a multiple of 32 (16-byte rows of packed codes)", k);
    return TNF_ERR_INVALID_ARGUMENT;
  }
  if (n % 8 != 0) {
    set_error("n=%u must be a multiple of 8 (16-byte output vectors)", n);
    return TNF_ERR_INVALID_ARGUMENT;
  }
  return TNF_OK;
}

// shared tail of tnf_linear_nvfp4 / tnf_gemm_nvfp4
// `a_raw` non-null: the skinny-M kernel takes the bf16 activations themselves (its prologue is the quantiser).
// `widened`: the dense arm's bf16 activations are the exact image (code x block scale) of NVFP4 activations, so
// the per-tensor activation scale still has to be applied.
static int32_t run_gemm(tnf_ctx* ctx, const tnf_linear_args* a, const uint8_t* a_codes, const uint8_t* a_scales,
                        const uint8_t* a_raw, bool widened) {
  int32_t st = TNF_OK;
  const bool swiglu = (a->flags & TNF_LINEAR_SWIGLU) != 0;
  const uint32_t n_out_cols = swiglu ? a->n / 2 : a->n;  // columns this call writes
  const uint32_t ldo = a->ldo ? a->ldo : n_out_cols;
  if (ldo % 8 != 0 || a->n_offset % 8 != 0 || a->n_offset + n_out_cols > ldo) {
    set_error("bad output window: n_offset %u + %u columns within ldo %u, all multiples of 8", a->n_offset, n_out_cols, ldo);
    return TNF_ERR_INVALID_ARGUMENT;
  }
  if (swiglu && (a->n % 16 != 0 || a->act != TNF_ACT_NONE || a->gate_bf16.len ||
                 (a->flags & (TNF_LINEAR_OUT_NVFP4 | TNF_LINEAR_SCATTER_PEERS | TNF_LINEAR_MULTICAST_OUT)))) {
    set_error("TNF_LINEAR_SWIGLU needs n %% 16 == 0 (n=%u), act none, no gated residual, and none of OUT_NVFP4 / SCATTER_PEERS / "
              "MULTICAST_OUT", a->n);
    return TNF_ERR_INVALID_ARGUMENT;
  }
  const bool dense = (a->flags & TNF_LINEAR_DENSE_ACT) != 0;
  uint8_t *w_codes = nullptr, *w_scales = nullptr;
  if (dense) {  // a_codes carries the bf16 activations, the weight is its dense image
    w_codes = resolve(ctx, a->w_dense, uint64_t(a->n) * a->k * 2, "w_dense", &st);
    if (!w_codes) return st;
  } else {
    w_codes = resolve(ctx, a->w_codes, uint64_t(a->n) * (a->k / 2), "w_codes", &st);
    if (!w_codes) return st;
    w_scales = resolve(ctx, a->w_scales, sf_device_bytes(a->n, a->k), "w_scales", &st);
    if (!w_scales) return st;
  }
  const bool q_out = (a->flags & TNF_LINEAR_OUT_NVFP4) != 0;
  const bool store_bf16 = !(q_out && (a->flags & TNF_LINEAR_NO_BF16_OUT));
  uint8_t* out = nullptr;
  if (store_bf16) {
    out = resolve(ctx, a->out_bf16, (uint64_t(a->m - 1) * ldo + a->n_offset + n_out_cols) * 2, "out_bf16", &st);
    if (!out) return st;
  }
  GemmParams p{};
  p.store_bf16 = store_bf16 ? 1u : 0u;
  const bool mc_out = (a->flags & TNF_LINEAR_MULTICAST_OUT) != 0;
  if (mc_out && ((a->flags & TNF_LINEAR_SCATTER_PEERS) || a->gate_bf16.len)) {
    set_error("TNF_LINEAR_MULTICAST_OUT cannot be combined with TNF_LINEAR_SCATTER_PEERS or a gated residual");
    return TNF_ERR_INVALID_ARGUMENT;
  }
  if (mc_out && store_bf16) {
    p.out_mc = reinterpret_cast<uint16_t*>(resolve_multicast(ctx, a->out_bf16, "out_bf16", &st));
    if (!p.out_mc) return st;
  }
  if (q_out) {
    if (a->n % 64 != 0 || a->n_offset % 64 != 0 || ldo % 64 != 0 || !(a->out_global > 0.0f) ||
        (a->flags & TNF_LINEAR_SCATTER_PEERS) || a->gate_bf16.len) {
      set_error("TNF_LINEAR_OUT_NVFP4 needs n, n_offset and ldo multiples of 64 (n=%u, n_offset=%u, ldo=%u), "
                "out_global > 0, no peer scatter and no gated residual", a->n, a->n_offset, ldo);
      return TNF_ERR_INVALID_ARGUMENT;
    }
    // the NVFP4 copy is the [m, ldo] operand of the next linear; this call fills columns n_offset .. n_offset + n
    p.q_codes = resolve(ctx, a->out_codes, uint64_t(a->m) * (ldo / 2), "out_codes", &st);
    if (!p.q_codes) return st;
    p.q_scales = resolve(ctx, a->out_scales, sf_device_bytes(a->m, ldo), "out_scales", &st);
    if (!p.q_scales) return st;
    if (mc_out) {
      p.q_codes_mc = resolve_multicast(ctx, a->out_codes, "out_codes", &st);
      if (!p.q_codes_mc) return st;
      p.q_scales_mc = resolve_multicast(ctx, a->out_scales, "out_scales", &st);
      if (!p.q_scales_mc) return st;
    }
    p.q_global = a->out_global;
    p.q_inv_t = 1.0f / (6.0f * a->out_global);
    p.q_k_atoms = sf_k_atoms(ldo);
    // The scale layout pads K to whole groups of four 512-byte atoms; the padding atoms of the next operand must
    // hold benign (zero) scales. Only those atoms are cleared (atoms ldo/64 .. k_atoms-1 of every 128-row block),
    // so an earlier window call's scales in the same buffer stay intact.
    const uint32_t used_atoms = ldo / 64;
    if (used_atoms < p.q_k_atoms)
      TNF_CUDA(cudaMemset2DAsync(p.q_scales + uint64_t(used_atoms) * 512u, uint64_t(p.q_k_atoms) * 512u, 0,
                                 uint64_t(p.q_k_atoms - used_atoms) * 512u, (a->m + 127u) / 128u, ctx->compute),
               "out_scales padding clear");
  }
  p.m = a->m; p.n = a->n; p.k = a->k;
  p.k_atoms = sf_k_atoms(a->k);
  p.alpha = (dense && !widened) ? a->w_global : a->a_global * a->w_global;
  p.dense = dense ? 1u : 0u;
  p.swiglu = swiglu ? 1u : 0u;
  p.sfa = a_scales;
  p.sfb = w_scales;
  if (a->bias_bf16.len) {
    p.bias = reinterpret_cast<const uint16_t*>(resolve(ctx, a->bias_bf16, uint64_t(a->n) * 2, "bias_bf16", &st));
    if (!p.bias) return st;
  }
  if (a->gate_bf16.len) {
    p.gate = reinterpret_cast<const uint16_t*>(resolve(ctx, a->gate_bf16, uint64_t(a->n) * 2, "gate_bf16", &st));
    if (!p.gate) return st;
    p.residual = reinterpret_cast<const uint16_t*>(
        resolve(ctx, a->residual_bf16, uint64_t(a->m) * a->n * 2, "residual_bf16", &st));
    if (!p.residual) return st;
  }
  p.out[0] = reinterpret_cast<uint16_t*>(out);
  p.n_out = 1;
  if (a->flags & TNF_LINEAR_SCATTER_PEERS) {
    const int set = int((a->flags >> 8) & 3u);
    if (ctx->n_peers[set] <= 0) {
      set_error("TNF_LINEAR_SCATTER_PEERS: peer set %d has no windows (tnf_peer_outputs)", set);
      return TNF_ERR_INVALID_ARGUMENT;
    }
    for (int i = 0; i < ctx->n_peers[set]; ++i) p.out[p.n_out++] = reinterpret_cast<uint16_t*>(ctx->peer_out[set][i]);
  }
  p.ldo = ldo;
  p.n_offset = a->n_offset;
  p.act = a->act;
  p.chain = a->parity_mode;
  p.status = ctx->dwords;
  p.wait_limit = ctx->wait_limit_cycles;
  p.trace = reinterpret_cast<unsigned long long*>(ctx->dwords + 64);
  if (a_raw) {
    if (skinny_tc_applies(a->m, a->n, a->k)) {
      CUtensorMap mw;
      if (!get_map(ctx, codes_spec(w_codes, a->n, a->k, 128), &mw)) return TNF_ERR_INVALID_ARGUMENT;
      TNF_CUDA(launch_skinny_tc(mw, a_raw, a->a_global, p, ctx->compute), "nvfp4 skinny-M tensor-core launch");
      return TNF_OK;
    }
    TNF_CUDA(launch_gemv_nvfp4(a_raw, a->a_global, w_codes, p, ctx->compute), "nvfp4 skinny-M launch");
    return TNF_OK;
  }
  CUtensorMap ma, mw;
  if (dense || swiglu || q_out || mc_out || gemm_use_pair(a->m, a->n, a->k)) {  // only the CTA-pair kernel has the dense arm and the NVFP4 / multicast epilogues
    const uint32_t kb = gemm_pair_kblocks();
    CUtensorMap msa, msb, outs[kMaxPeers];
    if (dense) {  // bf16 [rows, k]: boxes of 64 elements (128 bytes) x 128 rows, 128-byte swizzle; no scale maps
      if (!get_map(ctx, MapSpec{a_codes, 2, a->k, a->m, uint64_t(a->k) * 2, 64, 128, 128}, &ma) ||
          !get_map(ctx, MapSpec{w_codes, 2, a->k, a->n, uint64_t(a->k) * 2, 64, 128, 128}, &mw))
        return TNF_ERR_INVALID_ARGUMENT;
      msa = msb = ma;
    } else if (!get_map(ctx, pair_codes_spec(a_codes, a->m, a->k, kb), &ma) || !get_map(ctx, pair_codes_spec(w_codes, a->n, a->k, kb), &mw) ||
               !get_map(ctx, scales_spec(a_scales, a->m, a->k, kb), &msa) || !get_map(ctx, scales_spec(w_scales, a->n, a->k, kb), &msb))
      return TNF_ERR_INVALID_ARGUMENT;
    for (uint32_t d = 0; d < p.n_out; ++d) {
      // without a bf16 destination the map is never used; any valid one fills the slot
      if (!store_bf16) outs[d] = ma;
      else if (swiglu) {  // n/2 output columns; boxes of 32 columns x 32 rows, dense 64-byte rows in shared memory
        if (!get_map(ctx, MapSpec{p.out[d] + a->n_offset, 2, n_out_cols, a->m, uint64_t(ldo) * 2, 32, 32, 0}, &outs[d])) return TNF_ERR_INVALID_ARGUMENT;
      } else if (!get_map(ctx, out_spec(p.out[d] + a->n_offset, a->m, a->n, ldo), &outs[d])) return TNF_ERR_INVALID_ARGUMENT;
    }
    for (uint32_t d = p.n_out; d < kMaxPeers; ++d) outs[d] = outs[0];
    TNF_CUDA(launch_gemm_nvfp4_pair(ma, mw, msa, msb, outs, p, ctx->sm_count, ctx->compute), "nvfp4 pair gemm launch");
    return TNF_OK;
  }
  if (!get_map(ctx, codes_spec(a_codes, a->m, a->k, 128), &ma) ||
      !get_map(ctx, codes_spec(w_codes, a->n, a->k, gemm_tile_n(a->m, a->n)), &mw))
    return TNF_ERR_INVALID_ARGUMENT;
  TNF_CUDA(launch_gemm_nvfp4(ma, mw, p, ctx->sm_count, ctx->compute), "nvfp4 gemm launch");
  return TNF_OK;
}

}  // namespace tnf

using namespace tnf;

extern "C" {

uint32_t tnf_abi_version(void) { return 3; }
const char* tnf_last_error(void) { return g_err; }

int32_t tnf_create(int32_t device, uint64_t vram_budget_bytes, tnf_ctx** out) {
  if (!out) {
    set_error("tnf_create: null out");
    return TNF_ERR_INVALID_ARGUMENT;
  }
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || count == 0) {
    cudaGetLastError();
    set_error("no CUDA device is visible (%s); this library has no CPU path", cudaGetErrorString(e));
    return TNF_ERR_LAUNCH;
  }
  if (device < 0 || device >= count) {
    set_error("device %d out of range (0..%d)", device, count - 1);
    return TNF_ERR_INVALID_ARGUMENT;
  }
  TNF_CUDA(cudaSetDevice(device), "cudaSetDevice");
  cudaDeviceProp prop;
  TNF_CUDA(cudaGetDeviceProperties(&prop, device), "cudaGetDeviceProperties");
  if (prop.major != 10) {
    set_error("device %d is sm_%d%d; this library is built for sm_100a only", device, prop.major, prop.minor);
    return TNF_ERR_LAUNCH;
  }
  tnf_ctx* ctx = new tnf_ctx();
  ctx->device = device;
  ctx->sm_count = prop.multiProcessorCount;
  ctx->budget = vram_budget_bytes;
  TNF_CUDA(cudaStreamCreateWithFlags(&ctx->compute, cudaStreamNonBlocking), "cudaStreamCreate");
  TNF_CUDA(cudaStreamCreateWithFlags(&ctx->copy, cudaStreamNonBlocking), "cudaStreamCreate");
  TNF_CUDA(cudaStreamCreateWithFlags(&ctx->readback, cudaStreamNonBlocking), "cudaStreamCreate");
  TNF_CUDA(cudaMalloc(&ctx->dwords, 256 + 16384), "cudaMalloc(status words)");
  TNF_CUDA(cudaMemset(ctx->dwords, 0, 256 + 16384), "cudaMemset(status words)");
  *out = ctx;
  return TNF_OK;
}

int32_t tnf_destroy(tnf_ctx* ctx) {
  if (!ctx) return TNF_OK;
  cudaSetDevice(ctx->device);
  cudaDeviceSynchronize();
  tnf_comm_teardown(ctx);
  for (auto& kv : ctx->bufs)
    if (kv.second.owned) cudaFree(kv.second.ptr);
  for (auto& kv : ctx->hosts) {
    if (kv.second.owned) cudaFreeHost(kv.second.ptr);
    else cudaHostUnregister(kv.second.ptr);
  }
  for (auto& kv : ctx->events) cudaEventDestroy(kv.second);
  for (auto ev : ctx->event_pool) cudaEventDestroy(ev);
  for (int i = 0; i < 2; ++i) {
    if (ctx->stage_host[i]) cudaFreeHost(ctx->stage_host[i]);
    if (ctx->stage_done[i]) cudaEventDestroy(ctx->stage_done[i]);
  }
  cudaFree(ctx->dwords);
  cudaStreamDestroy(ctx->compute);
  cudaStreamDestroy(ctx->copy);
  cudaStreamDestroy(ctx->readback);
  for (int i = 0; i < 8; ++i) {
    if (ctx->push[i]) cudaStreamDestroy(ctx->push[i]);
    if (ctx->push_done[i]) cudaEventDestroy(ctx->push_done[i]);
  }
  cudaGetLastError();
  delete ctx;
  return TNF_OK;
}

int32_t tnf_alloc(tnf_ctx* ctx, uint64_t bytes, int32_t category, uint64_t* id) {
  TNF_CHECK_CTX(ctx);
  if (!id) {
    set_error("tnf_alloc: null id");
    return TNF_ERR_INVALID_ARGUMENT;
  }
  std::lock_guard<std::mutex> lk(ctx->mu);
  return alloc_locked(ctx, bytes, category, id);
}

int32_t tnf_free(tnf_ctx* ctx, uint64_t id) {
  TNF_CHECK_CTX(ctx);
  std::lock_guard<std::mutex> lk(ctx->mu);
  return free_locked(ctx, id);
}

static int32_t raw_range(tnf_ctx* ctx, uint64_t id, uint64_t off, uint64_t n, const char* what, uint8_t** p) {
  std::lock_guard<std::mutex> lk(ctx->mu);
  auto it = ctx->bufs.find(id);
  if (it == ctx->bufs.end()) {
    set_error("%s: unknown buffer id %llu", what, (unsigned long long)id);
    return TNF_ERR_UNKNOWN_BUFFER;
  }
  if (off > it->second.bytes || n > it->second.bytes - off) {
    set_error("%s: range [%llu, +%llu) outside buffer of %llu bytes", what, (unsigned long long)off,
              (unsigned long long)n, (unsigned long long)it->second.bytes);
    return TNF_ERR_INVALID_ARGUMENT;
  }
  *p = static_cast<uint8_t*>(it->second.ptr) + off;
  return TNF_OK;
}

int32_t tnf_write(tnf_ctx* ctx, uint64_t id, uint64_t dst_off, const void* src, uint64_t n) {
  TNF_CHECK_CTX(ctx);
  if (dst_off % 4 || n % 4) {  // same rule as Backend::write_buffer
    set_error("tnf_write: offset %llu and length %llu must be multiples of 4", (unsigned long long)dst_off,
              (unsigned long long)n);
    return TNF_ERR_INVALID_ARGUMENT;
  }
  if (n == 0) return TNF_OK;
  uint8_t* p = nullptr;
  int32_t st = raw_range(ctx, id, dst_off, n, "tnf_write", &p);
  if (st != TNF_OK) return st;
  TNF_CUDA(cudaMemcpyAsync(p, src, n, cudaMemcpyHostToDevice, ctx->compute), "tnf_write copy");
  // pageable sources are staged before the call returns; pinned ones are not, so wait
  TNF_CUDA(cudaStreamSynchronize(ctx->compute), "tnf_write sync");
  return TNF_OK;
}

int32_t tnf_read(tnf_ctx* ctx, uint64_t id, uint64_t off, void* dst, uint64_t n) {
  TNF_CHECK_CTX(ctx);
  if (n == 0) return TNF_OK;
  uint8_t* p = nullptr;
  int32_t st = raw_range(ctx, id, off, n, "tnf_read", &p);
  if (st != TNF_OK) return st;
  TNF_CUDA(cudaMemcpyAsync(dst, p, n, cudaMemcpyDeviceToHost, ctx->compute), "tnf_read copy");
  TNF_CUDA(cudaStreamSynchronize(ctx->compute), "tnf_read sync");
  return TNF_OK;
}

int32_t tnf_copy(tnf_ctx* ctx, uint64_t src_id, uint64_t src_off, uint64_t dst_id, uint64_t dst_off, uint64_t n) {
  TNF_CHECK_CTX(ctx);
  if (n == 0) return TNF_OK;
  uint8_t *s = nullptr, *d = nullptr;
  int32_t st = raw_range(ctx, src_id, src_off, n, "tnf_copy src", &s);
  if (st != TNF_OK) return st;
  st = raw_range(ctx, dst_id, dst_off, n, "tnf_copy dst", &d);
  if (st != TNF_OK) return st;
  TNF_CUDA(cudaMemcpyAsync(d, s, n, cudaMemcpyDeviceToDevice, ctx->compute), "tnf_copy");
  return TNF_OK;
}

int32_t tnf_buf_ptr(tnf_ctx* ctx, uint64_t id, void** device_ptr, uint64_t* bytes) {
  TNF_CHECK_CTX(ctx);
  std::lock_guard<std::mutex> lk(ctx->mu);
  auto it = ctx->bufs.find(id);
  if (it == ctx->bufs.end()) {
    set_error("tnf_buf_ptr: unknown buffer id %llu", (unsigned long long)id);
    return TNF_ERR_UNKNOWN_BUFFER;
  }
  if (device_ptr) *device_ptr = it->second.ptr;
  if (bytes) *bytes = it->second.bytes;
  return TNF_OK;
}

int32_t tnf_streams(tnf_ctx* ctx, void** compute_stream, void** copy_stream) {
  TNF_CHECK_CTX(ctx);
  if (compute_stream) *compute_stream = ctx->compute;
  if (copy_stream) *copy_stream = ctx->copy;
  return TNF_OK;
}

int32_t tnf_sync(tnf_ctx* ctx, uint32_t timeout_ms) {
  TNF_CHECK_CTX(ctx);
  cudaStream_t streams[11] = {ctx->compute, ctx->copy, ctx->readback};
  int n_streams = 3;
  for (int i = 0; i < 8; ++i)
    if (ctx->push[i]) streams[n_streams++] = ctx->push[i];
  auto t0 = std::chrono::steady_clock::now();
  for (int si = 0; si < n_streams; ++si) {
    cudaStream_t s = streams[si];
    if (timeout_ms == 0) {
      TNF_CUDA(cudaStreamSynchronize(s), "tnf_sync");
    } else {
      while (true) {
        cudaError_t e = cudaStreamQuery(s);
        if (e == cudaSuccess) break;
        if (e != cudaErrorNotReady) return cuda_fail(e, "tnf_sync");
        auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
        if (ms > timeout_ms) {
          set_error("tnf_sync: work still running after %u ms", timeout_ms);
          return TNF_ERR_TIMEOUT;
        }
        std::this_thread::sleep_for(std::chrono::microseconds(50));
      }
    }
  }
  uint32_t status = 0;
  TNF_CUDA(cudaMemcpy(&status, ctx->dwords, 4, cudaMemcpyDeviceToHost), "tnf_sync status read");
  if (status != 0) {
    cudaMemset(ctx->dwords, 0, 4);
    static const char* names[] = {"ok", "producer wait on a free stage", "MMA wait on a loaded stage",
                                  "epilogue wait on the accumulator", "MMA wait on a drained accumulator"};
    set_error("a device-side wait gave up: %s (code %u)", status < 5 ? names[status] : "unknown", status);
    return TNF_ERR_TIMEOUT;
  }
  return TNF_OK;
}

int32_t tnf_mem_snapshot(tnf_ctx* ctx, uint64_t out[8]) {
  if (!ctx || !out) {
    set_error("tnf_mem_snapshot: null argument");
    return TNF_ERR_INVALID_ARGUMENT;
  }
  std::lock_guard<std::mutex> lk(ctx->mu);
  for (int i = 0; i < 3; ++i) {
    out[i] = ctx->live[i];
    out[3 + i] = ctx->peak[i];
  }
  out[6] = ctx->true_peak;
  out[7] = ctx->streamed;
  return TNF_OK;
}

#ifdef TNF_GEMM_DIAG
// Diagnostic builds only (not part of the ABI): copies the clock64 stamps recorded with TNF_GEMM_DIAG bit 16.
int32_t tnf_debug_trace(tnf_ctx* ctx, unsigned long long* dst_2048) {
  TNF_CHECK_CTX(ctx);
  TNF_CUDA(cudaMemcpy(dst_2048, ctx->dwords + 64, 16384, cudaMemcpyDeviceToHost), "trace read");
  return TNF_OK;
}
#endif

int32_t tnf_reclaimed_bytes(tnf_ctx* ctx, uint64_t* bytes) {
  if (!ctx || !bytes) {
    set_error("tnf_reclaimed_bytes: null argument");
    return TNF_ERR_INVALID_ARGUMENT;
  }
  std::lock_guard<std::mutex> lk(ctx->mu);
  *bytes = ctx->reclaimed;
  return TNF_OK;
}

int32_t tnf_ws_alloc(tnf_ctx* ctx, uint64_t bytes, uint64_t* id) {
  if (!ctx || !id) {
    set_error("tnf_ws_alloc: null argument");
    return TNF_ERR_INVALID_ARGUMENT;
  }
  if (bytes > UINT64_MAX - 255) {
    set_error("tnf_ws_alloc: size %llu overflows its class", (unsigned long long)bytes);
    return TNF_ERR_INVALID_ARGUMENT;
  }
  const uint64_t cls = std::max<uint64_t>(256, (bytes + 255) / 256 * 256);
  std::lock_guard<std::mutex> lk(ctx->mu);
  auto c = ctx->ws_free.find(cls);
  if (c != ctx->ws_free.end()) {  // pool hit: the newest idle buffer of the class, no device call
    *id = c->second.back();
    c->second.pop_back();
    if (c->second.empty()) ctx->ws_free.erase(c);
    ctx->ws_pool_bytes -= cls;
    ctx->ws_hits++;
  } else {
    int32_t st = alloc_locked(ctx, cls, TNF_CAT_WORKSPACE, id);
    if (st != TNF_OK) return st;
    ctx->ws_misses++;
  }
  ctx->ws_rented[*id] = cls;
  return TNF_OK;
}

int32_t tnf_ws_release(tnf_ctx* ctx, uint64_t id) {
  TNF_CHECK_CTX(ctx);
  std::lock_guard<std::mutex> lk(ctx->mu);
  auto r = ctx->ws_rented.find(id);
  if (r == ctx->ws_rented.end()) {
    set_error("tnf_ws_release: buffer id %llu is not out on rent", (unsigned long long)id);
    return TNF_ERR_UNKNOWN_BUFFER;
  }
  ctx->ws_free[r->second].push_back(id);
  ctx->ws_pool_bytes += r->second;
  ctx->ws_rented.erase(r);
  return TNF_OK;
}

int32_t tnf_ws_drain(tnf_ctx* ctx, uint64_t* freed_bytes) {
  TNF_CHECK_CTX(ctx);
  std::lock_guard<std::mutex> lk(ctx->mu);
  const uint64_t spilled = ctx->ws_spilled;
  const uint64_t freed = ws_spill_locked(ctx, UINT64_MAX);
  ctx->ws_spilled = spilled;  // a drain is a phase boundary, not memory pressure
  if (freed_bytes) *freed_bytes = freed;
  return TNF_OK;
}

int32_t tnf_ws_stats(tnf_ctx* ctx, uint64_t out[6]) {
  if (!ctx || !out) {
    set_error("tnf_ws_stats: null argument");
    return TNF_ERR_INVALID_ARGUMENT;
  }
  std::lock_guard<std::mutex> lk(ctx->mu);
  uint64_t idle = 0;
  for (auto& c : ctx->ws_free) idle += c.second.size();
  out[0] = ctx->ws_pool_bytes;
  out[1] = idle;
  out[2] = ctx->ws_rented.size();
  out[3] = ctx->ws_hits;
  out[4] = ctx->ws_misses;
  out[5] = ctx->ws_spilled;
  return TNF_OK;
}

int32_t tnf_set_transient_reserve(tnf_ctx* ctx, uint64_t bytes) {
  if (!ctx) {
    set_error("null context");
    return TNF_ERR_INVALID_ARGUMENT;
  }
  std::lock_guard<std::mutex> lk(ctx->mu);
  ctx->transient_reserve = bytes;
  return TNF_OK;
}

int32_t tnf_set_device_wait_limit(tnf_ctx* ctx, uint64_t sm_cycles) {
  if (!ctx) {
    set_error("null context");
    return TNF_ERR_INVALID_ARGUMENT;
  }
  ctx->wait_limit_cycles = sm_cycles ? (long long)std::min<uint64_t>(sm_cycles, uint64_t(1) << 40) : kDefaultWaitLimitCycles;
  return TNF_OK;
}

int32_t tnf_selftest_stalled_wait(tnf_ctx* ctx) {
  TNF_CHECK_CTX(ctx);
  // A 512 x 512 x 512 problem on zeroed operands through the CTA-pair kernel with its producer switched off: no
  // copy and no MMA is ever in flight, the MMA warp's first wait on a loaded stage gives up after the context's
  // wait limit, every role falls through to the tear-down and the kernel returns normally with the status word set.
  const uint32_t m = 512, n = 512, k = 512;
  const uint64_t codes = uint64_t(m) * (k / 2), scales = sf_device_bytes(m, k), outb = uint64_t(m) * n * 2;
  uint64_t id = 0;
  uint8_t* base = nullptr;
  {
    std::lock_guard<std::mutex> lk(ctx->mu);
    int32_t st = alloc_locked(ctx, 2 * codes + 2 * scales + outb, TNF_CAT_WORKSPACE, &id);
    if (st != TNF_OK) return st;
    base = static_cast<uint8_t*>(ctx->bufs[id].ptr);
  }
  cudaError_t e = cudaMemsetAsync(base, 0, 2 * codes + 2 * scales + outb, ctx->compute);
  GemmParams p{};
  p.m = m; p.n = n; p.k = k;
  p.k_atoms = sf_k_atoms(k);
  p.alpha = 1.0f;
  p.sfa = base + 2 * codes;
  p.sfb = base + 2 * codes + scales;
  p.out[0] = reinterpret_cast<uint16_t*>(base + 2 * codes + 2 * scales);
  p.n_out = 1;
  p.ldo = n;
  p.store_bf16 = 1;
  p.status = ctx->dwords;
  p.wait_limit = ctx->wait_limit_cycles;
  p.stall = 1;
  p.trace = reinterpret_cast<unsigned long long*>(ctx->dwords + 64);
  CUtensorMap ma, mw, msa, msb, outs[kMaxPeers];
  const uint32_t kb = gemm_pair_kblocks();
  bool ok = e == cudaSuccess && make_tensor_map(&ma, pair_codes_spec(base, m, k, kb)) == TNF_OK &&
            make_tensor_map(&mw, pair_codes_spec(base + codes, n, k, kb)) == TNF_OK &&
            make_tensor_map(&msa, scales_spec(p.sfa, m, k, kb)) == TNF_OK &&
            make_tensor_map(&msb, scales_spec(p.sfb, n, k, kb)) == TNF_OK &&
            make_tensor_map(&outs[0], out_spec(p.out[0], m, n, n)) == TNF_OK;
  if (ok) {
    for (int d = 1; d < kMaxPeers; ++d) outs[d] = outs[0];
    e = launch_gemm_nvfp4_pair(ma, mw, msa, msb, outs, p, ctx->sm_count, ctx->compute);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->compute);
  }
  {
    std::lock_guard<std::mutex> lk(ctx->mu);
    free_locked(ctx, id);
  }
  if (!ok) return e != cudaSuccess ? cuda_fail(e, "tnf_selftest_stalled_wait set-up") : TNF_ERR_INVALID_ARGUMENT;
  if (e != cudaSuccess) return cuda_fail(e, "tnf_selftest_stalled_wait");
  return TNF_OK;  // the outcome is the status word: the next tnf_sync returns TNF_ERR_TIMEOUT
}

// ---- quantisers ----------------------------------------------------------------------------------

uint64_t tnf_device_scales_bytes(uint32_t rows, uint32_t k) { return sf_device_bytes(rows, k); }

int32_t tnf_quantize_weight(tnf_ctx* ctx, tnf_buf w_src, int32_t src_dtype, uint32_t n, uint32_t k, tnf_buf codes,
                            tnf_buf scales, float* global_scale) {
  TNF_CHECK_CTX(ctx);
  if (n == 0 || k == 0 || k % 32 != 0 || (src_dtype != TNF_DTYPE_F32 && src_dtype != TNF_DTYPE_BF16)) {
    set_error("tnf_quantize_weight: n=%u k=%u (k %% 32 == 0) dtype=%d", n, k, src_dtype);
    return TNF_ERR_INVALID_ARGUMENT;
  }
  int32_t st = TNF_OK;
  const uint64_t esz = src_dtype == TNF_DTYPE_BF16 ? 2 : 4;
  uint8_t* src = resolve(ctx, w_src, uint64_t(n) * k * esz, "w_src", &st);
  if (!src) return st;
  uint8_t* c = resolve(ctx, codes, uint64_t(n) * (k / 2), "codes", &st);
  if (!c) return st;
  uint8_t* s = resolve(ctx, scales, uint64_t(n) * (k / 16), "scales", &st);
  if (!s) return st;
  float* g = reinterpret_cast<float*>(ctx->dwords + 2);
  TNF_CUDA(launch_amax(src, src_dtype, uint64_t(n) * k, ctx->dwords + 1, ctx->compute), "amax launch");
  TNF_CUDA(launch_global_scale(ctx->dwords + 1, g, ctx->compute), "global scale launch");
  TNF_CUDA(launch_quantize(src, src_dtype, n, k, g, 0.0f, c, s, false, ctx->compute), "weight quantise launch");
  if (global_scale) {
    TNF_CUDA(cudaMemcpyAsync(global_scale, g, 4, cudaMemcpyDeviceToHost, ctx->compute), "global scale read");
    TNF_CUDA(cudaStreamSynchronize(ctx->compute), "tnf_quantize_weight sync");
  }
  return TNF_OK;
}

int32_t tnf_prepare_scales(tnf_ctx* ctx, tnf_buf scales_canonical, uint32_t rows, uint32_t k, tnf_buf scales_device) {
  TNF_CHECK_CTX(ctx);
  if (rows == 0 || k == 0 || k % 16 != 0) {
    set_error("tnf_prepare_scales: rows=%u k=%u", rows, k);
    return TNF_ERR_INVALID_ARGUMENT;
  }
  int32_t st = TNF_OK;
  uint8_t* in = resolve(ctx, scales_canonical, uint64_t(rows) * (k / 16), "scales_canonical", &st);
  if (!in) return st;
  uint8_t* out = resolve(ctx, scales_device, sf_device_bytes(rows, k), "scales_device", &st);
  if (!out) return st;
  TNF_CUDA(launch_scales_to_device(in, rows, k, out, ctx->compute), "scale layout launch");
  return TNF_OK;
}

static int32_t quantize_act_impl(tnf_ctx* ctx, const uint8_t* a, uint32_t m, uint32_t k, float g, bool device_layout,
                                 uint8_t* codes, uint8_t* scales, float* g_used) {
  const float* g_ptr = nullptr;
  if (!(g > 0.0f)) {
    float* gd = reinterpret_cast<float*>(ctx->dwords + 2);
    TNF_CUDA(launch_amax(a, TNF_DTYPE_BF16, uint64_t(m) * k, ctx->dwords + 1, ctx->compute), "amax launch");
    TNF_CUDA(launch_global_scale(ctx->dwords + 1, gd, ctx->compute), "global scale launch");
    g_ptr = gd;
  }
  TNF_CUDA(launch_quantize(a, TNF_DTYPE_BF16, m, k, g_ptr, g, codes, scales, device_layout, ctx->compute),
           "activation quantise launch");
  if (g_used) {
    if (g_ptr) {
      TNF_CUDA(cudaMemcpyAsync(g_used, g_ptr, 4, cudaMemcpyDeviceToHost, ctx->compute), "global scale read");
      TNF_CUDA(cudaStreamSynchronize(ctx->compute), "tnf_quantize_act sync");
    } else {
      *g_used = g;
    }
  }
  return TNF_OK;
}

int32_t tnf_quantize_act(tnf_ctx* ctx, tnf_buf a_bf16, uint32_t m, uint32_t k, float global_scale,
                         int32_t scales_layout, tnf_buf codes, tnf_buf scales, float* global_scale_used) {
  TNF_CHECK_CTX(ctx);
  if (m == 0 || k == 0 || k % 32 != 0) {
    set_error("tnf_quantize_act: m=%u k=%u (k %% 32 == 0)", m, k);
    return TNF_ERR_INVALID_ARGUMENT;
  }
  int32_t st = TNF_OK;
  const bool dev = scales_layout == TNF_SCALES_DEVICE;
  uint8_t* a = resolve(ctx, a_bf16, uint64_t(m) * k * 2, "a_bf16", &st);
  if (!a) return st;
  uint8_t* c = resolve(ctx, codes, uint64_t(m) * (k / 2), "codes", &st);
  if (!c) return st;
  uint8_t* s = resolve(ctx, scales, dev ? sf_device_bytes(m, k) : uint64_t(m) * (k / 16), "scales", &st);
  if (!s) return st;
  return quantize_act_impl(ctx, a, m, k, global_scale, dev, c, s, global_scale_used);
}

int32_t tnf_quantize_act_shared(tnf_ctx* ctx, tnf_buf a_bf16, uint32_t m, uint32_t k, float global_scale) {
  TNF_CHECK_CTX(ctx);
  if (m == 0 || k == 0 || k % 32 != 0 || !(global_scale > 0.0f)) {
    set_error("tnf_quantize_act_shared: m=%u k=%u (k %% 32 == 0), global_scale must be > 0", m, k);
    return TNF_ERR_INVALID_ARGUMENT;
  }
  int32_t st = TNF_OK;
  uint8_t* a = resolve(ctx, a_bf16, uint64_t(m) * k * 2, "a_bf16", &st);
  if (!a) return st;
  st = ensure_scratch(ctx, m, k);
  if (st != TNF_OK) return st;
  ctx->scratch_m = m;
  ctx->scratch_k = k;
  return quantize_act_impl(ctx, a, m, k, global_scale, true, static_cast<uint8_t*>(ctx->bufs[ctx->scratch_codes_id].ptr),
                           static_cast<uint8_t*>(ctx->bufs[ctx->scratch_scales_id].ptr), nullptr);
}

int32_t tnf_prepare_dense(tnf_ctx* ctx, tnf_buf w_codes, tnf_buf w_scales_device, uint32_t n, uint32_t k, tnf_buf out_bf16) {
  TNF_CHECK_CTX(ctx);
  if (n == 0 || k == 0 || k % 32 != 0) {
    set_error("tnf_prepare_dense: n=%u k=%u (k %% 32 == 0)", n, k);
    return TNF_ERR_INVALID_ARGUMENT;
  }
  int32_t st = TNF_OK;
  uint8_t* c = resolve(ctx, w_codes, uint64_t(n) * (k / 2), "w_codes", &st);
  if (!c) return st;
  uint8_t* s = resolve(ctx, w_scales_device, sf_device_bytes(n, k), "w_scales_device", &st);
  if (!s) return st;
  uint8_t* o = resolve(ctx, out_bf16, uint64_t(n) * k * 2, "out_bf16", &st);
  if (!o) return st;
  TNF_CUDA(launch_dequant_dense(c, s, n, k, reinterpret_cast<uint16_t*>(o), ctx->compute), "dense image launch");
  return TNF_OK;
}

uint32_t tnf_site_linear_flags(const tnf_dense_act_sites* policy, int32_t site) {
  if (!policy) return 0u;
  const uint32_t on[5] = {policy->qkv, policy->qkv_self, policy->proj, policy->ffn_up, policy->ffn_down};
  return (site >= 0 && site < 5 && on[site]) ? uint32_t(TNF_LINEAR_DENSE_ACT) : 0u;
}

// ---- the linear ------------------------------------------------------------------------------------

int32_t tnf_linear_nvfp4(tnf_ctx* ctx, const tnf_linear_args* a) {
  TNF_CHECK_CTX(ctx);
  if (!a) {
    set_error("tnf_linear_nvfp4: null args");
    return TNF_ERR_INVALID_ARGUMENT;
  }
  int32_t st = check_dims(a->m, a->n, a->k);
  if (st != TNF_OK) return st;
  const bool dense = (a->flags & TNF_LINEAR_DENSE_ACT) != 0;
  if ((!dense && !(a->a_global > 0.0f)) || !(a->w_global > 0.0f) || a->act > 1 || a->parity_mode > 1) {
    set_error("tnf_linear_nvfp4: scales must be > 0 (a %g, w %g), act %u, parity_mode %u", a->a_global, a->w_global,
              a->act, a->parity_mode);
    return TNF_ERR_INVALID_ARGUMENT;
  }
  if (dense) {
    if (a->k % 8 != 0) {
      set_error("TNF_LINEAR_DENSE_ACT: k=%u must be a multiple of 8", a->k);
      return TNF_ERR_INVALID_ARGUMENT;
    }
    if (a->flags & TNF_LINEAR_A_PREQUANTIZED) {
      // mixed arm: the NVFP4 activations in the shared scratch (tnf_quantize_act_shared) against the dense weight
      if (!(a->a_global > 0.0f) || ctx->scratch_m != a->m || ctx->scratch_k != a->k) {
        set_error("TNF_LINEAR_DENSE_ACT | TNF_LINEAR_A_PREQUANTIZED: a_global %g must be > 0 and the shared scratch must hold "
                  "m=%u k=%u (it holds m=%u k=%u)", a->a_global, a->m, a->k, ctx->scratch_m, ctx->scratch_k);
        return TNF_ERR_INVALID_ARGUMENT;
      }
      return run_mixed(ctx, a, static_cast<uint8_t*>(ctx->bufs[ctx->scratch_codes_id].ptr),
                       static_cast<uint8_t*>(ctx->bufs[ctx->scratch_scales_id].ptr));
    }
    // un-quantised activations: no quantiser launch, the GEMM reads a_bf16 itself
    uint8_t* src = resolve(ctx, a->a_bf16, uint64_t(a->m) * a->k * 2, "a_bf16", &st);
    if (!src) return st;
    return run_gemm(ctx, a, src, nullptr, nullptr, false);
  }
  // one launch for skinny M: the tensor-core kernel where it is the faster path, the CUDA-core one only for K too
  // long for it; everything else is quantiser + GEMM
  if (a->flags == 0 && (skinny_tc_applies(a->m, a->n, a->k) ||
                        (!skinny_tc_capable(a->m, a->n, a->k) && gemv_applies(a->m, a->n, a->k)))) {
    // a handful of rows: one launch that quantises A in its prologue and streams W (no scratch, no quantiser launch)
    uint8_t* src = resolve(ctx, a->a_bf16, uint64_t(a->m) * a->k * 2, "a_bf16", &st);
    if (!src) return st;
    return run_gemm(ctx, a, nullptr, nullptr, src, false);
  }
  if (!(a->flags & TNF_LINEAR_A_PREQUANTIZED)) {
    uint8_t* src = resolve(ctx, a->a_bf16, uint64_t(a->m) * a->k * 2, "a_bf16", &st);
    if (!src) return st;
    st = ensure_scratch(ctx, a->m, a->k);
    if (st != TNF_OK) return st;
    ctx->scratch_m = a->m;
    ctx->scratch_k = a->k;
    st = quantize_act_impl(ctx, src, a->m, a->k, a->a_global, true,
                           static_cast<uint8_t*>(ctx->bufs[ctx->scratch_codes_id].ptr),
                           static_cast<uint8_t*>(ctx->bufs[ctx->scratch_scales_id].ptr), nullptr);
    if (st != TNF_OK) return st;
  } else if (ctx->scratch_m != a->m || ctx->scratch_k != a->k) {
    // the scratch is tagged with the shape it was last filled for: a pre-quantised call for any other shape would
    // multiply stale codes (the scale layout depends on m and k), so it is refused
    set_error("TNF_LINEAR_A_PREQUANTIZED: the shared scratch holds the quantised activations of m=%u k=%u, not m=%u k=%u "
              "(call tnf_quantize_act_shared first)", ctx->scratch_m, ctx->scratch_k, a->m, a->k);
    return TNF_ERR_INVALID_ARGUMENT;
  }
  return run_gemm(ctx, a, static_cast<uint8_t*>(ctx->bufs[ctx->scratch_codes_id].ptr),
                  static_cast<uint8_t*>(ctx->bufs[ctx->scratch_scales_id].ptr), nullptr, false);
}

int32_t tnf_gemm_nvfp4(tnf_ctx* ctx, const tnf_linear_args* a, tnf_buf a_codes, tnf_buf a_scales_device) {
  TNF_CHECK_CTX(ctx);
  if (!a) {
    set_error("tnf_gemm_nvfp4: null args");
    return TNF_ERR_INVALID_ARGUMENT;
  }
  int32_t st = check_dims(a->m, a->n, a->k);
  if (st != TNF_OK) return st;
  if (!(a->a_global > 0.0f) || !(a->w_global > 0.0f) || a->act > 1 || a->parity_mode > 1) {
    set_error("tnf_gemm_nvfp4: scales must be > 0, act <= 1, parity_mode <= 1");
    return TNF_ERR_INVALID_ARGUMENT;
  }
  uint8_t* c = resolve(ctx, a_codes, uint64_t(a->m) * (a->k / 2), "a_codes", &st);
  if (!c) return st;
  uint8_t* s = resolve(ctx, a_scales_device, sf_device_bytes(a->m, a->k), "a_scales_device", &st);
  if (!s) return st;
  if (a->flags & TNF_LINEAR_DENSE_ACT) return run_mixed(ctx, a, c, s);
  return run_gemm(ctx, a, c, s, nullptr, false);
}

// ---- pinned host arenas and uploads -------------------------------------------------------------------

int32_t tnf_host_register(tnf_ctx* ctx, void* host_ptr, uint64_t bytes, uint64_t* host_id) {
  TNF_CHECK_CTX(ctx);
  if (!host_id || bytes == 0) {
    set_error("tnf_host_register: null id or zero size");
    return TNF_ERR_INVALID_ARGUMENT;
  }
  tnf_host_rec rec;
  rec.bytes = bytes;
  if (host_ptr) {
    TNF_CUDA(cudaHostRegister(host_ptr, bytes, cudaHostRegisterDefault), "cudaHostRegister");
    rec.ptr = host_ptr;
    rec.owned = false;
  } else {
    TNF_CUDA(cudaHostAlloc(&rec.ptr, bytes, cudaHostAllocDefault), "cudaHostAlloc");
    rec.owned = true;
  }
  std::lock_guard<std::mutex> lk(ctx->mu);
  uint64_t id = ctx->next_id++;
  ctx->hosts[id] = rec;
  *host_id = id;
  return TNF_OK;
}

int32_t tnf_host_ptr(tnf_ctx* ctx, uint64_t host_id, void** ptr, uint64_t* bytes) {
  if (!ctx) {
    set_error("null context");
    return TNF_ERR_INVALID_ARGUMENT;
  }
  std::lock_guard<std::mutex> lk(ctx->mu);
  auto it = ctx->hosts.find(host_id);
  if (it == ctx->hosts.end()) {
    set_error("tnf_host_ptr: unknown host arena %llu", (unsigned long long)host_id);
    return TNF_ERR_UNKNOWN_BUFFER;
  }
  if (ptr) *ptr = it->second.ptr;
  if (bytes) *bytes = it->second.bytes;
  return TNF_OK;
}

int32_t tnf_host_release(tnf_ctx* ctx, uint64_t host_id) {
  TNF_CHECK_CTX(ctx);
  TNF_CUDA(cudaStreamSynchronize(ctx->copy), "tnf_host_release sync");
  TNF_CUDA(cudaStreamSynchronize(ctx->readback), "tnf_host_release sync");
  std::lock_guard<std::mutex> lk(ctx->mu);
  auto it = ctx->hosts.find(host_id);
  if (it == ctx->hosts.end()) {
    set_error("tnf_host_release: unknown host arena %llu", (unsigned long long)host_id);
    return TNF_ERR_UNKNOWN_BUFFER;
  }
  cudaError_t e = it->second.owned ? cudaFreeHost(it->second.ptr) : cudaHostUnregister(it->second.ptr);
  ctx->hosts.erase(it);
  if (e != cudaSuccess) return cuda_fail(e, "tnf_host_release");
  return TNF_OK;
}

int32_t tnf_stream_upload(tnf_ctx* ctx, uint64_t host_id, uint64_t host_off, uint64_t dst_id, uint64_t dst_off,
                          uint64_t n, uint64_t* event) {
  TNF_CHECK_CTX(ctx);
  uint8_t* d = nullptr;
  int32_t st = raw_range(ctx, dst_id, dst_off, n, "tnf_stream_upload dst", &d);
  if (st != TNF_OK) return st;
  const uint8_t* h = nullptr;
  cudaEvent_t ev = nullptr;
  {
    std::lock_guard<std::mutex> lk(ctx->mu);
    auto it = ctx->hosts.find(host_id);
    if (it == ctx->hosts.end()) {
      set_error("tnf_stream_upload: unknown host arena %llu", (unsigned long long)host_id);
      return TNF_ERR_UNKNOWN_BUFFER;
    }
    if (host_off > it->second.bytes || n > it->second.bytes - host_off) {
      set_error("tnf_stream_upload: host range [%llu, +%llu) outside arena of %llu bytes",
                (unsigned long long)host_off, (unsigned long long)n, (unsigned long long)it->second.bytes);
      return TNF_ERR_INVALID_ARGUMENT;
    }
    h = static_cast<const uint8_t*>(it->second.ptr) + host_off;
    if (event) {
      if (!ctx->event_pool.empty()) {
        ev = ctx->event_pool.back();
        ctx->event_pool.pop_back();
      }
    }
    ctx->streamed += n;
  }
  if (n) TNF_CUDA(cudaMemcpyAsync(d, h, n, cudaMemcpyHostToDevice, ctx->copy), "tnf_stream_upload copy");
  if (event) {
    if (!ev) TNF_CUDA(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming), "cudaEventCreate");
    TNF_CUDA(cudaEventRecord(ev, ctx->copy), "cudaEventRecord");
    std::lock_guard<std::mutex> lk(ctx->mu);
    uint64_t id = ctx->next_id++;
    ctx->events[id] = ev;
    *event = id;
  }
  return TNF_OK;
}

int32_t tnf_wait_event(tnf_ctx* ctx, uint64_t event) {
  TNF_CHECK_CTX(ctx);
  cudaEvent_t ev;
  {
    std::lock_guard<std::mutex> lk(ctx->mu);
    auto it = ctx->events.find(event);
    if (it == ctx->events.end()) {
      set_error("tnf_wait_event: unknown event %llu", (unsigned long long)event);
      return TNF_ERR_UNKNOWN_BUFFER;
    }
    ev = it->second;
    ctx->events.erase(it);
  }
  cudaError_t e = cudaStreamWaitEvent(ctx->compute, ev, 0);
  {
    // the wait has captured the event's current record; the object can be recycled
    std::lock_guard<std::mutex> lk(ctx->mu);
    ctx->event_pool.push_back(ev);
  }
  if (e != cudaSuccess) return cuda_fail(e, "cudaStreamWaitEvent");
  return TNF_OK;
}

int32_t tnf_stream_download(tnf_ctx* ctx, uint64_t src_id, uint64_t src_off, uint64_t host_id, uint64_t host_off,
                            uint64_t n, uint64_t* event) {
  TNF_CHECK_CTX(ctx);
  uint8_t* d = nullptr;
  int32_t st = raw_range(ctx, src_id, src_off, n, "tnf_stream_download src", &d);
  if (st != TNF_OK) return st;
  uint8_t* h = nullptr;
  cudaEvent_t order = nullptr, done = nullptr;
  {
    std::lock_guard<std::mutex> lk(ctx->mu);
    auto it = ctx->hosts.find(host_id);
    if (it == ctx->hosts.end()) {
      set_error("tnf_stream_download: unknown host arena %llu", (unsigned long long)host_id);
      return TNF_ERR_UNKNOWN_BUFFER;
    }
    if (host_off > it->second.bytes || n > it->second.bytes - host_off) {
      set_error("tnf_stream_download: host range [%llu, +%llu) outside arena of %llu bytes",
                (unsigned long long)host_off, (unsigned long long)n, (unsigned long long)it->second.bytes);
      return TNF_ERR_INVALID_ARGUMENT;
    }
    h = static_cast<uint8_t*>(it->second.ptr) + host_off;
    for (cudaEvent_t* e : {&order, &done}) {
      if (!ctx->event_pool.empty()) {
        *e = ctx->event_pool.back();
        ctx->event_pool.pop_back();
      }
    }
  }
  if (!order) TNF_CUDA(cudaEventCreateWithFlags(&order, cudaEventDisableTiming), "cudaEventCreate");
  if (!done) TNF_CUDA(cudaEventCreateWithFlags(&done, cudaEventDisableTiming), "cudaEventCreate");
  // the copy starts when everything launched so far on the compute stream (the producer of src) is done
  TNF_CUDA(cudaEventRecord(order, ctx->compute), "cudaEventRecord");
  TNF_CUDA(cudaStreamWaitEvent(ctx->readback, order, 0), "cudaStreamWaitEvent");
  if (n) TNF_CUDA(cudaMemcpyAsync(h, d, n, cudaMemcpyDeviceToHost, ctx->readback), "tnf_stream_download copy");
  TNF_CUDA(cudaEventRecord(done, ctx->readback), "cudaEventRecord");
  std::lock_guard<std::mutex> lk(ctx->mu);
  ctx->event_pool.push_back(order);
  if (event) {
    uint64_t id = ctx->next_id++;
    ctx->events[id] = done;
    *event = id;
  } else {
    ctx->event_pool.push_back(done);
  }
  return TNF_OK;
}

int32_t tnf_event_sync(tnf_ctx* ctx, uint64_t event) {
  TNF_CHECK_CTX(ctx);
  cudaEvent_t ev;
  {
    std::lock_guard<std::mutex> lk(ctx->mu);
    auto it = ctx->events.find(event);
    if (it == ctx->events.end()) {
      set_error("tnf_event_sync: unknown event %llu", (unsigned long long)event);
      return TNF_ERR_UNKNOWN_BUFFER;
    }
    ev = it->second;
    ctx->events.erase(it);
  }
  cudaError_t e = cudaEventSynchronize(ev);
  {
    std::lock_guard<std::mutex> lk(ctx->mu);
    ctx->event_pool.push_back(ev);
  }
  if (e != cudaSuccess) return cuda_fail(e, "cudaEventSynchronize");
  return TNF_OK;
}

int32_t tnf_copy_after_compute(tnf_ctx* ctx) {
  TNF_CHECK_CTX(ctx);
  cudaEvent_t ev = nullptr;
  {
    std::lock_guard<std::mutex> lk(ctx->mu);
    if (!ctx->event_pool.empty()) {
      ev = ctx->event_pool.back();
      ctx->event_pool.pop_back();
    }
  }
  if (!ev) TNF_CUDA(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming), "cudaEventCreate");
  TNF_CUDA(cudaEventRecord(ev, ctx->compute), "cudaEventRecord");
  TNF_CUDA(cudaStreamWaitEvent(ctx->copy, ev, 0), "cudaStreamWaitEvent");
  std::lock_guard<std::mutex> lk(ctx->mu);
  ctx->event_pool.push_back(ev);
  return TNF_OK;
}

}  // extern "C"
