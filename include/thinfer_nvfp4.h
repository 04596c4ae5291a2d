/*
 * thinfer_nvfp4.h — C ABI of the B200 (sm_100a) NVFP4 linear path.
 *
 * This is the boundary a thinfer maintainer binds from Rust (`extern "C"`): plain
 * pointers and sizes, no C++ or torch types. Each entry point names the reference
 * interface it stands in for (paths are relative to the reference's `projects/`).
 *
 * Conventions kept from the reference: activations A are [M,K] row-major bf16, weights
 * are [N,K] ("N-major", blocks contiguous along K; thinfer-core/src/residency.rs:1026-1030),
 * outputs are [M,N] row-major bf16; buffers are opaque ids in a backend-owned table
 * (GpuBufferId, thinfer-core/src/tensor.rs:52-53) and `tnf_buf` is the non-owning
 * {id, offset, len} view (BufRef, thinfer-core/src/backend/mod.rs:12-33).
 *
 * Every function returns a status: 0 on success, a negative tnf_status otherwise;
 * tnf_last_error() gives the text of the calling thread's most recent failure.
 * Kernel launches are asynchronous on the context's compute stream; uploads issued with
 * tnf_stream_upload run on its copy stream. There is no CPU fallback anywhere: without a
 * CUDA device every call that needs one fails with TNF_ERR_LAUNCH.
 */
#ifndef THINFER_NVFP4_H_
#define THINFER_NVFP4_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Error classes; mirror WgpuError (thinfer-core/src/backend/wgpu.rs:115-159). */
typedef enum tnf_status {
  TNF_OK = 0,
  TNF_ERR_UNKNOWN_BUFFER = -1,  /* WgpuError::UnknownBuffer */
  TNF_ERR_ALLOCATE_OOM = -2,    /* WgpuError::AllocateOom: the device refused */
  TNF_ERR_BUDGET_EXCEEDED = -3, /* WgpuError::BudgetExceeded: refused on the host, device untouched */
  TNF_ERR_INVALID_ARGUMENT = -4,/* shape / alignment / range */
  TNF_ERR_LAUNCH = -5,          /* WgpuError::SubmitFailed: CUDA reported an error */
  TNF_ERR_TIMEOUT = -6,         /* a bounded device-side or host-side wait gave up */
  TNF_ERR_NCCL = -7
} tnf_status;

/* VramCategory (thinfer-core/src/mem.rs:14-26). */
enum { TNF_CAT_WEIGHTS = 0, TNF_CAT_WORKSPACE = 1, TNF_CAT_STAGING = 2 };

/* Source dtypes accepted by the weight quantiser. */
enum { TNF_DTYPE_F32 = 0, TNF_DTYPE_BF16 = 1 };

/* Scale layouts. CANONICAL is row-major [rows, K/16]; DEVICE is the 128x4 tiled layout
 * the block-scaled MMA reads (512-byte atoms [rows/128][K/64 rounded up to 4]; inside an
 * atom byte (r%32)*16 + ((r%128)/32)*4 + (b%4) holds row r, block b). */
enum { TNF_SCALES_CANONICAL = 0, TNF_SCALES_DEVICE = 1 };

/* Epilogue activation. GELU is the tanh form of thinfer-core/src/ops/gelu.rs:21-31. */
enum { TNF_ACT_NONE = 0, TNF_ACT_GELU_TANH = 1 };

typedef struct tnf_ctx tnf_ctx; /* one per device; Arc<WgpuBackend> in the reference */

typedef struct tnf_buf {
  uint64_t id, offset, len;
} tnf_buf;

/* ---- context and buffers ------------------------------------------------------------ */

/* WgpuBackend::new + MemArbiter budget (thinfer-core/src/backend/wgpu.rs:741-760,
 * thinfer-core/src/arbiter.rs:58-127). vram_budget_bytes == 0 means "no budget". */
int32_t tnf_create(int32_t device, uint64_t vram_budget_bytes, tnf_ctx** out);
int32_t tnf_destroy(tnf_ctx* ctx);
const char* tnf_last_error(void);
/* Bytes of the built library's ABI version; bumps on any signature change. */
uint32_t tnf_abi_version(void);

/* Backend::allocate_in (thinfer-core/src/backend/mod.rs:104-113): charged to `category`;
 * a request that would pass the budget fails with TNF_ERR_BUDGET_EXCEEDED before the
 * device is touched (budget_oom_error, :101-107). */
int32_t tnf_alloc(tnf_ctx* ctx, uint64_t bytes, int32_t category, uint64_t* id);
/* Backend::free (thinfer-core/src/backend/wgpu.rs:764-780). */
int32_t tnf_free(tnf_ctx* ctx, uint64_t id);
/* Backend::write_buffer (thinfer-core/src/backend/mod.rs:123-132): ordered before later
 * launches on the compute stream; the host memory may be reused on return. */
int32_t tnf_write(tnf_ctx* ctx, uint64_t id, uint64_t dst_off, const void* src, uint64_t n);
/* Backend::read_buffer (thinfer-core/src/backend/mod.rs:188-196): blocking. */
int32_t tnf_read(tnf_ctx* ctx, uint64_t id, uint64_t off, void* dst, uint64_t n);
/* Backend::copy_buffer_to_buffer (thinfer-core/src/backend/mod.rs:150-160). */
int32_t tnf_copy(tnf_ctx* ctx, uint64_t src_id, uint64_t src_off, uint64_t dst_id, uint64_t dst_off, uint64_t n);
/* Raw device address of a buffer, for callers that interoperate with other CUDA code
 * (no reference counterpart: wgpu hides addresses). */
int32_t tnf_buf_ptr(tnf_ctx* ctx, uint64_t id, void** device_ptr, uint64_t* bytes);
/* Awaited Backend::submit (thinfer-core/src/backend/wgpu.rs:941-1071): waits for the
 * compute and copy streams, then reports a device-side wait that gave up as
 * TNF_ERR_TIMEOUT. timeout_ms == 0 waits without a host limit. */
int32_t tnf_sync(tnf_ctx* ctx, uint32_t timeout_ms);
/* MemAccount snapshot (thinfer-core/src/mem.rs:105-196): out = {live weights, live
 * workspace, live staging, peak weights, peak workspace, peak staging, true concurrent
 * peak, bytes streamed host->device since creation}. */
int32_t tnf_mem_snapshot(tnf_ctx* ctx, uint64_t out[8]);
/* MemArbiter::reclaim_until_fits (thinfer-core/src/arbiter.rs:129-160): an allocation that does not fit the
 * budget first asks the registered holders of weight memory (every tnf_stack of the context: WeightReclaimer,
 * thinfer-core/src/residency.rs:1473-1547) to give memory back -- resident weight sets, largest first; a set that
 * is given back is streamed through its ring from the next step on -- and is refused with
 * TNF_ERR_BUDGET_EXCEEDED only if that was not enough. *bytes = total given back so far. */
int32_t tnf_reclaimed_bytes(tnf_ctx* ctx, uint64_t* bytes);
/* Workspace pool (Workspace::alloc / WsBuf::drop / drain_pool / pool_bytes / free_count,
 * thinfer-core/src/workspace.rs:131-316,318-420): scratch buffers rented by size class
 * (bytes rounded up to 256, at least 256), charged to the workspace category.
 *   tnf_ws_alloc    hands out the newest idle buffer of the class without a device call (a hit), else
 *                   allocates one (a miss) under the same budget rule as tnf_alloc. The buffer is at
 *                   least `bytes` long; views over it carry the requested length.
 *   tnf_ws_release  puts a rented buffer back as idle. Its bytes stay allocated and stay in the
 *                   workspace category of the snapshot; work already enqueued on the compute stream
 *                   that uses it is ordered before whatever the next renter enqueues there.
 *   tnf_ws_drain    frees every idle buffer (the phase boundary call); buffers out on rent stay.
 *   tnf_ws_stats    out = {idle bytes, idle buffers, buffers out on rent, hits, misses, bytes freed
 *                   under memory pressure}.
 * The idle pool is the first holder asked when an allocation does not fit the budget
 * (RECLAIM_IDLE_POOL before RECLAIM_EVICTABLE_WEIGHTS, thinfer-core/src/arbiter.rs:37-38): smallest
 * class first, until enough is back (spill_pool_locked, workspace.rs:52-85); only then are weights
 * given back. tnf_free on a pool buffer also takes it out of the pool's books. Releasing an id
 * that is not out on rent fails with TNF_ERR_UNKNOWN_BUFFER. */
int32_t tnf_ws_alloc(tnf_ctx* ctx, uint64_t bytes, uint64_t* id);
int32_t tnf_ws_release(tnf_ctx* ctx, uint64_t id);
int32_t tnf_ws_drain(tnf_ctx* ctx, uint64_t* freed_bytes);
int32_t tnf_ws_stats(tnf_ctx* ctx, uint64_t out[6]);
/* set_transient_reserve (thinfer-core/src/residency.rs:535-537): bytes of the budget that weight plans
 * (tnf_stack_create with a context budget, tnf_stack_restore) leave free for transient workspace. */
int32_t tnf_set_transient_reserve(tnf_ctx* ctx, uint64_t bytes);
/* Upper bound, in SM cycles, of every device-side wait of the kernels launched afterwards (a wait on a
 * loaded stage, a freed stage, a finished or drained accumulator). A wait that runs out makes its kernel
 * return normally with the status word set, and the next tnf_sync returns TNF_ERR_TIMEOUT: the analogue of a
 * submit whose error surfaces at the awaited future (thinfer-core/src/backend/wgpu.rs:948,1063-1068) instead
 * of a lost device. 0 restores the default (4e9 cycles, about two seconds). */
int32_t tnf_set_device_wait_limit(tnf_ctx* ctx, uint64_t sm_cycles);
/* Failure-detection self-test (the reference's counterpart is the submit-error path above, exercised
 * in its tests by a failing dispatch): launches the CTA-pair GEMM on a small zeroed problem with its
 * loader switched off, so that nothing is in flight and the first device-side wait runs out after the
 * context's wait limit. Blocks until the kernel has returned. The call itself returns TNF_OK; the
 * NEXT tnf_sync must return TNF_ERR_TIMEOUT, and the context stays usable afterwards. Set a short
 * limit first (tnf_set_device_wait_limit), or the call takes about two seconds. */
int32_t tnf_selftest_stalled_wait(tnf_ctx* ctx);
/* The context's CUDA streams (cudaStream_t as void*), for event timing by the caller. */
int32_t tnf_streams(tnf_ctx* ctx, void** compute_stream, void** copy_stream);

/* ---- quantisers (canonical layouts are bit-exact with the CPU oracle) ---------------- */

/* Load-time transcode of a dense weight to NVFP4; stands where the reference's upload-time
 * weight prep does (WeightPrep::Q8_0FromBf16, thinfer-core/src/backend/mod.rs:65-90,
 * thinfer-core/src/ops/weight_prep.rs:86-163). w_src is f32 or bf16 [n,k]; codes is
 * [n,k/2], scales [n,k/16] canonical. *global_scale receives amax/(6*448). Blocking. */
int32_t tnf_quantize_weight(tnf_ctx* ctx, tnf_buf w_src, int32_t src_dtype, uint32_t n, uint32_t k,
                            tnf_buf codes, tnf_buf scales, float* global_scale);
/* Bytes of the DEVICE scale layout for a [rows,k] operand. */
uint64_t tnf_device_scales_bytes(uint32_t rows, uint32_t k);
/* Canonical scales -> DEVICE layout (weights: once at load; PreparedWeight idea,
 * thinfer-models/src/common/block.rs:217-227). */
int32_t tnf_prepare_scales(tnf_ctx* ctx, tnf_buf scales_canonical, uint32_t rows, uint32_t k, tnf_buf scales_device);
/* Per-row, per-16 activation quantiser; stands where act_quant does
 * (thinfer-core/src/ops/act_quant.rs:58-191, BatchScope::act_quant
 * thinfer-core/src/workspace.rs:774-800). a_bf16 is [m,k]; global_scale > 0 is the
 * per-tensor scale to use, 0 computes amax/(6*448) on the device first.
 * *global_scale_used may be NULL; when not NULL the call blocks to report it. */
int32_t tnf_quantize_act(tnf_ctx* ctx, tnf_buf a_bf16, uint32_t m, uint32_t k, float global_scale,
                         int32_t scales_layout, tnf_buf codes, tnf_buf scales, float* global_scale_used);

/* ---- the linear ---------------------------------------------------------------------- */

/* out = epilogue(alpha * (Aq . Wq^T)): the dispatch arm Block::dispatch_matmul_site_diag
 * selects (thinfer-models/src/common/block.rs:2656-2882) plus the bias / GELU / gated
 * residual dispatches that follow it at the call sites
 * (thinfer-models/src/qwen_image/dit.rs:324-340,745-754; thinfer-core/src/ops/bcast_add.rs,
 * gelu.rs, bcast_fma.rs), fused. */
typedef struct tnf_linear_args {
  uint32_t m, n, k;
  float a_global;       /* per-tensor activation scale; > 0 */
  float w_global;       /* per-tensor weight scale from tnf_quantize_weight */
  tnf_buf a_bf16;       /* [m,k] bf16; quantised on the fly */
  tnf_buf w_codes;      /* [n,k/2] */
  tnf_buf w_scales;     /* DEVICE layout (tnf_prepare_scales) */
  tnf_buf bias_bf16;    /* [n] or len 0 */
  tnf_buf gate_bf16;    /* [n] or len 0: out = residual + gate*y (BcastFma) */
  tnf_buf residual_bf16;/* [m,n] (leading dim n) when gate is given */
  tnf_buf out_bf16;     /* [m, ldo] */
  uint32_t act;         /* TNF_ACT_* */
  uint32_t parity_mode; /* 0 fused (one rounding), 1 chain (reference's intermediate bf16 roundings) */
  uint32_t n_offset;    /* column offset into out (N-split) */
  uint32_t ldo;         /* leading dimension of out in elements; 0 = n */
  uint32_t flags;       /* TNF_LINEAR_* */
  float out_global;     /* TNF_LINEAR_OUT_NVFP4: per-tensor scale of the quantised output; > 0 */
  tnf_buf out_codes;    /* TNF_LINEAR_OUT_NVFP4: [m, ldo/2] E2M1 codes of the bf16-rounded output; this call fills
                           the bytes of columns n_offset .. n_offset+n of each row */
  tnf_buf out_scales;   /* TNF_LINEAR_OUT_NVFP4: DEVICE-layout scales of an [m, ldo] operand (same window) */
  tnf_buf w_dense;      /* TNF_LINEAR_DENSE_ACT: the weight's dense bf16 image [n,k] from tnf_prepare_dense */
} tnf_linear_args;

enum {
  TNF_LINEAR_A_PREQUANTIZED = 1u, /* a_bf16 unused; a_codes/a_scales of the ctx scratch come from tnf_quantize_act_shared */
  TNF_LINEAR_SCATTER_PEERS = 2u,  /* epilogue also stores to every peer registered with tnf_peer_outputs */
  /* The epilogue also quantises its bf16-rounded result to NVFP4 (same bits as tnf_quantize_act
   * on out_bf16 would give), ready to be the A operand of tnf_gemm_nvfp4: MLP up -> GELU -> down
   * (thinfer-models/src/qwen_image/dit.rs:745-754) without the act_quant dispatch between.
   * Requires n, n_offset and ldo to be multiples of 64; not combinable with gate_bf16 / residual_bf16
   * or TNF_LINEAR_SCATTER_PEERS. */
  TNF_LINEAR_OUT_NVFP4 = 4u,
  TNF_LINEAR_NO_BF16_OUT = 8u,    /* with OUT_NVFP4: skip the bf16 store (out_bf16 may have len 0) */
  /* The outputs of this call (out_bf16, and out_codes / out_scales with OUT_NVFP4) live in buffers
   * registered with tnf_import_symmetric: the epilogue stores them through the NVSwitch multicast
   * alias (multimem.st), so every rank of the group receives this rank's column window at the same
   * offsets while the GEMM is still running: the all-gather of an N-split output, fused into the
   * kernel that produces it. Follow with a barrier across the ranks before the result is read. */
  TNF_LINEAR_MULTICAST_OUT = 16u,
  /* The site keeps its activations un-quantised: out = epilogue(w_global * (A_bf16 . Wd^T)) with Wd the dense image
   * of the NVFP4 weight (w_dense). This is the reference's dense arm for sites whose A-side carries outliers
   * (DenseActSites, thinfer-models/src/common/block.rs:458-479; the "dequant once, then matmul" branch of
   * dispatch_matmul_site_diag, :2861-2881, with PreparedWeight::F16, :217-227). a_bf16 is required, a_global is
   * not used, no activation quantiser runs; bf16 x bf16 products on the tensor cores (tcgen05.mma kind::f16),
   * f32 accumulation, the same fused epilogue. k must be a multiple of 8.
   * w_dense may also be a weight that was never quantised (plain bf16 [n,k], w_global = 1): the reference's
   * refiner weights (thinfer-core/src/ops/matmul_i8_bf16.rs:15-17).
   * Mixed arm -- low-bit activations x dense bf16 weight, the role of the reference's matmul_i8_bf16
   * (thinfer-core/src/ops/matmul_i8_bf16.rs:1-17,113-292): with TNF_LINEAR_A_PREQUANTIZED as well (activations in
   * the shared scratch), or through tnf_gemm_nvfp4 with this flag (activations as codes + DEVICE scales), the
   * NVFP4 activations are first widened to bf16 in a workspace buffer (exact: a code times its block scale has
   * at most 6 significant bits) and out = epilogue(a_global * w_global * (Aq . Wd^T)). NVFP4 has no zero point, so
   * the reference's `za * sum_k b` correction term (bf16_block_sum.rs) has no counterpart. */
  TNF_LINEAR_DENSE_ACT = 32u,
  /* SwiGLU gating fused into the FFN-up GEMM: the weight is the ROW-INTERLEAVED pair [W1 row 0, W3 row 0,
   * W1 row 1, ...] (n = 2 x hidden rows, quantised as one tensor), and the epilogue writes
   * out[m, j] = silu(v[2j]) * v[2j+1] with silu(v) = v / (1 + exp(-v)): the reference's two matmul dispatches on
   * the same A plus its silu_mul dispatch (thinfer-models/src/common/block.rs:1720-1762,
   * thinfer-core/src/ops/silu_mul.rs) as one launch. out_bf16 is [m, ldo] with n/2 columns written at
   * n_offset (ldo = 0 means n/2); a bias, if given, is interleaved like the rows; act must be TNF_ACT_NONE;
   * n a multiple of 16; not combinable with a gated residual, OUT_NVFP4, SCATTER_PEERS or MULTICAST_OUT. */
  TNF_LINEAR_SWIGLU = 64u
};

/* Which linear sites of a block keep their activations dense; same fields as the reference's DenseActSites
 * (thinfer-models/src/common/block.rs:470-479). A site that is set runs with TNF_LINEAR_DENSE_ACT and needs
 * the weight's dense image; the others quantise their activations to NVFP4. */
typedef struct tnf_dense_act_sites {
  uint32_t qkv, qkv_self, proj, ffn_up, ffn_down;
} tnf_dense_act_sites;
enum { TNF_SITE_QKV = 0, TNF_SITE_QKV_SELF = 1, TNF_SITE_PROJ = 2, TNF_SITE_FFN_UP = 3, TNF_SITE_FFN_DOWN = 4 };
/* The tnf_linear_args.flags bits a site runs with under a policy (0 or TNF_LINEAR_DENSE_ACT). */
uint32_t tnf_site_linear_flags(const tnf_dense_act_sites* policy, int32_t site);

int32_t tnf_linear_nvfp4(tnf_ctx* ctx, const tnf_linear_args* args);
/* The dense bf16 image [n,k] of an NVFP4 weight for TNF_LINEAR_DENSE_ACT sites: code x block scale, exact in
 * bf16, without the per-tensor scale (the epilogue applies it). Made once per weight and kept resident, like
 * the reference's pre-dequantised PreparedWeight::F16 (thinfer-models/src/common/block.rs:211-227). */
int32_t tnf_prepare_dense(tnf_ctx* ctx, tnf_buf w_codes, tnf_buf w_scales_device, uint32_t n, uint32_t k, tnf_buf out_bf16);

/* LayerNorm (no affine) + AdaLN modulation + activation quantiser in one pass: the two
 * dispatches in front of every block linear, op_layernorm (thinfer-core/src/ops/layernorm.rs:95-125)
 * and op_modulate = x * (scale + mod_bias) + shift (thinfer-core/src/ops/bcast_modulate.rs:93-102;
 * call sites thinfer-models/src/qwen_image/dit.rs:521-532,757-768), followed by tnf_quantize_act
 * with a given per-tensor scale. The modulated row is rounded to bf16 once (parity_mode 1: also
 * after the LayerNorm, as the reference's two dispatches do) and quantised from those bits, so
 * out_codes / out_scales (DEVICE layout) hold what tnf_quantize_act would make of out_bf16; they
 * feed tnf_gemm_nvfp4. scale_bf16 / shift_bf16: [k] bf16, both or neither (len 0 = LayerNorm only);
 * out_bf16: [m, k] or len 0 to skip the bf16 store. k % 16 == 0, k <= 16384, out_global > 0. */
typedef struct {
  uint32_t m, k;
  float eps;       /* 1e-6 at the reference's call sites */
  float mod_bias;  /* 1.0 folds the "1 +" of AdaLN */
  tnf_buf x_bf16, scale_bf16, shift_bf16, out_bf16, out_codes, out_scales;
  float out_global;
  uint32_t parity_mode; /* 0 fused, 1 chain */
} tnf_norm_quant_args;
int32_t tnf_norm_modulate_quantize(tnf_ctx* ctx, const tnf_norm_quant_args* args);

/* Same linear, for callers that must not allocate device memory (a fixed memory plan, a
 * latency-critical thread, a host that forbids allocation after start-up). It has no counterpart
 * in the reference. The quantised activations go to a 16 MiB array built into the library
 * image (tnf_noalloc_scratch_bytes) instead of context scratch grown with cudaMalloc; a problem
 * whose m*k/2 + tnf_device_scales_bytes(m,k) exceeds it is refused with
 * TNF_ERR_INVALID_ARGUMENT. flags must be 0. The first call on a device resolves the array's
 * device address: make it before any stream capture. All calls share the array, which keeps the
 * last call's contents; calls whose kernels overlap on the GPU race on it. */
int32_t tnf_linear_nvfp4_noalloc(tnf_ctx* ctx, const tnf_linear_args* args);
uint64_t tnf_noalloc_scratch_bytes(void);

/* Quantise A once into context scratch so that several linears can share it (q, k and v
 * read one A: thinfer-models/src/qwen_image/dit.rs:511-560). Follow with
 * tnf_linear_nvfp4(flags = TNF_LINEAR_A_PREQUANTIZED). */
int32_t tnf_quantize_act_shared(tnf_ctx* ctx, tnf_buf a_bf16, uint32_t m, uint32_t k, float global_scale);

/* Pre-quantised operands on both sides (codes + DEVICE scales): the GEMM alone. With TNF_LINEAR_DENSE_ACT the
 * weight side is w_dense instead (mixed arm, see the flag). */
int32_t tnf_gemm_nvfp4(tnf_ctx* ctx, const tnf_linear_args* args, tnf_buf a_codes, tnf_buf a_scales_device);

/* ---- attention between the linears ------------------------------------------------------ */

/* op_sdpa (thinfer-core/src/ops/sdpa.rs:10-47; the DiT call site thinfer-models/src/qwen_image/dit.rs:618-655 runs it
 * over the joint [txt ++ img] sequence with has_mask = 0): out = softmax(Q K^T * scale) V per (batch, head).
 * q, out: bf16 [b, s_q, h_q, d]; k, v: bf16 [b, s_k, h_kv, d] (query head hq reads kv head hq * h_kv / h_q). d must be
 * 128, scale > 0, mask_mode 0 (no mask: the only mode the DiT blocks use). f32 softmax statistics and accumulation;
 * the probabilities are rounded to bf16 for the second product (relative Frobenius error <= 4e-3 against the
 * reference's f32 recurrence). Asynchronous on the compute stream. */
typedef struct tnf_sdpa_args {
  uint32_t b, s_q, s_k, h_q, h_kv, d;
  float scale;
  uint32_t mask_mode;
  tnf_buf q, k, v, out;
  uint32_t flags;       /* TNF_SDPA_* */
  float out_global;     /* TNF_SDPA_OUT_NVFP4: per-tensor scale of the quantised copy */
  tnf_buf out_codes;    /* TNF_SDPA_OUT_NVFP4: codes of the output viewed as [b * s_q, h_q * 128] ... */
  tnf_buf out_scales;   /* ... and its DEVICE-layout scales: the A operand of the out-projection (tnf_gemm_nvfp4) */
  uint32_t q_ld, kv_ld; /* elements between consecutive rows of q, and of k and v; 0 = dense (h * d). With the fused-QKV
                           output [rows, 3 * h * d] as the source, q / k / v are views at column 0, h*d, 2*h*d with
                           ld = 3 * h * d: no split copies (the reference concatenates and splits with buffer copies,
                           thinfer-models/src/qwen_image/dit.rs:605-616,648-654) */
} tnf_sdpa_args;
enum {
  /* The epilogue also quantises its bf16-rounded output to NVFP4 (the same bits tnf_quantize_act makes of `out`):
   * the out-projection that follows (thinfer-models/src/qwen_image/dit.rs:655-670) needs no act_quant dispatch and
   * never reads the bf16 tensor. */
  TNF_SDPA_OUT_NVFP4 = 1u,
  TNF_SDPA_NO_BF16_OUT = 2u /* with OUT_NVFP4: skip the bf16 store (out may have len 0) */
};
int32_t tnf_sdpa(tnf_ctx* ctx, const tnf_sdpa_args* args);

/* ---- streaming residency (WeightResidency, thinfer-core/src/residency.rs) ------------ */

/* Pinned host arena. host_ptr == NULL allocates `bytes` of pinned memory owned by the
 * context; otherwise the caller's range is page-locked in place. The reference has no
 * pinned memory (queue.write_buffer staging, thinfer-core/src/backend/wgpu.rs:782-803). */
int32_t tnf_host_register(tnf_ctx* ctx, void* host_ptr, uint64_t bytes, uint64_t* host_id);
int32_t tnf_host_ptr(tnf_ctx* ctx, uint64_t host_id, void** ptr, uint64_t* bytes);
int32_t tnf_host_release(tnf_ctx* ctx, uint64_t host_id);
/* stream_source_to_gpu (thinfer-core/src/residency.rs:1197-1341): asynchronous copy on
 * the copy stream; *event identifies its completion. */
int32_t tnf_stream_upload(tnf_ctx* ctx, uint64_t host_id, uint64_t host_off, uint64_t dst_id,
                          uint64_t dst_off, uint64_t n, uint64_t* event);
/* Compute stream waits for an upload event; the host does not block. */
int32_t tnf_wait_event(tnf_ctx* ctx, uint64_t event);
/* Asynchronous read-back into a pinned arena (the reference's read_buffer is awaited, not blocking:
 * thinfer-core/src/backend/mod.rs:180-185): once the work queued so far on the compute stream is
 * done, a read-back stream (separate from the upload stream: the link is full duplex) copies
 * src -> host; *event identifies completion. tnf_event_sync blocks
 * the HOST on an event (and retires it); tnf_wait_event makes the compute stream wait for it. */
int32_t tnf_stream_download(tnf_ctx* ctx, uint64_t src_id, uint64_t src_off, uint64_t host_id, uint64_t host_off,
                            uint64_t n, uint64_t* event);
int32_t tnf_event_sync(tnf_ctx* ctx, uint64_t event);
/* Copy stream waits until everything launched so far on the compute stream is done
 * (a ring slot may be overwritten only after its last reader). */
int32_t tnf_copy_after_compute(tnf_ctx* ctx);

/* Layer-stack driver: the block loop that joins {compute block i, acquire i+1, prefetch
 * i+2} (thinfer-models/src/qwen_image/dit.rs:1052-1180, thinfer-models/src/wan/dit.rs:520-640)
 * over weights registered in rings / a pin plan (register_in_ring :382-423, set_pin_plan
 * :440-457). See tnf_stack_* below. */
typedef struct tnf_stack tnf_stack;

typedef struct tnf_stack_linear {
  uint32_t n, k;
  uint32_t act;        /* TNF_ACT_* */
  uint32_t has_bias;
  uint32_t input;      /* 0: the stream's layer input X; 1: the previous linear's output; 2: the stream's
                          auxiliary input (stands for the attention output that feeds the out-projection) */
  uint32_t stream_id;  /* which activation stream (0 img, 1 txt, 2 mod ...) */
} tnf_stack_linear;

/* Describe a stack of `layers` identical layers, each `n_linears` linears applied to
 * `n_streams` activation streams of m_rows[s] rows. Weights wait in the pinned arena
 * `host_id`, layer-major then linear-minor, one record per linear: {codes [n,k/2], DEVICE
 * scales, bias bf16 [n], f32 per-tensor scale}, each section 256-byte aligned
 * (tnf_stack_record_offsets); tnf_stack_record_bytes gives the record size.
 * `weight_budget_bytes` (0 = unlimited) bounds resident + ring weight bytes: every linear
 * kind gets a ring of `ring_slots` records (0 = 4, thinfer-core/src/residency.rs:50) and the
 * rest of the budget pins whole linear kinds across all layers, largest first (role-major
 * pin plan). A budget below the ring reserve fails with TNF_ERR_BUDGET_EXCEEDED on the host.
 * The last linear of a stream feeds the next layer's X when its n equals `hidden`. */
uint64_t tnf_stack_record_bytes(uint32_t n, uint32_t k);
int32_t tnf_stack_record_offsets(uint32_t n, uint32_t k, uint64_t out[4]); /* codes, scales, bias, global */
int32_t tnf_stack_create(tnf_ctx* ctx, uint32_t layers, uint32_t n_linears, const tnf_stack_linear* linears,
                         uint32_t n_streams, const uint32_t* m_rows, uint32_t hidden, uint64_t host_id,
                         uint64_t weight_budget_bytes, uint32_t ring_slots, tnf_stack** out);
/* One pass over all layers (one "DiT step" of the GEMM stack), enqueued without blocking the
 * host: uploads on the copy stream run ring_slots layers ahead of the GEMMs and wrap around to
 * the next step's first layers. x_ids[s]: [m_rows[s], hidden] bf16 inputs; aux_ids[s]
 * (may be NULL when no linear has input 2): [m_rows[s], k]; out_ids[s] receives the last
 * layer's last linear of stream s. a_global: per-tensor activation scale used by every linear. */
int32_t tnf_stack_step(tnf_stack* st, const uint64_t* x_ids, const uint64_t* aux_ids, const uint64_t* out_ids,
                       float a_global);
/* out = {resident weight bytes, ring bytes, bytes uploaded by the last step, uploads in
 * the last step, resident (layer, linear) records, streamed records}. */
int32_t tnf_stack_stats(tnf_stack* st, uint64_t out[6]);
/* Phase eviction (evict_all_and_free, thinfer-core/src/residency.rs:1415-1465): waits for the work in flight and
 * frees every weight buffer of the stack (resident sets and rings), so that another consumer of the same budget
 * -- a VAE phase, a second model -- can run. The records stay in the pinned host arena; the next
 * tnf_stack_step (or tnf_stack_restore) re-plans under what the budget then allows and uploads again. */
int32_t tnf_stack_evict_all(tnf_stack* st);
/* Re-plans and re-uploads the stack's weights now. weight_budget_bytes = 0 keeps the budget given at creation;
 * either is capped by what the context's budget leaves beside the other live buffers and the transient
 * reserve. Also undoes demotions made by the reclaim chain once memory is free again. */
int32_t tnf_stack_restore(tnf_stack* st, uint64_t weight_budget_bytes);
int32_t tnf_stack_destroy(tnf_stack* st);

/* ---- host IO: readers with readahead hints ---------------------------------------------- */

/* A random-access reader over one file or one tensor's bytes: `trait WeightReader`
 * (thinfer-core/src/weight.rs:57-77) as a struct of function pointers, so that the embedding program can
 * pass its own readers. len and read_at are required; read_at lands exactly `n` bytes of [offset, offset+n)
 * in caller memory and returns TNF_OK or an error code. will_read is the prefetch hint "the next read_at
 * will be exactly (offset, n)" (:69-76): best effort, a wrong or ignored hint costs speed, never bytes; NULL
 * means "no hints". close releases `user` (NULL: nothing to release). One reader is used by one thread
 * at a time (the reference enforces that with `&mut self`). */
typedef struct tnf_reader {
  void* user;
  uint64_t (*len)(void* user);
  int32_t (*read_at)(void* user, uint64_t offset, void* dst, uint64_t n);
  void (*will_read)(void* user, uint64_t offset, uint64_t n);
  void (*close)(void* user);
} tnf_reader;

#define TNF_READER_DEFAULT_HINTS 0xFFFFFFFFu /* hint_chunks: the reference's READ_PREFETCH_CHUNKS (4) */

/* MmapFileOpener::new + FileOpener::open (thinfer-native/src/lib.rs:15-52): maps the whole file read-only.
 * read_at is a bounds-checked memcpy (:57-70); will_read is madvise(MADV_WILLNEED) on the range
 * (:72-86), which starts the page-in as large batched IOs. An empty file gives an empty reader. */
int32_t tnf_mmap_open(const char* path, tnf_reader* out);
/* out = {read_at calls, bytes read, hints accepted, bytes hinted} of a reader made by tnf_mmap_open. */
int32_t tnf_mmap_stats(const tnf_reader* r, uint64_t out[4]);
/* OffsetView (thinfer-core/src/weight.rs:102-127): restricts `inner` to [base, base+len) and rebases
 * offsets to [0, len). The view borrows `inner`, which must outlive it; closing the view leaves it open. */
int32_t tnf_reader_view(const tnf_reader* inner, uint64_t base, uint64_t len, tnf_reader* out);
void tnf_reader_close(tnf_reader* r);
/* The chunk loop of stream_source_to_gpu (thinfer-core/src/residency.rs:1253-1292) without a device: reads
 * [offset, offset+n) into `dst` in chunks of chunk_bytes (0 = 16 MiB), hinting the first hint_chunks
 * chunks up front and, after each chunk, the chunk hint_chunks ahead of it. Host only. */
int32_t tnf_reader_read(const tnf_reader* r, uint64_t offset, uint64_t n, void* dst, uint64_t chunk_bytes,
                        uint32_t hint_chunks);
/* The same loop into a pinned arena (tnf_host_register), e.g. one NVFP4 record of a container straight into
 * the arena a tnf_stack streams from: the bytes on disk are the bytes the copy engine sends. */
int32_t tnf_reader_read_to_arena(tnf_ctx* ctx, const tnf_reader* r, uint64_t offset, uint64_t n, uint64_t host_id,
                                 uint64_t host_off, uint64_t chunk_bytes, uint32_t hint_chunks);
/* stream_source_to_gpu (thinfer-core/src/residency.rs:1197-1341): streams `total` source bytes starting at
 * src_offset into the device view `dst`; dst.len >= total, and the bytes of the view past `total` are
 * zero-filled (the reference's padded_len). Chunks pass through two pinned staging slots kept by the
 * context, so reading chunk i+1 overlaps the copy of chunk i on the copy stream. *event (may be NULL)
 * identifies the completion of the last copy. */
int32_t tnf_upload_from_reader(tnf_ctx* ctx, const tnf_reader* r, uint64_t src_offset, uint64_t total, tnf_buf dst,
                               uint64_t chunk_bytes, uint32_t hint_chunks, uint64_t* event);

/* ---- container: GGUF-v3 header parser + tensor catalog ------------------------------- */

/* parse_header / catalog_from of the reference (thinfer-core/src/format/gguf.rs:122-250), host
 * only. tnf_gguf_parse reads a header from the first `len` bytes of a file: TNF_OK and a handle,
 * or TNF_GGUF_NEED_MORE with *need_at = the absolute offset it had to reach (read at least that
 * many bytes and call again: no whole-file load), or TNF_ERR_INVALID_ARGUMENT with the reference's
 * error variant in tnf_last_error() ("BadMagic(0x..)", "UnsupportedVersion(2)", "Oversized {..}",
 * "BadValueType(..)", "BadBool(..)", "BadUtf8", "BadAlignment(..)", "AlignmentTooLarge(..)",
 * "BadDimCount(..)"). tnf_gguf_info: out = {version, alignment, tensor-data offset, tensor count}.
 * tnf_gguf_tensor: catalog entry `index` (header order): dims OUTER-first (GGUF stores them
 * innermost-first), absolute file offset, size = distance to the next tensor in offset order
 * (the last one is bounded by file_size, or by its type's own size when file_size is 0). */
typedef struct tnf_gguf tnf_gguf;
#define TNF_GGUF_NEED_MORE 1
/* Added to ggml's type table: one linear as the streaming residency consumes it
 * (tnf_stack_record_offsets), GGUF dims [K, N]. "NVF4" in ASCII. */
#define TNF_GGML_TYPE_NVFP4_RECORD 0x4E564634u
typedef struct {
  const char* name; /* owned by the handle */
  uint32_t n_dims;
  uint64_t dims[8];
  uint32_t ggml_type;
  uint64_t offset, size;
  uint64_t on_disk_bytes; /* from dims and type; 0 for a type this build does not size */
} tnf_gguf_tensor_info;
int32_t tnf_gguf_parse(const void* buf, uint64_t len, tnf_gguf** out, uint64_t* need_at);
int32_t tnf_gguf_free(tnf_gguf* h);
int32_t tnf_gguf_info(const tnf_gguf* h, uint64_t out[4]);
int32_t tnf_gguf_tensor(const tnf_gguf* h, uint64_t index, uint64_t file_size, tnf_gguf_tensor_info* out);
const char* tnf_ggml_type_label(uint32_t ggml_type);

/* ---- multi-GPU (no reference counterpart: the reference is single-device) ------------ */

/* Join an NCCL communicator of `world` ranks. unique_id is the 128-byte ncclUniqueId
 * made by rank 0 with tnf_comm_unique_id and passed around by the caller. */
int32_t tnf_comm_unique_id(void* unique_id_128);
int32_t tnf_comm_init(tnf_ctx* ctx, int32_t world, int32_t rank, const void* unique_id_128);
/* All-gather the column slices of an N-split output: every rank holds out[m, n_total]
 * with its own n_local columns at rank*n_local filled; on return all columns are filled. */
int32_t tnf_all_gather_cols(tnf_ctx* ctx, tnf_buf out_bf16, uint32_t m, uint32_t n_total, uint32_t n_local);
/* The same gather for an output that the epilogue left in NVFP4 (TNF_LINEAR_OUT_NVFP4 with
 * n_offset = rank*n_local, ldo = n_total): codes[m, n_total/2] and the DEVICE-layout scales of the
 * [m, n_total] operand, both in one NCCL all-gather. Moves 0.5625 bytes per element instead of 2;
 * the gathered operand feeds tnf_gemm_nvfp4 and holds the same bits tnf_quantize_act would make
 * from the gathered bf16 output. n_local must be a multiple of 64. */
int32_t tnf_all_gather_nvfp4(tnf_ctx* ctx, tnf_buf codes, tnf_buf scales, uint32_t m, uint32_t n_total, uint32_t n_local);
/* Peer output windows for the fused epilogue scatter. tnf_ipc_export gives the 64-byte CUDA
 * IPC handle of a buffer; tnf_peer_outputs opens the other ranks' handles of the SAME logical
 * output as window set `set` (0..3). A linear with TNF_LINEAR_SCATTER_PEERS | TNF_LINEAR_PEER_SET(set)
 * then stores every output tile to its own out_bf16 and to each window of that set (plain
 * TMA stores into peer memory, no multicast). Follow with tnf_comm_barrier before any rank
 * reads the gathered output. */
int32_t tnf_ipc_export(tnf_ctx* ctx, uint64_t id, void* handle_64);
int32_t tnf_peer_outputs(tnf_ctx* ctx, int32_t set, int32_t n_peers, const void* handles_64xn);
#define TNF_LINEAR_PEER_SET(i) (((uint32_t)(i) & 3u) << 8)
/* Copy-engine delivery, overlapped by row bands: once the work queued so far on the compute
 * stream is done (the GEMM that produced rows [row0, row0+rows) of this rank's column slice),
 * the copy stream pushes that band of out[:, n_offset : n_offset+n] to every window of `set` with
 * one strided peer copy each. Call tnf_compute_after_copy, then tnf_comm_barrier, before any rank
 * reads the gathered output. */
int32_t tnf_scatter_rows(tnf_ctx* ctx, int32_t set, tnf_buf out_bf16, uint32_t row0, uint32_t rows, uint32_t n_offset,
                         uint32_t n, uint32_t ldo);
/* Contiguous copy-engine delivery. The linear writes its column slice PACKED (ldo = n, n_offset = 0;
 * an NVFP4 copy packs the same way); once the work queued so far on the compute stream is done the
 * copy stream copies src to byte dst_offset of every window of `set` (each peer's receive area,
 * which the caller sized; ring order, so every rank receives from one sender at a time) and to
 * self_dst, this rank's slot of its own receive area (len 0 to skip). Contiguous peer copies run
 * at link rate where the strided ones of tnf_scatter_rows do not. The pushes run on streams of
 * their own (not behind uploads or read-backs queued on the copy stream). Then
 * tnf_compute_after_push (the compute stream waits for the pushes queued so far, and only for
 * them), tnf_comm_barrier, and tnf_interleave_cols to lay the slices side by side. */
int32_t tnf_push_peers(tnf_ctx* ctx, int32_t set, tnf_buf src, uint64_t dst_offset, tnf_buf self_dst);
int32_t tnf_compute_after_push(tnf_ctx* ctx);
/* out[r*out_row_bytes + w*local_row_bytes + c] = gathered[w*rank_stride + r*src_row_bytes + c] for
 * w < world, r < rows, c < local_row_bytes: the receive area's per-rank blocks become the column
 * slices of one row-major matrix (bf16 rows, NVFP4 code rows, or 128-row blocks of device-layout
 * scales, whose rows may carry padding atoms). All byte counts are multiples of 16. */
int32_t tnf_interleave_cols(tnf_ctx* ctx, tnf_buf gathered, uint64_t rank_stride, uint32_t src_row_bytes, uint32_t world,
                            tnf_buf out, uint32_t out_row_bytes, uint32_t rows, uint32_t local_row_bytes);
/* Compute stream waits for everything queued so far on the copy stream and for the pushes. */
int32_t tnf_compute_after_copy(tnf_ctx* ctx);
/* Stream-ordered barrier across the communicator (after a scatter epilogue). */
int32_t tnf_comm_barrier(tnf_ctx* ctx);
/* Registers a device range this library did not allocate as a buffer: `local_ptr` is this rank's copy
 * of a symmetric allocation (same size and layout on every rank of the node) and `multicast_ptr`
 * the NVSwitch multicast alias of the same range (0 if the platform has none; the multicast
 * features then refuse the buffer). The range is charged to `category` but never freed here:
 * tnf_free only forgets it. The reference is single-device and has no counterpart; the nearest
 * idea is Backend::allocate_in (thinfer-core/src/backend/mod.rs:94-122) for memory owned elsewhere. */
int32_t tnf_import_symmetric(tnf_ctx* ctx, void* local_ptr, void* multicast_ptr, uint64_t bytes, int32_t category,
                             uint64_t* id);
/* Copies `n` bytes of `src` to offset `dst_off` of the symmetric buffer `dst_id` on EVERY rank
 * (this one included) with multicast stores; n, offsets 16-byte multiples. Asynchronous on the
 * compute stream. Used to hand every rank this rank's row block of a quantised activation. */
int32_t tnf_multicast_copy(tnf_ctx* ctx, tnf_buf src, uint64_t dst_id, uint64_t dst_off, uint64_t n);

#ifdef __cplusplus
}
#endif
#endif /* THINFER_NVFP4_H_ */
