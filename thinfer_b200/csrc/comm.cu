// Multi-GPU side of the ABI: NCCL communicator (loaded at run time), the all-gathers of an
// N-split output (bf16 columns, or the NVFP4 copy the epilogue made), CUDA IPC windows for the
// fused epilogue scatter and for the copy-engine deliveries (strided row bands; contiguous pushes
// of packed slices + an interleave kernel), a stream-ordered barrier.
// The reference is single-device; the N-split with an all-gather of the output is what the
// benchmark configuration adds. One process per GPU; NCCL is found with dlopen so that a
// process that already loaded a libnccl (torch) shares it.
#include <dlfcn.h>
#include <nccl.h>

#include <cstdlib>
#include <cstring>

#include "context.h"
#include "ptx.cuh"

namespace tnf {

struct NcclApi {
  void* handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
};

static NcclApi* nccl_api() {
  static NcclApi api;
  static bool tried = false;
  if (tried) return api.handle ? &api : nullptr;
  tried = true;
  void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD | RTLD_GLOBAL);
  if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
  if (!h) {
    set_error("libnccl.so.2 could not be loaded: %s", dlerror());
    return nullptr;
  }
  api.handle = h;
#define TNF_SYM(name)                                                           \
  api.name = reinterpret_cast<decltype(api.name)>(dlsym(h, "nccl" #name));      \
  if (!api.name) {                                                              \
    set_error("libnccl.so.2 lacks nccl" #name);                                 \
    api.handle = nullptr;                                                       \
    return nullptr;                                                             \
  }
  TNF_SYM(GetUniqueId)
  TNF_SYM(CommInitRank)
  TNF_SYM(CommDestroy)
  TNF_SYM(AllGather)
  TNF_SYM(AllReduce)
  TNF_SYM(GetErrorString)
#undef TNF_SYM
  return &api;
}

static int32_t nccl_fail(NcclApi* api, ncclResult_t r, const char* what) {
  set_error("%s: %s", what, api->GetErrorString(r));
  return TNF_ERR_NCCL;
}

// own column slice of a row-major matrix -> contiguous [rows, n_local]; all extents in 16-byte units
__global__ void pack_cols_kernel(const uint4* __restrict__ out, uint4* __restrict__ packed, uint32_t rows,
                                 uint32_t row_stride, uint32_t n_local, uint32_t col0) {
  uint64_t t = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t >= uint64_t(rows) * n_local) return;
  uint32_t r = uint32_t(t / n_local), c = uint32_t(t % n_local);
  packed[t] = out[uint64_t(r) * row_stride + col0 + c];
}
// gathered: rank w's [rows, n_local] block starts at w * rank_stride -> out columns w * n_local, skipping this rank's own
__global__ void unpack_cols_kernel(const uint4* __restrict__ gathered, uint4* __restrict__ out, uint32_t rows,
                                   uint32_t row_stride, uint32_t n_local, uint64_t rank_stride, uint32_t world,
                                   uint32_t self, uint32_t src_row_stride) {
  uint64_t t = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t >= uint64_t(world) * rows * n_local) return;
  uint32_t c = uint32_t(t % n_local);
  uint64_t q = t / n_local;
  uint32_t r = uint32_t(q % rows), w = uint32_t(q / rows);
  if (w == self) return;
  out[uint64_t(r) * row_stride + uint64_t(w) * n_local + c] = gathered[uint64_t(w) * rank_stride + uint64_t(r) * src_row_stride + c];
}

// Staging of the NCCL gathers (send slice + receive area). It is an ordinary workspace buffer of the context:
// charged to the budget, visible in tnf_mem_snapshot, refused on the host when it does not fit.
static int32_t ensure_gather_tmp(tnf_ctx* ctx, uint64_t need) {
  std::lock_guard<std::mutex> lk(ctx->mu);
  if (need <= ctx->gather_tmp_bytes) return TNF_OK;
  if (ctx->gather_tmp_id) free_locked(ctx, ctx->gather_tmp_id);
  ctx->gather_tmp_id = 0;
  ctx->gather_tmp = nullptr;
  ctx->gather_tmp_bytes = 0;
  int32_t st = alloc_locked(ctx, need, TNF_CAT_WORKSPACE, &ctx->gather_tmp_id);
  if (st != TNF_OK) return st;
  ctx->gather_tmp = ctx->bufs[ctx->gather_tmp_id].ptr;
  ctx->gather_tmp_bytes = need;
  return TNF_OK;
}

// src (local) -> the multicast alias of a symmetric buffer: one 16-byte multimem store per thread and round
__global__ void multicast_copy_kernel(const uint4* __restrict__ src, uint4* dst_mc, uint64_t n16) {
  for (uint64_t i = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n16; i += uint64_t(gridDim.x) * blockDim.x)
    multimem_st_v4(dst_mc + i, __ldg(src + i));
  __threadfence_system();
}

cudaError_t launch_multicast_copy(const uint8_t* src, uint8_t* dst_mc, uint64_t bytes, int sm_count, cudaStream_t s) {
  const uint64_t n16 = bytes / 16;
  if (n16 == 0) return cudaSuccess;
  const unsigned blocks = unsigned(std::min<uint64_t>((n16 + 255) / 256, uint64_t(sm_count) * 8));
  multicast_copy_kernel<<<blocks, 256, 0, s>>>(reinterpret_cast<const uint4*>(src), reinterpret_cast<uint4*>(dst_mc), n16);
  return cudaGetLastError();
}

}  // namespace tnf

using namespace tnf;

void tnf_comm_teardown(tnf_ctx* ctx) {
  if (ctx->nccl_comm) {
    NcclApi* api = nccl_api();
    if (api) api->CommDestroy(static_cast<ncclComm_t>(ctx->nccl_comm));
    ctx->nccl_comm = nullptr;
  }
  for (int s = 0; s < tnf_ctx::kPeerSets; ++s) {
    for (int i = 0; i < ctx->n_peers[s]; ++i)
      if (ctx->peer_out[s][i]) cudaIpcCloseMemHandle(ctx->peer_out[s][i]);
    ctx->n_peers[s] = 0;
  }
  ctx->gather_tmp = nullptr;  // the staging buffer is in the context's table and goes with it
  ctx->gather_tmp_bytes = 0;
}

extern "C" {

int32_t tnf_comm_unique_id(void* unique_id_128) {
  NcclApi* api = nccl_api();
  if (!api) return TNF_ERR_NCCL;
  static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId is 128 bytes");
  ncclUniqueId id;
  ncclResult_t r = api->GetUniqueId(&id);
  if (r != ncclSuccess) return nccl_fail(api, r, "ncclGetUniqueId");
  std::memcpy(unique_id_128, &id, 128);
  return TNF_OK;
}

int32_t tnf_comm_init(tnf_ctx* ctx, int32_t world, int32_t rank, const void* unique_id_128) {
  if (!ctx || !unique_id_128 || world < 1 || rank < 0 || rank >= world || world > kMaxPeers) {
    set_error("tnf_comm_init: bad arguments (world %d, rank %d, at most %d ranks)", world, rank, kMaxPeers);
    return TNF_ERR_INVALID_ARGUMENT;
  }
  NcclApi* api = nccl_api();
  if (!api) return TNF_ERR_NCCL;
  cudaError_t e = cudaSetDevice(ctx->device);
  if (e != cudaSuccess) return cuda_fail(e, "cudaSetDevice");
  ncclUniqueId id;
  std::memcpy(&id, unique_id_128, 128);
  ncclComm_t comm;
  ncclResult_t r = api->CommInitRank(&comm, world, id, rank);
  if (r != ncclSuccess) return nccl_fail(api, r, "ncclCommInitRank");
  ctx->nccl_comm = comm;
  ctx->world = world;
  ctx->rank = rank;
  return TNF_OK;
}

int32_t tnf_all_gather_cols(tnf_ctx* ctx, tnf_buf out_bf16, uint32_t m, uint32_t n_total, uint32_t n_local) {
  if (!ctx || !ctx->nccl_comm) {
    set_error("tnf_all_gather_cols: no communicator (call tnf_comm_init)");
    return TNF_ERR_INVALID_ARGUMENT;
  }
  cudaError_t e = cudaSetDevice(ctx->device);
  if (e != cudaSuccess) return cuda_fail(e, "cudaSetDevice");
  if (n_local % 8 || n_total != n_local * uint32_t(ctx->world) || m == 0) {
    set_error("tnf_all_gather_cols: n_total %u must be world %d x n_local %u, n_local a multiple of 8", n_total,
              ctx->world, n_local);
    return TNF_ERR_INVALID_ARGUMENT;
  }
  int32_t st = TNF_OK;
  uint8_t* out = resolve(ctx, out_bf16, uint64_t(m) * n_total * 2, "out_bf16", &st);
  if (!out) return st;
  NcclApi* api = nccl_api();
  const uint64_t slice = uint64_t(m) * n_local * 2;
  st = ensure_gather_tmp(ctx, slice * (uint64_t(ctx->world) + 1));
  if (st != TNF_OK) return st;
  uint8_t* send = static_cast<uint8_t*>(ctx->gather_tmp);
  uint8_t* recv = send + slice;
  const uint32_t nl8 = n_local / 8, nt8 = n_total / 8;
  uint64_t threads = uint64_t(m) * nl8;
  pack_cols_kernel<<<unsigned((threads + 255) / 256), 256, 0, ctx->compute>>>(
      reinterpret_cast<const uint4*>(out), reinterpret_cast<uint4*>(send), m, nt8, nl8, uint32_t(ctx->rank) * nl8);
  e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "pack launch");
  ncclResult_t r = api->AllGather(send, recv, slice / 2, ncclBfloat16, static_cast<ncclComm_t>(ctx->nccl_comm), ctx->compute);
  if (r != ncclSuccess) return nccl_fail(api, r, "ncclAllGather");
  threads *= uint64_t(ctx->world);
  unpack_cols_kernel<<<unsigned((threads + 255) / 256), 256, 0, ctx->compute>>>(
      reinterpret_cast<const uint4*>(recv), reinterpret_cast<uint4*>(out), m, nt8, nl8, uint64_t(m) * nl8,
      uint32_t(ctx->world), uint32_t(ctx->rank), nl8);
  e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "unpack launch");
  return TNF_OK;
}

int32_t tnf_all_gather_nvfp4(tnf_ctx* ctx, tnf_buf codes, tnf_buf scales, uint32_t m, uint32_t n_total, uint32_t n_local) {
  if (!ctx || !ctx->nccl_comm) {
    set_error("tnf_all_gather_nvfp4: no communicator (call tnf_comm_init)");
    return TNF_ERR_INVALID_ARGUMENT;
  }
  cudaError_t e = cudaSetDevice(ctx->device);
  if (e != cudaSuccess) return cuda_fail(e, "cudaSetDevice");
  if (n_local % 64 || n_total != n_local * uint32_t(ctx->world) || m == 0) {
    set_error("tnf_all_gather_nvfp4: n_total %u must be world %d x n_local %u, n_local a multiple of 64", n_total,
              ctx->world, n_local);
    return TNF_ERR_INVALID_ARGUMENT;
  }
  int32_t st = TNF_OK;
  uint8_t* pc = resolve(ctx, codes, uint64_t(m) * (n_total / 2), "codes", &st);
  if (!pc) return st;
  uint8_t* ps = resolve(ctx, scales, sf_device_bytes(m, n_total), "scales", &st);
  if (!ps) return st;
  NcclApi* api = nccl_api();
  // 16-byte units: a code row is n/32 of them; a 128-row block of scales is 32 per 64-column atom
  const uint32_t row_blocks = (m + 127) / 128;
  const uint32_t c_loc = n_local / 32, c_tot = n_total / 32;
  const uint32_t s_loc = (n_local / 64) * 32, s_tot = sf_k_atoms(n_total) * 32;
  const uint64_t c_units = uint64_t(m) * c_loc, s_units = uint64_t(row_blocks) * s_loc;
  const uint64_t slice = (c_units + s_units) * 16;
  st = ensure_gather_tmp(ctx, slice * (uint64_t(ctx->world) + 1));
  if (st != TNF_OK) return st;
  uint4* send = static_cast<uint4*>(ctx->gather_tmp);
  uint4* recv = send + slice / 16;
  const uint32_t rank = uint32_t(ctx->rank), world = uint32_t(ctx->world);
  pack_cols_kernel<<<unsigned((c_units + 255) / 256), 256, 0, ctx->compute>>>(reinterpret_cast<const uint4*>(pc), send, m,
                                                                             c_tot, c_loc, rank * c_loc);
  pack_cols_kernel<<<unsigned((s_units + 255) / 256), 256, 0, ctx->compute>>>(reinterpret_cast<const uint4*>(ps),
                                                                             send + c_units, row_blocks, s_tot, s_loc,
                                                                             rank * s_loc);
  e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "pack launch");
  ncclResult_t r = api->AllGather(send, recv, slice, ncclUint8, static_cast<ncclComm_t>(ctx->nccl_comm), ctx->compute);
  if (r != ncclSuccess) return nccl_fail(api, r, "ncclAllGather");
  unpack_cols_kernel<<<unsigned((c_units * world + 255) / 256), 256, 0, ctx->compute>>>(
      recv, reinterpret_cast<uint4*>(pc), m, c_tot, c_loc, slice / 16, world, rank, c_loc);
  unpack_cols_kernel<<<unsigned((s_units * world + 255) / 256), 256, 0, ctx->compute>>>(
      recv + c_units, reinterpret_cast<uint4*>(ps), row_blocks, s_tot, s_loc, slice / 16, world, rank, s_loc);
  e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "unpack launch");
  return TNF_OK;
}

int32_t tnf_ipc_export(tnf_ctx* ctx, uint64_t id, void* handle_64) {
  if (!ctx || !handle_64) {
    set_error("tnf_ipc_export: null argument");
    return TNF_ERR_INVALID_ARGUMENT;
  }
  cudaError_t e = cudaSetDevice(ctx->device);
  if (e != cudaSuccess) return cuda_fail(e, "cudaSetDevice");
  void* p = nullptr;
  {
    std::lock_guard<std::mutex> lk(ctx->mu);
    auto it = ctx->bufs.find(id);
    if (it == ctx->bufs.end()) {
      set_error("tnf_ipc_export: unknown buffer id %llu", (unsigned long long)id);
      return TNF_ERR_UNKNOWN_BUFFER;
    }
    p = it->second.ptr;
  }
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "cudaIpcMemHandle_t is 64 bytes");
  cudaIpcMemHandle_t h;
  e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) return cuda_fail(e, "cudaIpcGetMemHandle");
  std::memcpy(handle_64, &h, 64);
  return TNF_OK;
}

int32_t tnf_peer_outputs(tnf_ctx* ctx, int32_t set, int32_t n_peers, const void* handles_64xn) {
  if (!ctx || set < 0 || set >= tnf_ctx::kPeerSets || n_peers < 0 || n_peers > kMaxPeers - 1 || (n_peers > 0 && !handles_64xn)) {
    set_error("tnf_peer_outputs: bad arguments (set %d of %d, n_peers %d, at most %d)", set, tnf_ctx::kPeerSets, n_peers, kMaxPeers - 1);
    return TNF_ERR_INVALID_ARGUMENT;
  }
  cudaError_t e = cudaSetDevice(ctx->device);
  if (e != cudaSuccess) return cuda_fail(e, "cudaSetDevice");
  e = cudaStreamSynchronize(ctx->compute);
  if (e != cudaSuccess) return cuda_fail(e, "tnf_peer_outputs sync");
  for (int i = 0; i < ctx->n_peers[set]; ++i)
    if (ctx->peer_out[set][i]) cudaIpcCloseMemHandle(ctx->peer_out[set][i]);
  ctx->n_peers[set] = 0;
  for (int i = 0; i < n_peers; ++i) {
    cudaIpcMemHandle_t h;
    std::memcpy(&h, static_cast<const uint8_t*>(handles_64xn) + 64 * i, 64);
    void* p = nullptr;
    e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return cuda_fail(e, "cudaIpcOpenMemHandle");
    ctx->peer_out[set][ctx->n_peers[set]++] = p;
  }
  return TNF_OK;
}

int32_t tnf_scatter_rows(tnf_ctx* ctx, int32_t set, tnf_buf out_bf16, uint32_t row0, uint32_t rows, uint32_t n_offset,
                         uint32_t n, uint32_t ldo) {
  if (!ctx || set < 0 || set >= tnf_ctx::kPeerSets || rows == 0 || n == 0 || n_offset + n > ldo) {
    set_error("tnf_scatter_rows: bad arguments (set %d, rows %u, n_offset %u, n %u, ldo %u)", set, rows, n_offset, n, ldo);
    return TNF_ERR_INVALID_ARGUMENT;
  }
  cudaError_t e = cudaSetDevice(ctx->device);
  if (e != cudaSuccess) return cuda_fail(e, "cudaSetDevice");
  int32_t st = TNF_OK;
  uint8_t* base = resolve(ctx, out_bf16, (uint64_t(row0 + rows - 1) * ldo + n_offset + n) * 2, "out_bf16", &st);
  if (!base) return st;
  // the copies start when everything launched so far on the compute stream (the GEMM of these rows) is done
  cudaEvent_t ev = nullptr;
  {
    std::lock_guard<std::mutex> lk(ctx->mu);
    if (!ctx->event_pool.empty()) {
      ev = ctx->event_pool.back();
      ctx->event_pool.pop_back();
    }
  }
  if (!ev) {
    e = cudaEventCreateWithFlags(&ev, cudaEventDisableTiming);
    if (e != cudaSuccess) return cuda_fail(e, "cudaEventCreate");
  }
  e = cudaEventRecord(ev, ctx->compute);
  if (e == cudaSuccess) e = cudaStreamWaitEvent(ctx->copy, ev, 0);
  {
    std::lock_guard<std::mutex> lk(ctx->mu);
    ctx->event_pool.push_back(ev);
  }
  if (e != cudaSuccess) return cuda_fail(e, "tnf_scatter_rows: stream order");
  const uint64_t off = (uint64_t(row0) * ldo + n_offset) * 2;
  for (int i = 0; i < ctx->n_peers[set]; ++i) {
    e = cudaMemcpy2DAsync(static_cast<uint8_t*>(ctx->peer_out[set][i]) + off, uint64_t(ldo) * 2, base + off, uint64_t(ldo) * 2,
                          uint64_t(n) * 2, rows, cudaMemcpyDeviceToDevice, ctx->copy);
    if (e != cudaSuccess) return cuda_fail(e, "tnf_scatter_rows: peer copy");
  }
  return TNF_OK;
}

int32_t tnf_push_peers(tnf_ctx* ctx, int32_t set, tnf_buf src, uint64_t dst_offset, tnf_buf self_dst) {
  if (!ctx || set < 0 || set >= tnf_ctx::kPeerSets || src.len == 0 || (self_dst.len && self_dst.len != src.len)) {
    set_error("tnf_push_peers: bad arguments (set %d, %llu bytes, own copy of %llu)", set, (unsigned long long)src.len,
              (unsigned long long)self_dst.len);
    return TNF_ERR_INVALID_ARGUMENT;
  }
  cudaError_t e = cudaSetDevice(ctx->device);
  if (e != cudaSuccess) return cuda_fail(e, "cudaSetDevice");
  int32_t st = TNF_OK;
  const uint8_t* from = resolve(ctx, src, src.len, "src", &st);
  if (!from) return st;
  uint8_t* own = nullptr;
  if (self_dst.len) {
    own = resolve(ctx, self_dst, self_dst.len, "self_dst", &st);
    if (!own) return st;
  }
  // the copies start when everything launched so far on the compute stream (the GEMM that wrote src) is done
  cudaEvent_t ev = nullptr;
  {
    std::lock_guard<std::mutex> lk(ctx->mu);
    if (!ctx->event_pool.empty()) {
      ev = ctx->event_pool.back();
      ctx->event_pool.pop_back();
    }
  }
  if (!ev) {
    e = cudaEventCreateWithFlags(&ev, cudaEventDisableTiming);
    if (e != cudaSuccess) return cuda_fail(e, "cudaEventCreate");
  }
  // copies go out in ring order (next rank first), so with one lane every rank receives from one sender at a
  // time. More lanes measured no gain with 3 peers and a loss with 7; diagnostic builds can still try (TNF_PUSH_STREAMS).
  const int np = ctx->n_peers[set];
  static const int want_lanes = [] {
    const char* v = kDiag ? std::getenv("TNF_PUSH_STREAMS") : nullptr;
    const int k = v ? std::atoi(v) : 1;
    return k < 1 ? 1 : (k > 8 ? 8 : k);
  }();
  const int lanes = want_lanes < np + 1 ? want_lanes : np + 1;
  for (int i = 0; i < lanes; ++i) {
    if (!ctx->push[i]) {
      e = cudaStreamCreateWithFlags(&ctx->push[i], cudaStreamNonBlocking);
      if (e == cudaSuccess) e = cudaEventCreateWithFlags(&ctx->push_done[i], cudaEventDisableTiming);
      if (e != cudaSuccess) return cuda_fail(e, "tnf_push_peers: stream");
    }
  }
  e = cudaEventRecord(ev, ctx->compute);
  for (int i = 0; i < lanes && e == cudaSuccess; ++i) e = cudaStreamWaitEvent(ctx->push[i], ev, 0);
  {
    std::lock_guard<std::mutex> lk(ctx->mu);
    ctx->event_pool.push_back(ev);
  }
  if (e != cudaSuccess) return cuda_fail(e, "tnf_push_peers: stream order");
  // windows are kept in rank order without this rank; the copy stream then waits for every lane
  const int self = (ctx->world == np + 1) ? ctx->rank : 0;
  for (int d = 1; d <= np; ++d) {
    const int pr = (self + d) % (np + 1);
    const int i = pr < self ? pr : pr - 1;
    e = cudaMemcpyAsync(static_cast<uint8_t*>(ctx->peer_out[set][i]) + dst_offset, from, src.len, cudaMemcpyDeviceToDevice,
                        ctx->push[(d - 1) % lanes]);
    if (e != cudaSuccess) return cuda_fail(e, "tnf_push_peers: peer copy");
  }
  if (own) {
    e = cudaMemcpyAsync(own, from, src.len, cudaMemcpyDeviceToDevice, ctx->push[np % lanes]);
    if (e != cudaSuccess) return cuda_fail(e, "tnf_push_peers: own copy");
  }
  // the pushes stay on their own streams (host uploads and read-backs queued on the copy stream neither wait for
  // them nor delay them); tnf_compute_after_push / tnf_compute_after_copy / tnf_sync join them
  for (int i = 0; i < lanes; ++i) {
    e = cudaEventRecord(ctx->push_done[i], ctx->push[i]);
    if (e != cudaSuccess) return cuda_fail(e, "tnf_push_peers: record");
    ctx->push_pending[i] = true;
  }
  return TNF_OK;
}

int32_t tnf_compute_after_push(tnf_ctx* ctx) {
  if (!ctx) {
    set_error("null context");
    return TNF_ERR_INVALID_ARGUMENT;
  }
  cudaError_t e = cudaSetDevice(ctx->device);
  if (e != cudaSuccess) return cuda_fail(e, "cudaSetDevice");
  for (int i = 0; i < 8; ++i) {
    if (!ctx->push_pending[i]) continue;
    e = cudaStreamWaitEvent(ctx->compute, ctx->push_done[i], 0);
    if (e != cudaSuccess) return cuda_fail(e, "tnf_compute_after_push");
    ctx->push_pending[i] = false;
  }
  return TNF_OK;
}

int32_t tnf_interleave_cols(tnf_ctx* ctx, tnf_buf gathered, uint64_t rank_stride, uint32_t src_row_bytes, uint32_t world,
                            tnf_buf out, uint32_t out_row_bytes, uint32_t rows, uint32_t local_row_bytes) {
  if (!ctx || world == 0 || rows == 0 || local_row_bytes == 0 || (local_row_bytes | src_row_bytes | out_row_bytes) % 16 ||
      rank_stride % 16 || src_row_bytes < local_row_bytes || uint64_t(local_row_bytes) * world > out_row_bytes ||
      rank_stride < uint64_t(rows - 1) * src_row_bytes + local_row_bytes) {
    set_error("tnf_interleave_cols: bad arguments (world %u, rows %u, %u of %u bytes per source row, %u per output row, "
              "rank stride %llu; 16-byte units)", world, rows, local_row_bytes, src_row_bytes, out_row_bytes,
              (unsigned long long)rank_stride);
    return TNF_ERR_INVALID_ARGUMENT;
  }
  cudaError_t e = cudaSetDevice(ctx->device);
  if (e != cudaSuccess) return cuda_fail(e, "cudaSetDevice");
  int32_t st = TNF_OK;
  const uint8_t* g = resolve(ctx, gathered, uint64_t(world - 1) * rank_stride + uint64_t(rows - 1) * src_row_bytes + local_row_bytes,
                             "gathered", &st);
  if (!g) return st;
  uint8_t* o = resolve(ctx, out, uint64_t(rows - 1) * out_row_bytes + uint64_t(local_row_bytes) * world, "out", &st);
  if (!o) return st;
  if ((reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(o)) & 15) {
    set_error("tnf_interleave_cols: views must start on 16-byte boundaries");
    return TNF_ERR_INVALID_ARGUMENT;
  }
  const uint32_t nl = local_row_bytes / 16;
  const uint64_t threads = uint64_t(world) * rows * nl;
  unpack_cols_kernel<<<unsigned((threads + 255) / 256), 256, 0, ctx->compute>>>(
      reinterpret_cast<const uint4*>(g), reinterpret_cast<uint4*>(o), rows, out_row_bytes / 16, nl, rank_stride / 16, world,
      0xFFFFFFFFu, src_row_bytes / 16);
  e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "interleave launch");
  return TNF_OK;
}

int32_t tnf_compute_after_copy(tnf_ctx* ctx) {
  if (!ctx) {
    set_error("null context");
    return TNF_ERR_INVALID_ARGUMENT;
  }
  cudaError_t e = cudaSetDevice(ctx->device);
  if (e != cudaSuccess) return cuda_fail(e, "cudaSetDevice");
  int32_t st = tnf_compute_after_push(ctx);  // the copy-engine work of tnf_push_peers counts too
  if (st != TNF_OK) return st;
  cudaEvent_t ev = nullptr;
  {
    std::lock_guard<std::mutex> lk(ctx->mu);
    if (!ctx->event_pool.empty()) {
      ev = ctx->event_pool.back();
      ctx->event_pool.pop_back();
    }
  }
  if (!ev) {
    e = cudaEventCreateWithFlags(&ev, cudaEventDisableTiming);
    if (e != cudaSuccess) return cuda_fail(e, "cudaEventCreate");
  }
  e = cudaEventRecord(ev, ctx->copy);
  if (e == cudaSuccess) e = cudaStreamWaitEvent(ctx->compute, ev, 0);
  {
    std::lock_guard<std::mutex> lk(ctx->mu);
    ctx->event_pool.push_back(ev);
  }
  if (e != cudaSuccess) return cuda_fail(e, "tnf_compute_after_copy");
  return TNF_OK;
}

int32_t tnf_import_symmetric(tnf_ctx* ctx, void* local_ptr, void* multicast_ptr, uint64_t bytes, int32_t category, uint64_t* id) {
  if (!ctx || !local_ptr || !id || bytes == 0 || category < 0 || category > 2 || (reinterpret_cast<uintptr_t>(local_ptr) & 255) ||
      (reinterpret_cast<uintptr_t>(multicast_ptr) & 255)) {
    set_error("tnf_import_symmetric: null or misaligned pointer (256-byte alignment), zero size or bad category");
    return TNF_ERR_INVALID_ARGUMENT;
  }
  std::lock_guard<std::mutex> lk(ctx->mu);
  const uint64_t nid = ctx->next_id++;
  tnf_buffer_rec rec;
  rec.ptr = local_ptr;
  rec.bytes = bytes;
  rec.category = category;
  rec.owned = false;
  rec.mc = multicast_ptr;
  ctx->bufs[nid] = rec;
  ctx->live[category] += bytes;  // accounted like any other buffer; the memory itself belongs to the caller
  ctx->peak[category] = std::max(ctx->peak[category], ctx->live[category]);
  ctx->true_peak = std::max(ctx->true_peak, ctx->live[0] + ctx->live[1] + ctx->live[2]);
  *id = nid;
  return TNF_OK;
}

int32_t tnf_multicast_copy(tnf_ctx* ctx, tnf_buf src, uint64_t dst_id, uint64_t dst_off, uint64_t n) {
  if (!ctx || n == 0 || (n | dst_off | src.offset) % 16) {
    set_error("tnf_multicast_copy: size and offsets must be non-zero multiples of 16 bytes");
    return TNF_ERR_INVALID_ARGUMENT;
  }
  cudaError_t e = cudaSetDevice(ctx->device);
  if (e != cudaSuccess) return cuda_fail(e, "cudaSetDevice");
  int32_t st = TNF_OK;
  const uint8_t* from = resolve(ctx, src, n, "src", &st);
  if (!from) return st;
  tnf_buf dst{dst_id, dst_off, n};
  if (!resolve(ctx, dst, n, "dst", &st)) return st;
  uint8_t* mc = resolve_multicast(ctx, dst, "dst", &st);
  if (!mc) return st;
  e = launch_multicast_copy(from, mc, n, ctx->sm_count, ctx->compute);
  if (e != cudaSuccess) return cuda_fail(e, "multicast copy launch");
  return TNF_OK;
}

int32_t tnf_comm_barrier(tnf_ctx* ctx) {
  if (!ctx || !ctx->nccl_comm) {
    set_error("tnf_comm_barrier: no communicator (call tnf_comm_init)");
    return TNF_ERR_INVALID_ARGUMENT;
  }
  cudaError_t e = cudaSetDevice(ctx->device);
  if (e != cudaSuccess) return cuda_fail(e, "cudaSetDevice");
  NcclApi* api = nccl_api();
  float* word = reinterpret_cast<float*>(ctx->dwords + 8);
  ncclResult_t r = api->AllReduce(word, word, 1, ncclFloat, ncclSum, static_cast<ncclComm_t>(ctx->nccl_comm), ctx->compute);
  if (r != ncclSuccess) return nccl_fail(api, r, "ncclAllReduce (barrier)");
  return TNF_OK;
}

}  // extern "C"
