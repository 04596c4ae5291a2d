// The per-device context behind the C ABI: buffer table with category accounting, streams,
// scratch, tensor-map cache, pinned host arenas, upload events. Internal to the library.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <map>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/thinfer_nvfp4.h"
#include "internal.h"

struct tnf_buffer_rec {
  void* ptr = nullptr;
  uint64_t bytes = 0;
  int category = 0;
  bool owned = true;   // false: registered with tnf_import_symmetric, never freed here
  void* mc = nullptr;  // NVSwitch multicast alias of the same range (imported symmetric buffers only)
};

struct tnf_host_rec {
  void* ptr = nullptr;
  uint64_t bytes = 0;
  bool owned = false;  // cudaHostAlloc'ed by us (else cudaHostRegister'ed in place)
};

// A holder of device memory that can give some back when an allocation does not fit the budget: the
// WeightReclaimer the reference registers with its arbiter (thinfer-core/src/residency.rs:1473-1547,
// thinfer-core/src/arbiter.rs:129-160). `fn` is called with the context's mutex held and returns the bytes it freed.
struct tnf_reclaimer {
  void* owner = nullptr;
  uint64_t (*fn)(void* owner, uint64_t want_bytes) = nullptr;
};

struct tnf_ctx {
  int device = 0;
  int sm_count = 148;
  uint64_t budget = 0;
  cudaStream_t compute = nullptr, copy = nullptr;
  cudaStream_t readback = nullptr;  // device -> host copies of tnf_stream_download: full duplex beside the uploads on `copy`
  cudaStream_t push[8] = {};  // lanes of tnf_push_peers, made on first use
  cudaEvent_t push_done[8] = {};
  bool push_pending[8] = {};  // a push was recorded on lane i and nothing has waited for it yet
  std::mutex mu;
  uint64_t next_id = 1;
  std::unordered_map<uint64_t, tnf_buffer_rec> bufs;
  std::unordered_map<uint64_t, tnf_host_rec> hosts;
  std::unordered_map<uint64_t, cudaEvent_t> events;
  std::vector<cudaEvent_t> event_pool;
  // MemAccount: live and peak per category, true concurrent peak, streamed bytes
  uint64_t live[3] = {0, 0, 0}, peak[3] = {0, 0, 0}, true_peak = 0, streamed = 0;
  std::vector<tnf_reclaimer> reclaimers;  // asked in registration order by alloc_locked before it refuses
  bool in_reclaim = false;
  uint64_t reclaimed = 0;                 // bytes given back by reclaimers so far
  uint64_t transient_reserve = 0;         // bytes of the budget a weight plan leaves free for transient workspace
  // Workspace pool (thinfer-core/src/workspace.rs:131-316): idle scratch buffers by 256-byte size class, last in
  // first out within a class. Idle buffers stay in `bufs` and in `live[workspace]`; `ws_pool_bytes` is their sum.
  std::map<uint64_t, std::vector<uint64_t>> ws_free;  // class bytes -> ids of idle buffers
  std::unordered_map<uint64_t, uint64_t> ws_rented;   // id -> class of every buffer out on rent
  uint64_t ws_pool_bytes = 0, ws_hits = 0, ws_misses = 0, ws_spilled = 0;
  // scratch for on-the-fly activation quantisation (workspace category)
  uint64_t scratch_codes_id = 0, scratch_scales_id = 0;
  uint64_t scratch_codes_bytes = 0, scratch_scales_bytes = 0;
  uint32_t scratch_m = 0, scratch_k = 0;  // shape the scratch was last filled for (0 = never)
  uint64_t wide_id = 0, wide_bytes = 0;   // bf16 image of NVFP4 activations for the mixed arm (workspace category)
  long long wait_limit_cycles = tnf::kDefaultWaitLimitCycles;  // bound of every device-side mbarrier wait
  // small device words: [0] kernel status, [1] amax bits, [2] global scale (f32)
  uint32_t* dwords = nullptr;
  std::map<tnf::MapSpec, CUtensorMap> maps;
  // fused-scatter peer windows (opened CUDA IPC mappings), index 0 unused
  static constexpr int kPeerSets = 4;
  void* peer_out[kPeerSets][tnf::kMaxPeers] = {{nullptr}};
  int n_peers[kPeerSets] = {0, 0, 0, 0};
  // NCCL
  void* nccl_comm = nullptr;
  int world = 1, rank = 0;
  void* gather_tmp = nullptr;   // staging of the NCCL gathers: a workspace buffer of the table (gather_tmp_id)
  uint64_t gather_tmp_id = 0, gather_tmp_bytes = 0;
  // tnf_upload_from_reader: two pinned staging slots (reader -> slot -> device), each guarded by the event of the
  // copy that last read it
  void* stage_host[2] = {nullptr, nullptr};
  cudaEvent_t stage_done[2] = {nullptr, nullptr};
  uint64_t stage_bytes = 0;
};

void tnf_comm_teardown(tnf_ctx* ctx);  // comm.cu

namespace tnf {
void set_error(const char* fmt, ...);
int32_t cuda_fail(cudaError_t e, const char* what);
// Looks a view up and checks its range; returns the device address or null (error set).
uint8_t* resolve(tnf_ctx* ctx, const tnf_buf& b, uint64_t need_bytes, const char* name, int32_t* status);
// Multicast alias of a view already validated by resolve(); null (error set) if its buffer has none.
uint8_t* resolve_multicast(tnf_ctx* ctx, const tnf_buf& b, const char* name, int32_t* status);
int32_t alloc_locked(tnf_ctx* ctx, uint64_t bytes, int category, uint64_t* id);
int32_t free_locked(tnf_ctx* ctx, uint64_t id);
// Frees idle pool buffers, smallest class first, until `at_least` bytes are back; returns the bytes freed.
uint64_t ws_spill_locked(tnf_ctx* ctx, uint64_t at_least);
bool get_map(tnf_ctx* ctx, const MapSpec& spec, CUtensorMap* out);  // copies the (cached) map out under the lock
}  // namespace tnf
