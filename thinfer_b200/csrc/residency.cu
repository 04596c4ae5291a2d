// Layer-stack driver with weight streaming under a VRAM budget.
//
// Re-design of the reference's WeightResidency + block loops for a CUDA device
// (thinfer-core/src/residency.rs: register_in_ring :382-423, set_pin_plan :440-457,
// acquire_from_ring :760-902, stream_source_to_gpu :1197-1341, prefetch :1398-1408;
// thinfer-models/src/qwen_image/dit.rs:1052-1180 and thinfer-models/src/wan/dit.rs:520-640 for
// the join{compute block i, acquire i+1, prefetch i+2} loops). What changes on B200:
//   * weights wait in PINNED host memory and move with cudaMemcpyAsync on a copy stream, one
//     copy per weight record (codes + device-layout scales + bias are contiguous), instead of
//     mmap -> staging -> queue.write_buffer in 16 MiB chunks on the one compute queue;
//   * a ring slot is guarded by two events (uploaded / last reader done) instead of pin counts,
//     so the host never blocks: a whole step is enqueued asynchronously;
//   * the access pattern is a uniform cyclic scan (every weight once per step), so an LRU pool
//     gets no hits once the set exceeds the budget: the pin plan is static and role-major
//     (the same linears of every layer resident, the rest streamed through per-role rings), which
//     keeps the per-layer upload demand flat (thinfer-models/src/z_image/dit.rs:360-373);
//   * uploads run `ring_slots` layers ahead and wrap around to the next step's first layers.
#include <algorithm>
#include <cstring>
#include <vector>

#include "context.h"

namespace {

inline uint64_t align256(uint64_t x) { return (x + 255ull) & ~255ull; }

struct RecordLayout {
  uint64_t codes_off, scales_off, bias_off, global_off, bytes;
};

RecordLayout record_layout(uint32_t n, uint32_t k) {
  RecordLayout r;
  r.codes_off = 0;
  r.scales_off = align256(uint64_t(n) * (k / 2));
  r.bias_off = r.scales_off + align256(tnf::sf_device_bytes(n, k));
  r.global_off = r.bias_off + align256(uint64_t(n) * 2);
  r.bytes = r.global_off + 256;
  return r;
}

struct Role {  // one linear of the layer, across all layers
  tnf_stack_linear desc;
  RecordLayout lay;
  uint64_t layer_off = 0;        // offset of this linear's record inside a layer's block of the host arena
  uint32_t pinned_layers = 0;    // layers [0, pinned_layers) are resident
  uint64_t pinned_id = 0;        // one device buffer holding the resident records
  uint64_t ring_id = 0;          // ring_slots records
  uint32_t slots = 0;
  std::vector<cudaEvent_t> ready, freed;
  std::vector<int64_t> holds;    // streamed-layer sequence number each slot holds or is being filled with
  int64_t next_upload = 0;       // next streamed-layer sequence number to upload (monotonic, cyclic modulo streamed)
  int64_t epoch_step = 0;        // the stack's step count when this role's plan was last (re)made: sequences restart there
  uint64_t out_id = 0;           // workspace for this linear's output [m, n]
};

}  // namespace

struct tnf_stack {
  tnf_ctx* ctx = nullptr;
  uint32_t layers = 0, hidden = 0, n_streams = 0;
  std::vector<Role> roles;
  std::vector<uint32_t> m_rows;
  std::vector<uint64_t> x_ping, x_pong;  // per stream, [m, hidden] each
  uint64_t host_id = 0;
  const uint8_t* host_base = nullptr;
  uint64_t layer_bytes = 0;
  uint64_t pinned_bytes = 0, ring_bytes = 0, uploaded_last = 0, uploads_last = 0;
  int64_t steps_done = 0;
  uint64_t weight_budget = 0;  // as given at creation (0 = unlimited)
  uint32_t ring_slots = 4;
  bool in_step = false;        // a step is being enqueued: the reclaimer must not change the plan under it
  bool evicted = false;        // tnf_stack_evict_all ran: the next step (or tnf_stack_restore) brings the weights back
  uint64_t demoted_bytes = 0;  // resident bytes given back to the arbiter's reclaim chain so far
};

using namespace tnf;

static int32_t upload_record(tnf_stack* st, Role& r, int64_t seq) {
  const uint32_t streamed = st->layers - r.pinned_layers;
  const uint32_t layer = r.pinned_layers + uint32_t(seq % streamed);
  const uint32_t slot = uint32_t(seq % r.slots);
  tnf_ctx* ctx = st->ctx;
  // the slot's last reader must be done before the copy engine overwrites it
  cudaError_t e = cudaStreamWaitEvent(ctx->copy, r.freed[slot], 0);
  if (e != cudaSuccess) return cuda_fail(e, "stack: wait slot free");
  uint8_t* dst = static_cast<uint8_t*>(ctx->bufs[r.ring_id].ptr) + uint64_t(slot) * r.lay.bytes;
  const uint8_t* src = st->host_base + uint64_t(layer) * st->layer_bytes + r.layer_off;
  e = cudaMemcpyAsync(dst, src, r.lay.bytes, cudaMemcpyHostToDevice, ctx->copy);
  if (e != cudaSuccess) return cuda_fail(e, "stack: weight upload");
  e = cudaEventRecord(r.ready[slot], ctx->copy);
  if (e != cudaSuccess) return cuda_fail(e, "stack: record upload");
  r.holds[slot] = seq;
  ctx->streamed += r.lay.bytes;
  st->uploaded_last += r.lay.bytes;
  st->uploads_last += 1;
  return TNF_OK;
}


// ---- plan / materialise / release: the three steps behind create, restore, evict and reclaim --------------------
// Role-major pin plan under `budget` bytes for resident + ring weights (0 = unlimited): every role starts streamed
// (a ring of `slots` records); roles are then pinned whole, largest first, while the budget allows; one more role
// may be pinned in part. Returns false when the budget is below the ring reserve.
static bool plan_roles(tnf_stack* st, uint64_t budget, uint64_t* need_rings_out) {
  const uint32_t layers = st->layers, slots = std::min<uint32_t>(st->ring_slots, layers);
  uint64_t need_rings = 0;
  for (auto& r : st->roles) need_rings += uint64_t(slots) * r.lay.bytes;
  if (need_rings_out) *need_rings_out = need_rings;
  if (budget && need_rings > budget) return false;
  std::vector<uint32_t> order(st->roles.size());
  for (uint32_t j = 0; j < order.size(); ++j) order[j] = j;
  std::stable_sort(order.begin(), order.end(), [&](uint32_t a, uint32_t b) { return st->roles[a].lay.bytes > st->roles[b].lay.bytes; });
  uint64_t avail = budget ? budget - need_rings : ~0ull;
  bool partial_done = false;
  for (auto& r : st->roles) r.pinned_layers = 0;
  for (uint32_t j : order) {
    Role& r = st->roles[j];
    const uint64_t full_cost = uint64_t(layers - slots) * r.lay.bytes;  // the ring's bytes are given back
    if (layers <= slots || full_cost <= avail) {
      r.pinned_layers = layers;
      if (layers > slots) avail -= full_cost;
    } else if (!partial_done) {
      r.pinned_layers = uint32_t(std::min<uint64_t>(avail / r.lay.bytes, layers - slots));
      avail -= uint64_t(r.pinned_layers) * r.lay.bytes;
      partial_done = true;
    }
  }
  return true;
}

// Frees a role's weight buffers (resident set and ring) and its ring events. Context mutex held; the caller has
// made sure no work in flight still reads them.
static void release_role_locked(tnf_stack* st, Role& r) {
  tnf_ctx* ctx = st->ctx;
  if (r.pinned_id) {
    st->pinned_bytes -= ctx->bufs[r.pinned_id].bytes;
    free_locked(ctx, r.pinned_id);
  }
  if (r.ring_id) {
    st->ring_bytes -= ctx->bufs[r.ring_id].bytes;
    free_locked(ctx, r.ring_id);
  }
  r.pinned_id = r.ring_id = 0;
  for (auto e : r.ready) cudaEventDestroy(e);
  for (auto e : r.freed) cudaEventDestroy(e);
  r.ready.clear();
  r.freed.clear();
  r.holds.clear();
  r.slots = 0;
}

// Allocates what r.pinned_layers asks for (resident buffer, ring, ring events created signalled) and restarts the
// role's upload sequence at the current step. Context mutex held.
static int32_t materialise_role_locked(tnf_stack* st, Role& r) {
  tnf_ctx* ctx = st->ctx;
  const uint32_t layers = st->layers, slots = std::min<uint32_t>(st->ring_slots, layers);
  int32_t status = TNF_OK;
  if (r.pinned_layers) {
    status = alloc_locked(ctx, uint64_t(r.pinned_layers) * r.lay.bytes, TNF_CAT_WEIGHTS, &r.pinned_id);
    if (status != TNF_OK) return status;
    st->pinned_bytes += uint64_t(r.pinned_layers) * r.lay.bytes;
  }
  if (r.pinned_layers < layers) {
    r.slots = std::min<uint32_t>(slots, layers - r.pinned_layers);
    status = alloc_locked(ctx, uint64_t(r.slots) * r.lay.bytes, TNF_CAT_WEIGHTS, &r.ring_id);
    if (status != TNF_OK) return status;
    st->ring_bytes += uint64_t(r.slots) * r.lay.bytes;
  }
  for (uint32_t i = 0; i < r.slots; ++i) {
    cudaEvent_t a, b;
    cudaEventCreateWithFlags(&a, cudaEventDisableTiming);
    cudaEventCreateWithFlags(&b, cudaEventDisableTiming);
    r.ready.push_back(a);
    r.freed.push_back(b);
    r.holds.push_back(-1);
  }
  r.next_upload = 0;
  r.epoch_step = st->steps_done;
  return TNF_OK;
}

// Queues the upload of a role's resident records on the copy stream.
static int32_t upload_pinned(tnf_stack* st, Role& r) {
  if (!r.pinned_layers) return TNF_OK;
  tnf_ctx* ctx = st->ctx;
  uint8_t* dst = static_cast<uint8_t*>(ctx->bufs[r.pinned_id].ptr);
  for (uint32_t l = 0; l < r.pinned_layers; ++l) {
    cudaError_t ce = cudaMemcpyAsync(dst + uint64_t(l) * r.lay.bytes, st->host_base + uint64_t(l) * st->layer_bytes + r.layer_off,
                                     r.lay.bytes, cudaMemcpyHostToDevice, ctx->copy);
    if (ce != cudaSuccess) return cuda_fail(ce, "stack: resident upload");
  }
  return TNF_OK;
}

// The stack's entry in the arbiter's reclaim chain (WeightReclaimer, thinfer-core/src/residency.rs:1473-1547):
// resident weight sets are given back largest first; a role that loses its resident set is streamed through a ring
// from the next step on. Work in flight is waited for once, before the first free. Context mutex held.
static uint64_t stack_reclaim(void* owner, uint64_t want) {
  tnf_stack* st = static_cast<tnf_stack*>(owner);
  if (st->evicted || st->in_step) return 0;
  std::vector<uint32_t> order;
  for (uint32_t j = 0; j < st->roles.size(); ++j)
    if (st->roles[j].pinned_layers > std::min<uint32_t>(st->ring_slots, st->layers)) order.push_back(j);
  std::stable_sort(order.begin(), order.end(), [&](uint32_t a, uint32_t b) {
    return uint64_t(st->roles[a].pinned_layers) * st->roles[a].lay.bytes > uint64_t(st->roles[b].pinned_layers) * st->roles[b].lay.bytes;
  });
  uint64_t freed = 0;
  bool synced = false;
  for (uint32_t j : order) {
    if (freed >= want) break;
    Role& r = st->roles[j];
    if (!synced) {
      cudaStreamSynchronize(st->ctx->compute);
      cudaStreamSynchronize(st->ctx->copy);
      synced = true;
    }
    const uint64_t before = uint64_t(r.pinned_layers) * r.lay.bytes + uint64_t(r.slots) * r.lay.bytes;
    release_role_locked(st, r);
    r.pinned_layers = 0;
    if (materialise_role_locked(st, r) != TNF_OK) continue;  // the ring always fits: it is smaller than what was freed
    const uint64_t after = uint64_t(r.slots) * r.lay.bytes;
    freed += before - after;
  }
  st->demoted_bytes += freed;
  return freed;
}

// The weight budget a plan may use now: the configured one, capped by what the context's budget leaves after
// everything that is not this stack's weights and after the transient reserve.
static uint64_t effective_budget(tnf_stack* st, uint64_t configured) {
  tnf_ctx* ctx = st->ctx;
  if (!ctx->budget) return configured;
  const uint64_t live = ctx->live[0] + ctx->live[1] + ctx->live[2];
  const uint64_t own = st->pinned_bytes + st->ring_bytes;
  const uint64_t others = live - own + ctx->transient_reserve;
  const uint64_t room = ctx->budget > others ? ctx->budget - others : 1;  // 0 would read as "unlimited"
  return configured ? std::min(configured, room) : room;
}

extern "C" {

uint64_t tnf_stack_record_bytes(uint32_t n, uint32_t k) { return record_layout(n, k).bytes; }

int32_t tnf_stack_record_offsets(uint32_t n, uint32_t k, uint64_t out[4]) {
  RecordLayout r = record_layout(n, k);
  out[0] = r.codes_off;
  out[1] = r.scales_off;
  out[2] = r.bias_off;
  out[3] = r.global_off;
  return TNF_OK;
}

int32_t tnf_stack_create(tnf_ctx* ctx, uint32_t layers, uint32_t n_linears, const tnf_stack_linear* linears,
                         uint32_t n_streams, const uint32_t* m_rows, uint32_t hidden, uint64_t host_id,
                         uint64_t weight_budget_bytes, uint32_t ring_slots, tnf_stack** out) {
  if (!ctx || !linears || !m_rows || !out || layers == 0 || n_linears == 0 || n_streams == 0 || n_streams > 8) {
    set_error("tnf_stack_create: bad arguments");
    return TNF_ERR_INVALID_ARGUMENT;
  }
  cudaError_t ce = cudaSetDevice(ctx->device);
  if (ce != cudaSuccess) return cuda_fail(ce, "cudaSetDevice");
  if (ring_slots == 0) ring_slots = 4;  // the reference's ring depth (thinfer-core/src/residency.rs:50)
  if (ring_slots < 2) ring_slots = 2;
  tnf_stack* st = new tnf_stack();
  st->ctx = ctx;
  st->layers = layers;
  st->hidden = hidden;
  st->n_streams = n_streams;
  st->m_rows.assign(m_rows, m_rows + n_streams);
  st->host_id = host_id;
  uint64_t host_bytes = 0;
  {
    std::lock_guard<std::mutex> lk(ctx->mu);
    auto it = ctx->hosts.find(host_id);
    if (it == ctx->hosts.end()) {
      set_error("tnf_stack_create: unknown host arena %llu", (unsigned long long)host_id);
      delete st;
      return TNF_ERR_UNKNOWN_BUFFER;
    }
    st->host_base = static_cast<const uint8_t*>(it->second.ptr);
    host_bytes = it->second.bytes;
  }
  uint64_t off = 0;
  for (uint32_t j = 0; j < n_linears; ++j) {
    const tnf_stack_linear& d = linears[j];
    if (d.n == 0 || d.k == 0 || d.k % 32 || d.n % 8 || d.stream_id >= n_streams || d.input > 2 || d.act > 1) {
      set_error("tnf_stack_create: linear %u is malformed (n %u k %u stream %u input %u)", j, d.n, d.k, d.stream_id, d.input);
      delete st;
      return TNF_ERR_INVALID_ARGUMENT;
    }
    Role r;
    r.desc = d;
    r.lay = record_layout(d.n, d.k);
    r.layer_off = off;
    off += r.lay.bytes;
    st->roles.push_back(r);
  }
  st->layer_bytes = off;
  if (uint64_t(layers) * st->layer_bytes > host_bytes) {
    set_error("tnf_stack_create: host arena holds %llu bytes, the stack needs %llu", (unsigned long long)host_bytes,
              (unsigned long long)(uint64_t(layers) * st->layer_bytes));
    delete st;
    return TNF_ERR_INVALID_ARGUMENT;
  }
  // ---- pin plan, device memory, resident uploads
  st->weight_budget = weight_budget_bytes;
  st->ring_slots = ring_slots;
  uint64_t need_rings = 0;
  if (!plan_roles(st, weight_budget_bytes, &need_rings)) {
    set_error("weight budget %llu is below the ring reserve %llu (%u slots per linear)",
              (unsigned long long)weight_budget_bytes, (unsigned long long)need_rings, std::min<uint32_t>(ring_slots, layers));
    delete st;
    return TNF_ERR_BUDGET_EXCEEDED;  // refused on the host; the device is not touched
  }
  int32_t status = TNF_OK;
  {
    std::lock_guard<std::mutex> lk(ctx->mu);
    for (auto& r : st->roles) {
      status = materialise_role_locked(st, r);
      if (status != TNF_OK) break;
      status = alloc_locked(ctx, std::max<uint64_t>(uint64_t(st->m_rows[r.desc.stream_id]) * r.desc.n * 2, 256), TNF_CAT_WORKSPACE, &r.out_id);
      if (status != TNF_OK) break;
    }
    for (uint32_t s = 0; s < n_streams && status == TNF_OK; ++s) {
      uint64_t a = 0, b = 0;
      status = alloc_locked(ctx, std::max<uint64_t>(uint64_t(m_rows[s]) * hidden * 2, 256), TNF_CAT_WORKSPACE, &a);
      if (status == TNF_OK) status = alloc_locked(ctx, std::max<uint64_t>(uint64_t(m_rows[s]) * hidden * 2, 256), TNF_CAT_WORKSPACE, &b);
      st->x_ping.push_back(a);
      st->x_pong.push_back(b);
    }
  }
  if (status != TNF_OK) {
    tnf_stack_destroy(st);
    return status;
  }
  for (auto& r : st->roles) {
    status = upload_pinned(st, r);
    if (status != TNF_OK) {
      tnf_stack_destroy(st);
      return status;
    }
  }
  ce = cudaStreamSynchronize(ctx->copy);
  if (ce != cudaSuccess) {
    tnf_stack_destroy(st);
    return cuda_fail(ce, "stack: resident upload sync");
  }
  {
    std::lock_guard<std::mutex> lk(ctx->mu);
    ctx->reclaimers.push_back(tnf_reclaimer{st, stack_reclaim});
  }
  *out = st;
  return TNF_OK;
}

int32_t tnf_stack_evict_all(tnf_stack* st) {
  if (!st) {
    set_error("tnf_stack_evict_all: null stack");
    return TNF_ERR_INVALID_ARGUMENT;
  }
  tnf_ctx* ctx = st->ctx;
  cudaError_t ce = cudaSetDevice(ctx->device);
  if (ce != cudaSuccess) return cuda_fail(ce, "cudaSetDevice");
  cudaStreamSynchronize(ctx->compute);
  cudaStreamSynchronize(ctx->copy);
  std::lock_guard<std::mutex> lk(ctx->mu);
  for (auto& r : st->roles) {
    release_role_locked(st, r);
    r.pinned_layers = 0;
  }
  st->evicted = true;
  return TNF_OK;
}

int32_t tnf_stack_restore(tnf_stack* st, uint64_t weight_budget_bytes) {
  if (!st) {
    set_error("tnf_stack_restore: null stack");
    return TNF_ERR_INVALID_ARGUMENT;
  }
  tnf_ctx* ctx = st->ctx;
  cudaError_t ce = cudaSetDevice(ctx->device);
  if (ce != cudaSuccess) return cuda_fail(ce, "cudaSetDevice");
  cudaStreamSynchronize(ctx->compute);
  cudaStreamSynchronize(ctx->copy);
  if (weight_budget_bytes) st->weight_budget = weight_budget_bytes;
  int32_t status = TNF_OK;
  {
    std::lock_guard<std::mutex> lk(ctx->mu);
    for (auto& r : st->roles) release_role_locked(st, r);
    uint64_t need_rings = 0;
    const uint64_t budget = effective_budget(st, st->weight_budget);
    if (!plan_roles(st, budget, &need_rings)) {
      for (auto& r : st->roles) r.pinned_layers = 0;
      st->evicted = true;
      set_error("tnf_stack_restore: %llu bytes are available for weights, the rings alone need %llu",
                (unsigned long long)budget, (unsigned long long)need_rings);
      return TNF_ERR_BUDGET_EXCEEDED;
    }
    ctx->in_reclaim = true;  // a restore never asks other holders (or itself) to give memory back
    for (auto& r : st->roles) {
      status = materialise_role_locked(st, r);
      if (status != TNF_OK) break;
    }
    ctx->in_reclaim = false;
  }
  if (status != TNF_OK) return status;
  for (auto& r : st->roles) {
    status = upload_pinned(st, r);
    if (status != TNF_OK) return status;
  }
  ce = cudaStreamSynchronize(ctx->copy);
  if (ce != cudaSuccess) return cuda_fail(ce, "stack: resident upload sync");
  st->evicted = false;
  return TNF_OK;
}

int32_t tnf_stack_step(tnf_stack* st, const uint64_t* x_ids, const uint64_t* aux_ids, const uint64_t* out_ids,
                       float a_global) {
  if (!st || !x_ids || !out_ids || !(a_global > 0.0f)) {
    set_error("tnf_stack_step: bad arguments");
    return TNF_ERR_INVALID_ARGUMENT;
  }
  tnf_ctx* ctx = st->ctx;
  cudaError_t ce = cudaSetDevice(ctx->device);
  if (ce != cudaSuccess) return cuda_fail(ce, "cudaSetDevice");
  if (st->evicted) {  // a phase eviction happened: bring the weights back under what the budget allows now
    int32_t s = tnf_stack_restore(st, 0);
    if (s != TNF_OK) return s;
  }
  st->uploaded_last = 0;
  st->uploads_last = 0;
  struct InStep {
    tnf_stack* s;
    explicit InStep(tnf_stack* p) : s(p) { s->in_step = true; }
    ~InStep() { s->in_step = false; }
  } in_step_guard(st);
  // first use of a ring (after creation, a restore or a reclaim): fill it; later steps find their first layers in flight
  for (auto& r : st->roles) {
    while (r.slots && r.next_upload < int64_t(r.slots) && st->steps_done == r.epoch_step) {
      int32_t s = upload_record(st, r, r.next_upload);
      if (s != TNF_OK) return s;
      ++r.next_upload;
    }
  }
  const size_t R = st->roles.size();
  // which linear is the last of its stream (its output feeds the next layer when n == hidden)
  std::vector<int> last_of_stream(st->n_streams, -1);
  for (size_t j = 0; j < R; ++j) last_of_stream[st->roles[j].desc.stream_id] = int(j);
  for (uint32_t l = 0; l < st->layers; ++l) {
    for (size_t j = 0; j < R; ++j) {
      Role& r = st->roles[j];
      const uint32_t s = r.desc.stream_id;
      const uint32_t m = st->m_rows[s];
      const bool feeds = last_of_stream[s] == int(j) && r.desc.n == st->hidden;
      const bool stream_chains = st->roles[last_of_stream[s]].desc.n == st->hidden;
      // input
      uint64_t in_id;
      if (r.desc.input == 1) {
        if (j == 0 || st->roles[j - 1].desc.stream_id != s || st->roles[j - 1].desc.n != r.desc.k) {
          set_error("stack: linear %zu chains on a previous linear of another stream or width", j);
          return TNF_ERR_INVALID_ARGUMENT;
        }
        in_id = st->roles[j - 1].out_id;
      } else if (r.desc.input == 2) {
        if (!aux_ids) {
          set_error("stack: linear %zu needs an auxiliary input", j);
          return TNF_ERR_INVALID_ARGUMENT;
        }
        in_id = aux_ids[s];
      } else {
        in_id = (l == 0 || !stream_chains) ? x_ids[s] : ((l & 1u) ? st->x_ping[s] : st->x_pong[s]);
      }
      // output
      uint64_t out_id = r.out_id;
      if (last_of_stream[s] == int(j)) {
        if (l + 1 == st->layers) out_id = out_ids[s];
        else if (feeds) out_id = (l & 1u) ? st->x_pong[s] : st->x_ping[s];
      }
      // weight record
      uint64_t w_id, w_off;
      int slot = -1;
      if (l < r.pinned_layers) {
        w_id = r.pinned_id;
        w_off = uint64_t(l) * r.lay.bytes;
      } else {
        const uint32_t streamed = st->layers - r.pinned_layers;
        const int64_t seq = (st->steps_done - r.epoch_step) * int64_t(streamed) + int64_t(l - r.pinned_layers);
        slot = int(seq % r.slots);
        if (r.holds[slot] != seq) {
          set_error("stack: ring of linear %zu holds sequence %lld in slot %d, expected %lld", j, (long long)r.holds[slot],
                    slot, (long long)seq);
          return TNF_ERR_LAUNCH;
        }
        ce = cudaStreamWaitEvent(ctx->compute, r.ready[slot], 0);
        if (ce != cudaSuccess) return cuda_fail(ce, "stack: wait upload");
        w_id = r.ring_id;
        w_off = uint64_t(slot) * r.lay.bytes;
      }
      float w_global = 0.0f;
      {
        const uint32_t layer = l;
        std::memcpy(&w_global, st->host_base + uint64_t(layer) * st->layer_bytes + r.layer_off + r.lay.global_off, 4);
      }
      tnf_linear_args a{};
      a.m = m;
      a.n = r.desc.n;
      a.k = r.desc.k;
      a.a_global = a_global;
      a.w_global = w_global;
      a.a_bf16 = tnf_buf{in_id, 0, uint64_t(m) * r.desc.k * 2};
      a.w_codes = tnf_buf{w_id, w_off + r.lay.codes_off, uint64_t(r.desc.n) * (r.desc.k / 2)};
      a.w_scales = tnf_buf{w_id, w_off + r.lay.scales_off, sf_device_bytes(r.desc.n, r.desc.k)};
      if (r.desc.has_bias) a.bias_bf16 = tnf_buf{w_id, w_off + r.lay.bias_off, uint64_t(r.desc.n) * 2};
      a.out_bf16 = tnf_buf{out_id, 0, uint64_t(m) * r.desc.n * 2};
      a.act = r.desc.act;
      int32_t status = tnf_linear_nvfp4(ctx, &a);
      if (status != TNF_OK) return status;
      if (slot >= 0) {
        ce = cudaEventRecord(r.freed[slot], ctx->compute);
        if (ce != cudaSuccess) return cuda_fail(ce, "stack: record slot free");
        status = upload_record(st, r, r.next_upload);  // refill the slot with the layer `slots` ahead (cyclic)
        if (status != TNF_OK) return status;
        ++r.next_upload;
      }
    }
  }
  st->steps_done += 1;
  return TNF_OK;
}

int32_t tnf_stack_stats(tnf_stack* st, uint64_t out[6]) {
  if (!st || !out) {
    set_error("tnf_stack_stats: null argument");
    return TNF_ERR_INVALID_ARGUMENT;
  }
  uint64_t resident = 0, streamed = 0;
  for (auto& r : st->roles) {
    resident += r.pinned_layers;
    streamed += st->layers - r.pinned_layers;
  }
  out[0] = st->pinned_bytes;
  out[1] = st->ring_bytes;
  out[2] = st->uploaded_last;
  out[3] = st->uploads_last;
  out[4] = resident;
  out[5] = streamed;
  return TNF_OK;
}

int32_t tnf_stack_destroy(tnf_stack* st) {
  if (!st) return TNF_OK;
  tnf_ctx* ctx = st->ctx;
  cudaSetDevice(ctx->device);
  cudaStreamSynchronize(ctx->copy);
  cudaStreamSynchronize(ctx->compute);
  {
    std::lock_guard<std::mutex> lk(ctx->mu);
    for (auto it = ctx->reclaimers.begin(); it != ctx->reclaimers.end();)
      it = it->owner == st ? ctx->reclaimers.erase(it) : it + 1;
    for (auto& r : st->roles) {
      release_role_locked(st, r);
      if (r.out_id) free_locked(ctx, r.out_id);
    }
    for (auto id : st->x_ping) if (id) free_locked(ctx, id);
    for (auto id : st->x_pong) if (id) free_locked(ctx, id);
  }
  delete st;
  return TNF_OK;
}

}  // extern "C"
