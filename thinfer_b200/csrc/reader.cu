// Host IO: random-access readers with readahead hints, and the chunk loops that land a reader's bytes
// in caller memory, in a pinned arena, or in a device buffer.
//
// The reference reads weights through `trait WeightReader` (len / read_at / will_read,
// thinfer-core/src/weight.rs:57-77), opens whole files through `trait FileOpener` (:93-97), hands out
// per-tensor windows with `OffsetView` (:102-127), and on native targets backs them with an mmap whose
// will_read is madvise(WILLNEED) (thinfer-native/src/lib.rs:15-106). Its streaming loop hints
// READ_PREFETCH_CHUNKS = 4 chunks of 16 MiB ahead of the chunk it copies
// (thinfer-core/src/residency.rs:61-71,1253-1292). Here the trait is a C struct of function pointers,
// so the embedding program can keep its own readers (the Rust side passes trampolines to its
// WeightReader), and the built-in reader is the mmap one. Toward the device the loop is double
// buffered through two pinned staging slots: the read of chunk i+1 overlaps the DMA of chunk i.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <cerrno>
#include <cstring>
#include <new>

#include "../../include/thinfer_nvfp4.h"
#include "context.h"

namespace {

using tnf::set_error;

constexpr uint64_t kDefaultChunk = 16ull << 20;  // UPLOAD_CHUNK_BYTES of the reference
constexpr uint32_t kDefaultHints = 4;            // READ_PREFETCH_CHUNKS of the reference

struct MmapState {
  uint8_t* base = nullptr;
  uint64_t len = 0;
  long page = 4096;
  std::atomic<uint64_t> reads{0}, read_bytes{0}, hints{0}, hint_bytes{0};
};

uint64_t mmap_len(void* u) { return static_cast<MmapState*>(u)->len; }

int32_t mmap_read_at(void* u, uint64_t offset, void* dst, uint64_t n) {
  MmapState* m = static_cast<MmapState*>(u);
  if (offset > m->len || n > m->len - offset) {  // "read past mmap end" (UnexpectedEof); also the overflow case
    set_error("mmap reader: read [%llu, +%llu) past the end of a mapping of %llu bytes", (unsigned long long)offset,
              (unsigned long long)n, (unsigned long long)m->len);
    return TNF_ERR_INVALID_ARGUMENT;
  }
  if (n) std::memcpy(dst, m->base + offset, n);
  m->reads.fetch_add(1, std::memory_order_relaxed);
  m->read_bytes.fetch_add(n, std::memory_order_relaxed);
  return TNF_OK;
}

// Best effort: a hint that is out of range or refused only costs speed, never bytes.
void mmap_will_read(void* u, uint64_t offset, uint64_t n) {
  MmapState* m = static_cast<MmapState*>(u);
  if (n == 0 || offset > m->len || n > m->len - offset) return;
  const uint64_t lo = offset & ~uint64_t(m->page - 1);  // madvise wants a page-aligned start
  (void)madvise(m->base + lo, size_t(offset + n - lo), MADV_WILLNEED);
  m->hints.fetch_add(1, std::memory_order_relaxed);
  m->hint_bytes.fetch_add(n, std::memory_order_relaxed);
}

void mmap_close(void* u) {
  MmapState* m = static_cast<MmapState*>(u);
  if (m->base && m->len) munmap(m->base, size_t(m->len));
  delete m;
}

struct ViewState {
  tnf_reader inner;
  uint64_t base = 0, len = 0;
};

uint64_t view_len(void* u) { return static_cast<ViewState*>(u)->len; }

int32_t view_read_at(void* u, uint64_t offset, void* dst, uint64_t n) {
  ViewState* v = static_cast<ViewState*>(u);
  if (offset > v->len || n > v->len - offset) {
    set_error("reader view: read [%llu, +%llu) outside a window of %llu bytes", (unsigned long long)offset,
              (unsigned long long)n, (unsigned long long)v->len);
    return TNF_ERR_INVALID_ARGUMENT;
  }
  return v->inner.read_at(v->inner.user, v->base + offset, dst, n);
}

void view_will_read(void* u, uint64_t offset, uint64_t n) {
  ViewState* v = static_cast<ViewState*>(u);
  if (!v->inner.will_read || offset > v->len) return;
  v->inner.will_read(v->inner.user, v->base + offset, std::min(n, v->len - offset));
}

void view_close(void* u) { delete static_cast<ViewState*>(u); }  // the inner reader belongs to the caller

bool usable(const tnf_reader* r, const char* who) {
  if (!r || !r->len || !r->read_at) {
    set_error("%s: a reader needs len and read_at", who);
    return false;
  }
  return true;
}

// Checks [offset, offset + n) against the reader and fills in the chunking defaults.
int32_t check_range(const tnf_reader* r, uint64_t offset, uint64_t n, uint64_t* chunk, uint32_t* hints, const char* who) {
  if (!usable(r, who)) return TNF_ERR_INVALID_ARGUMENT;
  const uint64_t len = r->len(r->user);
  if (offset > len || n > len - offset) {
    set_error("%s: range [%llu, +%llu) outside a reader of %llu bytes", who, (unsigned long long)offset,
              (unsigned long long)n, (unsigned long long)len);
    return TNF_ERR_INVALID_ARGUMENT;
  }
  if (*chunk == 0) *chunk = kDefaultChunk;
  if (*hints == TNF_READER_DEFAULT_HINTS) *hints = kDefaultHints;
  return TNF_OK;
}

// The hint schedule of the reference's loop: the first `hints` chunks up front, then, after each chunk is read,
// the chunk `hints` ahead of it.
struct Hinter {
  const tnf_reader* r;
  uint64_t base, total, chunk;
  uint32_t ahead;
  void prime() const {
    if (!r->will_read) return;
    for (uint32_t i = 0; i < ahead && uint64_t(i) * chunk < total; ++i)
      r->will_read(r->user, base + uint64_t(i) * chunk, std::min(chunk, total - uint64_t(i) * chunk));
  }
  void after(uint64_t off) const {
    if (!r->will_read || ahead == 0) return;
    const uint64_t a = off + uint64_t(ahead) * chunk;
    if (a < total) r->will_read(r->user, base + a, std::min(chunk, total - a));
  }
};

int32_t read_loop(const tnf_reader* r, uint64_t offset, uint64_t n, uint8_t* dst, uint64_t chunk, uint32_t hints) {
  Hinter h{r, offset, n, chunk, hints};
  h.prime();
  for (uint64_t off = 0; off < n; off += chunk) {
    const uint64_t len = std::min(chunk, n - off);
    int32_t st = r->read_at(r->user, offset + off, dst + off, len);
    if (st != TNF_OK) return st;
    h.after(off);
  }
  return TNF_OK;
}

}  // namespace

extern "C" {

int32_t tnf_mmap_open(const char* path, tnf_reader* out) {
  if (!path || !out) {
    set_error("tnf_mmap_open: null path or reader");
    return TNF_ERR_INVALID_ARGUMENT;
  }
  const int fd = open(path, O_RDONLY | O_CLOEXEC);
  if (fd < 0) {
    set_error("tnf_mmap_open: %s: %s", path, std::strerror(errno));
    return TNF_ERR_INVALID_ARGUMENT;
  }
  struct stat sb;
  if (fstat(fd, &sb) != 0) {
    set_error("tnf_mmap_open: fstat %s: %s", path, std::strerror(errno));
    close(fd);
    return TNF_ERR_INVALID_ARGUMENT;
  }
  MmapState* m = new (std::nothrow) MmapState;
  if (!m) {
    close(fd);
    set_error("tnf_mmap_open: out of host memory");
    return TNF_ERR_ALLOCATE_OOM;
  }
  m->len = uint64_t(sb.st_size);
  const long pg = sysconf(_SC_PAGESIZE);
  if (pg > 0) m->page = pg;
  if (m->len) {  // an empty file maps to an empty reader (mmap refuses a zero length)
    void* p = mmap(nullptr, size_t(m->len), PROT_READ, MAP_PRIVATE, fd, 0);
    if (p == MAP_FAILED) {
      set_error("tnf_mmap_open: mmap %s: %s", path, std::strerror(errno));
      close(fd);
      delete m;
      return TNF_ERR_INVALID_ARGUMENT;
    }
    m->base = static_cast<uint8_t*>(p);
  }
  close(fd);  // the mapping keeps the file
  out->user = m;
  out->len = mmap_len;
  out->read_at = mmap_read_at;
  out->will_read = mmap_will_read;
  out->close = mmap_close;
  return TNF_OK;
}

int32_t tnf_mmap_stats(const tnf_reader* r, uint64_t out[4]) {
  if (!r || r->len != mmap_len || !out) {
    set_error("tnf_mmap_stats: not a reader made by tnf_mmap_open");
    return TNF_ERR_INVALID_ARGUMENT;
  }
  const MmapState* m = static_cast<const MmapState*>(r->user);
  out[0] = m->reads.load();
  out[1] = m->read_bytes.load();
  out[2] = m->hints.load();
  out[3] = m->hint_bytes.load();
  return TNF_OK;
}

int32_t tnf_reader_view(const tnf_reader* inner, uint64_t base, uint64_t len, tnf_reader* out) {
  if (!usable(inner, "tnf_reader_view") || !out) {
    if (inner && !out) set_error("tnf_reader_view: null output");
    return TNF_ERR_INVALID_ARGUMENT;
  }
  const uint64_t total = inner->len(inner->user);
  if (base > total || len > total - base) {
    set_error("tnf_reader_view: window [%llu, +%llu) outside a reader of %llu bytes", (unsigned long long)base,
              (unsigned long long)len, (unsigned long long)total);
    return TNF_ERR_INVALID_ARGUMENT;
  }
  ViewState* v = new (std::nothrow) ViewState;
  if (!v) {
    set_error("tnf_reader_view: out of host memory");
    return TNF_ERR_ALLOCATE_OOM;
  }
  v->inner = *inner;
  v->base = base;
  v->len = len;
  out->user = v;
  out->len = view_len;
  out->read_at = view_read_at;
  out->will_read = view_will_read;
  out->close = view_close;
  return TNF_OK;
}

void tnf_reader_close(tnf_reader* r) {
  if (!r) return;
  if (r->close) r->close(r->user);
  std::memset(r, 0, sizeof(*r));
}

int32_t tnf_reader_read(const tnf_reader* r, uint64_t offset, uint64_t n, void* dst, uint64_t chunk_bytes, uint32_t hint_chunks) {
  int32_t st = check_range(r, offset, n, &chunk_bytes, &hint_chunks, "tnf_reader_read");
  if (st != TNF_OK) return st;
  if (n && !dst) {
    set_error("tnf_reader_read: null destination");
    return TNF_ERR_INVALID_ARGUMENT;
  }
  return read_loop(r, offset, n, static_cast<uint8_t*>(dst), chunk_bytes, hint_chunks);
}

int32_t tnf_reader_read_to_arena(tnf_ctx* ctx, const tnf_reader* r, uint64_t offset, uint64_t n, uint64_t host_id,
                                 uint64_t host_off, uint64_t chunk_bytes, uint32_t hint_chunks) {
  if (!ctx) {
    set_error("null context");
    return TNF_ERR_INVALID_ARGUMENT;
  }
  int32_t st = check_range(r, offset, n, &chunk_bytes, &hint_chunks, "tnf_reader_read_to_arena");
  if (st != TNF_OK) return st;
  uint8_t* dst = nullptr;
  {
    std::lock_guard<std::mutex> lk(ctx->mu);
    auto it = ctx->hosts.find(host_id);
    if (it == ctx->hosts.end()) {
      set_error("tnf_reader_read_to_arena: unknown host arena %llu", (unsigned long long)host_id);
      return TNF_ERR_UNKNOWN_BUFFER;
    }
    if (host_off > it->second.bytes || n > it->second.bytes - host_off) {
      set_error("tnf_reader_read_to_arena: host range [%llu, +%llu) outside arena of %llu bytes", (unsigned long long)host_off,
                (unsigned long long)n, (unsigned long long)it->second.bytes);
      return TNF_ERR_INVALID_ARGUMENT;
    }
    dst = static_cast<uint8_t*>(it->second.ptr) + host_off;
  }
  return read_loop(r, offset, n, dst, chunk_bytes, hint_chunks);
}

int32_t tnf_upload_from_reader(tnf_ctx* ctx, const tnf_reader* r, uint64_t src_offset, uint64_t total, tnf_buf dst,
                               uint64_t chunk_bytes, uint32_t hint_chunks, uint64_t* event) {
  if (!ctx) {
    set_error("null context");
    return TNF_ERR_INVALID_ARGUMENT;
  }
  int32_t st = check_range(r, src_offset, total, &chunk_bytes, &hint_chunks, "tnf_upload_from_reader");
  if (st != TNF_OK) return st;
  const uint64_t padded = dst.len;  // bytes past `total` are zero-filled, as the reference pads its destination
  if (padded < total) {
    set_error("tnf_upload_from_reader: the destination view holds %llu bytes, the source range %llu",
              (unsigned long long)padded, (unsigned long long)total);
    return TNF_ERR_INVALID_ARGUMENT;
  }
  uint8_t* d = tnf::resolve(ctx, dst, padded, "tnf_upload_from_reader dst", &st);
  if (!d && padded) return st;
  if (cudaSetDevice(ctx->device) != cudaSuccess) return tnf::cuda_fail(cudaGetLastError(), "cudaSetDevice");
  // two pinned staging slots, kept by the context and grown when a larger chunk is asked for
  const uint64_t slot = std::min(chunk_bytes, std::max<uint64_t>(padded, 1));
  {
    std::lock_guard<std::mutex> lk(ctx->mu);
    if (ctx->stage_bytes < slot) {
      for (int i = 0; i < 2; ++i) {
        if (ctx->stage_host[i]) {
          if (ctx->stage_done[i]) cudaEventSynchronize(ctx->stage_done[i]);
          cudaFreeHost(ctx->stage_host[i]);
          ctx->stage_host[i] = nullptr;
        }
      }
      ctx->stage_bytes = 0;
      for (int i = 0; i < 2; ++i) {
        cudaError_t e = cudaHostAlloc(&ctx->stage_host[i], slot, cudaHostAllocDefault);
        if (e != cudaSuccess) return tnf::cuda_fail(e, "tnf_upload_from_reader staging slot");
        if (!ctx->stage_done[i]) {
          e = cudaEventCreateWithFlags(&ctx->stage_done[i], cudaEventDisableTiming);
          if (e != cudaSuccess) return tnf::cuda_fail(e, "cudaEventCreate");
        }
      }
      ctx->stage_bytes = slot;
    }
  }
  Hinter h{r, src_offset, total, chunk_bytes, hint_chunks};
  h.prime();
  int which = 0;
  for (uint64_t off = 0; off < padded; off += chunk_bytes, which ^= 1) {
    const uint64_t n_write = std::min(chunk_bytes, padded - off);
    const uint64_t n_read = off < total ? std::min(n_write, total - off) : 0;
    uint8_t* stage = static_cast<uint8_t*>(ctx->stage_host[which]);
    cudaError_t e = cudaEventSynchronize(ctx->stage_done[which]);  // the copy that last used this slot (a fresh event is complete)
    if (e != cudaSuccess) return tnf::cuda_fail(e, "staging slot wait");
    if (n_read) {
      st = r->read_at(r->user, src_offset + off, stage, n_read);
      if (st != TNF_OK) return st;
      h.after(off);
    }
    if (n_write > n_read) std::memset(stage + n_read, 0, size_t(n_write - n_read));
    e = cudaMemcpyAsync(d + off, stage, n_write, cudaMemcpyHostToDevice, ctx->copy);
    if (e != cudaSuccess) return tnf::cuda_fail(e, "tnf_upload_from_reader copy");
    e = cudaEventRecord(ctx->stage_done[which], ctx->copy);
    if (e != cudaSuccess) return tnf::cuda_fail(e, "cudaEventRecord");
  }
  cudaEvent_t ev = nullptr;
  {
    std::lock_guard<std::mutex> lk(ctx->mu);
    ctx->streamed += padded;
    if (event && !ctx->event_pool.empty()) {
      ev = ctx->event_pool.back();
      ctx->event_pool.pop_back();
    }
  }
  if (event) {  // completion of the last chunk, for tnf_wait_event / tnf_event_sync
    cudaError_t e = ev ? cudaSuccess : cudaEventCreateWithFlags(&ev, cudaEventDisableTiming);
    if (e != cudaSuccess) return tnf::cuda_fail(e, "cudaEventCreate");
    e = cudaEventRecord(ev, ctx->copy);
    if (e != cudaSuccess) return tnf::cuda_fail(e, "cudaEventRecord");
    std::lock_guard<std::mutex> lk(ctx->mu);
    const uint64_t id = ctx->next_id++;
    ctx->events[id] = ev;
    *event = id;
  }
  return TNF_OK;
}

}  // extern "C"
