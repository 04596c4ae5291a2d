// GGUF-v3 header parser and tensor catalog for the NVFP4 container. Host code only.
//
// Follows the reference's parser (thinfer-core/src/format/gguf.rs): pure "bytes in, catalog out";
// little-endian; strings are u64 length + bytes; a parse over a buffer that is too short reports
// the absolute offset it needed (`NeedMore { at }`, gguf.rs:49-58) so that a caller can read the
// header in pieces without loading the file; guardrails on counts and lengths (gguf.rs:80-84);
// `general.alignment` (default 32, a power of two, at most 64 KiB) positions the tensor data
// (gguf.rs:153-167,196-198); tensor sizes come from the NEXT tensor's offset in offset order and
// the file size bounds the last one (catalog_from, gguf.rs:206-250); GGUF dims are innermost-first
// and the catalog reverses them to the engine's outer-first [N, K] (gguf.rs:211-216).
//
// One tensor type is added to ggml's table: TNF_GGML_TYPE_NVFP4_RECORD, a whole linear as the
// streaming residency consumes it (tnf_stack_record_offsets: E2M1 codes, device-layout E4M3
// scales, bf16 bias, f32 per-tensor scale, sections 256-byte aligned), dims [K, N]. A container
// written with a 256-byte alignment can be read straight into the pinned arena and streamed
// unchanged (the reference's passthrough rule for quantised blocks, thinfer-core/src/residency.rs:155-162).
#include <algorithm>
#include <cstring>
#include <string>
#include <vector>

#include "context.h"

namespace {

constexpr uint32_t kMagic = 0x46554747u;  // "GGUF"
constexpr uint32_t kVersion = 3;
constexpr uint64_t kDefaultAlignment = 32;
constexpr uint64_t kMaxStringBytes = 16ull << 20, kMaxKvCount = 1000000, kMaxTensors = 1000000;
constexpr uint64_t kMaxArrayLen = 64ull << 20, kMaxAlignment = 64ull << 10;

struct TensorInfo {
  std::string name;
  std::vector<uint64_t> dims;  // as stored: innermost first
  uint32_t ggml_type = 0;
  uint64_t offset_in_data = 0;
};

struct NeedMore {
  uint64_t at;
};
struct Malformed {
  std::string what;
};

struct Cursor {
  const uint8_t* buf;
  uint64_t len, pos = 0;
  void ensure(uint64_t n) const {
    if (len < pos + n) throw NeedMore{pos + n};
  }
  template <typename T>
  T read() {
    ensure(sizeof(T));
    T v;
    std::memcpy(&v, buf + pos, sizeof(T));  // the library is built for little-endian hosts only
    pos += sizeof(T);
    return v;
  }
  std::string read_string() {
    const uint64_t n = read<uint64_t>();
    if (n > kMaxStringBytes) throw Malformed{"Oversized { field: string_len, got: " + std::to_string(n) + " }"};
    ensure(n);
    std::string s(reinterpret_cast<const char*>(buf + pos), size_t(n));
    pos += n;
    // UTF-8 well-formedness (overlong forms and surrogates are not singled out: names are ASCII in practice)
    for (size_t i = 0; i < s.size();) {
      const unsigned char c = static_cast<unsigned char>(s[i]);
      const int extra = c < 0x80 ? 0 : (c >> 5) == 6 ? 1 : (c >> 4) == 14 ? 2 : (c >> 3) == 30 ? 3 : -1;
      if (extra < 0 || i + size_t(extra) >= s.size() + (extra == 0 ? 1u : 0u)) throw Malformed{"BadUtf8"};  // bad lead byte or cut short
      for (int k = 1; k <= extra; ++k)
        if ((static_cast<unsigned char>(s[i + k]) >> 6) != 2) throw Malformed{"BadUtf8"};
      i += size_t(extra) + 1;
    }
    return s;
  }
};

// walks one typed value; integral unsigned kinds are returned (enough for general.alignment)
bool parse_value(Cursor& c, uint32_t vt, uint64_t* out) {
  switch (vt) {
    case 0: *out = c.read<uint8_t>(); return true;
    case 1: c.read<uint8_t>(); return false;
    case 2: *out = c.read<uint16_t>(); return true;
    case 3: c.read<uint16_t>(); return false;
    case 4: *out = c.read<uint32_t>(); return true;
    case 5: case 6: c.read<uint32_t>(); return false;
    case 7: {
      const uint8_t b = c.read<uint8_t>();
      if (b > 1) throw Malformed{"BadBool(" + std::to_string(b) + ")"};
      return false;
    }
    case 8: c.read_string(); return false;
    case 9: {
      const uint32_t inner = c.read<uint32_t>();
      const uint64_t n = c.read<uint64_t>();
      if (n > kMaxArrayLen) throw Malformed{"Oversized { field: array_len, got: " + std::to_string(n) + " }"};
      uint64_t ignored;
      for (uint64_t i = 0; i < n; ++i) parse_value(c, inner, &ignored);
      return false;
    }
    case 10: *out = c.read<uint64_t>(); return true;
    case 11: case 12: c.read<uint64_t>(); return false;
    default: throw Malformed{"BadValueType(" + std::to_string(vt) + ")"};
  }
}

uint64_t on_disk_bytes(uint32_t ggml_type, const std::vector<uint64_t>& dims) {
  uint64_t elems = 1;
  for (uint64_t d : dims) elems *= d;
  switch (ggml_type) {
    case 0: return elems * 4;                      // F32
    case 1: case 30: return elems * 2;             // F16, BF16
    case 2: return (elems / 32) * 18;              // Q4_0
    case 8: return (elems / 32) * 34;              // Q8_0
    case 12: return (elems / 256) * 144;           // Q4_K
    case 13: return (elems / 256) * 176;           // Q5_K
    case 14: return (elems / 256) * 210;           // Q6_K
    case 24: return elems;                         // I8
    case TNF_GGML_TYPE_NVFP4_RECORD:
      return dims.size() == 2 && dims[0] % 16 == 0 && dims[0] <= 0xFFFFFFFFull && dims[1] <= 0xFFFFFFFFull
                 ? tnf_stack_record_bytes(uint32_t(dims[1]), uint32_t(dims[0]))
                 : 0;
    default: return 0;  // a type this build does not size; the catalog still lists it
  }
}

}  // namespace

struct tnf_gguf {
  uint32_t version = 0;
  uint64_t alignment = kDefaultAlignment, data_offset = 0;
  std::vector<TensorInfo> tensors;
  std::vector<size_t> by_offset;  // indices of `tensors` in offset order
};

using namespace tnf;

extern "C" {

int32_t tnf_gguf_parse(const void* buf, uint64_t len, tnf_gguf** out, uint64_t* need_at) {
  if ((!buf && len) || !out) {
    set_error("tnf_gguf_parse: null argument");
    return TNF_ERR_INVALID_ARGUMENT;
  }
  *out = nullptr;
  tnf_gguf* h = new tnf_gguf();
  try {
    Cursor c{static_cast<const uint8_t*>(buf), len};
    const uint32_t magic = c.read<uint32_t>();
    if (magic != kMagic) {
      char t[48];
      snprintf(t, sizeof t, "BadMagic(0x%08x)", magic);
      throw Malformed{t};
    }
    h->version = c.read<uint32_t>();
    if (h->version != kVersion) throw Malformed{"UnsupportedVersion(" + std::to_string(h->version) + ")"};
    const uint64_t n_tensors = c.read<uint64_t>();
    if (n_tensors > kMaxTensors) throw Malformed{"Oversized { field: n_tensors, got: " + std::to_string(n_tensors) + " }"};
    const uint64_t n_kv = c.read<uint64_t>();
    if (n_kv > kMaxKvCount) throw Malformed{"Oversized { field: n_kv, got: " + std::to_string(n_kv) + " }"};
    for (uint64_t i = 0; i < n_kv; ++i) {
      const std::string key = c.read_string();
      const uint32_t vt = c.read<uint32_t>();
      uint64_t v = 0;
      if (parse_value(c, vt, &v) && key == "general.alignment") {
        if (v == 0 || (v & (v - 1))) throw Malformed{"BadAlignment(" + std::to_string(v) + ")"};
        if (v > kMaxAlignment) throw Malformed{"AlignmentTooLarge(" + std::to_string(v) + ")"};
        h->alignment = v;
      }
    }
    h->tensors.reserve(size_t(n_tensors));
    for (uint64_t i = 0; i < n_tensors; ++i) {
      TensorInfo t;
      t.name = c.read_string();
      const uint32_t n_dims = c.read<uint32_t>();
      if (n_dims < 1 || n_dims > 8) throw Malformed{"BadDimCount(" + std::to_string(n_dims) + ")"};
      for (uint32_t d = 0; d < n_dims; ++d) t.dims.push_back(c.read<uint64_t>());
      t.ggml_type = c.read<uint32_t>();
      t.offset_in_data = c.read<uint64_t>();
      h->tensors.push_back(std::move(t));
    }
    h->data_offset = c.pos + (h->alignment - c.pos % h->alignment) % h->alignment;
  } catch (const NeedMore& n) {
    delete h;
    if (need_at) *need_at = n.at;
    return TNF_GGUF_NEED_MORE;
  } catch (const Malformed& m) {
    delete h;
    set_error("tnf_gguf_parse: %s", m.what.c_str());
    return TNF_ERR_INVALID_ARGUMENT;
  }
  h->by_offset.resize(h->tensors.size());
  for (size_t i = 0; i < h->by_offset.size(); ++i) h->by_offset[i] = i;
  std::stable_sort(h->by_offset.begin(), h->by_offset.end(),
                   [&](size_t a, size_t b) { return h->tensors[a].offset_in_data < h->tensors[b].offset_in_data; });
  *out = h;
  return TNF_OK;
}

int32_t tnf_gguf_free(tnf_gguf* h) {
  delete h;
  return TNF_OK;
}

int32_t tnf_gguf_info(const tnf_gguf* h, uint64_t out[4]) {
  if (!h || !out) {
    set_error("tnf_gguf_info: null argument");
    return TNF_ERR_INVALID_ARGUMENT;
  }
  out[0] = h->version;
  out[1] = h->alignment;
  out[2] = h->data_offset;
  out[3] = h->tensors.size();
  return TNF_OK;
}

int32_t tnf_gguf_tensor(const tnf_gguf* h, uint64_t index, uint64_t file_size, tnf_gguf_tensor_info* out) {
  if (!h || !out || index >= h->tensors.size()) {
    set_error("tnf_gguf_tensor: index %llu of %llu tensors", (unsigned long long)index,
              (unsigned long long)(h ? h->tensors.size() : 0));
    return TNF_ERR_INVALID_ARGUMENT;
  }
  const TensorInfo& t = h->tensors[size_t(index)];
  std::memset(out, 0, sizeof(*out));
  out->name = t.name.c_str();
  out->n_dims = uint32_t(t.dims.size());
  for (size_t d = 0; d < t.dims.size(); ++d) out->dims[d] = t.dims[t.dims.size() - 1 - d];  // outer-first
  out->ggml_type = t.ggml_type;
  out->on_disk_bytes = on_disk_bytes(t.ggml_type, t.dims);
  out->offset = h->data_offset + t.offset_in_data;
  // size: up to the next tensor in offset order; the file size (or the type's own size) bounds the last
  const size_t rank = size_t(std::find(h->by_offset.begin(), h->by_offset.end(), size_t(index)) - h->by_offset.begin());
  uint64_t next_abs;
  if (rank + 1 < h->by_offset.size()) next_abs = h->data_offset + h->tensors[h->by_offset[rank + 1]].offset_in_data;
  else next_abs = file_size ? file_size : out->offset + out->on_disk_bytes;
  out->size = next_abs > out->offset ? next_abs - out->offset : 0;
  return TNF_OK;
}

const char* tnf_ggml_type_label(uint32_t t) {
  static const char* const kLabels[31] = {"F32",  "F16",  "Q4_0", "Q4_1",    "UNKNOWN", "UNKNOWN", "Q5_0",    "Q5_1",
                                          "Q8_0", "Q8_1", "Q2_K", "Q3_K",    "Q4_K",    "Q5_K",    "Q6_K",    "Q8_K",
                                          "IQ2_XXS", "IQ2_XS", "IQ3_XXS", "IQ1_S", "IQ4_NL", "IQ3_S", "IQ2_S", "IQ4_XS",
                                          "I8",   "I16",  "I32",  "I64",     "F64",     "IQ1_M",   "BF16"};
  if (t == TNF_GGML_TYPE_NVFP4_RECORD) return "NVFP4_RECORD";
  return t < 31 ? kLabels[t] : "UNKNOWN";
}

}  // extern "C"
