"""GGUF-v3 container for NVFP4 linears: writer, streaming reader, residency loader.

The reader mirrors the reference's ``GgufSource`` (thinfer-core/src/format/gguf.rs:440-525): it
reads the file head in growing pieces until the header parser stops answering "need more", then
serves tensors by (offset, size) from the catalog. The parser itself is the library's
``tnf_gguf_parse`` (C++). The writer is new (the reference only reads GGUF): it lays every
tensor out at the container's alignment, 256 bytes by default, so that an NVFP4 record
(``TNF_GGML_TYPE_NVFP4_RECORD``: codes, device-layout scales, bias, per-tensor scale, exactly
what ``tnf_stack_create`` expects in the pinned arena) can be read from the file straight into the
arena and streamed unchanged.
"""
from __future__ import annotations

import ctypes as C
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, Optional, Sequence, Tuple, Union

import numpy as np

from . import _lib as L

MAGIC = 0x46554747
VERSION = 3
GGML_F32, GGML_F16, GGML_Q8_0, GGML_BF16 = 0, 1, 8, 30
GGML_NVFP4_RECORD = L.GGML_TYPE_NVFP4_RECORD
_VT = {"u8": 0, "i8": 1, "u16": 2, "i16": 3, "u32": 4, "i32": 5, "f32": 6, "bool": 7, "str": 8, "u64": 10, "i64": 11, "f64": 12}
_FMT = {"u8": "<B", "i8": "<b", "u16": "<H", "i16": "<h", "u32": "<I", "i32": "<i", "f32": "<f", "bool": "<B",
        "u64": "<Q", "i64": "<q", "f64": "<d"}


class ContainerError(ValueError):
    """A malformed header (the text names the reference's ParseError variant) or an unknown tensor."""


def _string(s: str) -> bytes:
    b = s.encode("utf-8")
    return struct.pack("<Q", len(b)) + b


def _kv(key: str, kind: str, value) -> bytes:
    out = _string(key) + struct.pack("<I", _VT[kind])
    if kind == "str":
        return out + _string(value)
    return out + struct.pack(_FMT[kind], value)


def write_container(path: str, tensors: Sequence[Tuple[str, Sequence[int], int, Union[bytes, np.ndarray]]],
                    metadata: Optional[Iterable[Tuple[str, str, object]]] = None, alignment: int = 256) -> int:
    """Write a GGUF-v3 file. ``tensors``: (name, shape OUTER-first, ggml_type, data); ``metadata``:
    (key, kind, value) with kind in u8..f64/bool/str. Returns the file size."""
    if alignment <= 0 or alignment & (alignment - 1) or alignment > 64 * 1024:
        raise ValueError("alignment must be a power of two, at most 64 KiB")
    kvs = [("general.alignment", "u32", alignment)] + list(metadata or [])
    blobs = [np.ascontiguousarray(d).view(np.uint8).ravel() if isinstance(d, np.ndarray) else np.frombuffer(d, np.uint8)
             for _, _, _, d in tensors]
    offsets, pos = [], 0
    for b in blobs:
        offsets.append(pos)
        pos += (b.size + alignment - 1) // alignment * alignment
    head = struct.pack("<IIQQ", MAGIC, VERSION, len(tensors), len(kvs))
    for key, kind, value in kvs:
        head += _kv(key, kind, value)
    for (name, shape, ggml_type, _), off in zip(tensors, offsets):
        dims = list(shape)[::-1]  # GGUF stores the fastest axis first
        head += _string(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        head += struct.pack("<IQ", ggml_type, off)
    head += b"\0" * (-len(head) % alignment)
    with open(path, "wb") as f:
        f.write(head)
        for b, off in zip(blobs, offsets):
            f.seek(len(head) + off)
            f.write(b.tobytes())
        size = len(head) + pos
        f.truncate(size)
    return size


@dataclass
class TensorEntry:
    name: str
    shape: Tuple[int, ...]   # outer-first, e.g. (N, K)
    ggml_type: int
    label: str
    offset: int              # absolute file offset
    size: int                # bytes up to the next tensor
    on_disk_bytes: int       # bytes the type and shape need (0 if this build cannot size the type)


class Container:
    """An opened container: catalog by name + reads into caller memory."""

    def __init__(self, source: Union[str, "Reader"], first_read: int = 4096):
        """``source``: a file path (opened with the library's mmap reader) or any ``reader.Reader``."""
        from .reader import MmapReader, Reader

        self.path = source if isinstance(source, str) else None
        self.reader: Reader = MmapReader(source) if isinstance(source, str) else source
        self.file_size = len(self.reader)
        lib = L.load()
        handle, need = C.c_void_p(), C.c_uint64()
        want = min(first_read, self.file_size)
        name = self.path or "<reader>"
        while True:  # the reference's streaming pattern: read up to the offset the parser asked for, retry
            buf = self.reader.read(0, want).tobytes()
            rc = lib.tnf_gguf_parse(buf, len(buf), C.byref(handle), C.byref(need))
            if rc == 0:
                break
            if rc == L.GGUF_NEED_MORE:
                if need.value > self.file_size:
                    raise ContainerError(f"{name}: header runs past the end of the file (needs byte {need.value})")
                want = min(max(int(need.value), 2 * want), self.file_size)
                continue
            raise ContainerError(f"{name}: {lib.tnf_last_error().decode()}")
        self.header_reads_to = want
        info = (C.c_uint64 * 4)()
        lib.tnf_gguf_info(handle, info)
        self.version, self.alignment, self.data_offset, n = (int(v) for v in info)
        self.tensors: Dict[str, TensorEntry] = {}
        t = L.GgufTensorInfo()
        for i in range(n):
            if lib.tnf_gguf_tensor(handle, i, self.file_size, C.byref(t)) != 0:
                raise ContainerError(lib.tnf_last_error().decode())
            self.tensors[t.name.decode()] = TensorEntry(
                t.name.decode(), tuple(int(t.dims[d]) for d in range(t.n_dims)), int(t.ggml_type),
                lib.tnf_ggml_type_label(t.ggml_type).decode(), int(t.offset), int(t.size), int(t.on_disk_bytes))
        lib.tnf_gguf_free(handle)

    def read_into(self, name: str, dst: np.ndarray) -> int:
        """Read a tensor's bytes into `dst` (uint8 view of caller memory, e.g. a pinned arena record)."""
        e = self.tensors.get(name)
        if e is None:
            raise ContainerError(f"unknown tensor {name!r}")
        n = e.on_disk_bytes or e.size
        if n > e.size or e.offset + n > self.file_size:
            raise ContainerError(f"{name}: {n} bytes do not fit its slot of {e.size} bytes")
        if dst.dtype != np.uint8 or dst.size < n:
            raise ValueError(f"{name}: destination holds {dst.size} bytes, tensor has {n}")
        self.reader.read(e.offset, n, out=dst)
        return n

    def hint(self, name: str) -> None:
        """Readahead hint for a tensor about to be read (``WeightReader::will_read``)."""
        e = self.tensors.get(name)
        if e is not None:
            self.reader.will_read(e.offset, e.on_disk_bytes or e.size)

    def close(self) -> None:
        if self.path is not None:  # a reader passed in belongs to the caller
            self.reader.close()

    def read(self, name: str) -> np.ndarray:
        e = self.tensors[name] if name in self.tensors else None
        if e is None:
            raise ContainerError(f"unknown tensor {name!r}")
        out = np.empty(e.on_disk_bytes or e.size, np.uint8)
        self.read_into(name, out)
        return out


def record_name(layer: int, linear: int) -> str:
    return f"blk.{layer}.linear.{linear}.nvfp4"


def load_stack(container: Container, stack) -> int:
    """Fill a LayerStack's pinned arena from the container's NVFP4 records (no transcoding: the bytes
    on disk are the bytes the copy engine streams). Returns the bytes read."""
    total = 0
    names = [record_name(layer, j) for layer in range(stack.layers) for j in range(len(stack.linears))]
    for name in names[:2]:
        container.hint(name)
    for layer in range(stack.layers):
        for j, spec in enumerate(stack.linears):
            name = record_name(layer, j)
            ahead = layer * len(stack.linears) + j + 2
            if ahead < len(names):
                container.hint(names[ahead])  # the page-in of record i+2 runs under the copy of record i
            e = container.tensors.get(name)
            if e is None:
                raise ContainerError(f"unknown tensor {name!r}")
            if e.ggml_type != GGML_NVFP4_RECORD or e.shape != (spec.n, spec.k):
                raise ContainerError(f"{name}: {e.label} {e.shape}, the stack expects an NVFP4 record of {(spec.n, spec.k)}")
            total += container.read_into(name, stack.record_view(layer, j))
    return total


def pack_record(n: int, k: int, codes: np.ndarray, scales_device: np.ndarray, global_scale: float,
                bias_bf16: Optional[np.ndarray] = None) -> np.ndarray:
    """One linear as an NVFP4 record (the layout of tnf_stack_record_offsets)."""
    lib = L.load()
    rec = np.zeros(int(lib.tnf_stack_record_bytes(n, k)), np.uint8)
    offs = (C.c_uint64 * 4)()
    lib.tnf_stack_record_offsets(n, k, offs)
    oc, os_, ob, og = (int(v) for v in offs)
    c = np.ascontiguousarray(codes, np.uint8).ravel()
    s = np.ascontiguousarray(scales_device, np.uint8).ravel()
    rec[oc: oc + c.size] = c
    rec[os_: os_ + s.size] = s
    if bias_bf16 is not None:
        b = np.ascontiguousarray(bias_bf16, np.uint16).view(np.uint8).ravel()
        rec[ob: ob + b.size] = b
    rec[og: og + 4] = np.array([global_scale], np.float32).view(np.uint8)
    return rec


def transcode_linear(be, w_dense: np.ndarray, bias_bf16: Optional[np.ndarray] = None) -> np.ndarray:
    """Load-time transcode of one dense [N, K] weight (f32, or bf16 bits as uint16) to an NVFP4 record:
    the library's GPU quantiser + scale re-layout (the role of WeightMeta::transcode,
    thinfer-core/src/residency.rs:120-125, served by a GPU prep kernel as in weight_prep.rs)."""
    from .backend import Nvfp4Weight

    W = Nvfp4Weight.from_dense(be, w_dense, bias_bf16)
    rec = pack_record(W.n, W.k, be.read_buffer(W.codes), be.read_buffer(W.scales_device), W.global_scale, bias_bf16)
    W.free(be)
    return rec
