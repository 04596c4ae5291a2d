"""Host side of the streaming layer stack (``tnf_stack_*`` in the C ABI).

Mirrors what the reference's models do around ``WeightResidency``: register every linear of
every block (thinfer-models/src/common/loader.rs), choose what stays resident
(``set_pin_plan``, thinfer-core/src/residency.rs:440-457), then run the block loop that
overlaps block i's GEMMs with the upload of the following blocks
(thinfer-models/src/qwen_image/dit.rs:1052-1180). Here the weights wait in one pinned host
arena as fixed-size records and the C++ driver does the ring / event bookkeeping.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np

from . import _lib as L
from .backend import Backend, Buf, _check


@dataclass
class StackLinearSpec:
    """One linear of the layer: out = act(x @ W^T + b)."""
    n: int
    k: int
    act: int = L.ACT_NONE
    has_bias: bool = True
    input: int = 0      # 0 layer input, 1 previous linear's output, 2 the stream's auxiliary input
    stream_id: int = 0


def scales_to_device_layout(scales: np.ndarray) -> np.ndarray:
    """Canonical [rows, k/16] E4M3 scales -> the 128x4 tiled device layout (numpy, for packing records)."""
    rows, nb = scales.shape
    k_atoms = ((nb + 3) // 4 + 3) // 4 * 4
    out = np.zeros(((rows + 127) // 128) * k_atoms * 512, np.uint8)
    r = np.arange(rows)[:, None]
    b = np.arange(nb)[None, :]
    off = ((r // 128) * k_atoms + b // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + (b % 4)
    out[off] = scales
    return out


def record_bytes(n: int, k: int) -> int:
    return int(L.load().tnf_stack_record_bytes(n, k))


def record_offsets(n: int, k: int):
    out = (C.c_uint64 * 4)()
    L.load().tnf_stack_record_offsets(n, k, out)
    return [int(v) for v in out]


class HostArena:
    """Pinned host memory owned by the context (``tnf_host_register`` with a NULL pointer)."""

    def __init__(self, be: Backend, nbytes: int):
        self.be = be
        hid = C.c_uint64()
        _check(be.lib.tnf_host_register(be._ctx, None, nbytes, C.byref(hid)))
        self.id = hid.value
        p = C.c_void_p()
        _check(be.lib.tnf_host_ptr(be._ctx, self.id, C.byref(p), None))
        self.ptr = int(p.value)
        self.nbytes = nbytes
        self.np = np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_uint8)), shape=(nbytes,))

    def release(self) -> None:
        if self.id:
            self.np = None
            _check(self.be.lib.tnf_host_release(self.be._ctx, self.id))
            self.id = 0


class LayerStack:
    """`layers` x `linears` NVFP4 weights in a pinned arena, streamed under `weight_budget` bytes."""

    def __init__(self, be: Backend, layers: int, linears: Sequence[StackLinearSpec], m_rows: Sequence[int], hidden: int):
        self.be, self.layers, self.linears = be, layers, list(linears)
        self.m_rows, self.hidden = list(m_rows), hidden
        self.rec_bytes = [record_bytes(s.n, s.k) for s in self.linears]
        self.rec_offs = [record_offsets(s.n, s.k) for s in self.linears]
        self.layer_bytes = sum(self.rec_bytes)
        self.arena = HostArena(be, self.layer_bytes * layers)
        self._stack = C.c_void_p()

    # -- packing ------------------------------------------------------------------------------
    def record_view(self, layer: int, j: int) -> np.ndarray:
        off = layer * self.layer_bytes + sum(self.rec_bytes[:j])
        return self.arena.np[off: off + self.rec_bytes[j]]

    def pack(self, layer: int, j: int, codes: np.ndarray, scales_device: np.ndarray, global_scale: float,
             bias_bf16: Optional[np.ndarray] = None) -> None:
        """Write one record: packed codes, device-layout scales, bias (bf16 bits) and the f32 scale."""
        rec = self.record_view(layer, j)
        oc, os_, ob, og = self.rec_offs[j]
        c = np.ascontiguousarray(codes, np.uint8).ravel()
        rec[oc: oc + c.size] = c
        s = np.ascontiguousarray(scales_device, np.uint8).ravel()
        rec[os_: os_ + s.size] = s
        if bias_bf16 is not None:
            b = np.ascontiguousarray(bias_bf16, np.uint16).view(np.uint8).ravel()
            rec[ob: ob + b.size] = b
        rec[og: og + 4] = np.array([global_scale], np.float32).view(np.uint8)

    # -- residency ----------------------------------------------------------------------------
    def build(self, weight_budget: int = 0, ring_slots: int = 0) -> dict:
        """Allocate resident buffers and rings under the budget; uploads the resident records."""
        arr = (L.StackLinear * len(self.linears))()
        for i, s in enumerate(self.linears):
            arr[i] = L.StackLinear(s.n, s.k, s.act, int(s.has_bias), s.input, s.stream_id)
        rows = (C.c_uint32 * len(self.m_rows))(*self.m_rows)
        _check(self.be.lib.tnf_stack_create(self.be._ctx, self.layers, len(self.linears), arr, len(self.m_rows), rows,
                                            self.hidden, self.arena.id, weight_budget, ring_slots, C.byref(self._stack)))
        return self.stats()

    def step(self, x: Sequence[Buf], out: Sequence[Buf], a_global: float, aux: Optional[Sequence[Buf]] = None) -> None:
        """One pass over all layers; asynchronous (call ``Backend.submit`` to wait)."""
        n = len(self.m_rows)
        xs = (C.c_uint64 * n)(*[b.id for b in x])
        os_ = (C.c_uint64 * n)(*[b.id for b in out])
        ax = (C.c_uint64 * n)(*[b.id for b in aux]) if aux is not None else None
        _check(self.be.lib.tnf_stack_step(self._stack, xs, ax, os_, a_global))

    def evict_all(self) -> None:
        """Phase eviction: free every weight buffer of the stack (``evict_all_and_free`` in the reference); the
        next ``step`` brings the weights back under what the budget then allows."""
        _check(self.be.lib.tnf_stack_evict_all(self._stack))

    def restore(self, weight_budget: int = 0) -> dict:
        """Re-plan and re-upload now (also undoes demotions made by the reclaim chain once memory is free)."""
        _check(self.be.lib.tnf_stack_restore(self._stack, weight_budget))
        return self.stats()

    def stats(self) -> dict:
        out = (C.c_uint64 * 6)()
        _check(self.be.lib.tnf_stack_stats(self._stack, out))
        keys = ["resident_bytes", "ring_bytes", "uploaded_last_step", "uploads_last_step", "resident_records", "streamed_records"]
        return dict(zip(keys, [int(v) for v in out]))

    def close(self) -> None:
        if self._stack:
            self.be.lib.tnf_stack_destroy(self._stack)
            self._stack = C.c_void_p()
        self.arena.release()
