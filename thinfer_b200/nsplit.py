"""Column-parallel (N-split) execution of a linear over the ranks of one node.

The reference is single-device; this is the partition the benchmark configuration adds:
rank g keeps W[g*N/G:(g+1)*N/G, :] resident, computes out[:, slice] and the slices reach
every rank in one of several ways: packed slices pushed by the copy engines into every peer's
receive area and interleaved there (``PackedGather``), an NCCL all-gather of bf16 columns or of
the NVFP4 copy the epilogue made, the GEMM epilogue's own stores into the peers' output buffers
(opened over CUDA IPC), or strided copy-engine bands. ``torch.distributed`` is only the
plumbing that passes handles and the NCCL id around.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Tuple

from . import _lib as L
from .backend import Backend, Buf, _check


def column_partition(n: int, world: int) -> List[Tuple[int, int]]:
    """(offset, width) of each rank's output columns: equal widths, multiples of 8 (16-byte rows of bf16)."""
    if world < 1 or n % world or (n // world) % 8:
        raise ValueError(f"n={n} does not split into {world} equal column slices of a multiple of 8")
    w = n // world
    return [(g * w, w) for g in range(world)]


def all_gather_bytes(blob: bytes, world: int) -> List[bytes]:
    """Every rank's blob, in rank order (gloo or nccl process group)."""
    import torch.distributed as dist

    out = [None] * world
    dist.all_gather_object(out, blob)
    return out


class NSplitGroup:
    """One rank's view of the group: NCCL communicator inside the library + peer windows."""

    def __init__(self, be: Backend, rank: int, world: int):
        self.be, self.rank, self.world = be, rank, world
        uid = C.create_string_buffer(128)
        if rank == 0:
            _check(be.lib.tnf_comm_unique_id(uid))
        uid_all = all_gather_bytes(bytes(uid.raw), world)
        _check(be.lib.tnf_comm_init(be._ctx, world, rank, C.create_string_buffer(uid_all[0], 128)))

    def register_output(self, window_set: int, buf: Buf) -> None:
        """Open every other rank's copy of `buf` (the same logical output on each rank) as peer window set."""
        h = C.create_string_buffer(64)
        _check(self.be.lib.tnf_ipc_export(self.be._ctx, buf.id, h))
        handles = all_gather_bytes(bytes(h.raw), self.world)
        peers = b"".join(hd for r, hd in enumerate(handles) if r != self.rank)
        _check(self.be.lib.tnf_peer_outputs(self.be._ctx, window_set, self.world - 1,
                                            C.create_string_buffer(peers, len(peers)) if peers else None))

    def scatter_flags(self, window_set: int) -> int:
        return L.LINEAR_SCATTER_PEERS | ((window_set & 3) << 8) if self.world > 1 else 0

    def scatter_rows(self, window_set: int, out: Buf, row0: int, rows: int, n_offset: int, n: int, ldo: int) -> None:
        """Copy-engine push of a finished row band of this rank's slice to every peer (asynchronous)."""
        if self.world > 1:
            _check(self.be.lib.tnf_scatter_rows(self.be._ctx, window_set, out, row0, rows, n_offset, n, ldo))

    def wait_scatter(self) -> None:
        """Compute stream waits for the pushes queued so far; follow with ``barrier``."""
        _check(self.be.lib.tnf_compute_after_copy(self.be._ctx))

    def wait_pushes(self) -> None:
        """Compute stream waits for the ``push_peers`` copies queued so far (not for host uploads or read-backs)."""
        _check(self.be.lib.tnf_compute_after_push(self.be._ctx))

    def barrier(self) -> None:
        """Stream-ordered: later work on the compute stream starts after every rank got here."""
        _check(self.be.lib.tnf_comm_barrier(self.be._ctx))

    def all_gather_cols(self, out: Buf, m: int, n_total: int) -> None:
        _check(self.be.lib.tnf_all_gather_cols(self.be._ctx, out, m, n_total, n_total // self.world))

    def all_gather_nvfp4(self, codes: Buf, scales_device: Buf, m: int, n_total: int) -> None:
        """Gather an output the epilogue left in NVFP4 (codes + device-layout scales), 0.5625 B per element."""
        _check(self.be.lib.tnf_all_gather_nvfp4(self.be._ctx, codes, scales_device, m, n_total, n_total // self.world))

    def push_peers(self, window_set: int, src: Buf, dst_offset: int, self_dst: Buf) -> None:
        """Copy-engine push of a contiguous range to the same offset of every peer's receive area."""
        _check(self.be.lib.tnf_push_peers(self.be._ctx, window_set, src, dst_offset, self_dst))


class PackedGather:
    """One N-split output delivered by contiguous copy-engine pushes.

    The linear writes this rank's column slice PACKED into ``send`` (ldo = n_local); finished row
    bands are pushed to slot ``rank`` of every rank's receive area while the next band computes;
    ``finish`` waits, meets the other ranks and lays the slots side by side in the full output.
    ``kind`` is "bf16" (rows of n_local bf16) or "nvfp4" (rows of n_local/2 code bytes plus the
    device-layout scales of the [m, n_local] operand).
    """

    def __init__(self, grp: NSplitGroup, window_set: int, m: int, n_total: int, kind: str = "bf16"):
        from .backend import device_scales_bytes

        be = grp.be
        self.grp, self.set, self.m, self.n_total, self.kind = grp, window_set, m, n_total, kind
        self.n_local = n_total // grp.world
        if n_total % grp.world or self.n_local % (64 if kind == "nvfp4" else 8):
            raise ValueError(f"n={n_total} does not split into {grp.world} slices of whole 16-byte groups")
        self.row_bytes = self.n_local // 2 if kind == "nvfp4" else self.n_local * 2
        self.main_bytes = m * self.row_bytes
        self.main_cap = (self.main_bytes + 255) // 256 * 256
        self.scale_bytes = device_scales_bytes(m, self.n_local) if kind == "nvfp4" else 0
        self.scale_block = self.scale_bytes // ((m + 127) // 128) if kind == "nvfp4" else 0  # bytes per 128-row block
        self.slot = self.main_cap + (self.scale_bytes + 255) // 256 * 256
        self.send = be.allocate(self.slot)
        self.recv = be.allocate(self.slot * grp.world)
        grp.register_output(window_set, self.recv)

    # views of the packed slice for a row band (row0 a multiple of 128)
    def send_main(self, row0: int = 0, rows: int = 0) -> Buf:
        rows = rows or self.m - row0
        return Buf(self.send.id, self.send.offset + row0 * self.row_bytes, rows * self.row_bytes)

    def send_scales(self, row0: int = 0, rows: int = 0) -> Buf:
        rows = rows or self.m - row0
        return Buf(self.send.id, self.send.offset + self.main_cap + (row0 // 128) * self.scale_block,
                   ((rows + 127) // 128) * self.scale_block)

    def push(self, row0: int = 0, rows: int = 0) -> None:
        """Queue the delivery of a finished row band (after the compute work queued so far)."""
        base = self.grp.rank * self.slot
        parts = [self.send_main(row0, rows)] + ([self.send_scales(row0, rows)] if self.kind == "nvfp4" else [])
        for v in parts:
            off = base + (v.offset - self.send.offset)
            self.grp.push_peers(self.set, v, off, Buf(self.recv.id, self.recv.offset + off, v.len))

    def finish(self, out: Buf, out_scales: Buf = None, sync: bool = True) -> None:
        """Wait for the pushes, meet the other ranks (``sync=False``: the caller already did both),
        interleave the slots into the full output."""
        g, lib, ctx = self.grp, self.grp.be.lib, self.grp.be._ctx
        if sync:
            g.wait_pushes()
            g.barrier()
        _check(lib.tnf_interleave_cols(ctx, self.recv, self.slot, self.row_bytes, g.world, out, self.row_bytes * g.world,
                                       self.m, self.row_bytes))
        if self.kind == "nvfp4":
            k_atoms = ((self.n_total // 64) + 3) // 4 * 4
            src = Buf(self.recv.id, self.recv.offset + self.main_cap, self.recv.len - self.main_cap)
            _check(lib.tnf_interleave_cols(ctx, src, self.slot, self.scale_block, g.world, out_scales, k_atoms * 512,
                                           (self.m + 127) // 128, (self.n_local // 64) * 512))
