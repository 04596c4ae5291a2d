"""Column-parallel (N-split) execution of a linear over the ranks of one node.

The reference is single-device; this is the partition the benchmark configuration adds:
rank g keeps W[g*N/G:(g+1)*N/G, :] resident, computes out[:, slice] and the slices reach
every rank either through the GEMM epilogue itself (TMA stores into the peers' output
buffers, opened over CUDA IPC) or through an NCCL all-gather. ``torch.distributed`` is only
the plumbing that passes handles and the NCCL id around.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Sequence, Tuple

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

    def barrier(self) -> None:
        """Stream-ordered: later work on the compute stream starts after every rank got here."""
        _check(self.be.lib.tnf_comm_barrier(self.be._ctx))

    def all_gather_cols(self, out: Buf, m: int, n_total: int) -> None:
        _check(self.be.lib.tnf_all_gather_cols(self.be._ctx, out, m, n_total, n_total // self.world))

    def all_gather_nvfp4(self, codes: Buf, scales_device: Buf, m: int, n_total: int) -> None:
        """Gather an output the epilogue left in NVFP4 (codes + device-layout scales), 0.5625 B per element."""
        _check(self.be.lib.tnf_all_gather_nvfp4(self.be._ctx, codes, scales_device, m, n_total, n_total // self.world))
