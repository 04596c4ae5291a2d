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


def row_partition(m: int, world: int, align: int = 128) -> List[Tuple[int, int]]:
    """(row0, rows) of each rank's block of the activations: equal blocks of a multiple of `align` rows (a scale
    atom of the device layout covers 128 rows), the last one takes what is left (possibly nothing)."""
    per = ((m + world - 1) // world + align - 1) // align * align
    out = []
    for g in range(world):
        r0 = min(g * per, m)
        out.append((r0, min(per, m - r0)))
    return out


class SymmetricBuffer:
    """Device memory that exists with the same size on every rank of the node, plus its NVSwitch multicast
    alias: a store to the alias lands in every rank's copy at the same offset. The allocation and the exchange
    of handles between the processes are torch's (``torch.distributed._symmetric_memory``); the library only
    receives the two addresses (``tnf_import_symmetric``). Collective: every rank must create the same
    buffers in the same order."""

    def __init__(self, grp: NSplitGroup, nbytes: int, category: int = L.CAT_WORKSPACE, zero: bool = True):
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm

        be = grp.be
        self.grp = grp
        self.nbytes = (nbytes + 255) // 256 * 256
        self.tensor = symm.empty(self.nbytes, dtype=torch.uint8, device=f"cuda:{be.device}")
        if zero:
            self.tensor.zero_()
            torch.cuda.synchronize()
        self.handle = symm.rendezvous(self.tensor, dist.group.WORLD)
        self.multicast_ptr = int(self.handle.multicast_ptr or 0)
        bid = C.c_uint64()
        _check(be.lib.tnf_import_symmetric(be._ctx, C.c_void_p(self.tensor.data_ptr()), C.c_void_p(self.multicast_ptr),
                                           self.nbytes, category, C.byref(bid)))
        self.buf = Buf(bid.value, 0, nbytes)

    @property
    def has_multicast(self) -> bool:
        return self.multicast_ptr != 0

    def barrier(self, channel: int = 0) -> None:
        """Stream-ordered barrier of the ranks on the library's compute stream (signal pads of this buffer)."""
        import torch

        be = self.grp.be
        stream = torch.cuda.ExternalStream(be.streams()[0], device=f"cuda:{be.device}")
        with torch.cuda.stream(stream):
            self.handle.barrier(channel=channel)

    def free(self) -> None:
        if self.buf is not None:
            self.grp.be.free(self.buf)  # the library forgets the range; torch owns the memory
            self.buf = None


class MulticastFfn:
    """The N-split FFN pair (up + bias + GELU, down + bias) with each all-gather fused into the kernel that
    produces the data: rank g holds the column slices ``w_up`` [ffn/G, hidden] and ``w_dn`` [hidden/G, ffn];

      1. every rank quantises ITS row block of x and stores the codes and scales through the multicast alias,
         so that all ranks hold the whole NVFP4 operand (x is quantised once per step, not once per rank);
      2. the up GEMM's epilogue quantises its GELU output and stores its column window of H (codes + scales)
         through the multicast alias while the GEMM is still running;
      3. the down GEMM's epilogue does the same with its window of the bf16 output y.

    A barrier of the ranks follows each stage. Every rank ends with the full H (NVFP4) and the full y (bf16),
    which is what an all-gather after each linear would leave, bit for bit."""

    def __init__(self, grp: NSplitGroup, m: int, hidden: int, ffn: int, w_up, w_dn, ga_x: float, ga_h: float):
        from .backend import device_scales_bytes

        be = grp.be
        self.grp, self.m, self.hidden, self.ffn = grp, m, hidden, ffn
        self.w_up, self.w_dn, self.ga_x, self.ga_h = w_up, w_dn, ga_x, ga_h
        self.up_off, self.up_w = column_partition(ffn, grp.world)[grp.rank]
        self.dn_off, self.dn_w = column_partition(hidden, grp.world)[grp.rank]
        if self.up_w % 64 or self.up_off % 64:
            raise ValueError("the NVFP4 copy of H moves in whole 64-column groups: ffn / world must be a multiple of 64")
        self.row0, self.rows = row_partition(m, grp.world)[grp.rank]
        self.xq_c = SymmetricBuffer(grp, m * hidden // 2)
        self.xq_s = SymmetricBuffer(grp, device_scales_bytes(m, hidden))
        self.hq_c = SymmetricBuffer(grp, m * ffn // 2)
        self.hq_s = SymmetricBuffer(grp, device_scales_bytes(m, ffn))
        self.y = SymmetricBuffer(grp, m * hidden * 2)
        if not self.y.has_multicast:
            raise RuntimeError("this platform gave the symmetric allocation no multicast alias (no NVSwitch multicast)")
        self.x_scale_block = device_scales_bytes(128, hidden)  # bytes of one 128-row block of x's scales
        rows_cap = max(self.rows, 1)
        self.stage_c = be.allocate(max(rows_cap * hidden // 2, 256))
        self.stage_s = be.allocate(device_scales_bytes(rows_cap, hidden))

    def step(self, x_rows: Buf, mark=None, multicast: bool = True) -> None:
        """One pass. ``x_rows`` is this rank's row block of x (bf16 [rows, hidden], rows from ``row_partition``).
        ``mark(label)``, if given, is called after every stage has been queued (for event timing).
        ``multicast=False`` runs the same kernels with plain local stores and no barriers (each rank then only
        holds its own rows of x and its own column windows: for timing the arithmetic alone)."""
        be, lib, ctx = self.grp.be, self.grp.be.lib, self.grp.be._ctx
        sc = be.scope()
        mark = mark or (lambda label: None)
        flags = L.LINEAR_MULTICAST_OUT if multicast else 0
        if self.rows:
            nblk = (self.rows + 127) // 128
            c_bytes, s_bytes = self.rows * self.hidden // 2, nblk * self.x_scale_block
            c_off, s_off = self.row0 * self.hidden // 2, (self.row0 // 128) * self.x_scale_block
            if multicast:
                _check(lib.tnf_quantize_act(ctx, x_rows, self.rows, self.hidden, self.ga_x, L.SCALES_DEVICE, self.stage_c,
                                            self.stage_s, None))
                _check(lib.tnf_multicast_copy(ctx, Buf(self.stage_c.id, 0, c_bytes), self.xq_c.buf.id, c_off, c_bytes))
                _check(lib.tnf_multicast_copy(ctx, Buf(self.stage_s.id, 0, s_bytes), self.xq_s.buf.id, s_off, s_bytes))
            else:
                _check(lib.tnf_quantize_act(ctx, x_rows, self.rows, self.hidden, self.ga_x, L.SCALES_DEVICE,
                                            Buf(self.xq_c.buf.id, c_off, c_bytes), Buf(self.xq_s.buf.id, s_off, s_bytes), None))
        mark("quantise own rows of x" + (" + multicast" if multicast else ""))
        if multicast:
            self.y.barrier(0)
            mark("barrier")
        sc.matmul(self.xq_c.buf, self.xq_s.buf, self.m, self.w_up, self.ga_x, None, act=L.ACT_GELU_TANH, n_offset=self.up_off,
                  ldo=self.ffn, flags=flags, out_nvfp4=(self.hq_c.buf, self.hq_s.buf, self.ga_h))
        mark("up + GELU -> H (NVFP4)" + (", multicast" if multicast else ""))
        if multicast:
            self.y.barrier(1)
            mark("barrier")
        sc.matmul(self.hq_c.buf, self.hq_s.buf, self.m, self.w_dn, self.ga_h, self.y.buf, n_offset=self.dn_off, ldo=self.hidden,
                  flags=flags)
        mark("down -> y (bf16)" + (", multicast" if multicast else ""))
        if multicast:
            self.y.barrier(0)
            mark("barrier")

    def free(self) -> None:
        for b in (self.xq_c, self.xq_s, self.hq_c, self.hq_s, self.y):
            b.free()
        for b in (self.stage_c, self.stage_s):
            self.grp.be.free(b)
