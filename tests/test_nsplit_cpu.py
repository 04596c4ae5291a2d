"""N-split host logic on CPU ranks (gloo, world_size 2): partition arithmetic, the byte exchange used
for IPC handles / the NCCL id, and the gather emulated with the oracle as each rank's compute."""
import os
import socket

import numpy as np
import pytest
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, ret):
    import torch
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import oracle as O
    from thinfer_b200.nsplit import all_gather_bytes, column_partition

    m, n, k = 24, 64, 96
    a = O.f32_to_bf16(O.gaussian(m * k, 1).reshape(m, k))
    w = (O.gaussian(n * k, 2) * np.float32(0.05)).reshape(n, k)
    wc, ws, gw = O.quantize_weight(w)  # per-tensor scale of the FULL weight, shared by all slices
    ga = O.global_scale(O.amax_bf16(a))
    off, width = column_partition(n, world)[rank]
    mine = O.linear(a, ga, wc[off:off + width], ws[off:off + width], gw)  # this rank's column slice
    blobs = all_gather_bytes(mine.tobytes(), world)
    full = np.concatenate([np.frombuffer(b, np.uint16).reshape(m, -1) for b in blobs], axis=1)
    want = O.linear(a, ga, wc, ws, gw)
    ok = np.array_equal(full, want) and [len(b) for b in blobs] == [m * width * 2] * world
    t = torch.tensor([1 if ok else 0])
    dist.all_reduce(t)
    if rank == 0:
        ret.put(int(t.item()))
    dist.destroy_process_group()


def test_column_partition():
    from thinfer_b200.nsplit import column_partition

    assert column_partition(14336, 8) == [(g * 1792, 1792) for g in range(8)]
    assert column_partition(3072, 4)[3] == (2304, 768)
    with pytest.raises(ValueError):
        column_partition(3072 + 8, 8)


def test_two_rank_gather_matches_unsplit():
    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert ret.get(timeout=5) == 2


def test_row_partition_covers_rows_in_whole_scale_blocks():
    """Each rank quantises its own row block of the activations; blocks start on multiples of 128 rows (a scale
    atom of the device layout covers 128 rows), cover every row once and may leave the last ranks empty."""
    from thinfer_b200.nsplit import row_partition

    for m, world in [(26520, 1), (26520, 2), (26520, 4), (26520, 8), (2350, 2), (100, 4), (128, 8), (1, 2)]:
        parts = row_partition(m, world)
        assert len(parts) == world and sum(r for _, r in parts) == m
        nxt = 0
        for r0, rows in parts:
            assert r0 == nxt and r0 % 128 == 0 or rows == 0
            nxt = r0 + rows
        assert nxt == m
