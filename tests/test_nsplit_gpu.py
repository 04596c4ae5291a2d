"""N-split on real GPUs (2 ranks, one process per GPU): the fused peer-store epilogue, the copy-engine
deliveries (strided bands, packed pushes) and the NCCL all-gathers (bf16, NVFP4) must all reproduce the
unsplit result. Skipped when fewer than 2 GPUs are visible."""
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


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
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device(f"cuda:{rank}"))
    import oracle as O
    import thinfer_b200 as T
    from thinfer_b200.nsplit import NSplitGroup, column_partition

    m, n, k = 300, 1024, 512
    a = O.f32_to_bf16(O.gaussian(m * k, 1).reshape(m, k))
    w = (O.gaussian(n * k, 2) * np.float32(0.03)).reshape(n, k)
    bias = O.f32_to_bf16(O.gaussian(n, 3) * np.float32(0.01))
    wc, ws, gw = O.quantize_weight(w)
    ga = O.global_scale(O.amax_bf16(a))
    want = O.linear(a, ga, wc, ws, gw, bias=bias, act=1)
    be = T.Backend(rank)
    grp = NSplitGroup(be, rank, world)
    off, width = column_partition(n, world)[rank]
    W = T.Nvfp4Weight.from_packed(be, wc[off:off + width], ws[off:off + width], gw, bias[off:off + width])
    abuf = be.upload(a)
    ok = True
    for mode in ("fused", "copy", "nccl"):
        out = be.allocate(m * n * 2)
        be.write_buffer(out, np.full(m * n, 0x7FC0, np.uint16))
        be.submit()
        dist.barrier()
        sc = be.scope()
        if mode == "fused":
            grp.register_output(0, out)
            sc.linear(abuf, m, W, ga, out, act=1, n_offset=off, ldo=n, flags=grp.scatter_flags(0))
            grp.barrier()
        elif mode == "copy":  # two row bands pushed by the copy engines
            from thinfer_b200._lib import Buf
            grp.register_output(1, out)
            for r0, r1 in ((0, 256), (256, m)):
                sc.linear(Buf(abuf.id, r0 * k * 2, (r1 - r0) * k * 2), r1 - r0, W, ga, Buf(out.id, r0 * n * 2, (m - r0) * n * 2),
                          act=1, n_offset=off, ldo=n)
                grp.scatter_rows(1, out, r0, r1 - r0, off, width, n)
            grp.wait_scatter()
            grp.barrier()
        else:
            sc.linear(abuf, m, W, ga, out, act=1, n_offset=off, ldo=n)
            grp.all_gather_cols(out, m, n)
        be.submit(30000)
        dist.barrier()
        got = be.read_buffer(out, np.uint16).reshape(m, n)
        g, e = O.bf16_to_f32(got).astype(np.float64), O.bf16_to_f32(want).astype(np.float64)
        err = np.linalg.norm(g - e) / np.linalg.norm(e)
        ok = ok and bool(err <= 1e-3) and not np.isnan(g).any()
        dist.barrier()
    # NVFP4 gather: every rank's epilogue quantises its window; codes + scales are gathered; the gathered
    # operand must hold the bits the whole (unsplit) linear leaves on one GPU
    from thinfer_b200.backend import device_scales_bytes
    sc = be.scope()
    g_mid = 0.0009765625
    qc, qs = be.allocate(m * n // 2), be.allocate(device_scales_bytes(m, n))
    be.write_buffer(qs, np.zeros(qs.len, np.uint8))
    sc.linear(abuf, m, W, ga, None, act=1, n_offset=off, ldo=n, out_nvfp4=(qc, qs, g_mid))
    grp.all_gather_nvfp4(qc, qs, m, n)
    whole = T.Nvfp4Weight.from_packed(be, wc, ws, gw, bias)
    qc0, qs0 = be.allocate(m * n // 2), be.allocate(device_scales_bytes(m, n))
    be.write_buffer(qs0, np.zeros(qs0.len, np.uint8))
    sc.linear(abuf, m, whole, ga, None, act=1, out_nvfp4=(qc0, qs0, g_mid))
    be.submit(30000)
    ok = ok and np.array_equal(be.read_buffer(qc), be.read_buffer(qc0)) and np.array_equal(be.read_buffer(qs), be.read_buffer(qs0))
    dist.barrier()
    # packed slices pushed by the copy engines in two row bands, then interleaved: bf16 and NVFP4 outputs
    from thinfer_b200._lib import Buf
    from thinfer_b200.nsplit import PackedGather
    pg_b, pg_q = PackedGather(grp, 2, m, n, "bf16"), PackedGather(grp, 3, m, n, "nvfp4")
    out_p = be.allocate(m * n * 2)
    qc2, qs2 = be.allocate(m * n // 2), be.allocate(device_scales_bytes(m, n))
    be.write_buffer(qs2, np.zeros(qs2.len, np.uint8))
    be.write_buffer(pg_q.send, np.zeros(pg_q.send.len, np.uint8))
    be.submit()
    dist.barrier()
    for r0, r1 in ((0, 256), (256, m)):
        a_view = Buf(abuf.id, r0 * k * 2, (r1 - r0) * k * 2)
        sc.linear(a_view, r1 - r0, W, ga, pg_b.send_main(r0, r1 - r0), act=1)
        pg_b.push(r0, r1 - r0)
        sc.linear(a_view, r1 - r0, W, ga, None, act=1, out_nvfp4=(pg_q.send_main(r0, r1 - r0), pg_q.send_scales(r0, r1 - r0), g_mid))
        pg_q.push(r0, r1 - r0)
    pg_b.finish(out_p)
    pg_q.finish(qc2, qs2)
    be.submit(30000)
    got = O.bf16_to_f32(be.read_buffer(out_p, np.uint16).reshape(m, n)).astype(np.float64)
    e = O.bf16_to_f32(want).astype(np.float64)
    ok = ok and bool(np.linalg.norm(got - e) / np.linalg.norm(e) <= 1e-3)
    ok = ok and np.array_equal(be.read_buffer(qc2), be.read_buffer(qc0)) and np.array_equal(be.read_buffer(qs2), be.read_buffer(qs0))
    dist.barrier()
    t = torch.tensor([1 if ok else 0], device=f"cuda:{rank}")
    dist.all_reduce(t)
    if rank == 0:
        ret.put(int(t.item()))
    be.submit()
    dist.barrier()  # no rank leaves while a peer may still hold its windows
    be.close()
    dist.destroy_process_group()


def _worker_multicast(rank, world, port, ret):
    """The FFN pair with the all-gathers fused into the producing kernels (multicast stores through NVSwitch).
    Slices are large enough for the CTA-pair kernel to run several tiles per pair. Every rank must end with the
    bits the unsplit pair leaves on one GPU: H codes and scales, and y."""
    import torch
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device(f"cuda:{rank}"))
    import oracle as O
    import thinfer_b200 as T
    from thinfer_b200._lib import Buf
    from thinfer_b200.backend import device_scales_bytes
    from thinfer_b200.nsplit import MulticastFfn, NSplitGroup, column_partition, row_partition

    m, hidden, ffn = 2350, 512, 4608  # ragged rows; per-rank slices of 2304 and 256 columns
    x = O.f32_to_bf16(O.gaussian(m * hidden, 11).reshape(m, hidden))
    w1 = (O.gaussian(ffn * hidden, 12) * np.float32(0.03)).reshape(ffn, hidden)
    w2 = (O.gaussian(hidden * ffn, 13) * np.float32(0.03)).reshape(hidden, ffn)
    b1 = O.f32_to_bf16(O.gaussian(ffn, 14) * np.float32(0.01))
    b2 = O.f32_to_bf16(O.gaussian(hidden, 15) * np.float32(0.01))
    w1c, w1s, g1 = O.quantize_weight(w1)
    w2c, w2s, g2 = O.quantize_weight(w2)
    ga_x, ga_h = O.global_scale(O.amax_bf16(x)), 0.0009765625
    be = T.Backend(rank)
    grp = NSplitGroup(be, rank, world)
    uo, uw = column_partition(ffn, world)[rank]
    do, dw = column_partition(hidden, world)[rank]
    W1 = T.Nvfp4Weight.from_packed(be, w1c[uo:uo + uw], w1s[uo:uo + uw], g1, b1[uo:uo + uw])
    W2 = T.Nvfp4Weight.from_packed(be, w2c[do:do + dw], w2s[do:do + dw], g2, b2[do:do + dw])
    ok = True
    try:
        pair = MulticastFfn(grp, m, hidden, ffn, W1, W2, ga_x, ga_h)
    except RuntimeError:
        pair = None  # no multicast alias on this platform: nothing to test (every rank sees the same)
    if pair is not None:
        r0, rows = row_partition(m, world)[rank]
        xb = be.upload(x[r0:r0 + rows])
        for _ in range(2):  # twice: the second pass overwrites what the first delivered
            pair.step(Buf(xb.id, 0, rows * hidden * 2))
        be.submit(30000)
        dist.barrier()
        # the unsplit pair on this GPU
        whole1 = T.Nvfp4Weight.from_packed(be, w1c, w1s, g1, b1)
        whole2 = T.Nvfp4Weight.from_packed(be, w2c, w2s, g2, b2)
        xf = be.upload(x)
        qc, qs = be.allocate(m * ffn // 2), be.allocate(device_scales_bytes(m, ffn))
        be.write_buffer(qs, np.zeros(qs.len, np.uint8))
        yb = be.allocate(m * hidden * 2)
        sc = be.scope()
        sc.linear(xf, m, whole1, ga_x, None, act=1, out_nvfp4=(qc, qs, ga_h))
        sc.matmul(qc, qs, m, whole2, ga_h, yb)
        be.submit(30000)
        ok = ok and np.array_equal(be.read_buffer(pair.hq_c.buf), be.read_buffer(qc))
        ok = ok and np.array_equal(be.read_buffer(pair.hq_s.buf), be.read_buffer(qs))
        y_got, y_one = be.read_buffer(pair.y.buf, np.uint16), be.read_buffer(yb, np.uint16)
        ok = ok and np.array_equal(y_got, y_one)
        # and against the oracle: down projection on the gathered H
        from conftest import dev_scales_to_canonical
        hc = be.read_buffer(pair.hq_c.buf).reshape(m, ffn // 2)
        hs = dev_scales_to_canonical(be.read_buffer(pair.hq_s.buf), m, ffn)
        want = O.linear_q(hc, hs, ga_h, w2c, w2s, g2, bias=b2)
        g, e = O.bf16_to_f32(y_got.reshape(m, hidden)).astype(np.float64), O.bf16_to_f32(want).astype(np.float64)
        ok = ok and bool(np.linalg.norm(g - e) / np.linalg.norm(e) <= 1e-3)
    dist.barrier()
    t = torch.tensor([1 if ok else 0, 0 if pair is None else 1], device=f"cuda:{rank}")
    dist.all_reduce(t)
    if rank == 0:
        ret.put((int(t[0].item()), int(t[1].item())))
    be.submit()
    dist.barrier()  # no rank leaves while a peer may still write into its buffers
    if pair is not None:
        pair.free()
    be.close()
    dist.destroy_process_group()


def _run_two(worker):
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=worker, args=(r, 2, port, ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
        assert p.exitcode == 0
    return ret.get(timeout=5)


def test_two_gpu_multicast_ffn_pair():
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    ok, ran = _run_two(_worker_multicast)
    assert ok == 2
    if ran == 0:
        pytest.skip("the platform has no NVSwitch multicast alias for symmetric allocations")


def test_two_gpu_scatter_and_gather():
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(240)
        assert p.exitcode == 0
    assert ret.get(timeout=5) == 2
