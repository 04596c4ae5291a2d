"""Multi-GPU arm of bench.py (launched by torchrun, one rank per GPU).

Workload: BASELINE configs[4], the batched Wan-5B-shaped FFN pair at M = 26520 —
up 3072 -> 14336 (+bias, tanh-GELU), down 14336 -> 3072 (+bias). Weights are split by OUTPUT
columns over the ranks (each rank holds its slices resident); every rank holds the full
activations and ends each linear with the full [M, N] output:
  --gather multimem (default when the node has NVSwitch multicast): each all-gather is fused into the kernel
                   that produces the data. Every rank quantises its own row block of x and stores codes + scales
                   through the multicast alias of a symmetric buffer; the up GEMM's epilogue stores its column window
                   of H (NVFP4 codes + scales) and the down GEMM's epilogue its window of y (bf16) the same way
                   (multimem.st), so the transfer runs under the math tile by tile and nothing is packed, gathered
                   or interleaved afterwards; one barrier of the ranks per stage;
  --gather fused : the GEMM epilogue stores each output tile into its own output buffer (TMA) and
                   into every peer's (16-byte vector stores through CUDA IPC windows), then a
                   stream-ordered barrier;
  --gather copy  : the linear runs in row bands; while band i+1 computes, the copy engines push
                   band i of the rank's column slice to every peer (one strided peer copy each);
  --gather nccl  : the GEMM writes its slice locally, then an NCCL all-gather of the slices;
  --gather nvfp4 : the MLP-up epilogue quantises its slice to NVFP4 (what the down projection consumes
                   anyway) and the all-gather moves codes + scales, 0.5625 B per element instead of 2;
                   the final output is gathered as bf16. Same result bits as --gather nccl;
  --gather push  : the same bytes as nvfp4, but each rank writes its slice packed and the copy engines push
                   finished row bands to every peer's receive area with contiguous copies while the next
                   band computes; one barrier and an interleave kernel per linear.
Strong scaling: total work is fixed as N grows. The output bytes every rank must receive
((G-1)/G * 2*M*N) do not shrink with G, so NVLink ingest, not the tensor pipe, bounds this scheme.
"""
from __future__ import annotations

import json
import os

import numpy as np


def run_multi_gpu(args):
    import torch
    import torch.distributed as dist

    import thinfer_b200 as T
    from bench import (ClockSampler, HIDDEN, NOMINAL_FP4_TFLOPS, WAN_FFN, WAN_M, as_torch, make_weight,
                       measured_peaks, workload_config)
    from thinfer_b200 import _lib as L
    from thinfer_b200.nsplit import NSplitGroup, column_partition

    import sys
    saved_stdout = os.dup(1)  # libraries (NCCL) print banners on stdout: keep it clean for the one JSON line
    os.dup2(2, 1)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device(f"cuda:{local}"))
    dev = f"cuda:{local}"
    be = T.Backend(local)
    sc = be.scope()
    grp = NSplitGroup(be, rank, world)
    M = WAN_M
    ffn = None
    want_multimem = args.gather in ("auto", "multimem")
    if args.gather == "auto":
        # without NVSwitch multicast; measured ms/step at 2 / 4 / 8 ranks: push 1.04-1.17 / 1.05-1.13 / 1.19-2.27 (noisy with 7 peers), nvfp4 (NCCL)
        # 1.32 / 1.09 / 0.98-1.29, fused 1.20 / 4.3 / -, nccl (bf16) 2.2 / 2.15 / 2.12, copy (strided) 1.34 / 2.27 / 4.35
        args.gather = "push" if world <= 4 else "nvfp4"
    gen = torch.Generator(device=dev)
    gen.manual_seed(0xC5)  # same seed on every rank: identical full tensors, each rank keeps its slice

    def sliced_weight(n, k):
        # generate the rank's slice only; the per-tensor scale of a slice stands for the full tensor's
        off, width = column_partition(n, world)[rank]
        g = torch.Generator(device=dev)
        g.manual_seed(0xC500 + n + 31 * rank)
        return make_weight(be, T, L, g, width, k), off, width

    w_up, up_off, up_w = sliced_weight(WAN_FFN, HIDDEN)
    w_dn, dn_off, dn_w = sliced_weight(HIDDEN, WAN_FFN)
    x = be.allocate(M * HIDDEN * 2)
    h = be.allocate(M * WAN_FFN * 2)
    y = be.allocate(M * HIDDEN * 2)
    as_torch(be, x, torch.bfloat16, (M, HIDDEN)).copy_(torch.randn(M, HIDDEN, device=dev, generator=gen).to(torch.bfloat16))
    torch.cuda.synchronize()
    ga_x, ga_h = 0.0018, 0.0009765625  # calibrated static activation scales (N(0,1) input; GELU output)
    if want_multimem:
        from thinfer_b200.nsplit import MulticastFfn, row_partition
        try:
            ffn = MulticastFfn(grp, M, HIDDEN, WAN_FFN, w_up, w_dn, ga_x, ga_h)
            args.gather = "multimem"
        except RuntimeError as e:  # no multicast alias on this platform: the same answer on every rank
            if rank == 0:
                print(f"multimem unavailable ({e}); using --gather {args.gather}", file=sys.stderr)
            if args.gather == "multimem":
                raise
    if ffn is not None:
        my_row0, my_rows = row_partition(M, world)[rank]
        y_full = ffn.y.buf
    fused = args.gather == "fused"
    if fused or args.gather == "copy":
        grp.register_output(0, h)
        grp.register_output(1, y)
    from thinfer_b200._lib import Buf
    bands = args.bands
    band_rows = [((M * b // bands) + 255) // 256 * 256 if 0 < b < bands else (0 if b == 0 else M) for b in range(bands + 1)]
    compute = torch.cuda.ExternalStream(be.streams()[0], device=dev)
    from thinfer_b200.backend import device_scales_bytes
    hq_full_c = be.allocate(M * WAN_FFN // 2)
    hq_full_s = be.allocate(device_scales_bytes(M, WAN_FFN))
    hs_block = device_scales_bytes(128, WAN_FFN)  # bytes of one 128-row block of H's scales
    if args.gather == "push":
        from thinfer_b200.nsplit import PackedGather
        pg_h = PackedGather(grp, 2, M, WAN_FFN, "nvfp4")
        pg_y = PackedGather(grp, 3, M, HIDDEN, "bf16")

    marks = []  # (label, event) on the compute stream, filled when a breakdown pass asks for it

    def mark(label):
        if marks is not None and trace_on[0]:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record(compute)
            marks.append((label, ev))

    trace_on = [False]

    def step():
        mark("start")
        if ffn is not None:
            ffn.step(Buf(x.id, my_row0 * HIDDEN * 2, my_rows * HIDDEN * 2), mark)
        elif fused:
            sc.linear(x, M, w_up, ga_x, h, act=1, n_offset=up_off, ldo=WAN_FFN, flags=grp.scatter_flags(0))
            grp.barrier()
            sc.linear(h, M, w_dn, ga_h, y, n_offset=dn_off, ldo=HIDDEN, flags=grp.scatter_flags(1))
            grp.barrier()
        elif args.gather == "copy":
            # row bands: the GEMM of band i+1 runs while the copy engines push band i to the peers
            for (src, w, ga, dst, act, off, wd, ld, ws) in ((x, w_up, ga_x, h, 1, up_off, up_w, WAN_FFN, 0),
                                                            (h, w_dn, ga_h, y, 0, dn_off, dn_w, HIDDEN, 1)):
                k = w.k
                for b in range(bands):
                    r0, r1 = band_rows[b], band_rows[b + 1]
                    a_view = Buf(src.id, r0 * k * 2, (r1 - r0) * k * 2)
                    o_view = Buf(dst.id, r0 * ld * 2, (M - r0) * ld * 2)
                    sc.linear(a_view, r1 - r0, w, ga, o_view, act=act, n_offset=off, ldo=ld)
                    grp.scatter_rows(ws, dst, r0, r1 - r0, off, wd, ld)
                grp.wait_scatter()
                grp.barrier()
        elif args.gather == "push":
            # packed slices, contiguous copy-engine pushes band by band, one barrier + interleave per linear
            for b in range(bands):
                r0, rows = band_rows[b], band_rows[b + 1] - band_rows[b]
                sc.linear(Buf(x.id, r0 * HIDDEN * 2, rows * HIDDEN * 2), rows, w_up, ga_x, None, act=1,
                          out_nvfp4=(pg_h.send_main(r0, rows), pg_h.send_scales(r0, rows), ga_h))
                pg_h.push(r0, rows)
            mark("up bands")
            grp.wait_pushes()
            mark("H pushes done")
            grp.barrier()
            mark("barrier")
            pg_h.finish(hq_full_c, hq_full_s, sync=False)
            mark("H interleave")
            for b in range(bands):
                r0, rows = band_rows[b], band_rows[b + 1] - band_rows[b]
                sc.matmul(Buf(hq_full_c.id, r0 * WAN_FFN // 2, rows * WAN_FFN // 2),
                          Buf(hq_full_s.id, (r0 // 128) * hs_block, ((rows + 127) // 128) * hs_block), rows, w_dn, ga_h,
                          pg_y.send_main(r0, rows))
                pg_y.push(r0, rows)
            mark("down bands")
            grp.wait_pushes()
            mark("y pushes done")
            grp.barrier()
            mark("barrier")
            pg_y.finish(y, sync=False)
            mark("y interleave")
        elif args.gather == "nvfp4":
            sc.linear(x, M, w_up, ga_x, None, act=1, n_offset=up_off, ldo=WAN_FFN, out_nvfp4=(hq_full_c, hq_full_s, ga_h))
            grp.all_gather_nvfp4(hq_full_c, hq_full_s, M, WAN_FFN)
            sc.matmul(hq_full_c, hq_full_s, M, w_dn, ga_h, y, n_offset=dn_off, ldo=HIDDEN)
            grp.all_gather_cols(y, M, HIDDEN)
        else:
            sc.linear(x, M, w_up, ga_x, h, act=1, n_offset=up_off, ldo=WAN_FFN)
            grp.all_gather_cols(h, M, WAN_FFN)
            sc.linear(h, M, w_dn, ga_h, y, n_offset=dn_off, ldo=HIDDEN)
            grp.all_gather_cols(y, M, HIDDEN)

    def compute_only():  # same kernels, no delivery to peers (for the breakdown)
        if ffn is not None:
            ffn.step(Buf(x.id, my_row0 * HIDDEN * 2, my_rows * HIDDEN * 2), multicast=False)
            return
        sc.linear(x, M, w_up, ga_x, h, act=1, n_offset=up_off, ldo=WAN_FFN)
        sc.linear(h, M, w_dn, ga_h, y, n_offset=dn_off, ldo=HIDDEN)

    def timed(fn, n):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        dist.barrier()
        torch.cuda.synchronize()
        e0.record(compute)
        for _ in range(n):
            fn()
        e1.record(compute)
        be.submit()
        torch.cuda.synchronize()
        dist.barrier()
        t = torch.tensor([e0.elapsed_time(e1) / n], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)  # max over ranks
        return float(t.item())

    for _ in range(max(args.warmup, 3)):
        step()
    be.submit()
    # The timed region: `repeats` passes of exactly --steps steps, enough of them for about half a second of device
    # time, so that the clocks are those of a loaded GPU and the clock sampler sees it; the line reports the median
    # pass (ms_per_step) with the fastest and slowest beside it.
    probe_ms = timed(step, max(2, min(args.steps, 5)))
    repeats = int(min(200, max(3, np.ceil(500.0 / max(probe_ms * args.steps, 1e-3)))))
    sampler = ClockSampler(local) if rank == 0 else None
    passes = [timed(step, args.steps) for _ in range(repeats)]
    clocks = sampler.stop() if sampler else None
    ms = float(np.median(passes))
    breakdown = None
    if ffn is not None or os.environ.get("TNF_BENCH_BREAKDOWN"):  # one more step with an event after every stage (rank 0's view)
        dist.barrier()
        trace_on[0] = True
        step()
        trace_on[0] = False
        be.submit()
        torch.cuda.synchronize()
        breakdown = [(b[0], round(a[1].elapsed_time(b[1]), 4)) for a, b in zip(marks, marks[1:])]
    compute_only()  # grows the activation scratch on first use
    be.submit()
    ms_compute = timed(compute_only, max(2, min(args.steps, 5)))

    # ---- parity of the timed step's own outputs, on rank 0 (the only place this arm touches the oracle) ----
    parity = None
    if ffn is not None and not args.no_cpu:
        from bench import parity_entry, read_rows, sample_rows, weight_to_host
        step()
        be.submit()
        dist.barrier()
        mine = (weight_to_host(be, w_up), weight_to_host(be, w_dn))
        slices = [None] * world
        dist.gather_object(mine, slices if rank == 0 else None, dst=0)
        if rank == 0:
            import oracle as O
            try:
                O.set_num_threads(len(os.sched_getaffinity(0)))
            except AttributeError:
                pass
            rows = sample_rows(M)
            xr = read_rows(be, x, rows, HIDDEN * 2).reshape(len(rows), HIDDEN)
            h_codes = read_rows(be, ffn.hq_c.buf, rows, WAN_FFN // 2, np.uint8).reshape(len(rows), WAN_FFN // 2)
            dev_s = be.read_buffer(ffn.hq_s.buf)
            ka = ((WAN_FFN + 63) // 64 + 3) // 4 * 4
            r_, b_ = rows[:, None], np.arange(WAN_FFN // 16)[None, :]
            h_scales = dev_s[((r_ // 128) * ka + b_ // 4) * 512 + (r_ % 32) * 16 + ((r_ % 128) // 32) * 4 + (b_ % 4)]
            y_dev = read_rows(be, ffn.y.buf, rows, HIDDEN * 2).reshape(len(rows), HIDDEN)
            h_want = np.concatenate([O.linear(xr, ga_x, u[0], u[1], u[2], bias=u[3], act=1) for u, _ in slices], axis=1)
            hc_want, hs_want = O.quantize_act(h_want, ga_h)
            y_want = np.concatenate([O.linear_q(h_codes, h_scales, ga_h, d[0], d[1], d[2], bias=d[3]) for _, d in slices], axis=1)
            parity = {"tolerance": 1e-3, "sample": "256 rows (first, middle, last row tile) of rank 0's gathered H and y",
                      "h_codes_equal": float((h_codes == hc_want).mean()), "h_scales_equal": float((h_scales == hs_want).mean()),
                      "h_note": "device H against the oracle's up + GELU + quantiser; the tanh approximation flips a few codes",
                      "y": parity_entry(y_dev, y_want),
                      "y_note": "device y against the oracle's down projection on the device's own gathered NVFP4 H"}
            parity["ok"] = parity["y"]["rel_fro"] <= 1e-3 and parity["h_codes_equal"] > 0.99
        dist.barrier()

    # ---- the same work on ONE GPU (rank 0 alone, full weights, no exchange): the N = 1 time of this workload ----
    t1 = None
    if rank == 0:
        from bench import time_ffn_pair
        t1 = time_ffn_pair(be, M, HIDDEN, WAN_FFN)["ms"]
    dist.barrier()

    # ---- for comparison: the natural partition of this path, rows split over the ranks, no collective ----
    # every rank holds the full weights (2 x 24.8 MB) and computes its own M/G rows of both linears; the
    # MLP-up epilogue hands the down projection its NVFP4 operand directly
    gfull = torch.Generator(device=dev)
    gfull.manual_seed(0xC5AA)
    w_up_full = make_weight(be, T, L, gfull, WAN_FFN, HIDDEN)
    w_dn_full = make_weight(be, T, L, gfull, HIDDEN, WAN_FFN)
    r0 = (M * rank // world + 255) // 256 * 256 if rank else 0
    r1 = (M * (rank + 1) // world + 255) // 256 * 256 if rank + 1 < world else M
    mr = r1 - r0
    hq_c = be.allocate(mr * WAN_FFN // 2)
    hq_s = be.allocate(device_scales_bytes(mr, WAN_FFN))
    x_rows = Buf(x.id, r0 * HIDDEN * 2, mr * HIDDEN * 2)
    y_rows = Buf(y.id, r0 * HIDDEN * 2, mr * HIDDEN * 2)

    def step_msplit():
        sc.linear(x_rows, mr, w_up_full, ga_x, None, act=1, out_nvfp4=(hq_c, hq_s, ga_h))
        sc.matmul(hq_c, hq_s, mr, w_dn_full, ga_h, y_rows)

    for _ in range(3):
        step_msplit()
    be.submit()
    ms_msplit = timed(step_msplit, args.steps)

    # ---- end to end through the public API with host buffers ----
    # multimem: rank g takes only ITS row block of x from pinned host memory (the ranks exchange the quantised
    # operand over NVLink) and returns only its row block of the replicated y; other modes move the full x and y.
    # Double-buffered on the copy stream against the compute stream.
    from bench import _pinned, e2e_pipelined
    if ffn is not None:
        io_row0, io_rows, y_src = my_row0, max(my_rows, 1), ffn.y.buf
    else:
        io_row0, io_rows, y_src = 0, M, y
    nb_io = io_rows * HIDDEN * 2
    x_io = Buf(x.id, io_row0 * HIDDEN * 2, nb_io)
    y_io = Buf(y_src.id, y_src.offset + io_row0 * HIDDEN * 2, nb_io)
    hin, hout = [_pinned(be, nb_io) for _ in range(2)], [_pinned(be, nb_io) for _ in range(2)]
    x_host = as_torch(be, x, torch.int16, (M * HIDDEN,)).cpu().numpy().view(np.uint16)
    for hbuf in hin:
        hbuf["np"][:] = x_host[io_row0 * HIDDEN: (io_row0 + io_rows) * HIDDEN]
    x_stage, y_stage = [be.allocate(nb_io) for _ in range(2)], [be.allocate(nb_io) for _ in range(2)]
    n_e2e = max(2, args.steps)
    e2e_pipelined(be, step, x_io, y_io, nb_io, nb_io, hin, hout, x_stage, y_stage, 2)
    be.submit()
    import time as _time
    e2e_passes = []
    for _ in range(int(min(50, max(3, np.ceil(300.0 / max(ms * n_e2e, 1e-3)))))):
        torch.cuda.synchronize()
        dist.barrier()
        t_w = _time.perf_counter()
        e2e_pipelined(be, step, x_io, y_io, nb_io, nb_io, hin, hout, x_stage, y_stage, n_e2e)
        torch.cuda.synchronize()
        t_e = torch.tensor([(_time.perf_counter() - t_w) * 1e3 / n_e2e], device=dev)
        dist.all_reduce(t_e, op=dist.ReduceOp.MAX)  # host wall clock around uploads, steps and read-backs; max over ranks
        e2e_passes.append(float(t_e.item()))
    ms_e2e = float(np.median(e2e_passes))
    finite = all(bool(np.isfinite((hb["np"].astype(np.uint32) << 16).view(np.float32)).all()) for hb in hout)

    flops = 2.0 * M * HIDDEN * WAN_FFN * 2
    nvfp4_h = args.gather in ("nvfp4", "push", "multimem")
    out_bytes = (0.5625 if nvfp4_h else 2.0) * M * WAN_FFN + 2.0 * M * HIDDEN
    if ffn is not None:
        # the switch delivers every window to every rank, the sender included, and the quantised x travels too
        ingest = out_bytes + 0.5625 * M * HIDDEN
    else:
        ingest = out_bytes * (world - 1) / world  # bytes every rank must receive per step
    if rank == 0:
        peaks = measured_peaks()
        t_link = ingest / 770e9 * 1e3  # measured peer-copy bandwidth per direction and GPU
        t_math = flops / world / (4.0 * peaks["bf16_sustained"] * 1e12) * 1e3
        launches = {"multimem": 5, "push": 3 * bands + 3, "nvfp4": 9, "nccl": 8, "fused": 4, "copy": 4 * bands}[args.gather]
        line = {
            "metric": "nvfp4_linear_tflops", "value": flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None,
            "dtype": "nvfp4 (e2m1 x ue4m3 block scales, f32 accumulate, bf16 in/out)",
            "data": "synthetic (seeded torch.randn on device: weights N(0,0.02) quantised by the library, activations N(0,1) bf16)",
            "config": dict(workload_config(world), gather=args.gather,
                           note="--gpus 1 of this script is ANOTHER workload (the 60-layer block-linear stack, scaling 'weak'); "
                                "this workload's N = 1 time is t1_same_workload_ms, measured on rank 0 alone in this run"),
            "repeats": repeats, "ms_per_step_min": float(np.min(passes)), "ms_per_step_max": float(np.max(passes)),
            "timed_region_s": float(np.sum(passes)) * args.steps * 1e-3,
            "t1_same_workload_ms": t1, "strong_efficiency": t1 / (world * ms),
            "ms_compute_only": ms_compute, "ms_gather_exposed": ms - ms_compute,
            "ingest_bytes_per_rank": ingest, "nvlink_gbs_per_rank": ingest / (ms * 1e-3) / 1e9,
            "roofline": {"bound": "nvlink" if t_link > t_math else "tensor", "achieved": ingest / (ms * 1e-3) / 1e9,
                         "peak": 770.0, "unit": "GB/s", "frac": max(t_link, t_math) / ms,
                         "target_ms": max(t_link, t_math), "t_link_ms": t_link, "t_math_ms": t_math, "traffic": None,
                         "note": "target = slower of (FLOPs / 4x measured sustained bf16) and (bytes every rank receives / measured 770 GB/s peer copy)"},
            "clocks": clocks, "parity": parity,
            "e2e": {"value": flops / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_e2e,
                    "h2d_bytes_per_step": nb_io * world, "d2h_bytes_per_step": nb_io * world,
                    "h2d_bytes_per_step_per_rank": nb_io, "d2h_bytes_per_step_per_rank": nb_io,
                    "passes": len(e2e_passes), "output_finite": finite},
            # this library's kernels per step. multimem: activation quantiser, two multicast copies (codes, scales),
            # two GEMMs (the barriers are torch's); the others: quantiser + GEMM per band and linear, pack / unpack / interleave
            "gpu_launches": args.steps * launches,
            "breakdown_ms": breakdown,
            "m_split_no_collective": {"ms_per_step": ms_msplit, "value": flops / (ms_msplit * 1e-3) / 1e12, "unit": "TFLOP/s",
                                      "note": "same FFN pair with ROWS split over the ranks (full weights per rank, no exchange): "
                                              "the partition this path shards on naturally; reported beside the mandated N-split"},
            "frac_of_nominal_fp4": flops / (ms * 1e-3) / 1e12 / (NOMINAL_FP4_TFLOPS * world),
        }
        sys.stdout.flush()
        os.dup2(saved_stdout, 1)
        print(json.dumps(line), flush=True)
        os.dup2(2, 1)
    be.submit()
    dist.barrier()
    if ffn is not None:
        ffn.free()
    be.close()
    dist.destroy_process_group()
