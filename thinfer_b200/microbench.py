"""Times one NVFP4 linear shape through the C ABI (also the command the ncu captures run).

    python -m thinfer_b200.microbench --m 4352 --n 3072 --k 12288 [--act 1] [--iters 20]
                                      [--no-quant] [--flush-l2] [--out-nvfp4]

Prints one JSON line: average GEMM and activation-quantiser launch times (CUDA events on the
library's compute stream), TFLOP/s and the algorithmic bytes. Inputs are seeded random
operands; with --flush-l2 a 256 MB buffer is overwritten between iterations (untimed).
"""
from __future__ import annotations

import argparse
import ctypes as C
import json

import numpy as np


class _DevView:
    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


def _tview(be, buf, dtype, shape):
    import torch

    return torch.as_tensor(_DevView(be.device_ptr(buf), buf.len), device=f"cuda:{be.device}").view(dtype).view(*shape)


def random_weight(be, n, k, gen, sigma=0.02, bias=True):
    """N(0, sigma) weight generated on the device and quantised by the library."""
    import torch

    from . import _lib as L
    from .backend import Nvfp4Weight, _check, device_scales_bytes

    dev = f"cuda:{be.device}"
    src = be.allocate_in(n * k * 2, L.CAT_STAGING)
    _tview(be, src, torch.bfloat16, (n, k)).copy_((torch.randn(n, k, device=dev, generator=gen) * sigma).to(torch.bfloat16))
    torch.cuda.synchronize()
    codes = be.allocate_in(n * k // 2, L.CAT_WEIGHTS)
    canon = be.allocate_in(n * k // 16, L.CAT_STAGING)
    g = C.c_float()
    _check(be.lib.tnf_quantize_weight(be._ctx, src, L.DTYPE_BF16, n, k, codes, canon, C.byref(g)))
    devs = be.allocate_in(device_scales_bytes(n, k), L.CAT_WEIGHTS)
    _check(be.lib.tnf_prepare_scales(be._ctx, canon, n, k, devs))
    be.submit()
    be.free(src)
    be.free(canon)
    b = None
    if bias:
        b = be.allocate_in(n * 2, L.CAT_WEIGHTS)
        _tview(be, b, torch.bfloat16, (n,)).copy_((torch.randn(n, device=dev, generator=gen) * 0.01).to(torch.bfloat16))
        torch.cuda.synchronize()
    return Nvfp4Weight(n, k, codes, devs, float(g.value), b, None)


def run(m, n, k, act=0, iters=20, warmup=3, quant=True, flush_l2=False, device=0, out_nvfp4=False):
    import torch

    from . import Backend
    from . import _lib as L

    be = Backend(device)
    sc = be.scope()
    dev = f"cuda:{device}"
    torch.cuda.set_device(device)
    gen = torch.Generator(device=dev)
    gen.manual_seed(1234)
    W = random_weight(be, n, k, gen)
    a = be.allocate(m * k * 2)
    _tview(be, a, torch.bfloat16, (m, k)).copy_(torch.randn(m, k, device=dev, generator=gen).to(torch.bfloat16))
    out = be.allocate(m * n * 2)
    q_out = None
    if out_nvfp4:  # the epilogue also emits the result as the next linear's NVFP4 operand
        from .backend import device_scales_bytes
        q_out = (be.allocate(m * n // 2), be.allocate(device_scales_bytes(m, n)), 0.0009765625)
    torch.cuda.synchronize()
    _, _, ga = sc.act_quant(a, m, k, 0.0, device_layout=True)[0:3]
    stream = torch.cuda.ExternalStream(be.streams()[0], device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if flush_l2 else None
    tq, tg = [], []
    for it in range(warmup + iters):
        if flush is not None:
            flush.fill_(it & 0xFF)
            torch.cuda.synchronize()
        e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        e[0].record(stream)
        if quant or it == 0:
            sc.act_quant_shared(a, m, k, ga)
        e[1].record(stream)
        sc.linear(None, m, W, ga, out, act=act, flags=L.LINEAR_A_PREQUANTIZED, out_nvfp4=q_out)
        e[2].record(stream)
        be.submit(60000)
        torch.cuda.synchronize()
        if it >= warmup:
            tq.append(e[0].elapsed_time(e[1]))
            tg.append(e[1].elapsed_time(e[2]))
    flops = 2.0 * m * n * k
    gemm_ms, quant_ms = float(np.mean(tg)), float(np.mean(tq))
    res = {
        "m": m, "n": n, "k": k, "act": act, "out_nvfp4": bool(out_nvfp4), "iters": iters, "flush_l2": bool(flush_l2),
        "gemm_ms": gemm_ms, "gemm_ms_min": float(np.min(tg)), "quant_ms": quant_ms if quant else None,
        "gemm_tflops": flops / (gemm_ms * 1e-3) / 1e12,
        "linear_tflops": flops / ((gemm_ms + (quant_ms if quant else 0.0)) * 1e-3) / 1e12,
        "gemm_min_bytes": m * k // 2 + m * k // 16 + n * k // 2 + n * k // 16 + 2 * n + 2 * m * n,
        "quant_min_bytes": 2 * m * k + m * k // 2 + m * k // 16,
    }
    if quant:
        res["quant_gbs"] = res["quant_min_bytes"] / (quant_ms * 1e-3) / 1e9
    be.close()
    return res


def run_norm_quant(m, k, iters=20, warmup=3, device=0):
    """Times the fused LayerNorm + modulate + quantiser launch on [m, k] bf16 rows (no bf16 output)."""
    import torch

    from . import Backend
    from .backend import device_scales_bytes

    be = Backend(device)
    sc = be.scope()
    dev = f"cuda:{device}"
    torch.cuda.set_device(device)
    gen = torch.Generator(device=dev)
    gen.manual_seed(4321)
    x = be.allocate(m * k * 2)
    _tview(be, x, torch.bfloat16, (m, k)).copy_(torch.randn(m, k, device=dev, generator=gen).to(torch.bfloat16))
    s, t = be.allocate(k * 2), be.allocate(k * 2)
    _tview(be, s, torch.bfloat16, (k,)).copy_((torch.randn(k, device=dev, generator=gen) * 0.3).to(torch.bfloat16))
    _tview(be, t, torch.bfloat16, (k,)).copy_((torch.randn(k, device=dev, generator=gen) * 0.2).to(torch.bfloat16))
    codes, scales = be.allocate(m * k // 2), be.allocate(device_scales_bytes(m, k))
    torch.cuda.synchronize()
    stream = torch.cuda.ExternalStream(be.streams()[0], device=dev)
    ts = []
    for it in range(warmup + iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        sc.norm_modulate_quant(x, m, k, 0.002, codes, scales, scale=s, shift=t)
        e1.record(stream)
        be.submit(60000)
        torch.cuda.synchronize()
        if it >= warmup:
            ts.append(e0.elapsed_time(e1))
    ms = float(np.mean(ts))
    nbytes = 2 * m * k + m * k // 2 + m * k // 16 + 4 * k
    be.close()
    return {"op": "norm_modulate_quant", "m": m, "k": k, "ms": ms, "ms_min": float(np.min(ts)), "min_bytes": nbytes,
            "gbs": nbytes / (ms * 1e-3) / 1e9}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, required=True)
    ap.add_argument("--n", type=int, default=0)
    ap.add_argument("--k", type=int, required=True)
    ap.add_argument("--act", type=int, default=0)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-quant", action="store_true")
    ap.add_argument("--flush-l2", action="store_true")
    ap.add_argument("--out-nvfp4", action="store_true")
    ap.add_argument("--norm-quant", action="store_true", help="time tnf_norm_modulate_quantize on [m, k] instead of a linear")
    args = ap.parse_args()
    if args.norm_quant:
        print(json.dumps(run_norm_quant(args.m, args.k, args.iters, args.warmup)))
        return
    print(json.dumps(run(args.m, args.n, args.k, args.act, args.iters, args.warmup, not args.no_quant, args.flush_l2,
                         out_nvfp4=args.out_nvfp4)))


if __name__ == "__main__":
    main()
