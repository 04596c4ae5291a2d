"""Regenerates tests/golden/*.npz; the files are committed so that tests never read the reference.

    python tests/golden/make_golden.py --reference <path to a cretz/thinfer checkout>   # parts 1 and 2
    python tests/golden/make_golden.py                                                  # part 2 only

Part 1 — reference_fixtures.npz: the cases of the reference's committed conformance
fixtures (thinfer-conformance/fixtures/{fp32,bf16w,bf16p}.safetensors, spec in
fixtures/spec.json) that touch the linear path: matmul_basic, bcast_add (bias),
bcast_fma (gated residual), gelu_mul_basic (tanh-GELU gate), layernorm_basic and bcast_modulate
(the two steps in front of every block linear), and the sdpa cases (the attention between the
linears; the per-case scale is in fixtures/spec.json and repeated in the test). Copied as data, bit for bit;
bf16 tensors are stored as uint16 bit patterns.

Part 2 — nvfp4_golden.npz: small seeded NVFP4 cases produced by this repo's CPU oracle
(inputs and outputs), so that the GPU tests have fixed vectors to hit.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))

CASES = ["matmul_basic", "bcast_add", "bcast_fma", "gelu_mul_basic", "layernorm_basic", "bcast_modulate",
         "sdpa_basic", "sdpa_large_d_d128", "sdpa_decode_sq1", "sdpa_decode_multirow"]


def part1(reference_root):
    import torch
    from safetensors import safe_open

    REF_FIXTURES = os.path.join(reference_root, "projects", "thinfer-conformance", "fixtures")
    out = {}
    for variant in ("fp32", "bf16w", "bf16p"):
        with safe_open(os.path.join(REF_FIXTURES, f"{variant}.safetensors"), "pt") as h:
            for key in h.keys():
                case = key.split("/")[0]
                if case not in CASES:
                    continue
                t = h.get_tensor(key)
                if t.dtype == torch.bfloat16:
                    arr = t.view(torch.int16).numpy().view(np.uint16)
                else:
                    arr = t.numpy()
                out[f"{variant}/{key}"] = arr
    np.savez(os.path.join(HERE, "reference_fixtures.npz"), **out)
    print("reference_fixtures.npz:", len(out), "tensors")


def part2():
    import oracle as O

    out = {}
    for name, (m, n, k, seed) in {"small": (64, 64, 128, 11), "ragged": (40, 72, 96, 12), "c1_slice": (32, 256, 3072, 13)}.items():
        a = O.f32_to_bf16(O.gaussian(m * k, 0xA000 + seed).reshape(m, k))
        w = (O.gaussian(n * k, 0xB000 + seed) * np.float32(0.02)).reshape(n, k)
        bias = O.f32_to_bf16(O.gaussian(n, 0xC000 + seed) * np.float32(0.01))
        wc, ws, gw = O.quantize_weight(w)
        ga = O.global_scale(O.amax_bf16(a))
        ac, as_ = O.quantize_act(a, ga)
        y = O.linear(a, ga, wc, ws, gw, bias=bias)
        yg = O.linear(a, ga, wc, ws, gw, bias=bias, act=1)
        for key, val in dict(a=a, w=w, bias=bias, w_codes=wc, w_scales=ws, g_w=np.float32(gw), g_a=np.float32(ga),
                             a_codes=ac, a_scales=as_, out=y, out_gelu=yg).items():
            out[f"{name}/{key}"] = val
    np.savez_compressed(os.path.join(HERE, "nvfp4_golden.npz"), **out)
    print("nvfp4_golden.npz:", len(out), "tensors")


if __name__ == "__main__":
    import argparse

    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=None, help="root of a cretz/thinfer checkout; without it reference_fixtures.npz is left as committed")
    args = ap.parse_args()
    if args.reference:
        part1(args.reference)
    else:
        print("no --reference given: reference_fixtures.npz left as committed")
    part2()
