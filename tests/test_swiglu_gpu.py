"""SwiGLU pairwise gating fused into the FFN-up GEMM: one launch over the row-interleaved [W1; W3] weight whose
epilogue writes silu(A.W1^T) * (A.W3^T), against the reference's three dispatches (two matmuls on the same A,
then op_silu_mul: thinfer-models/src/common/block.rs:1720-1762, thinfer-core/src/ops/silu_mul.rs) restated with
the oracle's linear. Chain mode keeps the bf16 rounding of the two matmul outputs; fused mode does not.
Tolerance: relative Frobenius error <= 1e-3."""
import numpy as np
import pytest

import oracle as O
from conftest import rel_fro

pytestmark = pytest.mark.gpu


def _silu_mul(a, b):
    a, b = a.astype(np.float32), b.astype(np.float32)
    return (a / (np.float32(1.0) + np.exp(-a))) * b


@pytest.mark.parametrize("m,hid,k,chain,dense", [(200, 264, 512, False, False), (200, 264, 512, True, False),
                                                 (2304, 2304, 512, False, False), (300, 1280, 384, False, True)])
def test_swiglu_epilogue_matches_three_dispatches(backend, m, hid, k, chain, dense):
    import thinfer_b200 as T

    a = O.f32_to_bf16(O.gaussian(m * k, 0xA100 + m).reshape(m, k))
    w1 = (O.gaussian(hid * k, 0xB100 + m) * np.float32(0.03)).reshape(hid, k)
    w3 = (O.gaussian(hid * k, 0xB200 + m) * np.float32(0.03)).reshape(hid, k)
    w13 = T.interleave_swiglu(w1, w3)
    wc, ws, gw = O.quantize_weight(w13)  # quantised as one tensor: one per-tensor scale for both halves
    ga = O.global_scale(O.amax_bf16(a))
    be = backend
    W = T.Nvfp4Weight.from_packed(be, wc, ws, gw)
    if dense:
        W.prepare_dense(be)
    abuf = be.upload(a)
    out = be.allocate((m + 1) * hid * 2)
    be.write_buffer(out, np.full((m + 1) * hid, 0x7FC0, np.uint16))
    be.scope().linear(abuf, m, W, ga, out, chain=chain, swiglu=True, dense_act=dense)
    be.submit(30000)
    full = be.read_buffer(out, np.uint16).reshape(m + 1, hid)
    assert (full[m] == 0x7FC0).all()
    # the reference's way: two linears on the same A, then silu_mul
    kw = dict(quantize_a=not dense)
    if chain:
        h1 = O.bf16_to_f32(O.linear(a, ga, wc[0::2], ws[0::2], gw, **kw))
        h3 = O.bf16_to_f32(O.linear(a, ga, wc[1::2], ws[1::2], gw, **kw))
    else:
        scale = np.float32(gw) * (np.float32(ga) if not dense else np.float32(1.0))
        h1 = O.linear(a, ga, wc[0::2], ws[0::2], gw, return_acc=True, **kw)[1] * scale
        h3 = O.linear(a, ga, wc[1::2], ws[1::2], gw, return_acc=True, **kw)[1] * scale
    want = O.f32_to_bf16(_silu_mul(h1, h3))
    got = full[:m]
    assert not np.isnan(O.bf16_to_f32(got)).any()
    assert rel_fro(O.bf16_to_f32(got), O.bf16_to_f32(want)) <= 1e-3
    assert (got == want).mean() > 0.9  # exp is the hardware approximation
    be.free(abuf)
    be.free(out)
    W.free(be)
