"""LayerNorm + modulate + NVFP4 quantiser in one launch (tnf_norm_modulate_quantize) against the CPU
restatement of the reference's two dispatches (thinfer-core/src/ops/layernorm.rs,
bcast_modulate.rs) followed by the oracle quantiser."""
import numpy as np
import pytest

import oracle as O
from conftest import dev_scales_to_canonical, rel_fro

pytestmark = pytest.mark.gpu

G_OUT = 0.002  # static per-tensor scale of the quantised output (|y| up to ~5 after modulation)


def _run(be, x, s, t, chain, want_bf16=True, eps=1e-6):
    from thinfer_b200.backend import device_scales_bytes

    m, k = x.shape
    xb = be.upload(x)
    sb = be.upload(s) if s is not None else None
    tb = be.upload(t) if t is not None else None
    out = be.allocate(m * k * 2) if want_bf16 else None
    codes = be.allocate(m * k // 2)
    scales = be.allocate(device_scales_bytes(m, k))
    be.write_buffer(scales, np.full(scales.len, 0x7F, np.uint8))  # NaN canary in every scale byte
    be.scope().norm_modulate_quant(xb, m, k, G_OUT, codes, scales, scale=sb, shift=tb, out_bf16=out, eps=eps, chain=chain)
    be.submit(30000)
    y = be.read_buffer(out, np.uint16).reshape(m, k) if want_bf16 else None
    c = be.read_buffer(codes).reshape(m, k // 2)
    dev = be.read_buffer(scales)
    for b in (xb, sb, tb, out, codes, scales):
        if b is not None:
            be.free(b)
    return y, c, dev


def _inputs(m, k, seed):
    x = O.f32_to_bf16(O.gaussian(m * k, seed).reshape(m, k) * np.float32(2.5) + np.float32(0.3))
    s = O.f32_to_bf16(O.gaussian(k, seed + 1) * np.float32(0.3))
    t = O.f32_to_bf16(O.gaussian(k, seed + 2) * np.float32(0.2))
    return x, s, t


@pytest.mark.parametrize("m,k,seed", [(4, 16, 1), (3, 64, 2), (130, 96, 3), (200, 3072, 4), (33, 12288, 5), (5, 16384, 6)])
@pytest.mark.parametrize("chain", [False, True])
def test_norm_modulate_quant_against_oracle(backend, m, k, seed, chain):
    x, s, t = _inputs(m, k, seed)
    y, c, dev = _run(backend, x, s, t, chain)
    want = O.norm_modulate(x, s, t, 1e-6, 1.0, chain=chain)
    # the kernel adds the row sums in a tree, the reference sequentially: compare under a tolerance ...
    assert not np.isnan(O.bf16_to_f32(y)).any()
    assert rel_fro(O.bf16_to_f32(y), O.bf16_to_f32(want)) <= 1e-3
    assert (y == want).mean() >= 0.98
    # ... and the NVFP4 copy bit for bit against the oracle quantiser on the kernel's own bf16 output
    oc, os_ = O.quantize_act(y, G_OUT)
    assert np.array_equal(c, oc)
    assert np.array_equal(dev_scales_to_canonical(dev, m, k), os_)
    assert np.array_equal(dev, O.scales_to_device_layout(os_))  # padding bytes are zero


def test_layernorm_only_and_no_bf16_output(backend):
    x, _, _ = _inputs(150, 512, 9)
    y, c, dev = _run(backend, x, None, None, False)
    want = O.ref_layernorm(x, 1e-6)
    assert rel_fro(O.bf16_to_f32(y), O.bf16_to_f32(want)) <= 1e-3
    _, c2, dev2 = _run(backend, x, None, None, False, want_bf16=False)
    assert np.array_equal(c, c2) and np.array_equal(dev, dev2)


def test_reference_fixtures_through_the_kernel(backend, golden_ref):
    """layernorm_basic and bcast_modulate of the reference's committed fixtures (bf16 variant)."""
    x, out = golden_ref["bf16p/layernorm_basic/x"], golden_ref["bf16p/layernorm_basic/out"]
    y, _, _ = _run(backend, x, None, None, False)
    g, e = O.bf16_to_f32(y), O.bf16_to_f32(out)
    assert (np.abs(g - e) <= 2.0 ** -7 * np.abs(e) + 1e-5).all()


def test_feeds_the_gemm(backend):
    """norm -> modulate -> quantise -> GEMM equals the oracle's chain (norm_modulate, then the NVFP4 linear)."""
    import thinfer_b200 as T
    from thinfer_b200.backend import device_scales_bytes

    be = backend
    m, k, n = 300, 512, 384
    x, s, t = _inputs(m, k, 21)
    w = (O.gaussian(n * k, 22) * np.float32(0.02)).reshape(n, k)
    bias = O.f32_to_bf16(O.gaussian(n, 23) * np.float32(0.01))
    W = T.Nvfp4Weight.from_dense(be, w, bias)
    xb, sb, tb = be.upload(x), be.upload(s), be.upload(t)
    codes, scales = be.allocate(m * k // 2), be.allocate(device_scales_bytes(m, k))
    out = be.allocate(m * n * 2)
    sc = be.scope()
    sc.norm_modulate_quant(xb, m, k, G_OUT, codes, scales, scale=sb, shift=tb)
    sc.matmul(codes, scales, m, W, G_OUT, out)
    be.submit(30000)
    got = be.read_buffer(out, np.uint16).reshape(m, n)
    wc, ws, gw = O.quantize_weight(w)
    want = O.linear(O.norm_modulate(x, s, t), G_OUT, wc, ws, gw, bias=bias)
    assert rel_fro(O.bf16_to_f32(got), O.bf16_to_f32(want)) <= 5e-3  # a few FP4 codes flip with the summation order
    for b in (xb, sb, tb, codes, scales, out):
        be.free(b)
    W.free(be)


def test_argument_errors(backend):
    from thinfer_b200.backend import InvalidArgument, device_scales_bytes

    be = backend
    x = be.allocate(4 * 64 * 2)
    c, s = be.allocate(4 * 32), be.allocate(device_scales_bytes(4, 64))
    sc = be.scope()
    with pytest.raises(InvalidArgument):
        sc.norm_modulate_quant(x, 4, 24, G_OUT, c, s)          # k not a multiple of 16
    with pytest.raises(InvalidArgument):
        sc.norm_modulate_quant(x, 4, 64, 0.0, c, s)            # no per-tensor scale
    with pytest.raises(InvalidArgument):
        sc.norm_modulate_quant(x, 4, 64, G_OUT, c, s, scale=x)  # scale without shift
    for b in (x, c, s):
        be.free(b)
