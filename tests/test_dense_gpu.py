"""The dense-activation arm on the device: sites whose activations stay bf16 (the reference's DenseActSites,
thinfer-models/src/common/block.rs:458-479, served there by "dequantise once, then a dense matmul",
:2861-2881) multiply the NVFP4 weight's dense bf16 image with tcgen05.mma kind::f16 in the CTA-pair kernel.

Oracle: orc_linear with quantize_a = 0 (bf16 activations against the dequantised weight, f32 accumulation,
per-tensor weight scale in the epilogue). Tolerance: relative Frobenius error <= 1e-3 (in practice ~1e-6:
every product is exact in f32, only the summation order differs)."""
import numpy as np
import pytest

import oracle as O
from conftest import rel_fro

pytestmark = pytest.mark.gpu
TOL = 1e-3


def _inputs(m, n, k, seed):
    a = O.f32_to_bf16(O.gaussian(m * k, 0xA000 + seed).reshape(m, k))
    w = (O.gaussian(n * k, 0xB000 + seed) * np.float32(0.02)).reshape(n, k)
    b = O.f32_to_bf16(O.gaussian(n, 0xC000 + seed) * np.float32(0.01))
    return a, w, b


def test_dense_image_is_exact(backend):
    """code x block scale has at most six significant bits: the bf16 image equals the oracle's f32 dequantisation."""
    import thinfer_b200 as T

    n, k = 264, 320
    _, w, _ = _inputs(8, n, k, 81)
    wc, ws, gw = O.quantize_weight(w)
    W = T.Nvfp4Weight.from_packed(backend, wc, ws, gw)
    img = backend.read_buffer(W.prepare_dense(backend), np.uint16).reshape(n, k)
    want = O.dequant(wc, ws, 1.0)
    assert np.array_equal(O.bf16_to_f32(img), want)
    W.free(backend)


@pytest.mark.parametrize("m,n,k,act", [(200, 520, 512, 0), (37, 264, 96, 1), (2304, 4608, 512, 1), (2100, 2312, 320, 0)])
def test_dense_act_linear_matches_oracle(backend, m, n, k, act):
    import thinfer_b200 as T

    a, w, b = _inputs(m, n, k, m + n)
    wc, ws, gw = O.quantize_weight(w)
    be = backend
    W = T.Nvfp4Weight.from_packed(be, wc, ws, gw, b)
    W.prepare_dense(be)
    abuf = be.upload(a)
    out = be.allocate((m + 1) * n * 2)
    be.write_buffer(out, np.full((m + 1) * n, 0x7FC0, np.uint16))
    be.scope().linear(abuf, m, W, 0.0, out, act=act, dense_act=True)
    be.submit(30000)
    full = be.read_buffer(out, np.uint16).reshape(m + 1, n)
    assert (full[m] == 0x7FC0).all()
    want = O.linear(a, 1.0, wc, ws, gw, bias=b, act=act, quantize_a=False)
    assert not np.isnan(O.bf16_to_f32(full[:m])).any()
    assert rel_fro(O.bf16_to_f32(full[:m]), O.bf16_to_f32(want)) <= TOL
    assert (full[:m] == want).mean() > (0.9 if act else 0.98)
    be.free(abuf)
    be.free(out)
    W.free(be)


def test_site_policy_accuracy_on_device(backend):
    """The accuracy side of the site policy, measured on the GPU: error against the unquantised f64 product of
    FP4 activations x FP4 weights and of bf16 activations x FP4 weights, on Gaussian inputs and on inputs with
    30x outlier channels. The dense arm must recover what the activation quantiser costs."""
    import thinfer_b200 as T

    m, k, n = 256, 1024, 512
    w = (O.gaussian(n * k, 71) * np.float32(0.02)).reshape(n, k)
    gauss = O.gaussian(m * k, 72).reshape(m, k)
    heavy = gauss.copy()
    heavy[:, ::128] *= np.float32(30.0)
    be = backend
    W = T.Nvfp4Weight.from_dense(be, w)
    W.prepare_dense(be)
    policy = T.DenseActSites(proj=True, ffn_down=True)
    from thinfer_b200 import _lib as L
    assert policy.flags(L.SITE_PROJ) == L.LINEAR_DENSE_ACT and policy.flags(L.SITE_QKV) == 0
    errs = {}
    for name, a_f32 in (("gaussian", gauss), ("heavy", heavy)):
        a = O.f32_to_bf16(a_f32)
        exact = O.bf16_to_f32(a).astype(np.float64) @ w.astype(np.float64).T
        abuf = be.upload(a)
        out = be.allocate(m * n * 2)
        ga = O.global_scale(O.amax_bf16(a))
        res = []
        for site in (L.SITE_QKV, L.SITE_PROJ):  # a site with FP4 activations, a site the policy keeps dense
            be.scope().linear(abuf, m, W, ga, out, flags=policy.flags(site))
            be.submit(30000)
            res.append(rel_fro(O.bf16_to_f32(be.read_buffer(out, np.uint16).reshape(m, n)), exact))
        errs[name] = res
        be.free(abuf)
        be.free(out)
    W.free(be)
    for name, (e_fp4, e_dense) in errs.items():
        assert e_dense < e_fp4 < 0.16 and e_dense < 0.11, (name, e_fp4, e_dense)
        assert e_fp4 < 1.6 * e_dense
    print("site policy on device (rel. Frobenius error vs f64): " + ", ".join(f"{k} fp4 {v[0]:.4f} dense {v[1]:.4f}" for k, v in errs.items()))


@pytest.mark.parametrize("m,n,k,act", [(200, 520, 512, 1), (2100, 2312, 320, 0)])
def test_unquantised_bf16_weight_site(backend, m, n, k, act):
    """A weight that is never quantised (the reference's refiner weights, thinfer-core/src/ops/matmul_i8_bf16.rs:15-17)
    runs through the dense arm as it is: bf16 x bf16 on the tensor cores, f32 accumulation, per-tensor scale 1."""
    import thinfer_b200 as T

    a, w, b = _inputs(m, n, k, 3 * m + n)
    wb = O.f32_to_bf16(w)
    be = backend
    W = T.Nvfp4Weight.from_bf16(be, wb, b)
    abuf = be.upload(a)
    out = be.allocate(m * n * 2)
    be.scope().linear(abuf, m, W, 0.0, out, act=act, dense_act=True)
    be.submit(30000)
    got = be.read_buffer(out, np.uint16).reshape(m, n)
    want = O.epilogue(O.gemm_f32(O.bf16_to_f32(a), O.bf16_to_f32(wb)), 1.0, bias=b, act=act)
    assert rel_fro(O.bf16_to_f32(got), O.bf16_to_f32(want)) <= TOL
    assert (got == want).mean() > (0.9 if act else 0.98)
    with pytest.raises(T.InvalidArgument, match="dense_act"):
        be.scope().linear(abuf, m, W, 1.0, out)  # no NVFP4 form: the FP4 arm must refuse, not read null codes
    be.free(abuf)
    be.free(out)
    W.free(be)


@pytest.mark.parametrize("m,n,k,act,shared", [(200, 520, 512, 1, False), (2304, 2304, 256, 0, True), (37, 264, 96, 0, True)])
def test_mixed_arm_nvfp4_activations_times_bf16_weight(backend, m, n, k, act, shared):
    """Low-bit activations x dense bf16 weight (the role of the reference's matmul_i8_bf16,
    thinfer-core/src/ops/matmul_i8_bf16.rs:1-17): the NVFP4 activations are widened to bf16 exactly, so the result
    is the oracle's product of the dequantised activations with the bf16 weight, scaled by a_global * w_global in
    the epilogue. Both entries: the pre-quantised GEMM call and the shared-scratch linear."""
    import thinfer_b200 as T
    from thinfer_b200 import _lib as L

    a, w, b = _inputs(m, n, k, 5 * m + n)
    wb = O.f32_to_bf16(w)
    ga = O.global_scale(O.amax_bf16(a))
    ac, as_ = O.quantize_act(a, ga)
    want = O.epilogue(O.gemm_f32(O.dequant(ac, as_, 1.0), O.bf16_to_f32(wb)), ga * 1.0, bias=b, act=act)
    be = backend
    W = T.Nvfp4Weight.from_bf16(be, wb, b)
    abuf = be.upload(a)
    out = be.allocate(m * n * 2)
    sc = be.scope()
    if shared:
        sc.act_quant_shared(abuf, m, k, ga)
        sc.linear(None, m, W, ga, out, act=act, dense_act=True, flags=L.LINEAR_A_PREQUANTIZED)
    else:
        qc, qs, _ = sc.act_quant(abuf, m, k, ga, device_layout=True)
        sc.matmul(qc, qs, m, W, ga, out, act=act, dense_act=True)
    be.submit(30000)
    got = be.read_buffer(out, np.uint16).reshape(m, n)
    assert rel_fro(O.bf16_to_f32(got), O.bf16_to_f32(want)) <= TOL
    assert (got == want).mean() > (0.9 if act else 0.98)
    if shared:  # the scratch is tagged with its shape: another shape is refused
        with pytest.raises(T.InvalidArgument, match="shared scratch"):
            W2 = T.Nvfp4Weight(n, k + 32, None, None, 1.0, None, None, W.dense)
            sc.linear(None, m, W2, ga, out, dense_act=True, flags=L.LINEAR_A_PREQUANTIZED)
    else:
        be.free(qc)
        be.free(qs)
    be.free(abuf)
    be.free(out)
    W.free(be)
