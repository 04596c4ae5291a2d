"""GPU quantisers against the CPU oracle: packed codes and scales must match bit for bit."""
import numpy as np
import pytest

import oracle as O
from conftest import dev_scales_to_canonical

pytestmark = pytest.mark.gpu


def _weight_case(be, w):
    import thinfer_b200 as T

    n, k = w.shape
    W = T.Nvfp4Weight.from_dense(be, w, keep_canonical=True)
    codes = be.read_buffer(W.codes).reshape(n, k // 2)
    scales = be.read_buffer(W.scales_canonical)[: n * k // 16].reshape(n, k // 16)
    dev = be.read_buffer(W.scales_device)
    g = W.global_scale
    W.free(be)
    return codes, scales, dev, g


@pytest.mark.parametrize("n,k,seed", [(64, 64, 1), (384, 512, 2), (130, 96, 3), (3072, 3072, 0xB000)])
def test_weight_quantiser_bit_exact(backend, n, k, seed):
    w = (O.gaussian(n * k, seed) * np.float32(0.02)).reshape(n, k)
    w[0, :16] = 0.0  # an all-zero block
    oc, os_, og = O.quantize_weight(w)
    c, s, dev, g = _weight_case(backend, w)
    assert g == og
    assert np.array_equal(c, oc)
    assert np.array_equal(s, os_)
    assert np.array_equal(dev_scales_to_canonical(dev, n, k), os_)
    assert np.array_equal(dev, O.scales_to_device_layout(os_))  # padding bytes are zero


def test_weight_quantiser_bf16_source_and_subnormal_scales(backend):
    # weights small enough that block scales land in the E4M3 subnormal range (the idea of the
    # reference's f16-subnormal-scale regression, thinfer-conformance/tests/q8_0_matmul.rs:415-445)
    w = (O.gaussian(256 * 512, 0x5EED5AB0) * np.float32(5e-3)).reshape(256, 512)
    w[:, :16] *= np.float32(1e-3)
    w[3, 100] = 40.0  # one outlier sets the per-tensor scale
    wb = O.f32_to_bf16(w)
    oc, os_, og = O.quantize_weight(wb)
    assert (os_ < 8).any() and (os_ == 0).any()
    c, s, dev, g = _weight_case(backend, wb)
    assert g == og and np.array_equal(c, oc) and np.array_equal(s, os_)


def test_all_zero_weight(backend):
    c, s, dev, g = _weight_case(backend, np.zeros((128, 64), np.float32))
    assert g == 1.0 and not c.any() and not s.any() and not dev.any()


@pytest.mark.parametrize("m,k,seed", [(1, 32, 1), (2, 64, 0xC0FFEE), (3, 128, 0xBEEF), (200, 512, 4), (256, 3072, 0xA000)])
@pytest.mark.parametrize("device_layout", [False, True])
def test_act_quantiser_bit_exact(backend, m, k, seed, device_layout):
    a = O.f32_to_bf16(O.gaussian(m * k, seed).reshape(m, k))
    g = O.global_scale(O.amax_bf16(a))
    oc, os_ = O.quantize_act(a, g)
    sc = backend.scope()
    buf = backend.upload(a)
    c, s, gu = sc.act_quant(buf, m, k, g, device_layout=device_layout)
    codes = backend.read_buffer(c).reshape(m, k // 2)
    sraw = backend.read_buffer(s)
    scales = dev_scales_to_canonical(sraw, m, k) if device_layout else sraw[: m * k // 16].reshape(m, k // 16)
    for b in (buf, c, s):
        backend.free(b)
    assert gu == np.float32(g)
    assert np.array_equal(codes, oc)
    assert np.array_equal(scales, os_)
    if device_layout:
        assert np.array_equal(sraw, O.scales_to_device_layout(os_))


def test_act_quantiser_ties_saturation_and_dynamic_scale(backend):
    m, k = 8, 64
    a = np.zeros((m, k), np.float32)
    a[0, :16] = [6, 0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0, -0.0]
    a[1, :16] = 1e-30
    a[2, :16] = [3e38] + [1.0] * 15
    a[3, :] = O.gaussian(k, 5) * np.float32(40.0)  # heavy-tailed row (q8_0_matmul.rs:301-317 idea)
    a[3, 7] *= 8
    ab = O.f32_to_bf16(a)
    sc = backend.scope()
    buf = backend.upload(ab)
    for g in (1.0, 0.0):
        c, s, gu = sc.act_quant(buf, m, k, g)
        g_ref = g if g > 0 else O.global_scale(O.amax_bf16(ab))
        assert gu == np.float32(g_ref)
        oc, os_ = O.quantize_act(ab, g_ref)
        assert np.array_equal(backend.read_buffer(c).reshape(m, k // 2), oc)
        assert np.array_equal(backend.read_buffer(s)[: m * k // 16].reshape(m, k // 16), os_)
        backend.free(c)
        backend.free(s)
    backend.free(buf)


def test_quantiser_argument_errors(backend):
    import thinfer_b200 as T
    from thinfer_b200.backend import InvalidArgument

    buf = backend.allocate(4096)
    with pytest.raises(InvalidArgument):
        backend.scope().act_quant(buf, 4, 48)  # k % 32 != 0
    with pytest.raises(InvalidArgument):
        backend.scope().act_quant(buf, 64, 64)  # view too small
    backend.free(buf)
    with pytest.raises(T.UnknownBuffer):
        backend.free(buf)
