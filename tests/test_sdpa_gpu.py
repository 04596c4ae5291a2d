"""Attention between the linears on the device (tnf_sdpa: flash-attention tiling, both products on the tensor
cores) against the restated reference (oracle.ref_sdpa: thinfer-core/src/ops/sdpa.rs, online softmax in f32, one key
at a time), which tests/test_oracle_pins.py pins on the reference's own sdpa fixtures.

Tolerance: relative Frobenius error <= 4e-3. The kernel rounds the probabilities to bf16 for the second product and
evaluates exp as exp2 with the scale folded in; inputs and outputs are bf16 on both sides."""
import numpy as np
import pytest

import oracle as O
from conftest import rel_fro

pytestmark = pytest.mark.gpu
TOL = 4e-3


def _run(be, q, k, v, scale):
    b, s_q, h_q, d = q.shape
    _, s_k, h_kv, _ = k.shape
    qb, kb, vb = be.upload(q), be.upload(k), be.upload(v)
    out = be.allocate((b * s_q + 1) * h_q * d * 2)
    be.write_buffer(out, np.full((b * s_q + 1) * h_q * d, 0x7FC0, np.uint16))
    be.scope().sdpa(qb, kb, vb, out, b, s_q, s_k, h_q, h_kv, scale)
    be.submit(30000)
    full = be.read_buffer(out, np.uint16)
    for buf in (qb, kb, vb, out):
        be.free(buf)
    assert (full[b * s_q * h_q * d:] == 0x7FC0).all()  # nothing written past the last row
    return full[: b * s_q * h_q * d].reshape(b, s_q, h_q, d)


def _inputs(b, s_q, s_k, h_q, h_kv, seed, spread=1.0):
    d = 128
    q = O.f32_to_bf16(O.gaussian(b * s_q * h_q * d, 0x5100 + seed).reshape(b, s_q, h_q, d) * np.float32(spread))
    k = O.f32_to_bf16(O.gaussian(b * s_k * h_kv * d, 0x5200 + seed).reshape(b, s_k, h_kv, d))
    v = O.f32_to_bf16(O.gaussian(b * s_k * h_kv * d, 0x5300 + seed).reshape(b, s_k, h_kv, d))
    return q, k, v


@pytest.mark.parametrize("b,s_q,s_k,h_q,h_kv", [(1, 128, 128, 1, 1), (1, 256, 384, 2, 2), (1, 300, 200, 4, 2), (2, 129, 257, 2, 1),
                                                 (1, 1, 40, 2, 2), (1, 640, 1100, 3, 3)])
def test_sdpa_matches_reference_recurrence(backend, b, s_q, s_k, h_q, h_kv):
    q, k, v = _inputs(b, s_q, s_k, h_q, h_kv, s_q + s_k)
    scale = 1.0 / np.sqrt(128.0)
    got = _run(backend, q, k, v, float(scale))
    want = O.ref_sdpa(q, k, v, float(scale))
    assert not np.isnan(O.bf16_to_f32(got)).any()
    assert rel_fro(O.bf16_to_f32(got), O.bf16_to_f32(want)) <= TOL


@pytest.mark.parametrize("s_q,s_k,heads", [(256, 1024, 2), (128, 2176, 1), (384, 1536, 3)])
def test_sdpa_peaked_rows_rescale_the_running_output(backend, s_q, s_k, heads):
    """Scores with a large spread: the row maximum keeps growing from tile to tile, so the running output in TMEM is
    rescaled many times (by threads of both softmax groups, each waiting for the other's product), and most
    probabilities underflow to zero. Eight and more key tiles: every barrier goes through several phases."""
    q, k, v = _inputs(1, s_q, s_k, heads, heads, 77, spread=6.0)
    scale = 1.0 / np.sqrt(128.0)
    got = _run(backend, q, k, v, float(scale))
    want = O.ref_sdpa(q, k, v, float(scale))
    assert not np.isnan(O.bf16_to_f32(got)).any()
    assert rel_fro(O.bf16_to_f32(got), O.bf16_to_f32(want)) <= TOL


def test_sdpa_reference_fixture_d128(backend, golden_ref):
    """The reference's own D = 128 case (sdpa_large_d_d128: S = 4, one head, scale 0.088388346) through the kernel."""
    q, k, v, out = (golden_ref[f"fp32/sdpa_large_d_d128/{t}"] for t in "q k v out".split())
    got = _run(backend, O.f32_to_bf16(q), O.f32_to_bf16(k), O.f32_to_bf16(v), 0.088388346)
    assert rel_fro(O.bf16_to_f32(got), out) <= 8e-3  # the fixture's inputs are f32: narrowing them to bf16 is part of the error


def test_sdpa_argument_errors(backend):
    import thinfer_b200 as T
    from thinfer_b200 import _lib as L

    buf = backend.allocate(1 << 16)
    sc = backend.scope()
    with pytest.raises(T.InvalidArgument, match="d must be 128"):
        sc.sdpa(buf, buf, buf, buf, 1, 4, 4, 1, 1, 0.1, d=64)
    with pytest.raises(T.InvalidArgument, match="h_kv must divide"):
        sc.sdpa(buf, buf, buf, buf, 1, 4, 4, 3, 2, 0.1)
    with pytest.raises(T.TnfError):
        sc.sdpa(buf, buf, buf, buf, 1, 4096, 4, 1, 1, 0.1)  # q does not fit its buffer
    backend.free(buf)


@pytest.mark.parametrize("b,s_q,s_k,heads,keep_bf16", [(1, 300, 260, 2, True), (2, 200, 130, 3, True), (1, 257, 128, 4, False)])
def test_sdpa_fused_output_quantisation(backend, b, s_q, s_k, heads, keep_bf16):
    """TNF_SDPA_OUT_NVFP4: the attention epilogue also emits its output as the NVFP4 A operand of the out-projection.
    The codes and scales are bit for bit what the activation quantiser makes of the kernel's own bf16 output (oracle
    quantiser on those bits), padding of the scale layout is zero, and the operand feeds the GEMM directly."""
    import thinfer_b200 as T
    from thinfer_b200.backend import device_scales_bytes
    from conftest import dev_scales_to_canonical

    be = backend
    d, rows, cols = 128, b * s_q, heads * 128
    q, k, v = _inputs(b, s_q, s_k, heads, heads, 900 + s_q)
    scale = float(1.0 / np.sqrt(128.0))
    qb, kb, vb = be.upload(q), be.upload(k), be.upload(v)
    out = be.allocate(rows * cols * 2)
    codes = be.allocate(rows * cols // 2)
    nsc = device_scales_bytes(rows, cols)
    scales = be.allocate(nsc)
    be.write_buffer(scales, np.full(nsc, 0x7F, np.uint8))  # canary: stale NaN scales must not survive in the padding
    sc = be.scope()
    sc.sdpa(qb, kb, vb, out, b, s_q, s_k, heads, heads, scale)  # plain run: the bf16 reference output
    be.submit(30000)
    plain = be.read_buffer(out, np.uint16).reshape(rows, cols)
    g_out = O.global_scale(O.amax_bf16(plain))
    be.write_buffer(out, np.zeros(rows * cols, np.uint16))
    sc.sdpa(qb, kb, vb, out if keep_bf16 else None, b, s_q, s_k, heads, heads, scale, out_nvfp4=(codes, scales, g_out))
    be.submit(30000)
    if keep_bf16:
        assert np.array_equal(be.read_buffer(out, np.uint16).reshape(rows, cols), plain)
    else:
        assert not be.read_buffer(out, np.uint16).any()  # the bf16 tensor was not touched
    want_c, want_s = O.quantize_act(plain, g_out)
    got_c = be.read_buffer(codes).reshape(rows, cols // 2)
    dev = be.read_buffer(scales)
    assert np.array_equal(got_c, want_c)
    assert np.array_equal(dev_scales_to_canonical(dev, rows, cols), want_s)
    assert np.array_equal(dev, O.scales_to_device_layout(want_s))  # every padding byte is zero
    # and the out-projection runs on it: same bits as the linear that quantises the bf16 output itself
    n = 264
    w = (O.gaussian(n * cols, 0x7700) * np.float32(0.02)).reshape(n, cols)
    W = T.Nvfp4Weight.from_dense(be, w)
    y1, y2 = be.allocate(rows * n * 2), be.allocate(rows * n * 2)
    pb = be.upload(plain)
    sc.linear(pb, rows, W, g_out, y1)
    sc.matmul(codes, scales, rows, W, g_out, y2)
    be.submit(30000)
    assert np.array_equal(be.read_buffer(y1, np.uint16), be.read_buffer(y2, np.uint16))
    for buf in (qb, kb, vb, out, codes, scales, y1, y2, pb):
        be.free(buf)
    W.free(be)


def test_sdpa_reads_column_windows_of_the_fused_qkv_output(backend):
    """q, k and v as column windows of one [rows, 3 * h * d] matrix (the fused-QKV linear's output) with a leading
    dimension: the same bits as on separate dense tensors, without the reference's concatenate / split copies."""
    from thinfer_b200 import _lib as L

    be = backend
    b, s, heads = 1, 330, 3
    hd = heads * 128
    q, k, v = _inputs(b, s, s, heads, heads, 4242)
    scale = float(1.0 / np.sqrt(128.0))
    dense = _run(be, q, k, v, scale)
    qkv = np.concatenate([q.reshape(s, hd), k.reshape(s, hd), v.reshape(s, hd)], axis=1)  # [s, 3 * hd]
    buf = be.upload(qkv)
    out = be.allocate(s * hd * 2)
    win = lambda i: L.Buf(buf.id, i * hd * 2, s * 3 * hd * 2 - i * hd * 2)
    be.scope().sdpa(win(0), win(1), win(2), out, b, s, s, heads, heads, scale, q_ld=3 * hd, kv_ld=3 * hd)
    be.submit(30000)
    assert np.array_equal(be.read_buffer(out, np.uint16).reshape(b, s, heads, 128), dense)
    import thinfer_b200 as T
    with pytest.raises(T.InvalidArgument, match="must cover the heads"):
        be.scope().sdpa(win(0), win(1), win(2), out, b, s, s, heads, heads, scale, q_ld=hd - 8, kv_ld=3 * hd)
    be.free(buf)
    be.free(out)
