"""The NVFP4 linear through the C ABI against the CPU oracle.

Tolerance: relative Frobenius error <= 1e-3 (the bar stated for this path); most cases are
in fact bit-equal because the block-scaled products are exact in f32 and only the
accumulation order differs."""
import numpy as np
import pytest

import oracle as O
from conftest import rel_fro

pytestmark = pytest.mark.gpu
TOL = 1e-3


def _inputs(m, n, k, seed, bias=True):
    a = O.f32_to_bf16(O.gaussian(m * k, 0xA000 + seed).reshape(m, k))
    w = (O.gaussian(n * k, 0xB000 + seed) * np.float32(0.02)).reshape(n, k)
    b = O.f32_to_bf16(O.gaussian(n, 0xC000 + seed) * np.float32(0.01)) if bias else None
    return a, w, b


def _run(be, a, w, b, **kw):
    import thinfer_b200 as T

    m, k = a.shape
    n = w.shape[0]
    W = T.Nvfp4Weight.from_dense(be, w, b)
    ga = O.global_scale(O.amax_bf16(a))
    abuf = be.upload(a)
    out = be.allocate(m * n * 2)
    be.write_buffer(out, np.full(m * n, 0x7FC0, np.uint16))  # NaN canary
    be.scope().linear(abuf, m, W, ga, out, **kw)
    be.submit(30000)
    got = be.read_buffer(out, np.uint16).reshape(m, n)
    be.free(abuf)
    be.free(out)
    g_w = W.global_scale
    W.free(be)
    return got, ga, g_w


# shapes: reference conformance geometries (q4_0_matmul.rs:178-223 small / ragged / rectangular),
# tile-edge cases of this kernel (128x256 tiles, 256-element K tiles) and BASELINE config 1
SHAPES = [(16, 16, 32), (10, 16, 32), (8, 8, 128), (24, 48, 96), (128, 256, 256), (129, 264, 288),
          (200, 520, 1024), (256, 3072, 3072), (1, 3072, 3072), (2, 264, 96), (3, 18432, 3072), (8, 1000, 320), (5, 136, 12288),
          # the 1-CTA kernel's three tile widths: 64 (few tiles, above), 128 (76 tiles of 128) and 256 (148 of 256), ragged in n
          (100, 9608, 64), (40, 37896, 96)]


@pytest.mark.parametrize("m,n,k", SHAPES)
def test_linear_matches_oracle(backend, m, n, k):
    a, w, b = _inputs(m, n, k, m + n + k)
    got, ga, gw = _run(backend, a, w, b)
    wc, ws, ogw = O.quantize_weight(w)
    assert gw == ogw
    want = O.linear(a, ga, wc, ws, ogw, bias=b)
    assert not np.isnan(O.bf16_to_f32(got)).any()
    assert rel_fro(O.bf16_to_f32(got), O.bf16_to_f32(want)) <= TOL


@pytest.mark.parametrize("mode", ["none", "gelu", "gelu_chain", "chain", "gate"])
def test_epilogue_modes(backend, mode):
    m, n, k = 200, 520, 512
    a, w, b = _inputs(m, n, k, 77)
    wc, ws, gw = O.quantize_weight(w)
    ga = O.global_scale(O.amax_bf16(a))
    kw, okw = {}, {}
    gate = res = None
    if mode.startswith("gelu"):
        kw["act"] = okw["act"] = 1
    if mode.endswith("chain"):
        kw["chain"] = okw["chain"] = True
    if mode == "gate":
        gate = O.f32_to_bf16(O.gaussian(n, 0xD000))
        res = O.f32_to_bf16(O.gaussian(m * n, 0xE000).reshape(m, n))
        gb, rb = backend.upload(gate), backend.upload(res)
        kw.update(gate=gb, residual=rb)
        okw.update(gate=gate, residual=res)
    got, _, _ = _run(backend, a, w, b, **kw)
    want = O.linear(a, ga, wc, ws, gw, bias=b, **okw)
    assert rel_fro(O.bf16_to_f32(got), O.bf16_to_f32(want)) <= TOL
    # fused GELU: tanh.approx against libm tanh; chain mode evaluates the reference's formula with tanhf
    assert (got == want).mean() > (0.9 if mode == "gelu" else 0.99)
    if mode == "gate":
        backend.free(gb)
        backend.free(rb)


# one-launch kernels where they are the chosen path (m * k <= 12288, or 24576 from n = 12288 on; K beyond the
# tensor-core kernel's reach goes to the CUDA-core one) and shapes just outside it, which take quantiser + GEMM
@pytest.mark.parametrize("m,n,k", [(1, 18432, 3072), (3, 520, 1056), (8, 264, 4128), (4, 136, 64), (16, 1032, 3072), (13, 136, 352),
                                   (1, 264, 12288), (5, 136, 16384), (16, 264, 768), (8, 12296, 3072)])
@pytest.mark.parametrize("mode", ["gelu", "gelu_chain", "gate"])
def test_skinny_kernel_epilogue_modes(backend, m, n, k, mode):
    """A handful of rows runs a one-launch skinny kernel with the activation quantiser in its prologue: M <= 16 on the
    tensor cores with the operands swapped (the weight is the 128-row side), and for K too long for that kernel's
    shared memory (the last two shapes) M <= 8 with the weights streamed on the CUDA cores. Same contract, same
    epilogue variants; ragged N, K not a multiple of the 256-element tile, more K tiles than ring stages."""
    a, w, b = _inputs(m, n, k, 300 + m)
    wc, ws, gw = O.quantize_weight(w)
    ga = O.global_scale(O.amax_bf16(a))
    kw, okw, extra = {}, {}, []
    if mode.startswith("gelu"):
        kw["act"] = okw["act"] = 1
    if mode.endswith("chain"):
        kw["chain"] = okw["chain"] = True
    if mode == "gate":
        gate = O.f32_to_bf16(O.gaussian(n, 0xD200))
        res = O.f32_to_bf16(O.gaussian(m * n, 0xE200).reshape(m, n))
        gb, rb = backend.upload(gate), backend.upload(res)
        extra = [gb, rb]
        kw.update(gate=gb, residual=rb)
        okw.update(gate=gate, residual=res)
    got, _, _ = _run(backend, a, w, b, **kw)
    want = O.linear(a, ga, wc, ws, gw, bias=b, **okw)
    assert not np.isnan(O.bf16_to_f32(got)).any()
    assert rel_fro(O.bf16_to_f32(got), O.bf16_to_f32(want)) <= TOL
    assert (got == want).mean() > (0.9 if mode == "gelu" else 0.98)
    for buf in extra:
        backend.free(buf)


def test_golden_vectors(backend, golden_nvfp4):
    import thinfer_b200 as T

    for name in ("small", "ragged", "c1_slice"):
        g = {k.split("/", 1)[1]: golden_nvfp4[k] for k in golden_nvfp4.files if k.startswith(name + "/")}
        m, k = g["a"].shape
        n = g["w"].shape[0]
        W = T.Nvfp4Weight.from_dense(backend, g["w"], g["bias"], keep_canonical=True)
        assert np.float32(W.global_scale) == g["g_w"]
        assert np.array_equal(backend.read_buffer(W.codes).reshape(n, k // 2), g["w_codes"])
        abuf = backend.upload(g["a"])
        out = backend.allocate(m * n * 2)
        for act, key in ((0, "out"), (1, "out_gelu")):
            backend.scope().linear(abuf, m, W, float(g["g_a"]), out, act=act)
            backend.submit(30000)
            got = backend.read_buffer(out, np.uint16).reshape(m, n)
            assert rel_fro(O.bf16_to_f32(got), O.bf16_to_f32(g[key])) <= TOL
        backend.free(abuf)
        backend.free(out)
        W.free(backend)


def test_n_split_window_and_shared_activation(backend):
    """Column-parallel slices written into one [m, n_total] output, A quantised once."""
    import thinfer_b200 as T
    from thinfer_b200 import _lib as L

    m, n, k, parts = 160, 1024, 512, 4
    a, w, b = _inputs(m, n, k, 5)
    wc, ws, gw = O.quantize_weight(w)
    ga = O.global_scale(O.amax_bf16(a))
    abuf = backend.upload(a)
    out = backend.allocate(m * n * 2)
    sc = backend.scope()
    sc.act_quant_shared(abuf, m, k, ga)
    nl = n // parts
    Ws = []
    for p in range(parts):
        # each slice is quantised with the FULL tensor's scale: upload the oracle's packed slice
        Wp = T.Nvfp4Weight.from_packed(backend, wc[p * nl:(p + 1) * nl], ws[p * nl:(p + 1) * nl], gw, b[p * nl:(p + 1) * nl])
        Ws.append(Wp)
        sc.linear(None, m, Wp, ga, out, n_offset=p * nl, ldo=n, flags=L.LINEAR_A_PREQUANTIZED)
    backend.submit(30000)
    got = backend.read_buffer(out, np.uint16).reshape(m, n)
    want = O.linear(a, ga, wc, ws, gw, bias=b)
    assert rel_fro(O.bf16_to_f32(got), O.bf16_to_f32(want)) <= TOL
    for Wp in Ws:
        Wp.free(backend)
    backend.free(abuf)
    backend.free(out)


@pytest.mark.parametrize("m,hidden,ffn", [(256, 512, 1024), (200, 256, 320), (96, 128, 192)])
def test_fused_output_quantisation_mlp(backend, m, hidden, ffn):
    """MLP up -> GELU -> down with the up epilogue emitting the down's NVFP4 operand: the emitted
    codes/scales must equal what the standalone quantiser makes of the bf16 output, bit for bit,
    and the down result must match the oracle chain."""
    import thinfer_b200 as T
    from thinfer_b200.backend import device_scales_bytes
    from conftest import dev_scales_to_canonical

    a, w1, b1 = _inputs(m, ffn, hidden, 21)
    _, w2, b2 = _inputs(m, hidden, ffn, 22)
    be = backend
    W1, W2 = T.Nvfp4Weight.from_dense(be, w1, b1), T.Nvfp4Weight.from_dense(be, w2, b2)
    ga, g_mid = O.global_scale(O.amax_bf16(a)), 0.0009765625
    abuf = be.upload(a)
    mid = be.allocate(m * ffn * 2)
    qc = be.allocate(m * ffn // 2)
    qs = be.allocate(device_scales_bytes(m, ffn))
    be.write_buffer(qs, np.full(qs.len, 0x7F, np.uint8))  # NaN canary in every scale byte
    out = be.allocate(m * hidden * 2)
    sc = be.scope()
    sc.linear(abuf, m, W1, ga, mid, act=1, out_nvfp4=(qc, qs, g_mid))
    sc.matmul(qc, qs, m, W2, g_mid, out)
    be.submit(30000)
    mid_h = be.read_buffer(mid, np.uint16).reshape(m, ffn)
    codes = be.read_buffer(qc).reshape(m, ffn // 2)
    scales = dev_scales_to_canonical(be.read_buffer(qs), m, ffn)
    oc, os_ = O.quantize_act(mid_h, g_mid)  # oracle quantiser on the GPU's own bf16 output
    assert np.array_equal(codes, oc) and np.array_equal(scales, os_)
    got = be.read_buffer(out, np.uint16).reshape(m, hidden)
    assert not np.isnan(O.bf16_to_f32(got)).any()
    # bf16-free variant gives the same final result
    out2 = be.allocate(m * hidden * 2)
    sc.linear(abuf, m, W1, ga, None, act=1, out_nvfp4=(qc, qs, g_mid))
    sc.matmul(qc, qs, m, W2, g_mid, out2)
    be.submit(30000)
    assert np.array_equal(be.read_buffer(out2, np.uint16).reshape(m, hidden), got)
    # oracle chain
    w1c, w1s, g1 = O.quantize_weight(w1)
    w2c, w2s, g2 = O.quantize_weight(w2)
    mid_o = O.linear(a, ga, w1c, w1s, g1, bias=b1, act=1)
    want = O.linear(mid_o, g_mid, w2c, w2s, g2, bias=b2)
    assert rel_fro(O.bf16_to_f32(got), O.bf16_to_f32(want)) <= 5e-3  # GELU approximation flips a few FP4 codes
    for b in (abuf, mid, qc, qs, out, out2):
        be.free(b)
    W1.free(be)
    W2.free(be)


def test_fused_output_quantisation_column_windows(backend):
    """An N-split linear fills its own column window of the NVFP4 copy ([m, ldo] operand, columns
    n_offset .. n_offset+n): two window calls must leave the bytes one whole call leaves."""
    import thinfer_b200 as T
    from thinfer_b200.backend import device_scales_bytes

    m, hidden, ffn = 300, 256, 512
    a, w1, b1 = _inputs(m, ffn, hidden, 31)
    be = backend
    wc, ws, gw = O.quantize_weight(w1)
    ga, g_mid = O.global_scale(O.amax_bf16(a)), 0.0009765625
    abuf = be.upload(a)
    sc = be.scope()
    whole = T.Nvfp4Weight.from_packed(be, wc, ws, gw, b1)
    qc0, qs0 = be.allocate(m * ffn // 2), be.allocate(device_scales_bytes(m, ffn))
    be.write_buffer(qs0, np.zeros(qs0.len, np.uint8))  # rows past m of the last 128-row block are never written
    sc.linear(abuf, m, whole, ga, None, act=1, out_nvfp4=(qc0, qs0, g_mid))
    qc1, qs1 = be.allocate(m * ffn // 2), be.allocate(device_scales_bytes(m, ffn))
    be.write_buffer(qc1, np.full(qc1.len, 0xEE, np.uint8))
    be.write_buffer(qs1, np.zeros(qs1.len, np.uint8))
    halves = []
    for off in (0, ffn // 2):
        Wh = T.Nvfp4Weight.from_packed(be, wc[off:off + ffn // 2], ws[off:off + ffn // 2], gw, b1[off:off + ffn // 2])
        halves.append(Wh)
        sc.linear(abuf, m, Wh, ga, None, act=1, n_offset=off, ldo=ffn, out_nvfp4=(qc1, qs1, g_mid))
    be.submit(30000)
    assert np.array_equal(be.read_buffer(qc1), be.read_buffer(qc0))
    assert np.array_equal(be.read_buffer(qs1), be.read_buffer(qs0))
    with pytest.raises(T.backend.InvalidArgument):  # windows of the NVFP4 copy move in whole 64-column groups
        sc.linear(abuf, m, halves[1], ga, None, act=1, n_offset=32, ldo=ffn, out_nvfp4=(qc1, qs1, g_mid))
    for b in (abuf, qc0, qs0, qc1, qs1):
        be.free(b)
    for Wp in [whole] + halves:
        Wp.free(be)


def test_fused_output_quantisation_windows_keep_earlier_scales(backend):
    """ldo = 320 is five 64-column groups, so the scale layout pads every 128-row block to eight atoms and each
    window call clears the padding. A later window must not wipe the scales an earlier window wrote into the same
    buffer: two windows (192 + 128 columns) into canary-filled buffers equal one whole call, and the down
    projection that consumes the copy matches the oracle (stale or NaN padding scales would poison it)."""
    import thinfer_b200 as T
    from thinfer_b200.backend import device_scales_bytes
    from conftest import dev_scales_to_canonical

    m, hidden, ffn = 300, 256, 320
    a, w1, b1 = _inputs(m, ffn, hidden, 33)
    _, w2, b2 = _inputs(m, hidden, ffn, 34)
    be = backend
    wc, ws, gw = O.quantize_weight(w1)
    ga, g_mid = O.global_scale(O.amax_bf16(a)), 0.0009765625
    abuf = be.upload(a)
    sc = be.scope()
    W2 = T.Nvfp4Weight.from_dense(be, w2, b2)
    qc, qs = be.allocate(m * ffn // 2), be.allocate(device_scales_bytes(m, ffn))
    mid = be.allocate(m * ffn * 2)
    be.write_buffer(qc, np.full(qc.len, 0xEE, np.uint8))
    be.write_buffer(qs, np.full(qs.len, 0x7F, np.uint8))  # NaN canary in every scale byte, padding included
    parts = []
    for off, width in ((0, 192), (192, 128)):
        Wp = T.Nvfp4Weight.from_packed(be, wc[off:off + width], ws[off:off + width], gw, b1[off:off + width])
        parts.append(Wp)
        sc.linear(abuf, m, Wp, ga, mid, act=1, n_offset=off, ldo=ffn, out_nvfp4=(qc, qs, g_mid))
    out = be.allocate(m * hidden * 2)
    sc.matmul(qc, qs, m, W2, g_mid, out)
    be.submit(30000)
    mid_h = be.read_buffer(mid, np.uint16).reshape(m, ffn)
    oc, os_ = O.quantize_act(mid_h, g_mid)
    assert np.array_equal(be.read_buffer(qc).reshape(m, ffn // 2), oc)
    dev = be.read_buffer(qs)
    assert np.array_equal(dev_scales_to_canonical(dev, m, ffn), os_)  # both windows' scales are there
    atoms = dev.reshape(-1, 8, 512)  # [128-row block][atom][byte]
    assert not atoms[:, 5:, :].any()  # K-padding atoms are zero
    got = be.read_buffer(out, np.uint16).reshape(m, hidden)
    w2c, w2s, g2 = O.quantize_weight(w2)
    want = O.linear(mid_h, g_mid, w2c, w2s, g2, bias=b2)
    assert not np.isnan(O.bf16_to_f32(got)).any()
    assert rel_fro(O.bf16_to_f32(got), O.bf16_to_f32(want)) <= TOL
    for b in (abuf, qc, qs, mid, out):
        be.free(b)
    for Wp in parts + [W2]:
        Wp.free(be)


def test_prequantized_call_needs_matching_scratch(backend):
    """TNF_LINEAR_A_PREQUANTIZED reads the context's shared scratch; the scratch is tagged with the shape it was
    filled for, and a call for any other shape is refused instead of multiplying stale codes."""
    import thinfer_b200 as T
    from thinfer_b200 import _lib as L
    from thinfer_b200.backend import InvalidArgument

    be = backend
    a, w, b = _inputs(256, 128, 512, 3)
    a2, w2, b2 = _inputs(64, 128, 256, 4)
    W, W2 = T.Nvfp4Weight.from_dense(be, w, b), T.Nvfp4Weight.from_dense(be, w2, b2)
    abuf, a2buf = be.upload(a), be.upload(a2)
    out = be.allocate(256 * 128 * 2)
    sc = be.scope()
    sc.linear(abuf, 256, W, 0.002, out)  # grows the scratch beyond what the smaller problem needs
    with pytest.raises(InvalidArgument):
        sc.linear(None, 64, W2, 0.002, out, flags=L.LINEAR_A_PREQUANTIZED)
    sc.act_quant_shared(a2buf, 64, 256, 0.002)
    sc.linear(None, 64, W2, 0.002, out, flags=L.LINEAR_A_PREQUANTIZED)
    be.submit(30000)
    for buf in (abuf, a2buf, out):
        be.free(buf)
    W.free(be)
    W2.free(be)


def test_linearity_and_zero_activation(backend):
    """Size-independent properties: a zero A gives exactly the bias; doubling A's per-tensor
    scale with the same codes doubles the pre-bias result."""
    m, n, k = 256, 512, 1024
    a, w, b = _inputs(m, n, k, 9)
    got0, _, _ = _run(backend, np.zeros_like(a), w, b)
    assert np.array_equal(got0, np.tile(b, (m, 1)))
    got1, ga, gw = _run(backend, a, w, None)
    a2 = O.f32_to_bf16(O.bf16_to_f32(a) * np.float32(2.0))
    got2, ga2, _ = _run(backend, a2, w, None)
    assert ga2 == np.float32(ga) * 2
    assert np.array_equal(O.bf16_to_f32(got2), O.bf16_to_f32(got1) * 2)


def test_budget_and_argument_errors(backend):
    import thinfer_b200 as T
    from thinfer_b200.backend import BudgetExceeded, InvalidArgument

    small = T.Backend(0, vram_budget=1 << 20)
    b1 = small.allocate_in(512 << 10, 0)
    with pytest.raises(BudgetExceeded):
        small.allocate_in(768 << 10, 1)  # refused on the host, before the device is touched
    snap = small.mem_snapshot()
    assert snap["live_weights"] == 512 << 10 and snap["true_peak"] == 512 << 10
    small.free(b1)
    small.close()
    a, w, b = _inputs(32, 64, 64, 1)
    W = T.Nvfp4Weight.from_dense(backend, w, b)
    abuf = backend.upload(a)
    out = backend.allocate(32 * 64 * 2)
    with pytest.raises(InvalidArgument):
        backend.scope().linear(abuf, 32, W, 0.0, out)  # activation scale must be > 0
    with pytest.raises(InvalidArgument):
        backend.scope().linear(abuf, 64, W, 1.0, out)  # views too small for m=64
    W.free(backend)
    backend.free(abuf)
    backend.free(out)
