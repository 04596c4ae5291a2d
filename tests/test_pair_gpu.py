"""The CTA-pair kernel against the CPU oracle at the sizes that select it.

Every large-M linear (and every launch the benchmark times) runs nvfp4_gemm_pair_kernel: 256x256
tiles on SM pairs, a persistent loop in which a pair takes several tiles and alternates between two
accumulators that overlap in tensor memory. These tests give the pairs more tiles than there are
pairs (74 on a B200), so the second and third tile of a pair, both accumulator parities and every
epilogue variant are compared with the oracle; then the BASELINE shapes themselves run at full size
and a sample of rows from the first, a middle and the last row tile (the ragged one) is compared.
Rows of a linear are independent once the per-tensor activation scale is given, so the oracle only
has to evaluate the sampled rows.

Tolerance: relative Frobenius error <= 1e-3; in fact almost every output is bit-equal (the products
are exact in f32, only the summation order differs)."""
import numpy as np
import pytest

import oracle as O
from conftest import dev_scales_to_canonical, rel_fro

pytestmark = pytest.mark.gpu
TOL = 1e-3
G_MID = 0.0009765625  # static per-tensor scale of a GELU output (2^-10)


def _inputs(m, n, k, seed, bias=True):
    a = O.f32_to_bf16(O.gaussian(m * k, 0xA000 + seed).reshape(m, k))
    w = (O.gaussian(n * k, 0xB000 + seed) * np.float32(0.02)).reshape(n, k)
    b = O.f32_to_bf16(O.gaussian(n, 0xC000 + seed) * np.float32(0.01)) if bias else None
    return a, w, b


def _sample_rows(m, per_slab=86):
    """Row indices: the first rows, a slab around the middle, and the last rows (the ragged tile)."""
    if m <= 3 * per_slab:
        return np.arange(m)
    mid = (m // 2) // 256 * 256 + 100
    return np.concatenate([np.arange(per_slab), np.arange(mid, mid + per_slab), np.arange(m - per_slab, m)])


def _read_rows(be, buf, rows, row_bytes, dtype):
    """Reads the given rows (contiguous slabs) of a row-major device buffer."""
    out = []
    start = prev = int(rows[0])
    for r in list(rows[1:]) + [None]:
        if r is None or r != prev + 1:
            out.append(be.read_buffer(buf, dtype, count=(prev + 1 - start) * row_bytes // np.dtype(dtype).itemsize,
                                      offset=start * row_bytes))
            start = r
        prev = r
    return np.concatenate(out)


MODES = ["plain", "gelu", "chain", "gelu_chain", "gate", "gelu_gate", "chain_gate", "gelu_chain_gate"]


@pytest.mark.parametrize("mode", MODES)
def test_pair_multi_tile_epilogue_modes(backend, mode):
    """2304 x 4608 x 512: 162 pair tiles on 74 pairs, so pairs run a second and a third tile; the eight
    bf16 epilogue variants (GELU x chain x gated residual) over all rows."""
    import thinfer_b200 as T

    m, n, k = 2304, 4608, 512
    a, w, b = _inputs(m, n, k, 41)
    wc, ws, gw = O.quantize_weight(w)
    ga = O.global_scale(O.amax_bf16(a))
    be = backend
    W = T.Nvfp4Weight.from_packed(be, wc, ws, gw, b)
    abuf = be.upload(a)
    out = be.allocate(m * n * 2)
    be.write_buffer(out, np.full(m * n, 0x7FC0, np.uint16))  # NaN canary
    kw, okw, extra = {}, {}, []
    if "gelu" in mode:
        kw["act"] = okw["act"] = 1
    if "chain" in mode:
        kw["chain"] = okw["chain"] = True
    if "gate" in mode:
        gate = O.f32_to_bf16(O.gaussian(n, 0xD000))
        res = O.f32_to_bf16(O.gaussian(m * n, 0xE000).reshape(m, n))
        gb, rb = be.upload(gate), be.upload(res)
        extra = [gb, rb]
        kw.update(gate=gb, residual=rb)
        okw.update(gate=gate, residual=res)
    be.scope().linear(abuf, m, W, ga, out, **kw)
    be.submit(30000)
    got = be.read_buffer(out, np.uint16).reshape(m, n)
    want = O.linear(a, ga, wc, ws, gw, bias=b, **okw)
    assert not np.isnan(O.bf16_to_f32(got)).any()
    assert rel_fro(O.bf16_to_f32(got), O.bf16_to_f32(want)) <= TOL
    # fused GELU uses the hardware tanh approximation; chain mode evaluates the reference's formula with tanhf
    floor = 0.9 if mode in ("gelu", "gelu_gate") else 0.99
    assert (got == want).mean() > floor
    for buf in [abuf, out] + extra:
        be.free(buf)
    W.free(be)


@pytest.mark.parametrize("act,gated", [(1, False), (0, True)])
def test_pair_ragged_shape(backend, act, gated):
    """2100 x 2312 x 320: a ragged last row tile (52 rows), a ragged last column tile (8 columns) and a K that
    is not a multiple of the 256-element stage; 90 pair tiles."""
    import thinfer_b200 as T

    m, n, k = 2100, 2312, 320
    a, w, b = _inputs(m, n, k, 43)
    wc, ws, gw = O.quantize_weight(w)
    ga = O.global_scale(O.amax_bf16(a))
    be = backend
    W = T.Nvfp4Weight.from_packed(be, wc, ws, gw, b)
    abuf = be.upload(a)
    out = be.allocate((m + 1) * n * 2)
    be.write_buffer(out, np.full((m + 1) * n, 0x7FC0, np.uint16))
    kw, okw, extra = {"act": act}, {"act": act}, []
    if gated:
        gate = O.f32_to_bf16(O.gaussian(n, 0xD100))
        res = O.f32_to_bf16(O.gaussian(m * n, 0xE100).reshape(m, n))
        gb, rb = be.upload(gate), be.upload(res)
        extra = [gb, rb]
        kw.update(gate=gb, residual=rb)
        okw.update(gate=gate, residual=res)
    be.scope().linear(abuf, m, W, ga, out, **kw)
    be.submit(30000)
    full = be.read_buffer(out, np.uint16).reshape(m + 1, n)
    assert (full[m] == 0x7FC0).all()  # nothing is written past the last row
    want = O.linear(a, ga, wc, ws, gw, bias=b, **okw)
    assert rel_fro(O.bf16_to_f32(full[:m]), O.bf16_to_f32(want)) <= TOL
    assert (full[:m] == want).mean() > (0.9 if act else 0.99)
    for buf in [abuf, out] + extra:
        be.free(buf)
    W.free(be)


def test_pair_multi_tile_nvfp4_output(backend):
    """MLP up -> GELU -> down at 2304 rows with the up epilogue emitting the down operand in NVFP4 on a
    multi-tile launch: the codes and scales equal the oracle quantiser's on the kernel's own bf16 output."""
    import thinfer_b200 as T
    from thinfer_b200.backend import device_scales_bytes

    m, hidden, ffn = 2304, 512, 4608
    a, w1, b1 = _inputs(m, ffn, hidden, 51)
    _, w2, b2 = _inputs(8, hidden, ffn, 52)
    be = backend
    W1, W2 = T.Nvfp4Weight.from_dense(be, w1, b1), T.Nvfp4Weight.from_dense(be, w2, b2)
    ga = O.global_scale(O.amax_bf16(a))
    abuf = be.upload(a)
    mid, out = be.allocate(m * ffn * 2), be.allocate(m * hidden * 2)
    qc, qs = be.allocate(m * ffn // 2), be.allocate(device_scales_bytes(m, ffn))
    be.write_buffer(qs, np.full(qs.len, 0x7F, np.uint8))
    sc = be.scope()
    sc.linear(abuf, m, W1, ga, mid, act=1, out_nvfp4=(qc, qs, G_MID))
    sc.matmul(qc, qs, m, W2, G_MID, out)
    be.submit(30000)
    mid_h = be.read_buffer(mid, np.uint16).reshape(m, ffn)
    oc, os_ = O.quantize_act(mid_h, G_MID)
    assert np.array_equal(be.read_buffer(qc).reshape(m, ffn // 2), oc)
    assert np.array_equal(dev_scales_to_canonical(be.read_buffer(qs), m, ffn), os_)
    w1c, w1s, g1 = O.quantize_weight(w1)
    w2c, w2s, g2 = O.quantize_weight(w2)
    assert rel_fro(O.bf16_to_f32(mid_h), O.bf16_to_f32(O.linear(a, ga, w1c, w1s, g1, bias=b1, act=1))) <= TOL
    got = be.read_buffer(out, np.uint16).reshape(m, hidden)
    want = O.linear(mid_h, G_MID, w2c, w2s, g2, bias=b2)  # the oracle's down projection on the kernel's own H
    assert rel_fro(O.bf16_to_f32(got), O.bf16_to_f32(want)) <= TOL
    for buf in (abuf, mid, out, qc, qs):
        be.free(buf)
    W1.free(be)
    W2.free(be)


# BASELINE shapes at full size: (name, m, k, n, act). C2 = Qwen-Image block linears at 4352 rows, C3 = Wan FFN
# at 6630 rows (ragged last tile: 6630 = 25*256 + 230), C5 = one rank's 1/8 column slice of the batched Wan FFN.
BASELINE_SHAPES = [
    ("c2_qkv", 4352, 3072, 9216, 0), ("c2_out", 4352, 3072, 3072, 0), ("c2_up", 4352, 3072, 12288, 1),
    ("c2_down", 4352, 12288, 3072, 0), ("c3_up", 6630, 3072, 14336, 1), ("c3_down", 6630, 14336, 3072, 0),
    ("c5_up_slice", 26520, 3072, 1792, 1),
]


@pytest.mark.parametrize("name,m,k,n,act", BASELINE_SHAPES)
def test_baseline_shapes_sampled_rows(backend, name, m, k, n, act):
    import thinfer_b200 as T

    seed = 60 + [s[0] for s in BASELINE_SHAPES].index(name)
    a, w, b = _inputs(m, n, k, seed)
    be = backend
    W = T.Nvfp4Weight.from_dense(be, w, b, keep_canonical=True)
    wc, ws, gw = O.quantize_weight(w)
    assert np.float32(W.global_scale) == np.float32(gw)
    assert np.array_equal(be.read_buffer(W.codes).reshape(n, k // 2), wc)  # weight quantiser bit-exact at full size
    assert np.array_equal(be.read_buffer(W.scales_canonical).reshape(n, k // 16), ws)
    ga = O.global_scale(O.amax_bf16(a))
    abuf = be.upload(a)
    out = be.allocate(m * n * 2)
    be.scope().linear(abuf, m, W, ga, out, act=act)
    be.submit(60000)
    rows = _sample_rows(m)
    got = _read_rows(be, out, rows, n * 2, np.uint16).reshape(len(rows), n)
    want = O.linear(a[rows], ga, wc, ws, gw, bias=b, act=act)
    assert not np.isnan(O.bf16_to_f32(got)).any()
    err = rel_fro(O.bf16_to_f32(got), O.bf16_to_f32(want))
    assert err <= TOL, f"{name}: relative Frobenius error {err:.3e}"
    assert (got == want).mean() > (0.9 if act else 0.99)
    be.free(abuf)
    be.free(out)
    W.free(be)


def test_c2_mlp_chain_with_nvfp4_handoff(backend):
    """The benchmark's MLP at 4352 rows exactly as it is timed: up 3072 -> 12288 + bias + GELU whose epilogue
    emits only the NVFP4 operand (no bf16 store), then down 12288 -> 3072 on that operand. Sampled rows of the
    final output against the oracle chain; the GELU approximation may flip a few FP4 codes of H."""
    import thinfer_b200 as T
    from thinfer_b200.backend import device_scales_bytes

    m, hidden, ffn = 4352, 3072, 12288
    a, w1, b1 = _inputs(m, ffn, hidden, 71)
    _, w2, b2 = _inputs(8, hidden, ffn, 72)
    be = backend
    W1, W2 = T.Nvfp4Weight.from_dense(be, w1, b1), T.Nvfp4Weight.from_dense(be, w2, b2)
    ga = O.global_scale(O.amax_bf16(a))
    abuf = be.upload(a)
    out = be.allocate(m * hidden * 2)
    qc, qs = be.allocate(m * ffn // 2), be.allocate(device_scales_bytes(m, ffn))
    sc = be.scope()
    sc.linear(abuf, m, W1, ga, None, act=1, out_nvfp4=(qc, qs, G_MID))
    sc.matmul(qc, qs, m, W2, G_MID, out)
    be.submit(60000)
    rows = _sample_rows(m)
    got = _read_rows(be, out, rows, hidden * 2, np.uint16).reshape(len(rows), hidden)
    w1c, w1s, g1 = O.quantize_weight(w1)
    w2c, w2s, g2 = O.quantize_weight(w2)
    h = O.linear(a[rows], ga, w1c, w1s, g1, bias=b1, act=1)
    want = O.linear(h, G_MID, w2c, w2s, g2, bias=b2)
    codes = _read_rows(be, qc, rows, ffn // 2, np.uint8).reshape(len(rows), ffn // 2)
    oc, _ = O.quantize_act(h, G_MID)
    assert (codes == oc).mean() > 0.995  # H codes: only GELU-approximation flips
    assert rel_fro(O.bf16_to_f32(got), O.bf16_to_f32(want)) <= 5e-3
    for buf in (abuf, out, qc, qs):
        be.free(buf)
    W1.free(be)
    W2.free(be)
