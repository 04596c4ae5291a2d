"""Pins the CPU oracle against what the reference itself fixes: its committed conformance
fixtures and the properties its own unit tests assert. CPU only."""
import numpy as np
import pytest

import oracle as O
from conftest import rel_fro

TOL = 1e-5  # thinfer-core/src/conformance.rs:1308-1319: one tolerance for all three dtypes


# ---- committed fixtures (thinfer-conformance/fixtures/*.safetensors) ---------------------
@pytest.mark.parametrize("variant", ["fp32", "bf16w"])
def test_matmul_basic_fixture(golden_ref, variant):
    a, b, out = (golden_ref[f"{variant}/matmul_basic/{x}"] for x in "a b out".split())
    got = O.gemm_f32(a, np.ascontiguousarray(b.T))  # fixture b is [K,N]; oracle takes [N,K]
    if variant == "bf16w":  # fp32 inputs, output RNE-rounded through bf16 (stored as f32)
        got = O.bf16_to_f32(O.f32_to_bf16(got))
        # a sum that lands within 1e-5 of a bf16 tie may round either way
        assert (np.abs(got - out) <= 2.0 ** -7 * np.abs(out) + TOL).all() and (got == out).mean() >= 0.9
    else:
        assert np.abs(got - out).max() <= TOL


def test_matmul_basic_fixture_bf16p(golden_ref):
    a, b, out = (golden_ref[f"bf16p/matmul_basic/{x}"] for x in "a b out".split())
    got = O.gemm_f32(O.bf16_to_f32(a), np.ascontiguousarray(O.bf16_to_f32(b).T))
    assert np.array_equal(O.f32_to_bf16(got), out)  # f32 accumulate, one RNE narrowing


@pytest.mark.parametrize("variant", ["fp32", "bf16w"])
def test_bias_add_fixture(golden_ref, variant):
    x, s, out = (golden_ref[f"{variant}/bcast_add/{k}"] for k in "x s out".split())
    got = O.bf16_to_f32(O.epilogue(x, 1.0, bias=O.f32_to_bf16(s)))
    # the oracle's epilogue narrows to bf16: compare at bf16 resolution of the fixture
    assert np.abs(got - out).max() <= 2.0 ** -8 * np.abs(out).max() + TOL


def test_bias_add_fixture_bf16p(golden_ref):
    x, s, out = (golden_ref[f"bf16p/bcast_add/{k}"] for k in "x s out".split())
    got = O.epilogue(O.bf16_to_f32(x), 1.0, bias=s)
    assert np.array_equal(got, out)


def test_gated_residual_fixture_bf16p(golden_ref):
    keys = [k for k in golden_ref.files if k.startswith("bf16p/bcast_fma/")]
    if not keys:
        pytest.skip("reference fixtures hold no bcast_fma case")
    x, s, y, out = (golden_ref[f"bf16p/bcast_fma/{k}"] for k in "x s y out".split())
    # out = x + s*y ; oracle: residual + gate * v with v = acc
    yf = O.bf16_to_f32(y).reshape(x.shape)
    got = O.epilogue(yf, 1.0, gate=s.reshape(-1), residual=x)
    assert np.array_equal(got, out)


@pytest.mark.parametrize("variant", ["fp32", "bf16w", "bf16p"])
def test_layernorm_fixture(golden_ref, variant):
    """layernorm_basic (eps 1e-6, thinfer-conformance/fixtures/spec.json): the restated two-pass LayerNorm."""
    x, out = golden_ref[f"{variant}/layernorm_basic/x"], golden_ref[f"{variant}/layernorm_basic/out"]
    got = O.ref_layernorm(x, 1e-6)
    if variant == "bf16p":
        g, e = O.bf16_to_f32(got), O.bf16_to_f32(out)
        # torch's reduction order differs from the kernel's sequential sums: at most one bf16 step apart
        assert (np.abs(g - e) <= 2.0 ** -7 * np.abs(e) + TOL).all() and (got == out).mean() >= 0.9
    elif variant == "bf16w":  # f32 in, output narrowed through bf16
        assert (np.abs(got - out) <= 2.0 ** -7 * np.abs(out) + TOL).all()
    else:
        assert np.abs(got - out).max() <= TOL


SDPA_SCALES = {"sdpa_basic": 0.35355338, "sdpa_large_d_d128": 0.088388346, "sdpa_decode_sq1": 0.35355338,
               "sdpa_decode_multirow": 0.35355338}  # thinfer-conformance/fixtures/spec.json


@pytest.mark.parametrize("case", sorted(SDPA_SCALES))
@pytest.mark.parametrize("variant", ["fp32", "bf16w", "bf16p"])
def test_sdpa_fixture(golden_ref, variant, case):
    """The reference's attention cases (thinfer-core/src/ops/sdpa.rs test_cases, zero masks, GQA-free): the restated
    online-softmax SDPA against the committed outputs. sdpa_large_d_d128 has no packed-bf16 variant."""
    key = f"{variant}/{case}/q"
    if key not in golden_ref.files:
        pytest.skip("the reference's fixtures hold no such variant")
    q, k, v, mask, out = (golden_ref[f"{variant}/{case}/{t}"] for t in "q k v mask out".split())
    got = O.ref_sdpa(q, k, v, SDPA_SCALES[case], mask=mask)
    no_mask = O.ref_sdpa(q, k, v, SDPA_SCALES[case])
    assert np.array_equal(got, no_mask)  # the fixtures' masks are zero: mode 0 and mode 1 agree bit for bit
    if variant == "bf16p":
        g, e = O.bf16_to_f32(got), O.bf16_to_f32(out)
        assert (np.abs(g - e) <= 2.0 ** -7 * np.abs(e) + TOL).all() and (got == out).mean() >= 0.9
    elif variant == "bf16w":
        assert (np.abs(got - out) <= 2.0 ** -7 * np.abs(out) + TOL).all()
    else:
        assert np.abs(got - out).max() <= 1e-5


@pytest.mark.parametrize("variant", ["fp32", "bf16w", "bf16p"])
def test_bcast_modulate_fixture(golden_ref, variant):
    """bcast_modulate (bias 1.0): out = x * (s + 1) + t."""
    x, s, t, out = (golden_ref[f"{variant}/bcast_modulate/{k}"] for k in "x s t out".split())
    got = O.ref_bcast_modulate(x, s, t, 1.0)
    if variant == "bf16p":
        g, e = O.bf16_to_f32(got), O.bf16_to_f32(out)
        assert (np.abs(g - e) <= 2.0 ** -7 * np.abs(e) + TOL).all() and (got == out).mean() >= 0.9
    elif variant == "bf16w":
        assert (np.abs(got - out) <= 2.0 ** -7 * np.abs(out) + TOL).all()
    else:
        assert np.abs(got - out).max() <= TOL


def test_norm_modulate_fused_equals_the_two_dispatches():
    """The fused oracle routine in chain mode is the two restated dispatches back to back, bit for bit."""
    x = O.f32_to_bf16(O.gaussian(37 * 96, 5).reshape(37, 96) * np.float32(3.0) + np.float32(0.5))
    s = O.f32_to_bf16(O.gaussian(96, 6) * np.float32(0.3))
    t = O.f32_to_bf16(O.gaussian(96, 7) * np.float32(0.2))
    two = O.ref_bcast_modulate(O.ref_layernorm(x, 1e-6), s, t, 1.0)
    assert np.array_equal(O.norm_modulate(x, s, t, 1e-6, 1.0, chain=True), two)
    fused = O.bf16_to_f32(O.norm_modulate(x, s, t, 1e-6, 1.0, chain=False))
    assert rel_fro(fused, O.bf16_to_f32(two)) <= 4e-3  # one bf16 rounding less
    assert np.array_equal(O.norm_modulate(x, None, None, 1e-6), O.ref_layernorm(x, 1e-6))


def test_gelu_fixture(golden_ref):
    a, b, out = (golden_ref[f"fp32/gelu_mul_basic/{k}"] for k in "a b out".split())
    # fixture = gelu_tanh(a) * b ; take the oracle's GELU through its epilogue (bf16 out)
    g = O.bf16_to_f32(O.epilogue(a.reshape(1, -1), 1.0, act=1)).reshape(-1)
    ref_gelu = np.where(np.abs(b) > 1e-6, out / np.where(b == 0, 1, b), np.nan)
    ok = ~np.isnan(ref_gelu)
    assert np.abs(g[ok] - ref_gelu[ok]).max() <= 2.0 ** -8 * np.abs(ref_gelu[ok]).max() + 1e-4


# ---- properties of the reference's own unit tests ------------------------------------------
def test_q8_0_encode_roundtrip_bound():
    # thinfer-core/src/quant.rs:1314-1334 (encode_q8_0_roundtrip)
    vals = ((np.arange(64, dtype=np.float32)) - np.float32(31.5)) * np.float32(0.37)
    src = O.f32_to_bf16(vals)
    q = O.ref_encode_q8_0_from_bf16(src)
    deq = O.ref_dequantize_row_q8_0(q)
    want = O.bf16_to_f32(src)
    for bi in range(2):
        d = O.ref_f16_to_f32(int(q[bi * 34]) | (int(q[bi * 34 + 1]) << 8))
        err = np.abs(deq[bi * 32:(bi + 1) * 32] - want[bi * 32:(bi + 1) * 32])
        assert (err <= d * (0.5 + 127.0 / 2048.0) + 1e-6).all()


def test_q8_0_zero_block():
    # thinfer-core/src/quant.rs:1337-1344 (encode_q8_0_zero_block)
    assert not O.ref_encode_q8_0_from_bf16(np.zeros(32, np.uint16)).any()
    # the NVFP4 quantiser keeps the same rule: zero scale, zero codes
    c, s, g = O.quantize_weight(np.zeros((2, 32), np.float32))
    assert not c.any() and not s.any() and g == 1.0


def test_q4_0_matmul_reference_shapes():
    # thinfer-conformance/tests/q4_0_matmul.rs:178-200: GPU-vs-CPU there; here the restated
    # dequant+GEMM must agree with an f64 evaluation within the reference's tol = 1e-5*K.
    for (m, n, k, seed) in [(16, 16, 32, 0xC0FFEE), (10, 10, 32, 0xBEEF), (8, 8, 128, 0xDEAD), (24, 48, 96, 0x12345678)]:
        lcg = O.RefLcg(seed)
        a = lcg.fill(m * k, 0.5).reshape(m, k)
        b = lcg.fill(n * k, 0.5).reshape(n, k)
        bq = np.concatenate([O.ref_quantize_row_q4_0(b[i]) for i in range(n)])
        bd = O.ref_dequantize_row_q4_0(bq).reshape(n, k)
        got = O.gemm_f32(a, bd)
        want = a.astype(np.float64) @ bd.astype(np.float64).T
        assert np.abs(got - want).max() <= 1e-5 * k
        # quantisation error bound of Q4_0: half a step of d = |max|/8 per element
        assert np.abs(bd - b).max() <= np.abs(b).max() / 8.0 * 0.5 + 1e-3


def test_act_quant_i8_reference_cases():
    # thinfer-conformance/tests/act_quant_i8.rs:225-268: (2,64,0xC0FFEE), (3,128,0xBEEF)
    for (m, k, seed) in [(2, 64, 0xC0FFEE), (3, 128, 0xBEEF)]:
        raw = O.RefLcg(seed).fill(m * k, 0.5)
        a = np.array([O.ref_f16_to_f32(O.ref_f16_from_f32(float(v))) for v in raw], np.float32).reshape(m, k)
        q, params = O.ref_act_quant_i8(a)
        s, z = params[..., 0], params[..., 1]
        deq = q.reshape(m, k // 32, 32) * s[..., None] + z[..., None]
        err = np.abs(deq.reshape(m, k) - a)
        assert (err <= 0.51 * np.repeat(s, 32, axis=1) + 1e-3).all()
        assert q.min() >= -127 and q.max() <= 127
        # parameters are stored at f16 precision before the codes are computed
        for v in s.ravel():
            assert O.ref_f16_to_f32(O.ref_f16_from_f32(float(v))) == v


def test_matmul_i8_reference_case():
    # thinfer-conformance/tests/matmul_i8.rs:318-379 shapes; restated reference vs f64
    m, n, k = 8, 8, 64
    lcg = O.RefLcg(0xDEADBEEF)
    a = lcg.fill(m * k, 0.5).reshape(m, k)
    b = lcg.fill(n * k, 0.5).reshape(n, k)
    qa, pa = O.ref_act_quant_i8(a)
    bq = np.concatenate([O.ref_quantize_row_q8_0(b[i]) for i in range(n)]).reshape(n, k // 32, 34)
    qb = bq[:, :, 2:].view(np.int8).reshape(n, k)
    sb = np.array([[O.ref_f16_to_f32(int(bq[i, t, 0]) | (int(bq[i, t, 1]) << 8)) for t in range(k // 32)] for i in range(n)], np.float32)
    got = O.ref_matmul_i8(qa, pa[..., 0], pa[..., 1], qb, sb)
    want = a.astype(np.float64) @ b.astype(np.float64).T
    assert np.abs(got - want).max() <= max(5e-3 * np.abs(want).max(), 1e-4) * 4  # quantisation noise of both sides


def test_f16_roundtrip_all_bit_patterns():
    # half 2.7.1 behaviour pinned by thinfer-core/src/weight.rs:269-336
    import torch
    bits = np.arange(0, 0x7C00, dtype=np.uint16)
    f = torch.from_numpy(bits.view(np.int16)).view(torch.float16).float().numpy()
    for i in range(0, len(bits), 97):
        assert O.ref_f16_to_f32(int(bits[i])) == f[i]
        assert O.ref_f16_from_f32(float(f[i])) == int(bits[i])
    x = np.random.default_rng(0).standard_normal(2000).astype(np.float32) * np.float32(1e-3)
    want = torch.from_numpy(x).half().view(torch.int16).numpy().view(np.uint16)
    got = np.array([O.ref_f16_from_f32(float(v)) for v in x], np.uint16)
    assert np.array_equal(got, want)


# ---- independent known answers for the NVFP4 pieces (not from the reference) ----------------
def test_e4m3_against_torch():
    import torch
    xs = np.concatenate([np.linspace(0, 500, 5001, dtype=np.float32), np.float32(2.0) ** np.arange(-12, 9),
                         np.random.default_rng(0).random(5000, dtype=np.float32) * np.float32(0.05)])
    mine = np.array([O.e4m3_encode(float(x)) for x in xs], np.uint8)
    ref = torch.from_numpy(xs).clamp(max=448).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(mine, ref)
    dec = np.array([O.e4m3_decode(c) for c in range(127)], np.float32)
    ref_dec = torch.arange(0, 127, dtype=torch.uint8).view(torch.float8_e4m3fn).float().numpy()
    assert np.array_equal(dec, ref_dec)


def test_e2m1_table_and_ties():
    vals = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]
    for c, v in enumerate(vals):
        assert O.e2m1_decode(c) == v and O.e2m1_decode(c | 8) == -v
        assert O.e2m1_encode(v) == c
    ties = {0.25: 0, 0.75: 2, 1.25: 2, 1.75: 4, 2.5: 4, 3.5: 6, 5.0: 6}  # to the even code
    for x, c in ties.items():
        assert O.e2m1_encode(x) == c and O.e2m1_encode(-x) == (c | 8)
    assert O.e2m1_encode(100.0) == 7 and O.e2m1_encode(-100.0) == 15


def test_nvfp4_quantiser_properties():
    w = (O.gaussian(64 * 256, 7) * np.float32(0.02)).reshape(64, 256)
    c, s, g = O.quantize_weight(w)
    assert g == np.float32(np.abs(w).max()) / np.float32(2688.0)
    deq = O.dequant(c, s, g)
    # each element within half a grid step (<= 1.0 at the top of the E2M1 range) of its block scale
    d = np.repeat(np.array([O.e4m3_decode(int(x)) for x in s.ravel()], np.float32).reshape(s.shape) * np.float32(g), 16, axis=1)
    assert (np.abs(deq - w) <= d * 1.0 + 1e-12).all()
    # idempotence: quantising the dequantised tensor with the same scale reproduces the codes
    c2, s2 = O.quantize_act(O.f32_to_bf16(deq), g)  # bf16 is exact for code*scale only sometimes; compare where exact
    exact = O.bf16_to_f32(O.f32_to_bf16(deq)) == deq
    blocks_exact = exact.reshape(64, 16, 16).all(axis=2)
    assert np.array_equal(s2[blocks_exact], s[blocks_exact])
    # device layout is a bijection on the valid bytes
    from conftest import dev_scales_to_canonical
    assert np.array_equal(dev_scales_to_canonical(O.scales_to_device_layout(s), 64, 256), s)


def test_golden_nvfp4_regression(golden_nvfp4):
    for name in ("small", "ragged", "c1_slice"):
        g = {k.split("/", 1)[1]: golden_nvfp4[k] for k in golden_nvfp4.files if k.startswith(name + "/")}
        wc, ws, gw = O.quantize_weight(g["w"])
        assert np.array_equal(wc, g["w_codes"]) and np.array_equal(ws, g["w_scales"]) and np.float32(gw) == g["g_w"]
        ac, as_ = O.quantize_act(g["a"], float(g["g_a"]))
        assert np.array_equal(ac, g["a_codes"]) and np.array_equal(as_, g["a_scales"])
        y = O.linear(g["a"], float(g["g_a"]), wc, ws, gw, bias=g["bias"])
        assert np.array_equal(y, g["out"])


def test_gemm_f32_matches_f64_and_linearity():
    a = O.gaussian(32 * 128, 1).reshape(32, 128)
    w = O.gaussian(48 * 128, 2).reshape(48, 128)
    assert rel_fro(O.gemm_f32(a, w), O.gemm_f64(a, w)) < 1e-6
    assert np.array_equal(O.gemm_f32(a * np.float32(2), w), O.gemm_f32(a, w) * np.float32(2))
