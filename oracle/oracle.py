"""ctypes/numpy front end of the CPU oracle (TEST INFRASTRUCTURE, not a product path)."""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "build", "liboracle.so")


def build(force: bool = False) -> str:
    """Compile the oracle with the Makefile beside this file (needs g++)."""
    srcs = [os.path.join(_HERE, f) for f in ("nvfp4_oracle.cpp", "ref_restate.cpp", "Makefile")]
    stale = not os.path.exists(_SO) or any(os.path.getmtime(s) > os.path.getmtime(_SO) for s in srcs)
    if force or stale:
        subprocess.run(["make", "-C", _HERE, "-B"], check=True, capture_output=True)
    return _SO


def _load():
    try:
        build()  # recompiles when a source is newer than the library
    except (OSError, subprocess.CalledProcessError):
        if not os.path.exists(_SO):  # no compiler here: a prebuilt library is used as it is
            raise
    lib = C.CDLL(_SO)
    f32p, u16p, u8p, i8p = (C.POINTER(t) for t in (C.c_float, C.c_uint16, C.c_uint8, C.c_int8))
    i64, f32, vp = C.c_int64, C.c_float, C.c_void_p
    sig = {
        "orc_num_threads": (C.c_int, []),
        "orc_set_num_threads": (None, [C.c_int]),
        "orc_bf16_rne": (C.c_uint16, [f32]),
        "orc_e4m3_encode": (C.c_uint8, [f32]),
        "orc_e4m3_decode": (f32, [C.c_uint8]),
        "orc_e2m1_encode": (C.c_uint8, [f32]),
        "orc_e2m1_decode": (f32, [C.c_uint8]),
        "orc_f32_to_bf16": (None, [vp, vp, i64]),
        "orc_gaussian": (None, [vp, i64, C.c_uint64]),
        "orc_amax_f32": (f32, [vp, i64]),
        "orc_amax_bf16": (f32, [vp, i64]),
        "orc_global_scale": (f32, [f32]),
        "orc_quantize_weight": (f32, [vp, i64, i64, vp, vp]),
        "orc_quantize_weight_bf16": (f32, [vp, i64, i64, vp, vp]),
        "orc_quantize_act": (None, [vp, i64, i64, f32, vp, vp]),
        "orc_dequant": (None, [vp, vp, f32, i64, i64, vp]),
        "orc_scales_to_device_layout": (i64, [vp, i64, i64, vp]),
        "orc_gemm_f32": (None, [vp, vp, i64, i64, i64, vp]),
        "orc_gemm_f64": (None, [vp, vp, i64, i64, i64, vp]),
        "orc_epilogue": (None, [vp, i64, i64, f32, vp, C.c_int, vp, vp, C.c_int, vp]),
        "orc_linear": (None, [vp, i64, i64, f32, C.c_int, vp, vp, f32, i64, vp, C.c_int, vp, vp, C.c_int, vp, vp]),
        "orc_linear_q": (None, [vp, vp, i64, i64, f32, vp, vp, f32, i64, vp, C.c_int, vp, vp, C.c_int, vp]),
        "ref_f16_from_f32": (C.c_uint16, [f32]),
        "ref_f16_to_f32": (f32, [C.c_uint16]),
        "ref_lcg_fill": (None, [vp, i64, C.POINTER(C.c_uint64), f32]),
        "ref_quantize_row_q8_0": (None, [vp, i64, vp]),
        "ref_encode_q8_0_from_bf16": (None, [vp, i64, vp]),
        "ref_dequantize_row_q8_0": (None, [vp, i64, vp]),
        "ref_quantize_row_q4_0": (None, [vp, i64, vp]),
        "ref_dequantize_row_q4_0": (None, [vp, i64, vp]),
        "ref_act_quant_i8": (None, [vp, i64, i64, vp, vp]),
        "ref_matmul_i8": (None, [vp, vp, vp, vp, vp, i64, i64, i64, vp]),
        "ref_layernorm": (None, [vp, C.c_int, i64, i64, f32, vp]),
        "ref_bcast_modulate": (None, [vp, vp, vp, C.c_int, i64, i64, f32, vp]),
        "ref_sdpa": (None, [vp, vp, vp, vp, C.c_int, i64, i64, i64, i64, i64, i64, f32, C.c_int, vp]),
        "ref_norm_modulate_bf16": (None, [vp, vp, vp, i64, i64, f32, f32, C.c_int, vp]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    return lib


_lib = _load()


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _c(a, dt):
    return np.ascontiguousarray(a, dtype=dt)


def num_threads() -> int:
    return int(_lib.orc_num_threads())


def set_num_threads(n: int) -> None:
    """OpenMP threads of the following calls (torchrun exports OMP_NUM_THREADS=1 to its workers)."""
    _lib.orc_set_num_threads(int(n))


# ---- scalar conversions -------------------------------------------------------------
def bf16_rne(x: float) -> int:
    return int(_lib.orc_bf16_rne(x))


def e4m3_encode(x: float) -> int:
    return int(_lib.orc_e4m3_encode(x))


def e4m3_decode(c: int) -> float:
    return float(_lib.orc_e4m3_decode(c))


def e2m1_encode(x: float) -> int:
    return int(_lib.orc_e2m1_encode(x))


def e2m1_decode(c: int) -> float:
    return float(_lib.orc_e2m1_decode(c))


# ---- arrays -------------------------------------------------------------------------
def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    x = _c(x, np.float32)
    out = np.empty(x.shape, np.uint16)
    _lib.orc_f32_to_bf16(_p(x), _p(out), x.size)
    return out


def bf16_to_f32(h: np.ndarray) -> np.ndarray:
    return (_c(h, np.uint16).astype(np.uint32) << 16).view(np.float32)


def gaussian(n: int, seed: int) -> np.ndarray:
    out = np.empty(n, np.float32)
    _lib.orc_gaussian(_p(out), n, C.c_uint64(seed & (2**64 - 1)))
    return out


def global_scale(amax: float) -> float:
    return float(_lib.orc_global_scale(amax))


def amax_bf16(a: np.ndarray) -> float:
    a = _c(a, np.uint16)
    return float(_lib.orc_amax_bf16(_p(a), a.size))


def quantize_weight(w: np.ndarray):
    """f32 or bf16-bits (uint16) [rows, k] -> (codes [rows,k/2] u8, scales [rows,k/16] u8, g)."""
    rows, k = w.shape
    assert k % 16 == 0
    codes = np.empty((rows, k // 2), np.uint8)
    scales = np.empty((rows, k // 16), np.uint8)
    if w.dtype == np.uint16:
        w = _c(w, np.uint16)
        g = _lib.orc_quantize_weight_bf16(_p(w), rows, k, _p(codes), _p(scales))
    else:
        w = _c(w, np.float32)
        g = _lib.orc_quantize_weight(_p(w), rows, k, _p(codes), _p(scales))
    return codes, scales, float(g)


def quantize_act(a_bf16: np.ndarray, g: float):
    a = _c(a_bf16, np.uint16)
    m, k = a.shape
    assert k % 16 == 0
    codes = np.empty((m, k // 2), np.uint8)
    scales = np.empty((m, k // 16), np.uint8)
    _lib.orc_quantize_act(_p(a), m, k, g, _p(codes), _p(scales))
    return codes, scales


def dequant(codes: np.ndarray, scales: np.ndarray, g: float) -> np.ndarray:
    codes, scales = _c(codes, np.uint8), _c(scales, np.uint8)
    rows, k = codes.shape[0], codes.shape[1] * 2
    out = np.empty((rows, k), np.float32)
    _lib.orc_dequant(_p(codes), _p(scales), g, rows, k, _p(out))
    return out


def scales_to_device_layout(scales: np.ndarray) -> np.ndarray:
    scales = _c(scales, np.uint8)
    rows, nb = scales.shape
    out = np.empty(((rows + 127) // 128) * ((((nb + 3) // 4) + 3) // 4 * 4) * 512, np.uint8)
    _lib.orc_scales_to_device_layout(_p(scales), rows, nb, _p(out))
    return out


def gemm_f32(a: np.ndarray, w: np.ndarray) -> np.ndarray:
    """out[m,n] = sum_k a[m,k]*w[n,k], f32, K ascending."""
    a, w = _c(a, np.float32), _c(w, np.float32)
    m, k = a.shape
    n = w.shape[0]
    out = np.empty((m, n), np.float32)
    _lib.orc_gemm_f32(_p(a), _p(w), m, n, k, _p(out))
    return out


def gemm_f64(a: np.ndarray, w: np.ndarray) -> np.ndarray:
    a, w = _c(a, np.float32), _c(w, np.float32)
    m, k = a.shape
    n = w.shape[0]
    out = np.empty((m, n), np.float64)
    _lib.orc_gemm_f64(_p(a), _p(w), m, n, k, _p(out))
    return out


def epilogue(acc, scale=1.0, bias=None, act=0, gate=None, residual=None, chain=False) -> np.ndarray:
    acc = _c(acc, np.float32)
    m, n = acc.shape
    out = np.empty((m, n), np.uint16)
    bias = None if bias is None else _c(bias, np.uint16)
    gate = None if gate is None else _c(gate, np.uint16)
    residual = None if residual is None else _c(residual, np.uint16)
    _lib.orc_epilogue(_p(acc), m, n, scale, _p(bias), act, _p(gate), _p(residual), int(chain), _p(out))
    return out


def linear(a_bf16, g_a, w_codes, w_scales, g_w, bias=None, act=0, gate=None, residual=None,
           chain=False, quantize_a=True, return_acc=False):
    """The NVFP4 linear as the device computes it; returns bf16 bits [m, n]."""
    a = _c(a_bf16, np.uint16)
    w_codes, w_scales = _c(w_codes, np.uint8), _c(w_scales, np.uint8)
    m, k = a.shape
    n = w_codes.shape[0]
    out = np.empty((m, n), np.uint16)
    acc = np.empty((m, n), np.float32) if return_acc else None
    bias = None if bias is None else _c(bias, np.uint16)
    gate = None if gate is None else _c(gate, np.uint16)
    residual = None if residual is None else _c(residual, np.uint16)
    _lib.orc_linear(_p(a), m, k, g_a, int(quantize_a), _p(w_codes), _p(w_scales), g_w, n, _p(bias),
                    act, _p(gate), _p(residual), int(chain), _p(out), _p(acc))
    return (out, acc) if return_acc else out


def linear_q(a_codes, a_scales, g_a, w_codes, w_scales, g_w, bias=None, act=0, gate=None, residual=None, chain=False):
    """The linear on an activation operand that is already NVFP4 (canonical layouts); bf16 bits [m, n]."""
    a_codes, a_scales = _c(a_codes, np.uint8), _c(a_scales, np.uint8)
    w_codes, w_scales = _c(w_codes, np.uint8), _c(w_scales, np.uint8)
    m, k = a_codes.shape[0], a_codes.shape[1] * 2
    n = w_codes.shape[0]
    out = np.empty((m, n), np.uint16)
    bias = None if bias is None else _c(bias, np.uint16)
    gate = None if gate is None else _c(gate, np.uint16)
    residual = None if residual is None else _c(residual, np.uint16)
    _lib.orc_linear_q(_p(a_codes), _p(a_scales), m, k, g_a, _p(w_codes), _p(w_scales), g_w, n, _p(bias), act, _p(gate),
                      _p(residual), int(chain), _p(out))
    return out


# ---- restated reference routines (pinned by the reference's own unit tests) ----------
def ref_f16_from_f32(x: float) -> int:
    return int(_lib.ref_f16_from_f32(x))


def ref_f16_to_f32(h: int) -> float:
    return float(_lib.ref_f16_to_f32(h))


class RefLcg:
    """The LCG the reference's conformance tests draw inputs from."""

    def __init__(self, seed: int):
        self.state = C.c_uint64(seed)

    def fill(self, n: int, amp: float = 1.0) -> np.ndarray:
        out = np.empty(n, np.float32)
        _lib.ref_lcg_fill(_p(out), n, C.byref(self.state), amp)
        return out


def ref_quantize_row_q8_0(x):
    x = _c(x, np.float32)
    out = np.empty(x.size // 32 * 34, np.uint8)
    _lib.ref_quantize_row_q8_0(_p(x), x.size, _p(out))
    return out


def ref_encode_q8_0_from_bf16(h):
    h = _c(h, np.uint16)
    out = np.empty(h.size // 32 * 34, np.uint8)
    _lib.ref_encode_q8_0_from_bf16(_p(h), h.size, _p(out))
    return out


def ref_dequantize_row_q8_0(q):
    q = _c(q, np.uint8)
    n = q.size // 34 * 32
    out = np.empty(n, np.float32)
    _lib.ref_dequantize_row_q8_0(_p(q), n, _p(out))
    return out


def ref_quantize_row_q4_0(x):
    x = _c(x, np.float32)
    out = np.empty(x.size // 32 * 18, np.uint8)
    _lib.ref_quantize_row_q4_0(_p(x), x.size, _p(out))
    return out


def ref_dequantize_row_q4_0(q):
    q = _c(q, np.uint8)
    n = q.size // 18 * 32
    out = np.empty(n, np.float32)
    _lib.ref_dequantize_row_q4_0(_p(q), n, _p(out))
    return out


def ref_act_quant_i8(a):
    a = _c(a, np.float32)
    rows, k = a.shape
    q = np.empty((rows, k), np.int8)
    params = np.empty((rows, k // 32, 2), np.float32)
    _lib.ref_act_quant_i8(_p(a), rows, k, _p(q), _p(params))
    return q, params


def ref_matmul_i8(a, a_scale, a_zero, b, b_scale):
    a, b = _c(a, np.int8), _c(b, np.int8)
    m, k = a.shape
    n = b.shape[0]
    out = np.empty((m, n), np.float32)
    _lib.ref_matmul_i8(_p(a), _p(_c(a_scale, np.float32)), _p(_c(a_zero, np.float32)), _p(b),
                       _p(_c(b_scale, np.float32)), m, n, k, _p(out))
    return out


def ref_layernorm(x, eps: float):
    """Row LayerNorm without affine (thinfer-core/src/ops/layernorm.rs); f32 in -> f32 out, uint16 (bf16 bits) in -> bf16 bits out."""
    bf16 = x.dtype == np.uint16
    x = _c(x, np.uint16 if bf16 else np.float32)
    out = np.empty_like(x)
    _lib.ref_layernorm(_p(x), int(bf16), x.shape[0], x.shape[1], eps, _p(out))
    return out


def ref_bcast_modulate(x, s, t, bias: float = 1.0):
    """out = x * (s + bias) + t with s, t broadcast over rows (thinfer-core/src/ops/bcast_modulate.rs)."""
    bf16 = x.dtype == np.uint16
    dt = np.uint16 if bf16 else np.float32
    x, s, t = _c(x, dt), _c(s, dt), _c(t, dt)
    out = np.empty_like(x)
    _lib.ref_bcast_modulate(_p(x), _p(s), _p(t), int(bf16), x.size, s.size, bias, _p(out))
    return out


def ref_sdpa(q, k, v, scale: float, mask=None, mask_mode: int = 0):
    """Scaled-dot-product attention as the reference computes it (thinfer-core/src/ops/sdpa.rs: online softmax, keys in
    order, f32). q [B, Sq, Hq, D], k / v [B, Sk, Hkv, D]; float32 arrays, or uint16 bf16 bit patterns (output then bf16)."""
    bf16 = q.dtype == np.uint16
    dt = np.uint16 if bf16 else np.float32
    q, k, v = _c(q, dt), _c(k, dt), _c(v, dt)
    b, s_q, h_q, d = q.shape
    _, s_k, h_kv, _ = k.shape
    if mask is not None and mask_mode == 0:
        mask_mode = 2 if mask.ndim == 4 else 1
    mask = None if mask is None else _c(mask, dt)
    out = np.empty_like(q)
    _lib.ref_sdpa(_p(q), _p(k), _p(v), _p(mask), int(bf16), b, s_q, s_k, h_q, h_kv, d, scale, mask_mode if mask is not None else 0, _p(out))
    return out


def norm_modulate(x_bf16, scale_bf16=None, shift_bf16=None, eps: float = 1e-6, bias: float = 1.0, chain: bool = False):
    """LayerNorm + modulate fused on bf16 rows (the two reference dispatches; chain=True keeps their bf16 rounding between)."""
    x = _c(x_bf16, np.uint16)
    s = None if scale_bf16 is None else _c(scale_bf16, np.uint16)
    t = None if shift_bf16 is None else _c(shift_bf16, np.uint16)
    out = np.empty_like(x)
    _lib.ref_norm_modulate_bf16(_p(x), _p(s), _p(t), x.shape[0], x.shape[1], eps, bias, int(chain), _p(out))
    return out
