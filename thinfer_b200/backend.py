"""Host-side mirror of the reference's backend and op surface for the NVFP4 linear path.

Names follow the reference so that tests read like its own:

* :class:`Backend` — ``trait Backend`` (thinfer-core/src/backend/mod.rs:94-206):
  ``allocate_in`` / ``free`` / ``write_buffer`` / ``read_buffer`` /
  ``copy_buffer_to_buffer`` / ``submit`` / ``supports_weight_prep`` / ``weight_prep``.
* :class:`BatchScope` — the op-forwarding methods of ``BatchScope``
  (thinfer-core/src/workspace.rs:774-996): ``act_quant``, ``matmul`` and the fused
  ``linear`` that covers the ``biased`` call site (thinfer-models/src/qwen_image/dit.rs:324-340).
* :class:`Nvfp4Weight` — the ``PreparedWeight`` a site keeps resident
  (thinfer-models/src/common/block.rs:217-227), here codes + device-layout scales + bias.

Everything runs on the GPU through the C ABI (``include/thinfer_nvfp4.h``); host arrays are
numpy, bf16 carried as ``uint16`` bit patterns.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional

import numpy as np

from . import _lib as L
from ._lib import Buf, LinearArgs


class TnfError(RuntimeError):
    """WgpuError (thinfer-core/src/backend/wgpu.rs:115-159)."""

    def __init__(self, code: int, message: str):
        super().__init__(f"[{code}] {message}")
        self.code = code


class UnknownBuffer(TnfError):
    pass


class AllocateOom(TnfError):
    pass


class BudgetExceeded(TnfError):
    pass


class InvalidArgument(TnfError):
    pass


class LaunchFailed(TnfError):
    pass


class DeviceTimeout(TnfError):
    pass


class NcclError(TnfError):
    pass


_ERRORS = {
    L.ERR_UNKNOWN_BUFFER: UnknownBuffer, L.ERR_ALLOCATE_OOM: AllocateOom,
    L.ERR_BUDGET_EXCEEDED: BudgetExceeded, L.ERR_INVALID_ARGUMENT: InvalidArgument,
    L.ERR_LAUNCH: LaunchFailed, L.ERR_TIMEOUT: DeviceTimeout, L.ERR_NCCL: NcclError,
}


def _check(code: int) -> None:
    if code != L.OK:
        msg = L.load().tnf_last_error().decode("utf-8", "replace")
        raise _ERRORS.get(code, TnfError)(code, msg)


_NONE = Buf(0, 0, 0)


def _host(a: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(a)


class Backend:
    """One CUDA device behind the C ABI. ``vram_budget`` (bytes, 0 = none) is the arbiter's budget."""

    def __init__(self, device: int = 0, vram_budget: int = 0):
        self.lib = L.load()
        self._ctx = C.c_void_p()
        _check(self.lib.tnf_create(device, vram_budget, C.byref(self._ctx)))
        self.device = device

    # -- lifetime ---------------------------------------------------------------------
    def close(self) -> None:
        if self._ctx:
            self.lib.tnf_destroy(self._ctx)
            self._ctx = C.c_void_p()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def __del__(self):  # pragma: no cover
        try:
            self.close()
        except Exception:
            pass

    # -- trait Backend ------------------------------------------------------------------
    def allocate_in(self, nbytes: int, category: int = L.CAT_WORKSPACE) -> Buf:
        bid = C.c_uint64()
        _check(self.lib.tnf_alloc(self._ctx, nbytes, category, C.byref(bid)))
        return Buf(bid.value, 0, nbytes)

    def allocate(self, nbytes: int) -> Buf:
        return self.allocate_in(nbytes, L.CAT_WORKSPACE)

    def free(self, buf) -> None:
        _check(self.lib.tnf_free(self._ctx, buf.id if isinstance(buf, Buf) else int(buf)))

    def write_buffer(self, buf: Buf, data: np.ndarray, offset: int = 0) -> None:
        data = _host(data)
        _check(self.lib.tnf_write(self._ctx, buf.id, buf.offset + offset, data.ctypes.data_as(C.c_void_p), data.nbytes))

    def read_buffer(self, buf: Buf, dtype=np.uint8, count: Optional[int] = None, offset: int = 0) -> np.ndarray:
        dt = np.dtype(dtype)
        nbytes = (buf.len - offset) if count is None else count * dt.itemsize
        out = np.empty(nbytes // dt.itemsize, dt)
        _check(self.lib.tnf_read(self._ctx, buf.id, buf.offset + offset, out.ctypes.data_as(C.c_void_p), out.nbytes))
        return out

    def copy_buffer_to_buffer(self, src: Buf, dst: Buf, nbytes: int) -> None:
        _check(self.lib.tnf_copy(self._ctx, src.id, src.offset, dst.id, dst.offset, nbytes))

    def submit(self, timeout_ms: int = 0) -> None:
        """Awaited submit: waits for the device and surfaces device-side wait failures."""
        _check(self.lib.tnf_sync(self._ctx, timeout_ms))

    def supports_weight_prep(self) -> bool:
        return True

    def weight_prep(self, w: np.ndarray) -> "Nvfp4Weight":
        return Nvfp4Weight.from_dense(self, w)

    # -- helpers ------------------------------------------------------------------------
    def upload(self, data: np.ndarray, category: int = L.CAT_WORKSPACE) -> Buf:
        data = _host(data)
        buf = self.allocate_in(max(data.nbytes, 16), category)
        self.write_buffer(buf, data)
        return Buf(buf.id, 0, data.nbytes)

    def mem_snapshot(self) -> dict:
        out = (C.c_uint64 * 8)()
        _check(self.lib.tnf_mem_snapshot(self._ctx, out))
        keys = ["live_weights", "live_workspace", "live_staging", "peak_weights", "peak_workspace",
                "peak_staging", "true_peak", "streamed_bytes"]
        return dict(zip(keys, [int(v) for v in out]))

    def device_ptr(self, buf: Buf) -> int:
        p = C.c_void_p()
        _check(self.lib.tnf_buf_ptr(self._ctx, buf.id, C.byref(p), None))
        return int(p.value) + buf.offset

    def streams(self):
        a, b = C.c_void_p(), C.c_void_p()
        _check(self.lib.tnf_streams(self._ctx, C.byref(a), C.byref(b)))
        return int(a.value), int(b.value)

    # -- workspace pool (Workspace in the reference) ---------------------------------------
    def ws_alloc(self, nbytes: int) -> "WsBuf":
        """Rents a scratch buffer of at least ``nbytes`` from the pool (Workspace::alloc,
        thinfer-core/src/workspace.rs:196-260). Release it (or leave its ``with`` block) to make it idle."""
        bid = C.c_uint64()
        _check(self.lib.tnf_ws_alloc(self._ctx, nbytes, C.byref(bid)))
        return WsBuf(self, Buf(bid.value, 0, nbytes))

    def drain_pool(self) -> int:
        """Frees every idle pool buffer (Workspace::drain_pool); returns the bytes freed."""
        freed = C.c_uint64()
        _check(self.lib.tnf_ws_drain(self._ctx, C.byref(freed)))
        return int(freed.value)

    def pool_stats(self) -> dict:
        out = (C.c_uint64 * 6)()
        _check(self.lib.tnf_ws_stats(self._ctx, out))
        return dict(zip(["pool_bytes", "free_count", "rented", "hits", "misses", "spilled_bytes"], [int(v) for v in out]))

    def scope(self) -> "BatchScope":
        return BatchScope(self)


class WsBuf:
    """A rented pool buffer (WsBuf, thinfer-core/src/workspace.rs:318-420): ``buf`` is the view of the requested
    length; releasing returns the buffer to the pool, once."""

    def __init__(self, be: Backend, buf: Buf):
        self.be, self.buf = be, buf

    @property
    def id(self) -> int:
        return self.buf.id

    def __len__(self) -> int:
        return self.buf.len

    def release(self) -> None:
        if self.be is not None:
            be, self.be = self.be, None
            _check(be.lib.tnf_ws_release(be._ctx, self.buf.id))

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.release()


def device_scales_bytes(rows: int, k: int) -> int:
    return int(L.load().tnf_device_scales_bytes(rows, k))


@dataclass
class Nvfp4Weight:
    """A linear's resident weight: E2M1 codes [n,k/2], device-layout E4M3 scales, f32 scale, bias."""
    n: int
    k: int
    codes: Optional[Buf]          # None: a weight kept in bf16 only (from_bf16)
    scales_device: Optional[Buf]
    global_scale: float
    bias: Optional[Buf] = None
    scales_canonical: Optional[Buf] = None
    dense: Optional[Buf] = None  # bf16 [n,k] image for dense-activation sites (PreparedWeight::F16 in the reference)

    @staticmethod
    def from_dense(be: Backend, w: np.ndarray, bias_bf16: Optional[np.ndarray] = None,
                   keep_canonical: bool = False) -> "Nvfp4Weight":
        """Quantise a dense [n,k] weight (float32, or bf16 bits as uint16) on the device."""
        n, k = w.shape
        dtype = L.DTYPE_BF16 if w.dtype == np.uint16 else L.DTYPE_F32
        if dtype == L.DTYPE_F32:
            w = w.astype(np.float32, copy=False)
        src = be.upload(w, L.CAT_STAGING)
        codes = be.allocate_in(n * k // 2, L.CAT_WEIGHTS)
        canon = be.allocate_in(max(n * k // 16, 16), L.CAT_WEIGHTS if keep_canonical else L.CAT_STAGING)
        g = C.c_float()
        _check(be.lib.tnf_quantize_weight(be._ctx, src, dtype, n, k, codes, canon, C.byref(g)))
        dev = be.allocate_in(device_scales_bytes(n, k), L.CAT_WEIGHTS)
        _check(be.lib.tnf_prepare_scales(be._ctx, canon, n, k, dev))
        be.submit()
        be.free(src)
        if not keep_canonical:
            be.free(canon)
            canon = None
        bias = be.upload(bias_bf16.astype(np.uint16, copy=False), L.CAT_WEIGHTS) if bias_bf16 is not None else None
        return Nvfp4Weight(n, k, codes, dev, float(g.value), bias, canon)

    @staticmethod
    def from_packed(be: Backend, codes: np.ndarray, scales_canonical: np.ndarray, global_scale: float,
                    bias_bf16: Optional[np.ndarray] = None) -> "Nvfp4Weight":
        """Upload an already quantised weight (canonical layouts)."""
        n, k = codes.shape[0], codes.shape[1] * 2
        cb = be.upload(codes.astype(np.uint8, copy=False), L.CAT_WEIGHTS)
        canon = be.upload(scales_canonical.astype(np.uint8, copy=False), L.CAT_STAGING)
        dev = be.allocate_in(device_scales_bytes(n, k), L.CAT_WEIGHTS)
        _check(be.lib.tnf_prepare_scales(be._ctx, canon, n, k, dev))
        be.submit()
        be.free(canon)
        bias = be.upload(bias_bf16.astype(np.uint16, copy=False), L.CAT_WEIGHTS) if bias_bf16 is not None else None
        return Nvfp4Weight(n, k, cb, dev, float(global_scale), bias, None)

    @staticmethod
    def from_bf16(be: Backend, w_bf16: np.ndarray, bias_bf16: Optional[np.ndarray] = None) -> "Nvfp4Weight":
        """A weight that is never quantised (bf16 bits as uint16, [n,k]): only the dense arm (``dense_act=True``) and the
        mixed arm (NVFP4 activations x this weight) can use it. The reference keeps its refiner weights this way
        (thinfer-core/src/ops/matmul_i8_bf16.rs:15-17)."""
        if w_bf16.dtype != np.uint16 or w_bf16.ndim != 2:
            raise InvalidArgument(L.ERR_INVALID_ARGUMENT, "from_bf16 takes bf16 bits as a uint16 [n,k] array")
        n, k = w_bf16.shape
        dense = be.upload(w_bf16, L.CAT_WEIGHTS)
        bias = be.upload(bias_bf16.astype(np.uint16, copy=False), L.CAT_WEIGHTS) if bias_bf16 is not None else None
        return Nvfp4Weight(n, k, None, None, 1.0, bias, None, dense)

    def prepare_dense(self, be: Backend) -> Buf:
        """Make (once) and keep the dense bf16 image a ``dense_act`` site multiplies with: code x block scale, exact."""
        if self.dense is None:
            self.dense = be.allocate_in(self.n * self.k * 2, L.CAT_WEIGHTS)
            _check(be.lib.tnf_prepare_dense(be._ctx, self.codes, self.scales_device, self.n, self.k, self.dense))
        return self.dense

    def free(self, be: Backend) -> None:
        for b in (self.codes, self.scales_device, self.bias, self.scales_canonical, self.dense):
            if b is not None:
                be.free(b)


def interleave_swiglu(w1: np.ndarray, w3: np.ndarray) -> np.ndarray:
    """[W1 row 0, W3 row 0, W1 row 1, ...]: the weight (or bias) layout of a ``swiglu`` linear."""
    assert w1.shape == w3.shape
    out = np.empty((2 * w1.shape[0],) + w1.shape[1:], w1.dtype)
    out[0::2], out[1::2] = w1, w3
    return out


@dataclass
class DenseActSites:
    """Which linear sites of a block keep un-quantised activations; the reference's ``DenseActSites``
    (thinfer-models/src/common/block.rs:470-479). ``flags(site)`` gives the linear flags for that site."""
    qkv: bool = False
    qkv_self: bool = False
    proj: bool = False
    ffn_up: bool = False
    ffn_down: bool = False

    def flags(self, site: int) -> int:
        c = L.DenseActSites(int(self.qkv), int(self.qkv_self), int(self.proj), int(self.ffn_up), int(self.ffn_down))
        return int(L.load().tnf_site_linear_flags(C.byref(c), site))


class BatchScope:
    """Op surface used by the linear call sites; launches are asynchronous until ``submit``."""

    def __init__(self, backend: Backend):
        self.be = backend
        self._guards = []  # pool buffers rented through the scope: none returns to the pool before submit

    def alloc(self, nbytes: int) -> Buf:
        """Scratch for the launches of this scope (BatchScope::alloc, thinfer-core/src/workspace.rs:452-467): rented
        from the pool and held until ``submit``, so no launch of the scope sees a buffer recycled under it."""
        g = self.be.ws_alloc(nbytes)
        self._guards.append(g)
        return g.buf

    def act_quant(self, a_bf16: Buf, m: int, k: int, global_scale: float = 0.0, device_layout: bool = False):
        """Per-row per-16 NVFP4 activation quantiser. Returns (codes, scales, global_scale_used)."""
        be = self.be
        codes = be.allocate(m * k // 2)
        nscale = device_scales_bytes(m, k) if device_layout else max(m * k // 16, 16)
        scales = be.allocate(nscale)
        g = C.c_float()
        _check(be.lib.tnf_quantize_act(be._ctx, a_bf16, m, k, global_scale,
                                       L.SCALES_DEVICE if device_layout else L.SCALES_CANONICAL, codes, scales,
                                       C.byref(g)))
        return codes, scales, float(g.value)

    def act_quant_shared(self, a_bf16: Buf, m: int, k: int, global_scale: float) -> None:
        _check(self.be.lib.tnf_quantize_act_shared(self.be._ctx, a_bf16, m, k, global_scale))

    def _args(self, m, w: Nvfp4Weight, a, a_global, out, act, gate, residual, chain, n_offset, ldo, flags, bias,
              out_nvfp4=None):
        args = LinearArgs()
        args.m, args.n, args.k = m, w.n, w.k
        args.a_global, args.w_global = a_global, w.global_scale
        args.a_bf16 = a if a is not None else _NONE
        if w.codes is None and not flags & L.LINEAR_DENSE_ACT:
            raise InvalidArgument(L.ERR_INVALID_ARGUMENT, "a bf16-only weight needs dense_act=True")
        args.w_codes, args.w_scales = w.codes or _NONE, w.scales_device or _NONE
        use_bias = w.bias if bias is None else (None if bias is False else bias)
        args.bias_bf16 = use_bias if use_bias is not None else _NONE
        args.gate_bf16 = gate if gate is not None else _NONE
        args.residual_bf16 = residual if residual is not None else _NONE
        args.out_bf16 = out if out is not None else _NONE
        args.act, args.parity_mode = act, int(chain)
        if out_nvfp4 is not None:  # (codes, device-layout scales, per-tensor scale): quantised copy of the output
            args.out_codes, args.out_scales, args.out_global = out_nvfp4
            flags |= L.LINEAR_OUT_NVFP4 | (L.LINEAR_NO_BF16_OUT if out is None else 0)
        else:
            args.out_codes, args.out_scales = _NONE, _NONE
        args.w_dense = _NONE
        if flags & L.LINEAR_DENSE_ACT:
            if w.dense is None:
                raise InvalidArgument(L.ERR_INVALID_ARGUMENT, "dense_act site: call Nvfp4Weight.prepare_dense first")
            args.w_dense = w.dense
        args.n_offset, args.ldo, args.flags = n_offset, ldo, flags
        return args

    def norm_modulate_quant(self, x_bf16: Buf, m: int, k: int, out_global: float, out_codes: Buf, out_scales_device: Buf,
                            scale: Optional[Buf] = None, shift: Optional[Buf] = None, out_bf16: Optional[Buf] = None,
                            eps: float = 1e-6, mod_bias: float = 1.0, chain: bool = False) -> None:
        """op_layernorm + op_modulate + act_quant of the reference's block in one launch
        (thinfer-models/src/qwen_image/dit.rs:521-532); the NVFP4 copy feeds ``matmul``."""
        none = Buf(0, 0, 0)
        args = L.NormQuantArgs(m, k, eps, mod_bias, x_bf16, scale or none, shift or none, out_bf16 or none, out_codes,
                               out_scales_device, out_global, int(chain))
        _check(self.be.lib.tnf_norm_modulate_quantize(self.be._ctx, C.byref(args)))

    def linear(self, a_bf16: Optional[Buf], m: int, w: Nvfp4Weight, a_global: float, out: Optional[Buf],
               act: int = L.ACT_NONE, gate: Optional[Buf] = None, residual: Optional[Buf] = None, chain: bool = False,
               n_offset: int = 0, ldo: int = 0, flags: int = 0, bias=None, out_nvfp4=None, dense_act: bool = False,
               swiglu: bool = False) -> None:
        """out = epilogue(a_global*w_global * (quant(A) . Wq^T)): the ``biased`` call site, fused.

        ``dense_act=True`` is the reference's dense arm for outlier-carrying sites (``DenseActSites``): the
        activations stay bf16 and multiply the weight's dense image (``Nvfp4Weight.prepare_dense``); ``a_global``
        is ignored. ``swiglu=True``: ``w`` is the row-interleaved pair from :func:`interleave_swiglu` and the
        epilogue writes ``silu(A.W1^T) * (A.W3^T)``, ``w.n // 2`` columns (the reference's ``op_silu_mul`` after its
        two FFN-up matmuls, thinfer-models/src/common/block.rs:1720-1762).

        ``out_nvfp4=(codes, scales_device, g)`` also emits the result quantised to NVFP4 (the A operand
        of the next linear: MLP up -> GELU -> down); ``out=None`` then skips the bf16 store."""
        if dense_act:
            flags |= L.LINEAR_DENSE_ACT
        if swiglu:
            flags |= L.LINEAR_SWIGLU
        args = self._args(m, w, a_bf16, a_global, out, act, gate, residual, chain, n_offset, ldo, flags, bias, out_nvfp4)
        _check(self.be.lib.tnf_linear_nvfp4(self.be._ctx, C.byref(args)))

    def matmul(self, a_codes: Buf, a_scales_device: Buf, m: int, w: Nvfp4Weight, a_global: float, out: Optional[Buf],
               act: int = L.ACT_NONE, gate=None, residual=None, chain: bool = False, n_offset: int = 0, ldo: int = 0,
               flags: int = 0, bias=None, out_nvfp4=None, dense_act: bool = False) -> None:
        """The GEMM alone on pre-quantised operands. ``dense_act=True`` is the mixed arm: the NVFP4 activations are
        widened to bf16 (exact) and multiply the weight's dense image, or a weight that was never quantised
        (``Nvfp4Weight.from_bf16``) -- the role of the reference's matmul_i8_bf16."""
        if dense_act:
            flags |= L.LINEAR_DENSE_ACT
        args = self._args(m, w, None, a_global, out, act, gate, residual, chain, n_offset, ldo, flags, bias, out_nvfp4)
        _check(self.be.lib.tnf_gemm_nvfp4(self.be._ctx, C.byref(args), a_codes, a_scales_device))

    def sdpa(self, q: Buf, k: Buf, v: Buf, out: Optional[Buf], b: int, s_q: int, s_k: int, h_q: int, h_kv: int, scale: float,
             d: int = 128, out_nvfp4=None, q_ld: int = 0, kv_ld: int = 0) -> None:
        """Joint attention between the linears (``op_sdpa``, thinfer-core/src/ops/sdpa.rs): q / out bf16 [b, s_q, h_q, d],
        k / v bf16 [b, s_k, h_kv, d], no mask, d = 128. ``out_nvfp4=(codes, scales_device, g)`` also emits the output
        quantised to NVFP4 as the [b*s_q, h_q*d] operand of the out-projection; ``out=None`` then skips the bf16 store.
        ``q_ld`` / ``kv_ld`` (elements, 0 = dense) let q, k and v be column windows of a wider matrix, e.g. of the fused-QKV
        linear's output."""
        flags, none = 0, Buf(0, 0, 0)
        oc, os_, og = none, none, 0.0
        if out_nvfp4 is not None:
            oc, os_, og = out_nvfp4
            flags = L.SDPA_OUT_NVFP4 | (L.SDPA_NO_BF16_OUT if out is None else 0)
        args = L.SdpaArgs(b, s_q, s_k, h_q, h_kv, d, scale, 0, q, k, v, out if out is not None else none, flags, og, oc, os_, q_ld, kv_ld)
        _check(self.be.lib.tnf_sdpa(self.be._ctx, C.byref(args)))

    def submit(self, timeout_ms: int = 0) -> None:
        try:
            self.be.submit(timeout_ms)
        finally:
            guards, self._guards = self._guards, []
            for g in guards:
                g.release()
