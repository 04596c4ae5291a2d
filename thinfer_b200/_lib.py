"""ctypes binding of libthinfer_nvfp4.so. There is no fallback: a missing library raises."""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# THINFER_B200_LIB points at another build of the same library (a variant compiled with different options)
LIB_PATH = os.environ.get("THINFER_B200_LIB") or os.path.join(_HERE, "libthinfer_nvfp4.so")

OK = 0
ERR_UNKNOWN_BUFFER, ERR_ALLOCATE_OOM, ERR_BUDGET_EXCEEDED = -1, -2, -3
ERR_INVALID_ARGUMENT, ERR_LAUNCH, ERR_TIMEOUT, ERR_NCCL = -4, -5, -6, -7
CAT_WEIGHTS, CAT_WORKSPACE, CAT_STAGING = 0, 1, 2
DTYPE_F32, DTYPE_BF16 = 0, 1
SCALES_CANONICAL, SCALES_DEVICE = 0, 1
ACT_NONE, ACT_GELU_TANH = 0, 1
LINEAR_A_PREQUANTIZED, LINEAR_SCATTER_PEERS, LINEAR_OUT_NVFP4, LINEAR_NO_BF16_OUT, LINEAR_MULTICAST_OUT = 1, 2, 4, 8, 16
LINEAR_DENSE_ACT, LINEAR_SWIGLU = 32, 64


class Buf(C.Structure):
    """tnf_buf: the non-owning {id, offset, len} view (BufRef in the reference)."""
    _fields_ = [("id", C.c_uint64), ("offset", C.c_uint64), ("len", C.c_uint64)]


class LinearArgs(C.Structure):
    _fields_ = [
        ("m", C.c_uint32), ("n", C.c_uint32), ("k", C.c_uint32),
        ("a_global", C.c_float), ("w_global", C.c_float),
        ("a_bf16", Buf), ("w_codes", Buf), ("w_scales", Buf), ("bias_bf16", Buf),
        ("gate_bf16", Buf), ("residual_bf16", Buf), ("out_bf16", Buf),
        ("act", C.c_uint32), ("parity_mode", C.c_uint32), ("n_offset", C.c_uint32),
        ("ldo", C.c_uint32), ("flags", C.c_uint32), ("out_global", C.c_float),
        ("out_codes", Buf), ("out_scales", Buf), ("w_dense", Buf),
    ]


class DenseActSites(C.Structure):
    """tnf_dense_act_sites: which sites keep un-quantised activations (DenseActSites in the reference)."""
    _fields_ = [("qkv", C.c_uint32), ("qkv_self", C.c_uint32), ("proj", C.c_uint32), ("ffn_up", C.c_uint32), ("ffn_down", C.c_uint32)]


SITE_QKV, SITE_QKV_SELF, SITE_PROJ, SITE_FFN_UP, SITE_FFN_DOWN = range(5)


class SdpaArgs(C.Structure):
    _fields_ = [("b", C.c_uint32), ("s_q", C.c_uint32), ("s_k", C.c_uint32), ("h_q", C.c_uint32), ("h_kv", C.c_uint32),
                ("d", C.c_uint32), ("scale", C.c_float), ("mask_mode", C.c_uint32), ("q", Buf), ("k", Buf), ("v", Buf), ("out", Buf),
                ("flags", C.c_uint32), ("out_global", C.c_float), ("out_codes", Buf), ("out_scales", Buf),
                ("q_ld", C.c_uint32), ("kv_ld", C.c_uint32)]


SDPA_OUT_NVFP4, SDPA_NO_BF16_OUT = 1, 2


class NormQuantArgs(C.Structure):
    _fields_ = [
        ("m", C.c_uint32), ("k", C.c_uint32), ("eps", C.c_float), ("mod_bias", C.c_float),
        ("x_bf16", Buf), ("scale_bf16", Buf), ("shift_bf16", Buf), ("out_bf16", Buf), ("out_codes", Buf), ("out_scales", Buf),
        ("out_global", C.c_float), ("parity_mode", C.c_uint32),
    ]


class GgufTensorInfo(C.Structure):
    _fields_ = [("name", C.c_char_p), ("n_dims", C.c_uint32), ("dims", C.c_uint64 * 8), ("ggml_type", C.c_uint32),
                ("offset", C.c_uint64), ("size", C.c_uint64), ("on_disk_bytes", C.c_uint64)]


GGUF_NEED_MORE = 1
GGML_TYPE_NVFP4_RECORD = 0x4E564634


class StackLinear(C.Structure):
    _fields_ = [("n", C.c_uint32), ("k", C.c_uint32), ("act", C.c_uint32), ("has_bias", C.c_uint32),
                ("input", C.c_uint32), ("stream_id", C.c_uint32)]


READER_DEFAULT_HINTS = 0xFFFFFFFF
READER_LEN = C.CFUNCTYPE(C.c_uint64, C.c_void_p)
READER_READ_AT = C.CFUNCTYPE(C.c_int32, C.c_void_p, C.c_uint64, C.c_void_p, C.c_uint64)
READER_WILL_READ = C.CFUNCTYPE(None, C.c_void_p, C.c_uint64, C.c_uint64)
READER_CLOSE = C.CFUNCTYPE(None, C.c_void_p)


class Reader(C.Structure):
    """tnf_reader: len / read_at / will_read / close over an opaque `user` (WeightReader in the reference)."""
    _fields_ = [("user", C.c_void_p), ("len", READER_LEN), ("read_at", READER_READ_AT), ("will_read", READER_WILL_READ),
                ("close", READER_CLOSE)]


_u64p, _u32p, _vpp = C.POINTER(C.c_uint64), C.POINTER(C.c_uint32), C.POINTER(C.c_void_p)
_ctx = C.c_void_p

# name -> (restype, argtypes); must list every symbol include/thinfer_nvfp4.h declares
SIGNATURES = {
    "tnf_create": (C.c_int32, [C.c_int32, C.c_uint64, C.POINTER(_ctx)]),
    "tnf_destroy": (C.c_int32, [_ctx]),
    "tnf_last_error": (C.c_char_p, []),
    "tnf_abi_version": (C.c_uint32, []),
    "tnf_alloc": (C.c_int32, [_ctx, C.c_uint64, C.c_int32, _u64p]),
    "tnf_free": (C.c_int32, [_ctx, C.c_uint64]),
    "tnf_write": (C.c_int32, [_ctx, C.c_uint64, C.c_uint64, C.c_void_p, C.c_uint64]),
    "tnf_read": (C.c_int32, [_ctx, C.c_uint64, C.c_uint64, C.c_void_p, C.c_uint64]),
    "tnf_copy": (C.c_int32, [_ctx, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint64]),
    "tnf_buf_ptr": (C.c_int32, [_ctx, C.c_uint64, _vpp, _u64p]),
    "tnf_sync": (C.c_int32, [_ctx, C.c_uint32]),
    "tnf_mem_snapshot": (C.c_int32, [_ctx, _u64p]),
    "tnf_streams": (C.c_int32, [_ctx, _vpp, _vpp]),
    "tnf_set_device_wait_limit": (C.c_int32, [_ctx, C.c_uint64]),
    "tnf_selftest_stalled_wait": (C.c_int32, [_ctx]),
    "tnf_quantize_weight": (C.c_int32, [_ctx, Buf, C.c_int32, C.c_uint32, C.c_uint32, Buf, Buf, C.POINTER(C.c_float)]),
    "tnf_device_scales_bytes": (C.c_uint64, [C.c_uint32, C.c_uint32]),
    "tnf_prepare_scales": (C.c_int32, [_ctx, Buf, C.c_uint32, C.c_uint32, Buf]),
    "tnf_quantize_act": (C.c_int32, [_ctx, Buf, C.c_uint32, C.c_uint32, C.c_float, C.c_int32, Buf, Buf, C.POINTER(C.c_float)]),
    "tnf_linear_nvfp4": (C.c_int32, [_ctx, C.POINTER(LinearArgs)]),
    "tnf_prepare_dense": (C.c_int32, [_ctx, Buf, Buf, C.c_uint32, C.c_uint32, Buf]),
    "tnf_site_linear_flags": (C.c_uint32, [C.POINTER(DenseActSites), C.c_int32]),
    "tnf_linear_nvfp4_noalloc": (C.c_int32, [_ctx, C.POINTER(LinearArgs)]),
    "tnf_sdpa": (C.c_int32, [_ctx, C.POINTER(SdpaArgs)]),
    "tnf_norm_modulate_quantize": (C.c_int32, [_ctx, C.POINTER(NormQuantArgs)]),
    "tnf_noalloc_scratch_bytes": (C.c_uint64, []),
    "tnf_quantize_act_shared": (C.c_int32, [_ctx, Buf, C.c_uint32, C.c_uint32, C.c_float]),
    "tnf_gemm_nvfp4": (C.c_int32, [_ctx, C.POINTER(LinearArgs), Buf, Buf]),
    "tnf_host_register": (C.c_int32, [_ctx, C.c_void_p, C.c_uint64, _u64p]),
    "tnf_host_ptr": (C.c_int32, [_ctx, C.c_uint64, _vpp, _u64p]),
    "tnf_host_release": (C.c_int32, [_ctx, C.c_uint64]),
    "tnf_stream_upload": (C.c_int32, [_ctx, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint64, _u64p]),
    "tnf_wait_event": (C.c_int32, [_ctx, C.c_uint64]),
    "tnf_stream_download": (C.c_int32, [_ctx, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint64, _u64p]),
    "tnf_event_sync": (C.c_int32, [_ctx, C.c_uint64]),
    "tnf_copy_after_compute": (C.c_int32, [_ctx]),
    "tnf_stack_record_bytes": (C.c_uint64, [C.c_uint32, C.c_uint32]),
    "tnf_stack_create": (C.c_int32, [_ctx, C.c_uint32, C.c_uint32, C.POINTER(StackLinear), C.c_uint32, _u32p,
                                     C.c_uint32, C.c_uint64, C.c_uint64, C.c_uint32, C.POINTER(C.c_void_p)]),
    "tnf_stack_record_offsets": (C.c_int32, [C.c_uint32, C.c_uint32, _u64p]),
    "tnf_stack_step": (C.c_int32, [C.c_void_p, _u64p, _u64p, _u64p, C.c_float]),
    "tnf_stack_stats": (C.c_int32, [C.c_void_p, _u64p]),
    "tnf_stack_destroy": (C.c_int32, [C.c_void_p]),
    "tnf_stack_evict_all": (C.c_int32, [C.c_void_p]),
    "tnf_stack_restore": (C.c_int32, [C.c_void_p, C.c_uint64]),
    "tnf_reclaimed_bytes": (C.c_int32, [_ctx, _u64p]),
    "tnf_set_transient_reserve": (C.c_int32, [_ctx, C.c_uint64]),
    "tnf_ws_alloc": (C.c_int32, [_ctx, C.c_uint64, _u64p]),
    "tnf_ws_release": (C.c_int32, [_ctx, C.c_uint64]),
    "tnf_ws_drain": (C.c_int32, [_ctx, _u64p]),
    "tnf_ws_stats": (C.c_int32, [_ctx, _u64p]),
    "tnf_mmap_open": (C.c_int32, [C.c_char_p, C.POINTER(Reader)]),
    "tnf_mmap_stats": (C.c_int32, [C.POINTER(Reader), _u64p]),
    "tnf_reader_view": (C.c_int32, [C.POINTER(Reader), C.c_uint64, C.c_uint64, C.POINTER(Reader)]),
    "tnf_reader_close": (None, [C.POINTER(Reader)]),
    "tnf_reader_read": (C.c_int32, [C.POINTER(Reader), C.c_uint64, C.c_uint64, C.c_void_p, C.c_uint64, C.c_uint32]),
    "tnf_reader_read_to_arena": (C.c_int32, [_ctx, C.POINTER(Reader), C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint64,
                                             C.c_uint64, C.c_uint32]),
    "tnf_upload_from_reader": (C.c_int32, [_ctx, C.POINTER(Reader), C.c_uint64, C.c_uint64, Buf, C.c_uint64, C.c_uint32, _u64p]),
    "tnf_gguf_parse": (C.c_int32, [C.c_void_p, C.c_uint64, C.POINTER(C.c_void_p), _u64p]),
    "tnf_gguf_free": (C.c_int32, [C.c_void_p]),
    "tnf_gguf_info": (C.c_int32, [C.c_void_p, _u64p]),
    "tnf_gguf_tensor": (C.c_int32, [C.c_void_p, C.c_uint64, C.c_uint64, C.POINTER(GgufTensorInfo)]),
    "tnf_ggml_type_label": (C.c_char_p, [C.c_uint32]),
    "tnf_comm_unique_id": (C.c_int32, [C.c_void_p]),
    "tnf_comm_init": (C.c_int32, [_ctx, C.c_int32, C.c_int32, C.c_void_p]),
    "tnf_all_gather_cols": (C.c_int32, [_ctx, Buf, C.c_uint32, C.c_uint32, C.c_uint32]),
    "tnf_all_gather_nvfp4": (C.c_int32, [_ctx, Buf, Buf, C.c_uint32, C.c_uint32, C.c_uint32]),
    "tnf_ipc_export": (C.c_int32, [_ctx, C.c_uint64, C.c_void_p]),
    "tnf_peer_outputs": (C.c_int32, [_ctx, C.c_int32, C.c_int32, C.c_void_p]),
    "tnf_scatter_rows": (C.c_int32, [_ctx, C.c_int32, Buf, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32]),
    "tnf_push_peers": (C.c_int32, [_ctx, C.c_int32, Buf, C.c_uint64, Buf]),
    "tnf_interleave_cols": (C.c_int32, [_ctx, Buf, C.c_uint64, C.c_uint32, C.c_uint32, Buf, C.c_uint32, C.c_uint32, C.c_uint32]),
    "tnf_compute_after_copy": (C.c_int32, [_ctx]),
    "tnf_compute_after_push": (C.c_int32, [_ctx]),
    "tnf_comm_barrier": (C.c_int32, [_ctx]),
    "tnf_import_symmetric": (C.c_int32, [_ctx, C.c_void_p, C.c_void_p, C.c_uint64, C.c_int32, _u64p]),
    "tnf_multicast_copy": (C.c_int32, [_ctx, Buf, C.c_uint64, C.c_uint64, C.c_uint64]),
}

_lib = None


def load() -> C.CDLL:
    """Load the CUDA library. Raises if it has not been built; nothing stands in for it."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m thinfer_b200.build` "
                "(nvcc, sm_100a). thinfer_b200 has no CPU or PyTorch fallback.")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError if the library lacks a declared symbol
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib
