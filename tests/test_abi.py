"""The C-ABI library loads and exports every symbol include/thinfer_nvfp4.h declares (CPU only;
no compute call is made here)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "thinfer_nvfp4.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tnf_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_exported_and_bound():
    from thinfer_b200 import _lib

    names = declared_symbols()
    assert len(names) >= 30
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for n in names:
        assert hasattr(lib, n), f"{n} declared in the header but not exported"
    assert sorted(_lib.SIGNATURES) == names, "ctypes binding table and header disagree"


def test_struct_layouts_match_header():
    from thinfer_b200._lib import Buf, LinearArgs, StackLinear

    assert ctypes.sizeof(Buf) == 24
    assert ctypes.sizeof(LinearArgs) == 5 * 4 + 4 + 7 * 24 + 6 * 4 + 3 * 24  # 5 scalars (+pad), 7 views, 6 words, 3 views
    assert ctypes.sizeof(StackLinear) == 24
    from thinfer_b200._lib import Reader, SdpaArgs
    assert ctypes.sizeof(SdpaArgs) == 8 * 4 + 4 * 24 + 2 * 4 + 2 * 24 + 2 * 4  # 8 words, 4 views, 2 words, 2 views, 2 words
    assert ctypes.sizeof(Reader) == 5 * 8


def test_no_device_fails_loudly():
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    import thinfer_b200 as T

    with pytest.raises(T.TnfError) as e:
        T.Backend(0)
    assert "no CPU path" in str(e.value)


def test_abi_version_and_sizes():
    from thinfer_b200 import _lib

    lib = _lib.load()
    assert lib.tnf_abi_version() == 3
    # 128-row x 4-block atoms of 512 bytes; K atoms rounded up to a multiple of 4
    assert lib.tnf_device_scales_bytes(128, 256) == 4 * 512
    assert lib.tnf_device_scales_bytes(129, 3072) == 2 * 48 * 512
    assert lib.tnf_device_scales_bytes(1, 64) == 4 * 512


def test_rust_bindings_declare_every_header_symbol():
    """rust/thinfer-native-cuda/src/ffi.rs (generated from the header) lists exactly the header's functions, and its
    struct fields follow the ctypes mirror (same order, so the same layout under repr(C))."""
    text = open(os.path.join(ROOT, "rust", "thinfer-native-cuda", "src", "ffi.rs")).read()
    rust = sorted(set(re.findall(r"pub fn (tnf_[a-z0-9_]+)\s*\(", text)))
    assert rust == declared_symbols()
    from thinfer_b200._lib import DenseActSites, LinearArgs, NormQuantArgs, Reader, SdpaArgs, StackLinear

    for rust_name, ct in (("TnfLinearArgs", LinearArgs), ("TnfNormQuantArgs", NormQuantArgs), ("TnfStackLinear", StackLinear),
                          ("TnfDenseActSites", DenseActSites), ("TnfSdpaArgs", SdpaArgs), ("TnfReader", Reader)):
        body = re.search(r"pub struct %s \{(.*?)\n?\}" % rust_name, text, flags=re.S).group(1)
        fields = re.findall(r"pub (\w+):", body)
        assert fields == [f[0] for f in ct._fields_], rust_name


def test_site_policy_flags_are_host_only():
    from thinfer_b200 import DenseActSites, _lib as L

    pol = DenseActSites(proj=True, ffn_down=True)
    assert [pol.flags(s) for s in range(5)] == [0, 0, L.LINEAR_DENSE_ACT, 0, L.LINEAR_DENSE_ACT]
    assert DenseActSites().flags(L.SITE_QKV) == 0 and pol.flags(7) == 0
