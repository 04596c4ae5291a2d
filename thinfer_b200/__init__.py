"""thinfer_b200 — the NVFP4 linear path of thinfer for B200 (sm_100a).

Host-side mirror of the reference's backend / op surface for this one path, over the
C ABI in ``include/thinfer_nvfp4.h``. Everything computes on the GPU through
``libthinfer_nvfp4.so``; there is no CPU or PyTorch fallback.
"""
from . import _lib  # noqa: F401
from .backend import (  # noqa: F401
    Backend, BatchScope, BudgetExceeded, DenseActSites, DeviceTimeout, InvalidArgument, Nvfp4Weight, TnfError, UnknownBuffer, WsBuf,
    interleave_swiglu,
)
from .reader import CallbackReader, MmapReader, Reader, ReaderError, ReaderView  # noqa: F401
