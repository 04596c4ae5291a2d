"""Host IO: random-access readers with readahead hints, over the library's ``tnf_reader``.

Mirrors the reference's ``WeightReader`` / ``FileOpener`` / ``OffsetView``
(thinfer-core/src/weight.rs:57-127) and its native mmap reader (thinfer-native/src/lib.rs:15-106).
``MmapReader`` is the library's own reader (mmap + ``madvise(WILLNEED)`` hints); ``CallbackReader``
wraps any Python object with ``len() / read_at(offset, dst) / will_read(offset, n)`` — the way an
embedding program passes its own reader through the C ABI. The chunk loops (hint ``hint_chunks``
chunks ahead, read a chunk, land it) run in the library.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import numpy as np

from . import _lib as L


class ReaderError(IOError):
    """A read outside the reader's range, a failing ``read_at``, or a file that cannot be opened."""


def _check(rc: int) -> None:
    if rc != L.OK:
        raise ReaderError(L.load().tnf_last_error().decode())


class Reader:
    """Base: owns one ``tnf_reader`` struct; subclasses fill it."""

    def __init__(self):
        self._r = L.Reader()
        self._open = False

    @property
    def raw(self):
        if not self._open:
            raise ReaderError("reader is closed")
        return C.byref(self._r)

    def __len__(self) -> int:
        return int(self._r.len(self._r.user)) if self._open else 0

    def will_read(self, offset: int, n: int) -> None:
        if self._open and self._r.will_read:
            self._r.will_read(self._r.user, offset, n)

    def read(self, offset: int, n: int, chunk_bytes: int = 0, hint_chunks: int = L.READER_DEFAULT_HINTS,
             out: Optional[np.ndarray] = None) -> np.ndarray:
        """[offset, offset+n) into ``out`` (uint8, made if absent) through the library's chunk loop."""
        if out is None:
            out = np.empty(n, np.uint8)
        if out.dtype != np.uint8 or out.size < n or not out.flags.c_contiguous:
            raise ValueError(f"destination must be contiguous uint8 with at least {n} bytes")
        _check(L.load().tnf_reader_read(self.raw, offset, n, out.ctypes.data_as(C.c_void_p), chunk_bytes, hint_chunks))
        return out[:n]

    def read_to_arena(self, be, offset: int, n: int, arena, arena_off: int, chunk_bytes: int = 0,
                      hint_chunks: int = L.READER_DEFAULT_HINTS) -> None:
        """[offset, offset+n) into a pinned ``HostArena`` at ``arena_off``."""
        _check(L.load().tnf_reader_read_to_arena(be._ctx, self.raw, offset, n, arena.id, arena_off, chunk_bytes, hint_chunks))

    def upload(self, be, offset: int, total: int, dst: L.Buf, chunk_bytes: int = 0,
               hint_chunks: int = L.READER_DEFAULT_HINTS, want_event: bool = False) -> Optional[int]:
        """Stream [offset, offset+total) into the device view ``dst`` (zero-filled past ``total``) on the copy
        stream, double-buffered through pinned staging. Returns the completion event id if asked for."""
        ev = C.c_uint64()
        _check(L.load().tnf_upload_from_reader(be._ctx, self.raw, offset, total, dst, chunk_bytes, hint_chunks,
                                               C.byref(ev) if want_event else None))
        return int(ev.value) if want_event else None

    def view(self, base: int, length: int) -> "ReaderView":
        return ReaderView(self, base, length)

    def close(self) -> None:
        if self._open:
            L.load().tnf_reader_close(C.byref(self._r))
            self._open = False

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


class MmapReader(Reader):
    """The whole file mapped read-only; ``will_read`` starts the page-in of a range."""

    def __init__(self, path: str):
        super().__init__()
        _check(L.load().tnf_mmap_open(path.encode(), C.byref(self._r)))
        self._open = True

    def stats(self) -> dict:
        out = (C.c_uint64 * 4)()
        _check(L.load().tnf_mmap_stats(self.raw, out))
        return dict(reads=int(out[0]), read_bytes=int(out[1]), hints=int(out[2]), hint_bytes=int(out[3]))


class ReaderView(Reader):
    """``inner`` restricted to [base, base+length), offsets rebased to 0. Keeps ``inner`` alive; closing the
    view leaves ``inner`` open."""

    def __init__(self, inner: Reader, base: int, length: int):
        super().__init__()
        self._inner = inner
        _check(L.load().tnf_reader_view(inner.raw, base, length, C.byref(self._r)))
        self._open = True


class CallbackReader(Reader):
    """Adapts a Python object with ``__len__``, ``read_at(offset, dst: memoryview)`` and optionally
    ``will_read(offset, n)`` to a ``tnf_reader``. An exception in ``read_at`` becomes an error return."""

    def __init__(self, obj):
        super().__init__()
        self._obj = obj
        self.error: Optional[BaseException] = None

        def _len(_u):
            return len(obj)

        def _read_at(_u, offset, dst, n):
            try:
                obj.read_at(int(offset), memoryview((C.c_uint8 * n).from_address(dst)).cast("B") if n else memoryview(b""))
                return L.OK
            except BaseException as e:  # the C loop stops at the first failing chunk
                self.error = e
                return L.ERR_INVALID_ARGUMENT

        def _will_read(_u, offset, n):
            obj.will_read(int(offset), int(n))

        self._keep = [L.READER_LEN(_len), L.READER_READ_AT(_read_at)]  # the struct holds raw pointers: keep the thunks
        self._r.user = None
        self._r.len, self._r.read_at = self._keep
        if hasattr(obj, "will_read"):
            self._keep.append(L.READER_WILL_READ(_will_read))
            self._r.will_read = self._keep[-1]
        self._open = True

    def close(self) -> None:  # nothing of the library's to release
        self._open = False
