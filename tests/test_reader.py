"""Host IO readers: the mmap reader, offset views, readers passed in by the caller, the chunk loop's
hint schedule (the reference's: READ_PREFETCH_CHUNKS chunks primed, then one hint per chunk read,
thinfer-core/src/residency.rs:1253-1292), and on a GPU the double-buffered upload from a reader.
The cases follow the reference's reader contract (thinfer-core/src/weight.rs:57-127) and its mmap
reader (thinfer-native/src/lib.rs:54-106): bounds-checked reads, hints that never change bytes."""
import ctypes as C

import numpy as np
import pytest


def _file(tmp_path, n, seed=1):
    data = np.random.default_rng(seed).integers(0, 256, n, dtype=np.uint8)
    p = tmp_path / "blob.bin"
    p.write_bytes(data.tobytes())
    return str(p), data


class _MemSource:
    """A reader kept by the caller: bytes in memory, every call logged."""

    def __init__(self, data, fail_at=None):
        self.data, self.log, self.fail_at = data, [], fail_at

    def __len__(self):
        return self.data.size

    def read_at(self, offset, dst):
        self.log.append(("read", offset, len(dst)))
        if self.fail_at is not None and offset >= self.fail_at:
            raise IOError("disk went away")
        dst[:] = self.data[offset: offset + len(dst)].tobytes()

    def will_read(self, offset, n):
        self.log.append(("hint", offset, n))


def test_mmap_reader_reads_and_bounds(tmp_path):
    from thinfer_b200.reader import MmapReader, ReaderError

    path, data = _file(tmp_path, 100_003)
    with MmapReader(path) as r:
        assert len(r) == data.size
        assert np.array_equal(r.read(0, data.size), data)
        assert np.array_equal(r.read(77, 1000, chunk_bytes=64), data[77:1077])
        assert r.read(data.size, 0).size == 0  # an empty read at the end is fine
        with pytest.raises(ReaderError, match="outside a reader"):
            r.read(data.size - 10, 11)
        from thinfer_b200 import _lib as L
        small = (C.c_uint8 * 8)()  # offset + n overflows 64 bits: refused, nothing written
        assert L.load().tnf_reader_read(r.raw, 2**63, 2**63, small, 0, 0) == L.ERR_INVALID_ARGUMENT
        s = r.stats()
        assert s["read_bytes"] == data.size + 1000 and s["reads"] == 1 + 16
    with pytest.raises(ReaderError, match="No such file"):
        MmapReader(str(tmp_path / "missing.bin"))


def test_mmap_reader_empty_file(tmp_path):
    from thinfer_b200.reader import MmapReader

    p = tmp_path / "empty.bin"
    p.write_bytes(b"")
    with MmapReader(str(p)) as r:
        assert len(r) == 0 and r.read(0, 0).size == 0


def test_mmap_hints_are_counted_and_never_change_bytes(tmp_path):
    from thinfer_b200.reader import MmapReader

    path, data = _file(tmp_path, 1 << 20)
    with MmapReader(path) as r:
        r.will_read(123, 4567)            # unaligned start: the library rounds down to the page
        r.will_read(data.size - 5, 100)   # out of range: ignored
        r.will_read(0, 0)                 # empty: ignored
        out = r.read(0, data.size, chunk_bytes=1 << 16, hint_chunks=4)
        assert np.array_equal(out, data)
        s = r.stats()
        # 1 explicit hint + 4 primed + one per chunk that still has a chunk 4 ahead (16 chunks -> 12)
        assert s["hints"] == 1 + 4 + 12 and s["hint_bytes"] == 4567 + (1 << 20)


def test_chunk_loop_hint_schedule_matches_the_reference_loop():
    from thinfer_b200.reader import CallbackReader

    data = np.arange(10_500, dtype=np.uint32).astype(np.uint8)
    src = _MemSource(data)
    r = CallbackReader(src)
    out = r.read(200, 10_000, chunk_bytes=1000, hint_chunks=4)
    assert np.array_equal(out, data[200:10_200])
    want = [("hint", 200 + i * 1000, 1000) for i in range(4)]
    for i in range(10):
        want.append(("read", 200 + i * 1000, 1000))
        if i + 4 < 10:
            want.append(("hint", 200 + (i + 4) * 1000, 1000))
    assert src.log == want
    # ragged tail, fewer chunks than the hint depth, and no hints at all
    src.log.clear()
    r.read(0, 2500, chunk_bytes=1000, hint_chunks=4)
    assert src.log == [("hint", 0, 1000), ("hint", 1000, 1000), ("hint", 2000, 500),
                       ("read", 0, 1000), ("read", 1000, 1000), ("read", 2000, 500)]
    src.log.clear()
    r.read(0, 2500, chunk_bytes=1000, hint_chunks=0)
    assert [e[0] for e in src.log] == ["read"] * 3


def test_failing_read_stops_the_loop_and_is_reported():
    from thinfer_b200.reader import CallbackReader, ReaderError

    src = _MemSource(np.zeros(5000, np.uint8), fail_at=2000)
    r = CallbackReader(src)
    with pytest.raises(ReaderError):
        r.read(0, 5000, chunk_bytes=1000, hint_chunks=0)
    assert isinstance(r.error, IOError)
    assert [e[1] for e in src.log if e[0] == "read"] == [0, 1000, 2000]  # nothing after the failing chunk


def test_offset_view_rebases_reads_and_hints(tmp_path):
    from thinfer_b200.reader import CallbackReader, ReaderError

    data = np.random.default_rng(3).integers(0, 256, 4096, dtype=np.uint8)
    src = _MemSource(data)
    whole = CallbackReader(src)
    v = whole.view(1000, 512)
    assert len(v) == 512
    assert np.array_equal(v.read(10, 100, hint_chunks=0), data[1010:1110])
    v.will_read(500, 100)  # clipped to the window
    assert src.log[-1] == ("hint", 1500, 12)
    with pytest.raises(ReaderError, match="outside a reader"):
        v.read(500, 13)
    with pytest.raises(ReaderError, match="outside a reader"):
        whole.view(4000, 97)
    vv = v.view(100, 50)  # views nest
    assert np.array_equal(vv.read(0, 50, hint_chunks=0), data[1100:1150])
    v.close()
    assert np.array_equal(whole.read(0, 16, hint_chunks=0), data[:16])  # closing a view leaves the inner reader open


def test_container_opens_from_a_callers_reader(tmp_path):
    from thinfer_b200.container import Container, write_container, GGML_F32
    from thinfer_b200.reader import CallbackReader

    a = np.arange(64, dtype=np.float32)
    b = np.arange(96, dtype=np.float32).reshape(3, 32)
    p = str(tmp_path / "c.gguf")
    write_container(p, [("a", (64,), GGML_F32, a), ("b", (3, 32), GGML_F32, b)], alignment=64)
    raw = np.fromfile(p, np.uint8)
    src = _MemSource(raw)
    c = Container(CallbackReader(src), first_read=16)  # the header needs several growing reads
    assert set(c.tensors) == {"a", "b"} and c.file_size == raw.size
    assert np.array_equal(c.read("b").view(np.float32).reshape(3, 32), b)
    c.hint("a")
    assert src.log[-1] == ("hint", c.tensors["a"].offset, 256)
    c2 = Container(p)  # a path goes through the mmap reader
    assert np.array_equal(c2.read("a").view(np.float32), a)
    c2.close()


def test_null_reader_is_refused():
    from thinfer_b200 import _lib as L

    lib = L.load()
    r = L.Reader()  # no len, no read_at
    buf = (C.c_uint8 * 8)()
    assert lib.tnf_reader_read(C.byref(r), 0, 8, buf, 0, 0) == L.ERR_INVALID_ARGUMENT
    assert b"needs len and read_at" in lib.tnf_last_error()


@pytest.mark.gpu
def test_upload_from_reader_pads_and_matches(backend, tmp_path):
    """Reader -> pinned staging -> device, chunked and double buffered: the device bytes are the file's bytes, the
    tail of the view is zero, and a caller's reader sees the reference's hint schedule."""
    from thinfer_b200 import _lib as L
    from thinfer_b200.reader import CallbackReader, MmapReader
    from thinfer_b200.residency import HostArena

    be = backend
    path, data = _file(tmp_path, 3_000_001, seed=5)
    dst = be.allocate_in(3_100_000, L.CAT_WEIGHTS)
    be.write_buffer(dst, np.full(3_100_000, 0xAB, np.uint8))
    with MmapReader(path) as r:
        ev = r.upload(be, 1, 3_000_000, L.Buf(dst.id, 0, 3_100_000), chunk_bytes=1 << 18, want_event=True)
        assert be.lib.tnf_event_sync(be._ctx, ev) == 0
        got = be.read_buffer(dst)
        assert np.array_equal(got[:3_000_000], data[1:]) and not got[3_000_000:].any()
        # a second upload with a larger chunk regrows the staging slots
        ev = r.upload(be, 0, 2_000_000, L.Buf(dst.id, 4096, 2_000_000), chunk_bytes=1 << 20, want_event=True)
        assert be.lib.tnf_event_sync(be._ctx, ev) == 0
        assert np.array_equal(be.read_buffer(dst)[4096: 4096 + 2_000_000], data[:2_000_000])
        # into a pinned arena
        arena = HostArena(be, 1 << 20)
        r.read_to_arena(be, 5, 1 << 19, arena, 100, chunk_bytes=1 << 16)
        assert np.array_equal(arena.np[100: 100 + (1 << 19)], data[5: 5 + (1 << 19)])
        with pytest.raises(IOError, match="outside arena"):
            r.read_to_arena(be, 0, 1 << 20, arena, 1)
        arena.release()
    src = _MemSource(data)
    cr = CallbackReader(src)
    ev = cr.upload(be, 0, 1_000_000, L.Buf(dst.id, 0, 1_000_000), chunk_bytes=250_000, hint_chunks=2, want_event=True)
    assert be.lib.tnf_event_sync(be._ctx, ev) == 0
    assert [e for e in src.log if e[0] == "hint"] == [("hint", i * 250_000, 250_000) for i in range(4)]
    assert np.array_equal(be.read_buffer(dst)[:1_000_000], data[:1_000_000])
    be.free(dst)
