"""GGUF-v3 container: the header parser against the cases of the reference's own unit tests
(thinfer-core/src/format/gguf.rs:549-668), its error variants, the writer/reader round trip and,
on a GPU, a checkpoint transcoded to NVFP4 records, written, read back into the pinned arena and
streamed."""
import ctypes as C
import struct

import numpy as np
import pytest

import oracle as O


def _s(t: str) -> bytes:
    b = t.encode()
    return struct.pack("<Q", len(b)) + b


def _minimal(alignment=32, version=3, magic=0x46554747):
    """Two Q8_0 tensors, "a" [32] at 0 and "bb" GGUF dims [32, 2] at 34, one alignment key: the file the
    reference's tests build."""
    b = struct.pack("<IIQQ", magic, version, 2, 1)
    b += _s("general.alignment") + struct.pack("<II", 4, alignment)
    b += _s("a") + struct.pack("<IQIQ", 1, 32, 8, 0)
    b += _s("bb") + struct.pack("<IQQIQ", 2, 32, 2, 8, 34)
    b += b"\0" * (-len(b) % 32)
    data_offset = len(b)
    b += b"\0" * (34 + 68)
    return b, data_offset


def _parse(buf: bytes):
    from thinfer_b200 import _lib as L

    lib = L.load()
    h, need = C.c_void_p(), C.c_uint64()
    rc = lib.tnf_gguf_parse(buf, len(buf), C.byref(h), C.byref(need))
    return lib, rc, h, int(need.value)


def test_parse_minimal_header_and_catalog():
    from thinfer_b200 import _lib as L

    buf, data_offset = _minimal()
    lib, rc, h, _ = _parse(buf)
    assert rc == 0
    info = (C.c_uint64 * 4)()
    lib.tnf_gguf_info(h, info)
    assert list(info) == [3, 32, data_offset, 2]
    t = L.GgufTensorInfo()
    assert lib.tnf_gguf_tensor(h, 0, len(buf), C.byref(t)) == 0
    assert (t.name, t.n_dims, t.dims[0], t.ggml_type, t.on_disk_bytes, t.size, t.offset) == (b"a", 1, 32, 8, 34, 34, data_offset)
    assert lib.tnf_gguf_tensor(h, 1, len(buf), C.byref(t)) == 0
    # GGUF dims [32, 2] are innermost-first; the catalog is outer-first [2, 32]; size runs to the end of the file
    assert (t.name, t.n_dims, t.dims[0], t.dims[1], t.on_disk_bytes, t.size) == (b"bb", 2, 2, 32, 68, 68)
    assert lib.tnf_gguf_tensor(h, 1, 0, C.byref(t)) == 0 and t.size == 68  # no file size: the type's own size
    assert lib.tnf_gguf_tensor(h, 2, 0, C.byref(t)) != 0
    assert lib.tnf_ggml_type_label(8) == b"Q8_0" and lib.tnf_ggml_type_label(30) == b"BF16"
    assert lib.tnf_ggml_type_label(L.GGML_TYPE_NVFP4_RECORD) == b"NVFP4_RECORD" and lib.tnf_ggml_type_label(99) == b"UNKNOWN"
    lib.tnf_gguf_free(h)


def test_truncated_buffer_yields_need_more():
    from thinfer_b200 import _lib as L

    buf, _ = _minimal()
    for cut in (0, 4, 16, 32, 64, 100):
        lib, rc, h, need = _parse(buf[:cut])
        assert rc == L.GGUF_NEED_MORE and need > cut and not h.value


@pytest.mark.parametrize("mutate,variant", [
    (lambda: _minimal(magic=0xDEADBEEF)[0], "BadMagic(0xdeadbeef)"),
    (lambda: _minimal(version=2)[0], "UnsupportedVersion(2)"),
    (lambda: _minimal(alignment=0)[0], "BadAlignment(0)"),
    (lambda: _minimal(alignment=48)[0], "BadAlignment(48)"),
    (lambda: _minimal(alignment=1 << 17)[0], "AlignmentTooLarge(131072)"),
    (lambda: struct.pack("<IIQQ", 0x46554747, 3, 0, 1) + _s("k") + struct.pack("<IB", 7, 2), "BadBool(2)"),
    (lambda: struct.pack("<IIQQ", 0x46554747, 3, 0, 1) + _s("k") + struct.pack("<I", 13), "BadValueType(13)"),
    (lambda: struct.pack("<IIQQ", 0x46554747, 3, 1, 0) + _s("t") + struct.pack("<I", 0), "BadDimCount(0)"),
    (lambda: struct.pack("<IIQQ", 0x46554747, 3, 1, 0) + _s("t") + struct.pack("<I", 9), "BadDimCount(9)"),
    (lambda: struct.pack("<IIQQ", 0x46554747, 3, 0, 1) + struct.pack("<Q", 1 << 30), "Oversized { field: string_len"),
    (lambda: struct.pack("<IIQQ", 0x46554747, 3, 2_000_000, 0), "Oversized { field: n_tensors"),
    (lambda: struct.pack("<IIQQ", 0x46554747, 3, 0, 1) + struct.pack("<Q", 2) + b"\xff\xfe", "BadUtf8"),
])
def test_malformed_headers_name_the_reference_error(mutate, variant):
    lib, rc, h, _ = _parse(mutate())
    assert rc == -4 and not h.value
    assert variant in lib.tnf_last_error().decode()


def test_metadata_of_every_kind_is_walked():
    """Values the catalog does not need are skipped byte-accurately, nested arrays included."""
    b = struct.pack("<IIQQ", 0x46554747, 3, 1, 6)
    b += _s("a.u8") + struct.pack("<IB", 0, 7) + _s("a.f64") + struct.pack("<Id", 12, 2.5) + _s("a.str") + struct.pack("<I", 8) + _s("héllo")
    b += _s("a.arr") + struct.pack("<IIQ", 9, 5, 3) + struct.pack("<iii", 1, -2, 3)
    b += _s("a.nested") + struct.pack("<IIQ", 9, 9, 2) + struct.pack("<IQ", 8, 1) + _s("x") + struct.pack("<IQ", 2, 2) + struct.pack("<HH", 1, 2)
    b += _s("general.alignment") + struct.pack("<IQ", 10, 64)
    b += _s("w") + struct.pack("<IQQIQ", 2, 16, 4, 30, 0)
    lib, rc, h, _ = _parse(b)
    assert rc == 0
    info = (C.c_uint64 * 4)()
    lib.tnf_gguf_info(h, info)
    assert info[1] == 64 and info[2] == (len(b) + 63) // 64 * 64 and info[3] == 1
    lib.tnf_gguf_free(h)


def test_writer_reader_round_trip(tmp_path):
    from thinfer_b200.container import GGML_BF16, GGML_F32, GGML_NVFP4_RECORD, Container, ContainerError, write_container
    from thinfer_b200.residency import record_bytes

    rng = np.random.default_rng(3)
    n, k = 136, 96
    rec = rng.integers(0, 256, record_bytes(n, k), dtype=np.uint8)
    f32 = rng.standard_normal((5, 7)).astype(np.float32)
    bf = rng.integers(0, 65536, (3, 8), dtype=np.uint16)
    tensors = [(f"blk.{i}.pad", (1 + i,), GGML_F32, np.zeros(1 + i, np.float32)) for i in range(300)]  # a header of > 4 KiB
    tensors += [("blk.0.linear.0.nvfp4", (n, k), GGML_NVFP4_RECORD, rec), ("norm.w", f32.shape, GGML_F32, f32), ("emb", bf.shape, GGML_BF16, bf)]
    path = str(tmp_path / "m.gguf")
    size = write_container(path, tensors, metadata=[("general.name", "str", "tiny"), ("tnf.layers", "u32", 1)])
    c = Container(path)
    assert c.file_size == size and c.alignment == 256 and c.data_offset % 256 == 0 and c.header_reads_to > 4096
    e = c.tensors["blk.0.linear.0.nvfp4"]
    assert e.shape == (n, k) and e.label == "NVFP4_RECORD" and e.on_disk_bytes == rec.size and e.offset % 256 == 0
    assert e.size == (rec.size + 255) // 256 * 256
    assert np.array_equal(c.read("blk.0.linear.0.nvfp4"), rec)
    assert np.array_equal(c.read("norm.w").view(np.float32).reshape(5, 7), f32)
    assert np.array_equal(c.read("emb").view(np.uint16).reshape(3, 8), bf)
    dst = np.zeros(rec.size + 10, np.uint8)
    assert c.read_into("blk.0.linear.0.nvfp4", dst) == rec.size and not dst[rec.size:].any()
    with pytest.raises(ContainerError):
        c.read("missing")
    with pytest.raises(ValueError):
        c.read_into("norm.w", np.zeros(4, np.uint8))
    # a file cut inside its header
    with open(path, "rb") as f:
        head = f.read(1000)
    cut = str(tmp_path / "cut.gguf")
    with open(cut, "wb") as f:
        f.write(head)
    with pytest.raises(ContainerError):
        Container(cut)


@pytest.mark.gpu
def test_transcoded_checkpoint_streams_from_the_container(backend, tmp_path):
    """Dense weights -> NVFP4 records on the GPU -> container -> pinned arena -> streamed stack: the records
    equal the ones packed from the oracle quantiser and the stack computes the same outputs."""
    from thinfer_b200.container import GGML_NVFP4_RECORD, Container, load_stack, record_name, transcode_linear, write_container
    from thinfer_b200.residency import LayerStack, StackLinearSpec as S, record_bytes, scales_to_device_layout

    be = backend
    hidden, layers, a_global = 128, 3, 0.004
    specs = [S(384, 128, 0, True, 0, 0), S(128, 128, 0, True, 2, 0), S(256, 128, 1, True, 1, 0), S(128, 256, 0, True, 1, 0)]
    m_rows = [96]
    direct = LayerStack(be, layers, specs, m_rows, hidden)
    tensors = []
    for l in range(layers):
        for j, s in enumerate(specs):
            w = (O.gaussian(s.n * s.k, 900 + 10 * l + j) * np.float32(1.0 / np.sqrt(s.k))).reshape(s.n, s.k)
            b = O.f32_to_bf16(O.gaussian(s.n, 950 + 10 * l + j) * np.float32(0.01))
            c, sc, g = O.quantize_weight(w)
            direct.pack(l, j, c, scales_to_device_layout(sc), g, b)
            rec = transcode_linear(be, w, b)  # the GPU quantiser
            assert rec.size == record_bytes(s.n, s.k) and np.array_equal(rec, direct.record_view(l, j))
            tensors.append((record_name(l, j), (s.n, s.k), GGML_NVFP4_RECORD, rec))
    path = str(tmp_path / "ckpt.gguf")
    write_container(path, tensors, metadata=[("tnf.layers", "u32", layers)])
    cont = Container(path)
    loaded = LayerStack(be, layers, specs, m_rows, hidden)
    assert load_stack(cont, loaded) == layers * sum(record_bytes(s.n, s.k) for s in specs)
    assert np.array_equal(loaded.arena.np, direct.arena.np)
    x = O.f32_to_bf16(O.gaussian(96 * hidden, 77).reshape(96, hidden))
    aux = O.f32_to_bf16(O.gaussian(96 * hidden, 78).reshape(96, hidden))
    outs = []
    for st in (direct, loaded):
        xb, ab, ob = be.upload(x), be.upload(aux), be.allocate(96 * hidden * 2)
        st.build(weight_budget=2 * sum(record_bytes(s.n, s.k) for s in specs), ring_slots=2)  # everything streams
        st.step([xb], [ob], a_global, aux=[ab])
        be.submit(30000)
        outs.append(be.read_buffer(ob, np.uint16))
        st.close()
        for b in (xb, ab, ob):
            be.free(b)
    assert np.array_equal(outs[0], outs[1]) and not np.isnan(O.bf16_to_f32(outs[0])).any()
