"""Streaming layer stack: resident vs streamed weights give identical results, the budget is
honoured, the ring wraps across steps. Host-side packing helpers are checked on the CPU."""
import numpy as np
import pytest

import oracle as O
from conftest import rel_fro


def test_device_layout_helper_matches_oracle():
    from thinfer_b200.residency import scales_to_device_layout

    rng = np.random.default_rng(0)
    for rows, nb in [(1, 2), (130, 6), (256, 192), (200, 20)]:
        s = rng.integers(0, 127, (rows, nb), dtype=np.uint8)
        assert np.array_equal(scales_to_device_layout(s), O.scales_to_device_layout(s))


def test_record_layout_is_aligned_and_sized():
    from thinfer_b200.residency import record_bytes, record_offsets

    for n, k in [(3072, 3072), (9216, 3072), (136, 96)]:
        oc, os_, ob, og = record_offsets(n, k)
        assert oc == 0 and os_ >= n * k // 2 and all(o % 256 == 0 for o in (os_, ob, og))
        assert record_bytes(n, k) == og + 256


def _build(be, layers, specs, m_rows, hidden, seed):
    from thinfer_b200.residency import LayerStack, scales_to_device_layout

    st = LayerStack(be, layers, specs, m_rows, hidden)
    ws = []
    for l in range(layers):
        row = []
        for j, s in enumerate(specs):
            w = (O.gaussian(s.n * s.k, seed + 100 * l + j) * np.float32(1.0 / np.sqrt(s.k))).reshape(s.n, s.k)
            b = O.f32_to_bf16(O.gaussian(s.n, seed + 7 + 100 * l + j) * np.float32(0.01)) if s.has_bias else None
            c, sc, g = O.quantize_weight(w)  # packing a checkpoint is offline work; the oracle quantiser stands in for it
            st.pack(l, j, c, scales_to_device_layout(sc), g, b)
            row.append((c, sc, g, b))
        ws.append(row)
    return st, ws


@pytest.mark.gpu
def test_stack_streamed_equals_resident_and_oracle(backend):
    from thinfer_b200.residency import StackLinearSpec as S, record_bytes

    be = backend
    hidden, layers, a_global = 128, 7, 0.004
    specs = [S(384, 128, 0, True, 0, 0), S(128, 128, 0, True, 2, 0), S(256, 128, 1, True, 1, 0), S(128, 256, 0, True, 1, 0),
             S(192, 128, 0, False, 0, 1)]
    m_rows = [200, 1]
    st, ws = _build(be, layers, specs, m_rows, hidden, 500)
    x = [O.f32_to_bf16(O.gaussian(m * hidden, 40 + i).reshape(m, hidden)) for i, m in enumerate(m_rows)]
    aux = [O.f32_to_bf16(O.gaussian(m * hidden, 50 + i).reshape(m, hidden)) for i, m in enumerate(m_rows)]
    xb = [be.upload(v) for v in x]
    ab = [be.upload(v) for v in aux]
    ob = [be.allocate(200 * 128 * 2), be.allocate(max(1 * 192 * 2, 256))]

    # oracle chain
    def oracle_step():
        cur = x[0]
        for l in range(layers):
            (c0, s0, g0, b0), (c1, s1, g1, b1), (c2, s2, g2, b2), (c3, s3, g3, b3), _ = ws[l]
            O.linear(cur, a_global, c0, s0, g0, bias=b0)  # qkv: output unused downstream
            h1 = O.linear(aux[0], a_global, c1, s1, g1, bias=b1)
            h2 = O.linear(h1, a_global, c2, s2, g2, bias=b2, act=1)
            cur = O.linear(h2, a_global, c3, s3, g3, bias=b3)
        c4, s4, g4, _ = ws[layers - 1][4]
        return cur, O.linear(x[1], a_global, c4, s4, g4)

    want0, want1 = oracle_step()
    results = []
    ring_need = 2 * sum(record_bytes(s.n, s.k) for s in specs)
    for budget, slots in [(0, 0), (ring_need + record_bytes(384, 128) * 3, 2), (ring_need, 2)]:
        info = st.build(weight_budget=budget, ring_slots=slots)
        if budget:
            assert info["resident_bytes"] + info["ring_bytes"] <= budget
            assert info["streamed_records"] > 0
        else:
            assert info["streamed_records"] == 0
        for step in range(3):  # the ring wraps: later steps find their first layers already uploaded
            st.step(xb, ob, a_global, aux=ab)
            be.submit(30000)
            got0 = be.read_buffer(ob[0], np.uint16).reshape(200, 128)
            got1 = be.read_buffer(ob[1], np.uint16)[:192].reshape(1, 192)
            results.append((got0, got1))
            s = st.stats()
            if budget and step > 0:  # the first step also fills the rings; afterwards: each streamed record once
                assert s["uploads_last_step"] == s["streamed_records"]
        be.lib.tnf_stack_destroy(st._stack)
        st._stack = type(st._stack)()
    for got0, got1 in results:
        assert np.array_equal(got0, results[0][0]) and np.array_equal(got1, results[0][1])
    assert rel_fro(O.bf16_to_f32(results[0][0]), O.bf16_to_f32(want0)) <= 2e-2  # 7 chained FP4 layers: GELU approx flips codes
    assert rel_fro(O.bf16_to_f32(results[0][1]), O.bf16_to_f32(want1)) <= 1e-3
    st.close()
    for b in xb + ab + ob:
        be.free(b)


@pytest.mark.gpu
def test_reclaim_chain_phase_eviction_and_restore():
    """The reclaim side of the residency manager. Under a context budget: (1) an allocation that does not fit first
    makes the stack give resident weight sets back (they are streamed from then on) and then succeeds; (2) a
    phase eviction frees every weight buffer; the next step brings the weights back by itself; (3) a restore after
    the other consumer is gone pins everything again. The step's outputs never change."""
    import thinfer_b200 as T
    from thinfer_b200.backend import BudgetExceeded
    from thinfer_b200.residency import StackLinearSpec as S, record_bytes

    hidden, layers, a_global = 128, 9, 0.004
    specs = [S(384, 128, 0, True, 0, 0), S(128, 384, 0, True, 1, 0)]
    weights = layers * sum(record_bytes(s.n, s.k) for s in specs)
    be = T.Backend(0, vram_budget=weights + (6 << 20))  # everything resident fits, with 6 MiB to spare
    try:
        st, _ = _build(be, layers, specs, [160], hidden, 700)
        x = O.f32_to_bf16(O.gaussian(160 * hidden, 41).reshape(160, hidden))
        xb, ob = [be.upload(x)], [be.allocate(160 * hidden * 2)]
        info = st.build(weight_budget=0, ring_slots=2)
        assert info["streamed_records"] == 0

        def run():
            st.step(xb, ob, a_global)
            be.submit(30000)
            return be.read_buffer(ob[0], np.uint16).copy()

        ref = run()
        # (1) another consumer takes most of the spare room and then some: the stack must give memory back
        spare = be.mem_snapshot()
        room = weights + (6 << 20) - (spare["live_weights"] + spare["live_workspace"] + spare["live_staging"])
        other = be.allocate_in(room + weights // 3, 1)
        got = C_u64()
        be.lib.tnf_reclaimed_bytes(be._ctx, got)
        assert got.value >= weights // 3 - 2 * max(record_bytes(s.n, s.k) for s in specs) * 2
        s1 = st.stats()
        assert s1["streamed_records"] > 0 and s1["resident_bytes"] < info["resident_bytes"]
        assert np.array_equal(run(), ref) and np.array_equal(run(), ref)  # the second step finds its rings in flight
        with pytest.raises(BudgetExceeded):  # nothing more to give that would make this fit
            be.allocate_in(weights * 4, 1)
        # (2) phase eviction: all weight memory goes, the records stay in the pinned arena
        st.evict_all()
        assert be.mem_snapshot()["live_weights"] == 0
        assert np.array_equal(run(), ref)  # the step restored what the budget allows by itself
        # (3) the other consumer leaves: restore pins everything again
        be.free(other)
        s3 = st.restore()
        assert s3["streamed_records"] == 0 and s3["resident_bytes"] == info["resident_bytes"]
        assert np.array_equal(run(), ref)
        # transient reserve: a plan leaves that much of the budget free
        from thinfer_b200.backend import _check
        snap = be.mem_snapshot()
        budget = weights + (6 << 20)
        reserve = budget - snap["live_workspace"] - snap["live_staging"] - int(0.6 * weights)  # leaves room for 60 % of the weights
        _check(be.lib.tnf_set_transient_reserve(be._ctx, reserve))
        s4 = st.restore()
        live = be.mem_snapshot()
        assert live["live_weights"] + live["live_workspace"] + live["live_staging"] + reserve <= budget
        _check(be.lib.tnf_set_transient_reserve(be._ctx, budget))  # no room at all: refused on the host, weights stay evicted
        with pytest.raises(BudgetExceeded):
            st.restore()
        _check(be.lib.tnf_set_transient_reserve(be._ctx, reserve))
        s4 = st.restore()
        assert s4["streamed_records"] > 0 and np.array_equal(run(), ref)
        st.close()
    finally:
        be.close()


def C_u64():
    import ctypes

    return ctypes.c_uint64()


@pytest.mark.gpu
def test_stack_budget_below_ring_reserve_is_refused(backend):
    from thinfer_b200.backend import BudgetExceeded
    from thinfer_b200.residency import StackLinearSpec as S

    st, _ = _build(backend, 4, [S(128, 128)], [64], 128, 900)
    before = backend.mem_snapshot()["live_weights"]
    with pytest.raises(BudgetExceeded):
        st.build(weight_budget=1024, ring_slots=2)
    assert backend.mem_snapshot()["live_weights"] == before  # nothing was allocated
    st.close()


@pytest.mark.gpu
def test_stream_upload_download_round_trip(backend):
    """Pinned arena -> device on the copy stream, a compute-stream copy in between, device -> pinned arena
    with tnf_stream_download; tnf_event_sync makes the host wait for exactly that read-back."""
    import ctypes as C

    from thinfer_b200.backend import UnknownBuffer, _check
    from thinfer_b200.residency import HostArena

    be = backend
    n = 1 << 20
    src, dst = HostArena(be, n), HostArena(be, n)
    src.np[:] = (np.arange(n, dtype=np.uint32) * 2654435761 >> 24).astype(np.uint8)
    dst.np[:] = 0
    a, b = be.allocate(n), be.allocate(n)
    ev = C.c_uint64()
    _check(be.lib.tnf_stream_upload(be._ctx, src.id, 0, a.id, 0, n, C.byref(ev)))
    _check(be.lib.tnf_wait_event(be._ctx, ev.value))
    _check(be.lib.tnf_copy(be._ctx, a.id, 0, b.id, 0, n))
    _check(be.lib.tnf_stream_download(be._ctx, b.id, 4096, dst.id, 4096, n - 4096, C.byref(ev)))
    _check(be.lib.tnf_event_sync(be._ctx, ev.value))
    assert np.array_equal(dst.np[4096:], src.np[4096:]) and not dst.np[:4096].any()
    with pytest.raises(UnknownBuffer):
        _check(be.lib.tnf_event_sync(be._ctx, ev.value))  # an event is retired by its first wait
    be.free(a)
    be.free(b)
    src.release()
    dst.release()
