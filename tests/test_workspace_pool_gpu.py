"""The workspace pool behind the scope's scratch buffers. The cases follow the reference's pool tests
(thinfer-core/src/workspace.rs:2313-2474: distinct buffers per rent, recycle within a size class, classes do not
share, draining frees the idle buffers) and its reclaim order (idle pool before weights,
thinfer-core/src/arbiter.rs:37-38, smallest class first, thinfer-core/src/workspace.rs:52-85)."""
import ctypes as C

import numpy as np
import pytest

from oracle import oracle as O


def _live(be):
    s = be.mem_snapshot()
    return s["live_weights"] + s["live_workspace"] + s["live_staging"]


@pytest.mark.gpu
def test_rent_recycle_classes_and_drain(backend):
    from thinfer_b200.backend import UnknownBuffer, _check

    be = backend
    be.drain_pool()
    base, s0 = be.mem_snapshot()["live_workspace"], be.pool_stats()
    r1, r2 = be.ws_alloc(100), be.ws_alloc(100)
    assert r1.id != r2.id and len(r1) == 100 and r1.buf.offset == 0  # the view keeps the requested length
    assert be.mem_snapshot()["live_workspace"] == base + 512         # two buffers of the 256-byte class
    id1, id2 = r1.id, r2.id
    r1.release(), r2.release()
    r1.release()  # a second release of the same guard does nothing
    s = be.pool_stats()
    assert s["free_count"] == 2 and s["pool_bytes"] == 512 and s["rented"] == 0
    assert be.mem_snapshot()["live_workspace"] == base + 512  # idle buffers stay allocated and charged
    r3, r4 = be.ws_alloc(200), be.ws_alloc(256)               # same class: both come from the pool, newest first
    assert (r3.id, r4.id) == (id2, id1)
    s = be.pool_stats()
    assert s["hits"] - s0["hits"] == 2 and s["misses"] - s0["misses"] == 2 and s["free_count"] == 0
    r5 = be.ws_alloc(257)  # next class: 512 bytes, a new buffer
    assert r5.id not in (id1, id2) and be.mem_snapshot()["live_workspace"] == base + 1024
    with pytest.raises(UnknownBuffer, match="not out on rent"):
        _check(be.lib.tnf_ws_release(be._ctx, 0xDEAD))
    # a rented buffer works like any other: bytes written are bytes read, also after a recycle
    data = np.arange(200, dtype=np.uint8)
    be.write_buffer(r3.buf, data)
    assert np.array_equal(be.read_buffer(r3.buf), data)
    r3.release(), r4.release()
    with be.ws_alloc(64) as again:  # `with` releases at the end of the block
        assert again.id == id1
    assert be.drain_pool() == 512 and be.pool_stats()["free_count"] == 0
    assert be.mem_snapshot()["live_workspace"] == base + 512  # r5 is still out on rent and untouched by the drain
    be.free(r5.buf)  # freeing a pool buffer directly takes it off the pool's books
    assert be.pool_stats()["rented"] == 0 and be.mem_snapshot()["live_workspace"] == base
    r5.be = None


@pytest.mark.gpu
def test_scope_holds_its_scratch_until_submit(backend):
    be = backend
    be.drain_pool()
    sc = be.scope()
    a, b = sc.alloc(1000), sc.alloc(1000)
    assert a.id != b.id and be.pool_stats()["rented"] == 2  # nothing rented in a scope is recycled inside it
    sc.submit()
    s = be.pool_stats()
    assert s["rented"] == 0 and s["free_count"] == 2
    sc2 = be.scope()
    c = sc2.alloc(1024)
    assert c.id in (a.id, b.id)  # the next scope reuses them
    sc2.submit()
    be.drain_pool()


@pytest.mark.gpu
def test_idle_pool_is_given_back_before_weights():
    """Under a budget the reclaim chain asks the idle pool first, smallest class first, and touches resident
    weights only when the pool was not enough."""
    import thinfer_b200 as T
    from thinfer_b200.backend import BudgetExceeded
    from thinfer_b200.residency import StackLinearSpec as S, record_bytes
    from test_residency import _build

    hidden, layers = 128, 6
    specs = [S(384, 128, 0, True, 0, 0), S(128, 384, 0, True, 1, 0)]
    weights = layers * sum(record_bytes(s.n, s.k) for s in specs)
    budget = weights + (8 << 20)
    be = T.Backend(0, vram_budget=budget)
    try:
        st, _ = _build(be, layers, specs, [160], hidden, 900)
        info = st.build(weight_budget=0, ring_slots=2)
        assert info["streamed_records"] == 0
        x = O.f32_to_bf16(O.gaussian(160 * hidden, 43).reshape(160, hidden))
        xb, ob = [be.upload(x)], [be.allocate(160 * hidden * 2)]
        st.step(xb, ob, 0.004)
        be.submit(30000)
        ref = be.read_buffer(ob[0], np.uint16).copy()
        # fill the spare room with idle pool buffers of three classes
        small = [be.ws_alloc(64 << 10) for _ in range(4)]
        mid = [be.ws_alloc(512 << 10) for _ in range(2)]
        big = [be.ws_alloc(2 << 20)]
        for g in small + mid + big:
            g.release()
        idle = be.pool_stats()["pool_bytes"]
        assert idle == 4 * (64 << 10) + 2 * (512 << 10) + (2 << 20)
        room = budget - _live(be)
        # (1) needs 100 KiB more than the room: two of the smallest class go, nothing else
        o1 = be.allocate_in(room + (100 << 10), 1)
        s = be.pool_stats()
        assert s["spilled_bytes"] == 2 * (64 << 10) and s["free_count"] == 5
        got = C.c_uint64()
        be.lib.tnf_reclaimed_bytes(be._ctx, C.byref(got))
        assert got.value == 0 and st.stats()["streamed_records"] == 0  # weights untouched
        # (2) needs more than the whole pool: the pool empties, then the stack gives weight sets back
        room = budget - _live(be)
        o2 = be.allocate_in(room + be.pool_stats()["pool_bytes"] + weights // 4, 1)
        s = be.pool_stats()
        assert s["free_count"] == 0 and s["pool_bytes"] == 0 and s["spilled_bytes"] == idle
        be.lib.tnf_reclaimed_bytes(be._ctx, C.byref(got))
        assert got.value > 0 and st.stats()["streamed_records"] > 0
        st.step(xb, ob, 0.004)
        be.submit(30000)
        assert np.array_equal(be.read_buffer(ob[0], np.uint16), ref)
        # (3) a rent that cannot fit is refused like any allocation
        with pytest.raises(BudgetExceeded):
            be.ws_alloc(budget)
        be.free(o1), be.free(o2)
        st.close()
    finally:
        be.close()
