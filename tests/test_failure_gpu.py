"""Failure detection on the device without faulting it: a bounded wait runs out.

Every wait inside the GEMM kernels (on a loaded stage, a freed stage, a finished or drained accumulator) has
a cycle limit; a wait that gives up raises a flag, every role of the kernel falls through to its tear-down,
the kernel returns normally with a status word set and the awaited submit reports a timeout. The self-test
launches the CTA-pair kernel with its loader switched off, so nothing is ever in flight: no trap, no bad
address, no endless loop. Afterwards the same context must run a correct linear."""
import numpy as np
import pytest

import oracle as O
from conftest import rel_fro

pytestmark = pytest.mark.gpu


def test_bounded_device_wait_reports_timeout_and_context_survives():
    import thinfer_b200 as T
    from thinfer_b200.backend import DeviceTimeout, _check

    be = T.Backend(0)
    try:
        _check(be.lib.tnf_set_device_wait_limit(be._ctx, 2_000_000))  # about a millisecond
        _check(be.lib.tnf_selftest_stalled_wait(be._ctx))             # returns once the kernel has left
        with pytest.raises(DeviceTimeout) as e:
            be.submit(10000)
        assert "wait gave up" in str(e.value)
        be.submit(10000)  # the status word was consumed: the next submit is clean
        _check(be.lib.tnf_set_device_wait_limit(be._ctx, 0))
        # the context is still usable: a pair-kernel linear right after, against the oracle
        m, n, k = 1024, 2048, 256
        a = O.f32_to_bf16(O.gaussian(m * k, 0xA0F0).reshape(m, k))
        w = (O.gaussian(n * k, 0xB0F0) * np.float32(0.02)).reshape(n, k)
        W = T.Nvfp4Weight.from_dense(be, w)
        ga = O.global_scale(O.amax_bf16(a))
        abuf, out = be.upload(a), be.allocate(m * n * 2)
        be.scope().linear(abuf, m, W, ga, out)
        be.submit(30000)
        got = be.read_buffer(out, np.uint16).reshape(m, n)
        wc, ws, gw = O.quantize_weight(w)
        assert rel_fro(O.bf16_to_f32(got), O.bf16_to_f32(O.linear(a, ga, wc, ws, gw))) <= 1e-3
    finally:
        be.close()
