"""The way out after a device-side wait that runs out, exercised without faulting anything: a self-test kernel
waits (bounded, a few thousand probes) on a barrier nobody arrives at, gives up, reports and returns; the host
gets LUTAMM_EDEVICE; the same context then computes bit-exact results again, split tiles included."""
import numpy as np
import pytest

import oracle
import pim_dl_asplos_b200 as P
from pim_dl_asplos_b200 import synth

pytestmark = pytest.mark.gpu


def test_a_wait_that_runs_out_reports_and_leaves_the_context_usable(ctx):
    c = synth.make_case(M=300, K=768, N=768, v=2, CT=16, seed=31)
    want = oracle.amm(c.x, c.centroid, c.lut, c.bias, c.scale, 0.0)[0]
    ctx.load_weights(30, c.centroid, c.lut, c.bias, c.scale)
    ctx.set_plan(30, variant=P.VARIANT_UMMA, umma_split=3)      # split tiles: the counters that an error re-arms
    y = np.zeros_like(want)
    ctx.amm_host(30, c.x, y)
    assert np.array_equal(y.view(np.uint32), want.view(np.uint32))
    for _ in range(2):
        rc = ctx._L.lutamm_selftest_bounded_wait(ctx._h, 4096)
        assert rc == P.EDEVICE
        assert b"bounded wait" in ctx._L.lutamm_last_error(ctx._h)
        y[:] = 0
        ctx.amm_host(30, c.x, y)                                 # the very next ordinary call
        assert np.array_equal(y.view(np.uint32), want.view(np.uint32))
    ctx.sync()                                                   # no stale error left behind
    assert ctx._L.lutamm_selftest_bounded_wait(ctx._h, 0) == P.EINVAL
    ctx.unload_weights(30)
