"""Failure detection without a fault: every device-side wait in the library is bounded, and a wait
that runs out must surface as NNE_ERR_TIMEOUT on the host while the kernel returns and the context
stays usable.  The library's self-test entry runs a one-CTA kernel that waits a few milliseconds
for an event nothing will ever produce (a barrier nobody arrives at; an arrival word of the
column-shard exchange nothing raises).  Nothing here traps, faults or hangs the GPU."""
import time

import numpy as np
import pytest

import oracle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("which", [0, 1])
def test_a_wait_that_runs_out_becomes_a_timeout_status(nne, which):
    lib = nne.load()
    ctx = nne.CudaContext(0)
    ctx.check()                                      # clean to begin with
    t0 = time.perf_counter()
    assert lib.nne_cuda_ctx_selftest_wait(ctx.handle, which, 3000) == 0   # 3 ms limit
    took = time.perf_counter() - t0
    assert took < 1.0, f"the bounded wait took {took:.2f} s"
    assert lib.nne_cuda_ctx_check(ctx.handle) == nne._lib.TIMEOUT
    assert "bounded wait ran out" in nne._lib.last_error()
    with pytest.raises(nne.GpuError):
        lib.nne_cuda_ctx_selftest_wait(ctx.handle, which, 2000)
        ctx.check()
    assert lib.nne_cuda_ctx_check(ctx.handle) == 0   # reported once, then clear
    # the context still computes
    w = oracle.normal(90, 0, (128, 256), 0.0, 0.02)
    ql = nne.QLinear.from_linear(nne.Linear(w), ctx)
    x = oracle.normal(90, 1, (1, 256))
    qo, so = oracle.quantize_rows(w)
    tol, _ = oracle.tolerance(qo, so, x)
    assert float((np.abs(ql.forward(x) - oracle.forward(qo, so, None, x)) / tol).max()) <= 1.0
    # a host-pointer forward right after a timed-out kernel reports it too
    assert lib.nne_cuda_ctx_selftest_wait(ctx.handle, which, 2000) == 0
    with pytest.raises(nne.GpuError, match="bounded wait"):
        ql.forward(x)
    ql.forward(x)
    assert lib.nne_cuda_ctx_selftest_wait(ctx.handle, 5, 1000) == 1
    assert lib.nne_cuda_ctx_selftest_wait(ctx.handle, 0, 0) == 1
    ql.close()
    ctx.close()
