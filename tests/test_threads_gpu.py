"""`Module: Send + Sync`: the reference's HTTP server calls `forward(&self)` on one layer from a
pool of worker threads (src/bin/server.rs:219-259).  The host entry points serialise per context;
this test hammers one layer from several threads with different batch sizes (three different
kernels) and checks every result against the same call made alone."""
import threading

import numpy as np
import pytest

import oracle

pytestmark = pytest.mark.gpu


def test_concurrent_forward_on_one_layer(nne, ctx):
    n, k = 1536, 2048
    w = oracle.normal(41, 0, (n, k), 0.0, 0.02)
    b = oracle.normal(41, 1, (n,), 0.0, 0.1)
    ql = nne.QLinear.from_linear(nne.Linear(w, b), ctx)
    cases = []
    for t, m in enumerate((1, 2, 5, 16, 40, 130, 1, 8)):
        x = oracle.normal(41, 10 + t, (m, k))
        cases.append((x, ql.forward(x)))
    ctx.check()
    errors = []

    def worker(idx):
        x, want = cases[idx]
        try:
            for _ in range(25):
                got = ql.forward(x)
                if not np.array_equal(got.view(np.uint32), want.view(np.uint32)):
                    errors.append(f"thread {idx}: result differs")
                    return
        except Exception as e:  # pragma: no cover - reported below
            errors.append(f"thread {idx}: {type(e).__name__}: {e}")

    threads = [threading.Thread(target=worker, args=(i,)) for i in range(len(cases))]
    for th in threads:
        th.start()
    for th in threads:
        th.join(timeout=120)
    assert not any(th.is_alive() for th in threads), "a worker did not finish"
    assert not errors, errors
    ctx.check()


def test_concurrent_quantize_and_clone(nne, ctx):
    """from_linear / clone on several threads at once (each builds its own device handle)."""
    results = [None] * 6

    def worker(i):
        w = oracle.normal(43, i, (256, 512), 0.0, 0.02)
        ql = nne.QLinear.from_linear(nne.Linear(w, None), ctx)
        qo, so = oracle.quantize_rows(w)
        c = ql.clone()
        x = oracle.normal(43, 100 + i, (3, 512))
        results[i] = (np.array_equal(ql.qweight.reshape(256, 512), qo)
                      and np.array_equal(ql.scales.view(np.uint32), so.view(np.uint32))
                      and np.array_equal(c.forward(x).view(np.uint32), ql.forward(x).view(np.uint32)))

    threads = [threading.Thread(target=worker, args=(i,)) for i in range(6)]
    for th in threads:
        th.start()
    for th in threads:
        th.join(timeout=120)
    assert all(results), results
    ctx.check()
