"""The allocation-free forward (nne_qlinear_forward_dev_static) against the ordinary device
forward, through the C ABI.

Who needs it: callers that must not allocate device memory while they run - a serving loop whose
memory was handed out in full at start-up, or a thread issuing work while a collective is in
flight, for which an allocation could mean a device-wide synchronisation.  The entry point keeps
its activation workspace in a fixed array inside the library instead.  The file name sorts last so
that a run that stops at the first failure has already run every other test."""
import ctypes as C

import numpy as np
import pytest

import oracle

pytestmark = pytest.mark.gpu


def test_static_forward_matches_ordinary_forward_twice(nne, ctx):
    import torch
    lib = nne.load()
    n, k = 640, 1024
    w = oracle.normal(120, 0, (n, k), 0.0, 0.02)
    b = oracle.normal(120, 1, (n,), 0.0, 0.1)
    ql = nne.QLinear.from_linear(nne.Linear(w, b), ctx)
    s = torch.cuda.current_stream().cuda_stream
    # two calls in a row; the second is smaller, so it runs over what the first left in the array
    for call, m in enumerate((300, 130)):
        x = oracle.normal(121, call, (m, k))
        xd = torch.from_numpy(x).cuda()
        y_ref = torch.full((m, n), float("nan"), device="cuda")
        y_new = torch.full((m, n), float("nan"), device="cuda")
        assert lib.nne_qlinear_forward_dev(ql._handle, xd.data_ptr(), m, k, y_ref.data_ptr(), s) == 0
        st = lib.nne_qlinear_forward_dev_static(ql._handle, xd.data_ptr(), m, k, y_new.data_ptr(), s)
        assert st == 0, nne._lib.last_error()
        torch.cuda.synchronize()
        ctx.check()
        a, r = y_new.cpu().numpy(), y_ref.cpu().numpy()
        assert ql.kernel_for(m) == 2          # the ordinary forward took a tensor-core kernel too
        # Same contraction, two tensor-core kernels: this entry point runs the bf16 one (codes
        # dequantized to bf16 in shared memory, x rounded to bf16), the ordinary forward the
        # integer one.  They must agree within the tolerance of the forward tests,
        # tol_j = 1e-3 * ||x||inf * scale_j * sum_k |q_jk|, and so must each with the oracle.
        tol, _ = oracle.tolerance(ql.qweight.reshape(n, k), ql.scales, x)
        y_oracle = oracle.forward(ql.qweight.reshape(n, k), ql.scales, b, x)
        assert float((np.abs(a - r) / tol).max()) <= 1.0
        assert float((np.abs(a - y_oracle) / tol).max()) <= 1.0
        assert float((np.abs(r - y_oracle) / tol).max()) <= 1.0
        # with integer-valued activations every kernel is exact, so there the two agree bit for bit
        xi = np.random.default_rng(call).integers(-8, 9, size=(m, k)).astype(np.float32)
        xid = torch.from_numpy(xi).cuda()
        assert lib.nne_qlinear_forward_dev(ql._handle, xid.data_ptr(), m, k, y_ref.data_ptr(), s) == 0
        assert lib.nne_qlinear_forward_dev_static(ql._handle, xid.data_ptr(), m, k, y_new.data_ptr(), s) == 0
        torch.cuda.synchronize()
        assert np.array_equal(y_new.cpu().numpy().view(np.uint32), y_ref.cpu().numpy().view(np.uint32))


def test_static_forward_refuses_what_it_cannot_take(nne, ctx):
    import torch
    lib = nne.load()
    ql = nne.QLinear.from_linear(nne.Linear(oracle.normal(122, 0, (64, 4096), 0.0, 0.02)), ctx)
    x = torch.zeros(2048, 4096, device="cuda")
    y = torch.zeros(2048, 64, device="cuda")
    # 2048 * 4096 = 8 Mi elements > 4 Mi: refused, with the limit in the message
    st = lib.nne_qlinear_forward_dev_static(ql._handle, x.data_ptr(), 2048, 4096, y.data_ptr(), 0)
    assert st == 1 and "4194304" in nne._lib.last_error()
    # exactly at the limit is accepted
    assert lib.nne_qlinear_forward_dev_static(ql._handle, x.data_ptr(), 1024, 4096, y.data_ptr(), 0) == 0
    torch.cuda.synchronize()
    assert lib.nne_qlinear_forward_dev_static(ql._handle, x.data_ptr(), 4, 4095, y.data_ptr(), 0) == 2
    odd = nne.QLinear.from_linear(nne.Linear(oracle.normal(122, 1, (8, 24), 0.0, 0.02)), ctx)
    assert lib.nne_qlinear_forward_dev_static(odd._handle, x.data_ptr(), 4, 24, y.data_ptr(), 0) == 7
