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


def test_static_forward_worst_case_stays_inside_its_own_bound(nne, ctx):
    """The entry point's documented bound is the bf16 kernel's, 2^-8 * ||x||inf * scale_j * sum|q_jk|,
    which is looser than the 1e-3 tolerance of the ordinary forward.  Activations that sit on bf16
    half-way points (1 + 2^-8 rounds to 1), with signs chosen so that every rounding error pulls
    channel 0 the same way, come close to that bound and stay inside it; the ordinary forward
    (integer kernel) keeps its 1e-3 tolerance on the same input."""
    import torch
    lib = nne.load()
    n, k, m = 256, 1024, 32
    w = oracle.normal(123, 0, (n, k), 0.0, 0.02)
    ql = nne.QLinear.from_linear(nne.Linear(w), ctx)
    q = ql.qweight.reshape(n, k)
    sign = np.where(q[0] >= 0, -1.0, 1.0).astype(np.float32)   # error of bf16(x_k) gets q's sign
    x = np.tile((sign * np.float32(1.0 + 2.0 ** -8))[None, :], (m, 1)).astype(np.float32)
    xd = torch.from_numpy(x).cuda()
    y_new = torch.empty(m, n, device="cuda")
    y_ord = torch.empty(m, n, device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    assert lib.nne_qlinear_forward_dev_static(ql._handle, xd.data_ptr(), m, k, y_new.data_ptr(), s) == 0
    assert lib.nne_qlinear_forward_dev(ql._handle, xd.data_ptr(), m, k, y_ord.data_ptr(), s) == 0
    torch.cuda.synchronize()
    ctx.check()
    exact = oracle.forward_f64(q, ql.scales, None, x)
    tol, xinf = oracle.tolerance(q, ql.scales, x)              # 1e-3 * ||x||inf * scale_j * sum|q_jk|
    bound_bf16 = tol * (2.0 ** -8 / 1e-3)
    err_new = np.abs(y_new.cpu().numpy() - exact)
    err_ord = np.abs(y_ord.cpu().numpy() - exact)
    print(f"bf16 worst case: channel 0 err / (1e-3 bound) = {float(err_new[0, 0] / tol[0]):.2f}, "
          f"err / (2^-8 bound) = {float(err_new[0, 0] / bound_bf16[0]):.3f}")
    assert float((err_new / (bound_bf16 * 1.001)).max()) <= 1.0
    assert float(err_new[0, 0] / tol[0]) > 1.0    # the case really is outside the ordinary tolerance
    assert float((err_ord / tol).max()) <= 1.0


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
