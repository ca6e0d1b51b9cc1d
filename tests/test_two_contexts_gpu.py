"""One process, two contexts on two GPUs: kernel attributes (the opt-in for more than 48 KB of
dynamic shared memory) are per device, so every kernel class must work on the second device too.
Runs one forward per kernel class, the quantize kernels and the allocation-free entry point on each
device and checks them against the oracle.  No peer memory is used.  Skipped with one GPU."""
import ctypes as C

import numpy as np
import pytest

import oracle

pytestmark = pytest.mark.gpu


def test_every_kernel_class_on_two_devices_in_one_process(nne):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    lib = nne.load()
    n, k = 640, 1024
    w = oracle.normal(77, 0, (n, k), 0.0, 0.02)
    b = oracle.normal(77, 1, (n,), 0.0, 0.1)
    qo, so = oracle.quantize_rows(w)
    # device 1 first: a process-wide "already set" flag would then break device 0, and vice versa
    for dev in (1, 0, 1):
        ctx = nne.CudaContext(dev)
        ql = nne.QLinear.from_linear(nne.Linear(w, b), ctx)    # 1024 columns: the warp-per-row quantize kernel
        assert np.array_equal(ql.qweight.reshape(n, k), qo)
        wide = oracle.normal(78, dev, (64, 4096), 0.0, 0.02)    # 4096 columns: the bulk-copy quantize kernel
        qw, sw = oracle.quantize_rows(wide)
        qlw = nne.QLinear.from_linear(nne.Linear(wide), ctx)
        assert np.array_equal(qlw.qweight.reshape(64, 4096), qw)
        assert np.array_equal(qlw.scales.view(np.uint32), sw.view(np.uint32))
        for m, kernel in ((1, 1), (2, 1), (8, 4), (160, 2)):
            assert ql.kernel_for(m) == kernel
            x = oracle.normal(79, m, (m, k))
            y = ql.forward(x)
            tol, _ = oracle.tolerance(qo, so, x)
            ratio = float((np.abs(y - oracle.forward(qo, so, b, x)) / tol).max())
            assert ratio <= 1.0, f"device {dev} m={m}: err/tol {ratio}"
        # a plan (streaming kernel over a list) and the allocation-free entry point
        with torch.cuda.device(dev):
            xd = torch.from_numpy(oracle.normal(80, 0, (40, k))).cuda()
            yd = torch.empty(40, n, device=f"cuda:{dev}")
            st = lib.nne_qlinear_forward_dev_static(ql._handle, xd.data_ptr(), 40, k, yd.data_ptr(),
                                                    torch.cuda.current_stream().cuda_stream)
            assert st == 0, nne._lib.last_error()
            torch.cuda.synchronize()
            tol, _ = oracle.tolerance(qo, so, xd.cpu().numpy())
            y_ref = oracle.forward(qo, so, b, xd.cpu().numpy())
            assert float((np.abs(yd.cpu().numpy() - y_ref) / tol).max()) <= 1.0
            x1 = torch.from_numpy(oracle.normal(80, 1, (1, k))).cuda()
            y1 = torch.empty(2, n, device=f"cuda:{dev}")
            plan = nne.QLinearPlan([ql, ql], [x1.data_ptr(), x1.data_ptr()],
                                   [y1[0].data_ptr(), y1[1].data_ptr()], 1, ctx)
            plan.run(torch.cuda.current_stream().cuda_stream)
            torch.cuda.synchronize()
            want = ql.forward(x1.cpu().numpy())
            assert np.array_equal(y1[0].cpu().numpy().view(np.uint32), want[0].view(np.uint32))
            assert np.array_equal(y1[1].cpu().numpy().view(np.uint32), want[0].view(np.uint32))
            plan.close()
        ctx.check()
        ql.close()
        qlw.close()
        ctx.close()


def test_rows_too_long_for_int32_sums_leave_the_tensor_core_kernels(nne, ctx):
    """The integer tensor-core kernels keep int32 sums in TMEM: exact below 2^17 terms.  A layer
    with longer rows must be sent elsewhere, whatever m is, and still be right."""
    n, k = 2, (1 << 17) + 16
    w = oracle.normal(81, 0, (n, k), 0.0, 0.02)
    ql = nne.QLinear.from_linear(nne.Linear(w), ctx)
    qo, so = oracle.quantize_rows(w)
    assert np.array_equal(ql.qweight.reshape(n, k), qo)
    for m in (1, 8, 17):
        assert ql.kernel_for(m) in (1, 3), f"m={m} took kernel {ql.kernel_for(m)}"
        x = oracle.normal(81, 10 + m, (m, k))
        y = ql.forward(x)
        tol, _ = oracle.tolerance(qo, so, x)
        assert float((np.abs(y - oracle.forward(qo, so, None, x)) / tol).max()) <= 1.0
    short = nne.QLinear.from_linear(nne.Linear(oracle.normal(81, 1, (2, (1 << 17) - 128), 0.0, 0.02)), ctx)
    assert short.kernel_for(8) == 4 and short.kernel_for(17) == 2
    ctx.check()
