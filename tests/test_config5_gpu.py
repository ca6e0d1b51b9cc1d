"""Config 5 of the benchmark plan on ONE GPU: the LLaMA-70B-shaped FFN projections
(8192 -> 28672 and 28672 -> 8192, 235 MB of int8 codes each, weights ~ N(0, 0.015)) at M = 1, 8 and
2048.  (The column-sharded form over 2 GPUs is tests/test_sharded_gpu.py.)

The f32 weights are drawn on the device (235 M values take minutes on the CPU generator); the codes
are downloaded through the C ABI and a SAMPLE of output channels is recomputed on the host in
float64 for every activation row.  Besides that, size-independent properties over the whole
output: the M = 8 rows equal the M = 1 forwards bit for bit, and the M = 2048 rows agree with the
M = 8 rows within the stated tolerance."""
import ctypes as C

import numpy as np
import pytest

import oracle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n,k", [(28672, 8192), (8192, 28672)])
def test_config5_70b_ffn_single_gpu(nne, ctx, n, k):
    import torch
    lib = nne.load()
    dev = torch.device("cuda", 0)
    gen = torch.Generator(device=dev)
    gen.manual_seed(5)
    stream = torch.cuda.current_stream().cuda_stream
    w = torch.randn(n, k, generator=gen, device=dev) * 0.015
    h = C.c_void_p()
    assert lib.nne_qlinear_create_from_f32_dev(ctx.handle, w.data_ptr(), None, n, k, stream, C.byref(h)) == 0
    torch.cuda.synchronize()

    # quantize parity on sampled rows: the oracle on the same f32 rows gives the same codes and scales
    rng = np.random.default_rng(n)
    ch = np.sort(rng.choice(n, 96, replace=False))
    w_rows = w[torch.from_numpy(ch).to(dev)].cpu().numpy()
    del w
    qw = np.empty((n, k), dtype=np.int8)
    sc = np.empty(n, dtype=np.float32)
    assert lib.nne_qlinear_download(h, qw.ctypes.data_as(C.c_void_p), sc.ctypes.data_as(C.c_void_p)) == 0
    q_ref, s_ref = oracle.quantize_rows(w_rows)
    assert np.array_equal(qw[ch], q_ref) and np.array_equal(sc[ch].view(np.uint32), s_ref.view(np.uint32))

    m_big = 2048
    x = torch.randn(m_big, k, generator=gen, device=dev)
    outs = {}
    for m in (1, 8, m_big):
        y = torch.empty(m, n, device=dev)
        assert lib.nne_qlinear_forward_dev(h, x.data_ptr(), m, k, y.data_ptr(), stream) == 0
        torch.cuda.synchronize()
        outs[m] = y.cpu().numpy()
    ctx.check()
    xh = x.cpu().numpy()

    # sampled channels against a float64 contraction of the downloaded codes
    q64 = qw[ch].astype(np.float64)
    bound = np.abs(q64).sum(axis=1) * sc[ch].astype(np.float64)          # scale_j * sum_k |q_jk|
    for m in (1, 8, m_big):
        xm = xh[:m].astype(np.float64)
        y_ref = (xm @ q64.T) * sc[ch].astype(np.float64)
        tol = 1e-3 * np.abs(xm).max() * bound
        ratio = float((np.abs(outs[m][:, ch] - y_ref) / tol).max())
        print(f"config5 {k}->{n} M={m}: kernel {lib.nne_qlinear_kernel_for(h, m)}, "
              f"max err/tol on 96 sampled channels {ratio:.3e}")
        assert ratio <= 1.0
    # properties over the whole output
    assert np.array_equal(outs[8][0].view(np.uint32), outs[1][0].view(np.uint32))
    full_bound = 1e-3 * np.abs(xh[:8]).max() * (np.abs(qw).astype(np.float32).sum(axis=1) * sc)
    assert float((np.abs(outs[m_big][:8] - outs[8]) / full_bound).max()) <= 1.0
    assert np.isfinite(outs[m_big]).all()
    lib.nne_qlinear_destroy(h)
