"""Regenerates tests/golden/qlinear_golden.npz.

The reference keeps no golden vectors for this path and cannot be run here (Rust crate, no Rust
toolchain), so these fixtures are produced by the C oracle (oracle/qlinear_ref.c) and are written
only if the independent numpy restatement of the quantize step agrees with it byte for byte.
Run from the repo root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import oracle  # noqa: E402


def edge_rows(cols: int) -> np.ndarray:
    """Rows that exercise every branch of the quantize arithmetic."""
    rows = []
    rows.append(np.zeros(cols, np.float32))                                   # all zero -> scale 1
    r = oracle.normal(101, 0, (cols,), 0.0, 0.02); r[3] = np.nan; rows.append(r)            # NaN ignored, coded 0
    r = oracle.normal(101, 1, (cols,), 0.0, 0.02); r[5] = np.inf; r[6] = -np.inf; rows.append(r)  # Inf -> scale inf
    r = oracle.normal(101, 2, (cols,), 0.0, 1.0) * np.float32(1e-42); rows.append(r.astype(np.float32))  # denormals
    r = np.zeros(cols, np.float32); r[0] = np.float32(1e-44); r[1] = -np.float32(1e-45); rows.append(r)  # max/127 underflows to 0
    r = np.zeros(cols, np.float32); r[0] = 127.0                             # scale exactly 1: exact .5 ties
    r[1:9] = [0.5, -0.5, 1.5, -1.5, 2.5, -2.5, 126.5, -126.5]; rows.append(r)
    r = oracle.normal(101, 3, (cols,), 0.0, 3.0e38); rows.append(r)          # huge values, some overflow to inf
    r = -np.abs(oracle.normal(101, 4, (cols,), 0.0, 0.02)); rows.append(r)   # all negative
    return np.stack(rows).astype(np.float32)


def main():
    n, k, m = 24, 48, 3
    w = oracle.normal(7, 0, (n, k), 0.0, 0.02)
    w = np.concatenate([w, edge_rows(k)], axis=0)
    bias = oracle.normal(7, 1, (w.shape[0],), 0.0, 0.1)
    x = oracle.normal(7, 2, (m, k), 0.0, 1.0)
    with np.errstate(all="ignore"):
        q, s = oracle.quantize_rows(w)
        q_np, s_np = oracle.numpy_quantize_rows(w)
    assert np.array_equal(q, q_np), "C oracle and numpy restatement disagree on codes"
    assert np.array_equal(s.view(np.uint32), s_np.view(np.uint32)), "scales disagree"
    # forward fixtures use only rows whose scale is finite and non-zero (the first n rows)
    qf, sf, bf = q[:n], s[:n], bias[:n]
    y_avx2 = oracle.forward(qf, sf, bf, x, threads=1, use_avx2=1)
    y_scalar = oracle.forward(qf, sf, bf, x, threads=1, use_avx2=0)
    y_nobias = oracle.forward(qf, sf, None, x, threads=1, use_avx2=1)
    y_f64 = oracle.forward_f64(qf, sf, bf, x)
    t = oracle.normal(7, 3, (4, 5, 6), 0.0, 1.0)
    tq, ts = oracle.int8tensor_from_raw(t)
    tdq = oracle.dequantize(tq, ts)
    out = os.path.join(HERE, "qlinear_golden.npz")
    np.savez_compressed(out, w=w, bias=bias, x=x, q=q, scales=s, n_forward=np.int64(n),
                        y_avx2=y_avx2, y_scalar=y_scalar, y_nobias=y_nobias, y_f64=y_f64,
                        t=t, t_q=tq, t_scale=np.float32(ts), t_dq=tdq)
    print("wrote", out, os.path.getsize(out), "bytes")


if __name__ == "__main__":
    main()
