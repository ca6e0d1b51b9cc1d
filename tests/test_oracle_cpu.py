"""CPU tests of the oracle (oracle/qlinear_ref.c): golden fixtures, the independent numpy
restatement, hand-derived known answers for the rounding rule, and the four assertions of the
reference's own tests (tests/nn/quantization_tests.rs) replayed on seeded inputs."""
import os

import numpy as np
import pytest

import oracle

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "qlinear_golden.npz")


@pytest.fixture(scope="module")
def golden():
    return np.load(GOLDEN)


def bits(a):
    return np.asarray(a, dtype=np.float32).view(np.uint32)


def test_golden_quantize(golden):
    with np.errstate(all="ignore"):
        q, s = oracle.quantize_rows(golden["w"])
    assert np.array_equal(q, golden["q"])
    assert np.array_equal(bits(s), bits(golden["scales"]))


def test_golden_forward(golden):
    n = int(golden["n_forward"])
    q, s, b, x = golden["q"][:n], golden["scales"][:n], golden["bias"][:n], golden["x"]
    assert np.array_equal(bits(oracle.forward(q, s, b, x, 1, 1)), bits(golden["y_avx2"]))
    assert np.array_equal(bits(oracle.forward(q, s, b, x, 1, 0)), bits(golden["y_scalar"]))
    assert np.array_equal(bits(oracle.forward(q, s, None, x, 1, 1)), bits(golden["y_nobias"]))
    assert np.allclose(oracle.forward_f64(q, s, b, x), golden["y_f64"], rtol=0, atol=0)
    # threading must not change any bit: rows are independent tasks (reference :179-182)
    assert np.array_equal(bits(oracle.forward(q, s, b, x, 3, 1)), bits(golden["y_avx2"]))


def test_golden_int8tensor(golden):
    q, s = oracle.int8tensor_from_raw(golden["t"])
    assert np.array_equal(q, golden["t_q"])
    assert bits(s) == bits(golden["t_scale"])
    assert np.array_equal(bits(oracle.dequantize(q, s)), bits(golden["t_dq"]))


def test_rounding_known_answers():
    """scale = 127/127 = 1 exactly, so codes are round-half-AWAY of the values themselves
    (reference src/nn/quantized.rs:124, f32::round).  Expected codes written out by hand."""
    row = np.array([[127.0, 0.5, -0.5, 1.5, -1.5, 2.5, -2.5, 126.5, -126.5, 0.49999997, -0.49999997,
                     1.0, -0.0, 63.5]], dtype=np.float32)
    q, s = oracle.quantize_rows(row)
    assert s[0] == np.float32(1.0)
    assert q[0].tolist() == [127, 1, -1, 2, -2, 3, -3, 127, -127, 0, 0, 1, 0, 64]
    # half-to-even would give 0,0,2,-2,2,-2,126,-126 for the eight ties above


def test_edge_rows_known_answers():
    with np.errstate(all="ignore"):
        # all-zero row: scale 1.0, codes 0 (reference :119)
        q, s = oracle.quantize_rows(np.zeros((1, 8), np.float32))
        assert s[0] == 1.0 and not q.any()
        # NaN never wins the absmax and is coded 0 (Rust `as i8`)
        q, s = oracle.quantize_rows(np.array([[np.nan, 2.0, -1.0]], np.float32))
        assert bits(s)[0] == bits(np.float32(2.0) / np.float32(127.0)) and q[0].tolist() == [0, 127, -64]
        # Inf: scale inf, inv 0, finite -> 0, inf*0 = NaN -> 0
        q, s = oracle.quantize_rows(np.array([[np.inf, 2.0, -np.inf]], np.float32))
        assert np.isinf(s[0]) and q[0].tolist() == [0, 0, 0]
        # max/127 underflows to 0: inv = inf, codes saturate, zero stays 0 (0*inf = NaN -> 0)
        q, s = oracle.quantize_rows(np.array([[1e-44, -1e-45, 0.0]], np.float32))
        assert s[0] == 0.0 and q[0].tolist() == [127, -128, 0]


def test_c_oracle_matches_numpy_restatement():
    w = oracle.normal(0, 0, (512, 1024), 0.0, 0.02)
    q, s = oracle.quantize_rows(w)
    qn, sn = oracle.numpy_quantize_rows(w)
    assert np.array_equal(q, qn)
    assert np.array_equal(bits(s), bits(sn))
    assert int(q.min()) >= -127 and int(q.max()) == 127  # -128 is unreachable on finite rows


def test_forward_oracle_matches_the_second_restatement_of_the_avx2_dot(golden):
    """The forward has two restatements written from the Rust lines independently: the C oracle
    (AVX2 intrinsics, as the reference) and numpy with an emulated fused multiply-add.  They must
    agree BIT FOR BIT on the golden case, on lengths that end in a scalar tail, and on inputs with a
    wide dynamic range (where a double-rounded FMA emulation would show)."""
    if not oracle.lib().nne_ref_has_avx2_fma():
        pytest.skip("host without AVX2/FMA: the C oracle cannot run the reference's SIMD branch")
    n = int(golden["n_forward"])
    q, s, b, x = golden["q"][:n], golden["scales"][:n], golden["bias"][:n], golden["x"]
    y_np = oracle.numpy_forward_avx2(q, s, b, x)
    assert np.array_equal(y_np.view(np.uint32), golden["y_avx2"].view(np.uint32))
    assert np.array_equal(oracle.numpy_forward_avx2(q, s, None, x).view(np.uint32),
                          golden["y_nobias"].view(np.uint32))
    rng = np.random.default_rng(11)
    for k in (1, 15, 16, 17, 31, 250, 1003):
        w = oracle.normal(70, k, (6, k), 0.0, 0.02)
        qq, ss = oracle.quantize_rows(w)
        xx = (rng.standard_normal((2, k)) * np.exp2(rng.integers(-18, 18, (2, k)))).astype(np.float32)
        a = oracle.forward(qq, ss, None, xx, threads=1, use_avx2=1)
        assert np.array_equal(a.view(np.uint32), oracle.numpy_forward_avx2(qq, ss, None, xx).view(np.uint32)), k


def test_rms_norm_and_silu_mul_restatements():
    """RMSNorm (src/nn/norm.rs:517-577, both branches) and silu(gate) * up against float64 numpy."""
    x = oracle.normal(71, 0, (5, 1003), 0.0, 2.0)
    g = oracle.normal(71, 1, (1003,), 1.0, 0.2)
    ref = x.astype(np.float64) / np.sqrt((x.astype(np.float64) ** 2).mean(-1, keepdims=True) + 1e-6) * g
    for avx in (0, 1):
        if avx and not oracle.lib().nne_ref_has_avx2_fma():
            continue
        assert np.abs(oracle.rms_norm(x, g, 1e-6, avx) - ref).max() <= 1e-5 * np.abs(ref).max()
    ones = oracle.rms_norm(np.full((1, 8), 3.0, np.float32), np.ones(8, np.float32), 0.0, 0)
    assert np.array_equal(ones, np.ones((1, 8), np.float32))          # 3 / sqrt(9) = 1 exactly
    gate = np.array([0.0, 1.0, -1.0, 30.0, -30.0], np.float32)
    up = np.array([2.0, 2.0, 2.0, 0.5, 4.0], np.float32)
    want = gate.astype(np.float64) / (1 + np.exp(-gate.astype(np.float64))) * up
    assert np.abs(oracle.silu_mul(gate, up) - want).max() <= 1e-6


def test_generator_is_deterministic_and_normal():
    a = oracle.normal(3, 5, (1 << 16,))
    b = oracle.normal(3, 5, (1 << 16,))
    c = oracle.normal(3, 6, (1 << 16,))
    assert np.array_equal(bits(a), bits(b)) and not np.array_equal(a, c)
    assert abs(float(a.mean())) < 0.02 and abs(float(a.std()) - 1.0) < 0.02
    # a prefix of a longer stream is the shorter stream (counter based)
    assert np.array_equal(bits(oracle.normal(3, 5, (100,))), bits(a[:100]))


def test_avx2_and_scalar_dots_agree_within_rounding():
    x = oracle.normal(11, 0, (1, 4099))
    w = oracle.normal(11, 1, (3, 4099), 0.0, 0.02)
    q, s = oracle.quantize_rows(w)
    ya = oracle.forward(q, s, None, x, 1, 1)
    ys = oracle.forward(q, s, None, x, 1, 0)
    y64 = oracle.forward_f64(q, s, None, x)
    assert np.abs(ya - y64).max() < 1e-4 and np.abs(ys - y64).max() < 1e-4


# ---- the reference's own four tests, on seeded inputs -----------------------------------------
def kaiming_like(seed, out_f, in_f):
    """Linear::new draws kaiming-uniform weights and a uniform bias (src/nn/linear.rs:28-36);
    any bounded weights do for these assertions, so a seeded normal of the same scale is used."""
    bound = 1.0 / np.sqrt(in_f)
    w = oracle.normal(seed, 0, (out_f, in_f), 0.0, bound / np.sqrt(3.0))
    b = oracle.normal(seed, 1, (out_f,), 0.0, bound / np.sqrt(3.0))
    return w, b


def test_ref_int8_tensor_roundtrip():
    """tests/nn/quantization_tests.rs:4-29."""
    raw = oracle.normal(21, 0, (32, 64))
    q, scale = oracle.int8tensor_from_raw(raw)
    assert q.shape == (32, 64) and q.size == 32 * 64 and scale > 0
    deq = oracle.dequantize(q, scale)
    rmse = np.sqrt(np.mean((raw - deq) ** 2, dtype=np.float32))
    assert rmse < 0.05


def test_ref_qlinear_from_linear_and_forward():
    """tests/nn/quantization_tests.rs:32-74."""
    w, b = kaiming_like(22, 128, 64)
    q, s = oracle.quantize_rows(w)
    assert q.size == 64 * 128 and s.size == 128
    x = oracle.normal(22, 2, (8, 64))
    out_fp32 = x @ w.T + b
    out_int8 = oracle.forward(q, s, b, x)
    assert out_fp32.shape == out_int8.shape
    cos = float((out_fp32 * out_int8).sum() / (np.linalg.norm(out_fp32) * np.linalg.norm(out_int8)))
    assert cos > 0.995
    x3 = oracle.normal(22, 3, (4, 10, 64))
    out3 = oracle.forward(q, s, b, x3.reshape(-1, 64)).reshape(4, 10, 128)
    assert out3.shape == (4, 10, 128)


def test_ref_qlinear_memory_compression():
    """tests/nn/quantization_tests.rs:77-90."""
    fp32_bytes = 256 * 512 * 4 + 512 * 4
    int8_bytes = oracle.lib().nne_ref_qlinear_memory_bytes(512, 256, 1)
    assert fp32_bytes / int8_bytes > 3.8


def test_ref_qlinear_to_linear_roundtrip():
    """tests/nn/quantization_tests.rs:93-116: int8 forward vs f32 forward of the dequantized layer."""
    w, b = kaiming_like(24, 64, 32)
    q, s = oracle.quantize_rows(w)
    w_rec = oracle.to_linear(q, s)
    x = oracle.normal(24, 2, (2, 32))
    out_q = oracle.forward(q, s, b, x)
    out_rec = (x.astype(np.float32) @ w_rec.T.astype(np.float32) + b).astype(np.float32)
    assert np.abs(out_q - out_rec).max() < 1e-4
