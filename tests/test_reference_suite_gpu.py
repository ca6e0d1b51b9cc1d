"""The reference's own tests for this path (tests/nn/quantization_tests.rs), replayed through
the host mirror of nn::quantized on the GPU, with the same assertions and thresholds."""
import numpy as np
import pytest

import oracle

pytestmark = pytest.mark.gpu


def new_linear(nne, seed, in_f, out_f):
    """Linear::new(in, out): random weights and bias of the usual fan-in scale."""
    bound = 1.0 / np.sqrt(in_f)
    w = oracle.normal(seed, 0, (out_f, in_f), 0.0, bound / np.sqrt(3.0))
    b = oracle.normal(seed, 1, (out_f,), 0.0, bound / np.sqrt(3.0))
    return nne.Linear(w, b)


def linear_forward_f32(lin, x):
    """f32 Linear::forward (src/nn/linear.rs:47-55), the comparison target of the tests."""
    y = x.reshape(-1, lin.in_features).astype(np.float32) @ lin.weight.T
    if lin.bias is not None:
        y = y + lin.bias
    return y.reshape(list(x.shape[:-1]) + [lin.out_features]).astype(np.float32)


def test_int8_tensor_roundtrip(nne, ctx):
    raw = oracle.normal(21, 0, (32, 64))
    q_tensor = nne.Int8Tensor.from_raw(raw, ctx)
    assert q_tensor.shape == [32, 64]
    assert len(q_tensor.data) == 32 * 64
    assert q_tensor.scale > 0.0
    dequant = q_tensor.dequantize(ctx)
    assert dequant.shape == raw.shape
    rmse = np.sqrt(np.mean((raw - dequant) ** 2, dtype=np.float32))
    assert rmse < 0.05, f"INT8 quantization error too high: RMSE = {rmse}"


def test_qlinear_from_linear_and_forward(nne, ctx):
    linear = new_linear(nne, 22, 64, 128)
    qlinear = nne.QLinear.from_linear(linear, ctx)
    assert qlinear.in_features == 64 and qlinear.out_features == 128
    assert len(qlinear.qweight) == 64 * 128 and len(qlinear.scales) == 128
    x_2d = oracle.normal(22, 2, (8, 64))
    out_fp32 = linear_forward_f32(linear, x_2d)
    out_int8 = qlinear.forward(x_2d)
    assert out_fp32.shape == out_int8.shape
    cos = float((out_fp32 * out_int8).sum() / (np.linalg.norm(out_fp32) * np.linalg.norm(out_int8)))
    assert cos > 0.995, f"QLinear 2D cosine similarity too low: {cos}"
    x_3d = oracle.normal(22, 3, (4, 10, 64))
    out_3d_int8 = qlinear.forward(x_3d)
    assert out_3d_int8.shape == linear_forward_f32(linear, x_3d).shape == (4, 10, 128)


def test_qlinear_memory_compression(nne, ctx):
    linear = new_linear(nne, 23, 256, 512)
    qlinear = nne.QLinear.from_linear(linear, ctx)
    fp32_bytes = 256 * 512 * 4 + 512 * 4
    assert fp32_bytes / qlinear.memory_bytes() > 3.8


def test_qlinear_to_linear_roundtrip(nne, ctx):
    linear = new_linear(nne, 24, 32, 64)
    qlinear = nne.QLinear.from_linear(linear, ctx)
    recovered = qlinear.to_linear()
    assert recovered.in_features == 32 and recovered.out_features == 64
    assert np.array_equal(recovered.weight.view(np.uint32),
                          oracle.to_linear(qlinear.qweight.reshape(64, 32), qlinear.scales).view(np.uint32))
    x = oracle.normal(24, 2, (2, 32))
    out_q = qlinear.forward(x)
    out_rec = linear_forward_f32(recovered, x)
    assert np.abs(out_q - out_rec).max() < 1e-4


def test_example16_layer(nne, ctx):
    """examples/16_kvcache_and_int8_quantization.rs:105-146: 512 -> 1024, batch 16."""
    linear = new_linear(nne, 25, 512, 1024)
    q = nne.QLinear.from_linear(linear, ctx)
    fp32_bytes = 512 * 1024 * 4 + 1024 * 4
    assert fp32_bytes / q.memory_bytes() > 3.9
    x = oracle.normal(25, 2, (16, 512))
    a, b = linear_forward_f32(linear, x), q.forward(x)
    cos = float((a * b).sum() / (np.linalg.norm(a) * np.linalg.norm(b)))
    assert cos > 0.999


def test_qlinear_saved_as_int8_loads_straight_onto_the_device(nne, ctx, tmp_path):
    """The int8 on-disk format: a QLinear saved with I8 codes + F32 scales/bias comes back through
    nne_qlinear_create_from_i8 with identical fields and an identical forward (nothing re-quantized)."""
    w = oracle.normal(60, 0, (192, 320), 0.0, 0.02)
    b = oracle.normal(60, 1, (192,), 0.0, 0.1)
    ql = nne.QLinear.from_linear(nne.Linear(w, b), ctx)
    nb = nne.QLinear.from_linear(nne.Linear(w[:64], None), ctx)
    path = str(tmp_path / "layers.safetensors")
    nne.save_qlinears({"blk.0.up_proj": ql, "blk.0.gate_proj": nb}, path)
    back = nne.load_qlinear(path, "blk.0.up_proj", ctx)
    assert np.array_equal(back.qweight, ql.qweight) and np.array_equal(back.scales.view(np.uint32), ql.scales.view(np.uint32))
    assert np.array_equal(back.bias.view(np.uint32), ql.bias.view(np.uint32))
    back_nb = nne.load_qlinear(path, "blk.0.gate_proj", ctx)
    assert back_nb.bias is None
    for m in (1, 5, 40):
        x = oracle.normal(61, m, (m, 320))
        assert np.array_equal(back.forward(x).view(np.uint32), ql.forward(x).view(np.uint32))
        assert np.array_equal(back_nb.forward(x).view(np.uint32), nb.forward(x).view(np.uint32))
    ctx.check()


def test_device_tensor_chain_stays_on_the_device(nne, ctx):
    """`ToGpu for QLinear` + `CudaTensor` (the GpuLinear / GpuTensor pattern of the reference's device
    backend, src/gpu/layers.rs:12-57, src/gpu/tensor.rs:12-100): three layers chained on device
    tensors give what three host forwards give, bit for bit, with one upload and one download."""
    dims = [(256, 192), (320, 256), (128, 320)]
    layers = [nne.QLinear.from_linear(new_linear(nne, 70 + i, k, n), ctx) for i, (n, k) in enumerate(dims)]
    gpu_layers = [l.to_gpu(ctx) for l in layers]
    for shape in ([1, 192], [5, 192], [2, 3, 192], [40, 192]):
        x = oracle.normal(71, len(shape) * shape[0], shape)
        t = nne.CudaTensor.from_raw(x, ctx)
        assert t.shape == shape
        for gl in gpu_layers:
            t = gl.forward(t)
        want = x
        for l in layers:
            want = l.forward(want)
        got = t.to_cpu()
        assert got.shape == want.shape and np.array_equal(got.view(np.uint32), want.view(np.uint32))
    with pytest.raises(nne.ShapeMismatch):
        gpu_layers[0].forward(nne.CudaTensor.from_raw(np.zeros((2, 100), np.float32), ctx))
    with pytest.raises(nne.InvalidArgument):
        gpu_layers[0].forward(nne.CudaTensor.from_raw(np.zeros((192,), np.float32), ctx))
    with pytest.raises(nne.InvalidArgument):
        nne.CudaTensor.from_slice([1.0, 2.0, 3.0], [2, 2], ctx)
    assert np.array_equal(nne.CudaTensor.from_slice([1.0, 2.0, 3.0, 4.0], [2, 2], ctx).to_cpu(),
                          np.array([[1, 2], [3, 4]], np.float32))
    ctx.check()
