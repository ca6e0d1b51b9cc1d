// The reference's four tests for this path (tests/nn/quantization_tests.rs) plus the example-16
// layer, written against the C++ mirror of nn::quantized with the same assertions.  Needs a B200.
// Inputs are seeded (the reference draws from an unseeded RNG).  Exit code 0 = all passed.
#include <cmath>
#include <cstdio>
#include <random>

#include "nn_quantized.hpp"

using namespace nne;
using nne::quantized::Int8Tensor;
using nne::quantized::QLinear;

static int failures = 0;
#define CHECK(cond)                                                         \
    do {                                                                    \
        if (!(cond)) {                                                      \
            std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond);   \
            ++failures;                                                     \
        }                                                                   \
    } while (0)

static RawTensor randn(std::mt19937 &g, std::vector<size_t> shape, float std_) {
    size_t n = 1;
    for (size_t s : shape) n *= s;
    std::normal_distribution<float> d(0.0f, std_);
    std::vector<float> v(n);
    for (auto &x : v) x = d(g);
    return RawTensor::from_vec(std::move(v), std::move(shape));
}

static Linear new_linear(std::mt19937 &g, size_t in_f, size_t out_f) {
    const float s = 1.0f / std::sqrt(3.0f * (float)in_f);
    return Linear{Tensor(randn(g, {out_f, in_f}, s), true), Tensor(randn(g, {out_f}, s), true), in_f, out_f};
}

static std::vector<float> linear_forward(const Linear &l, const Tensor &x) {  // f32 Linear::forward
    const size_t m = x.data().len() / l.in_features;
    std::vector<float> y(m * l.out_features);
    for (size_t r = 0; r < m; ++r)
        for (size_t j = 0; j < l.out_features; ++j) {
            float s = 0.0f;
            for (size_t i = 0; i < l.in_features; ++i)
                s += x.data().data[r * l.in_features + i] * l.weight.data().data[j * l.in_features + i];
            y[r * l.out_features + j] = s + (l.bias ? l.bias->data().data[j] : 0.0f);
        }
    return y;
}

int main() {
    std::mt19937 g(1234);
    {  // test_int8_tensor_roundtrip (:4-29)
        RawTensor raw = randn(g, {32, 64}, 1.0f);
        Int8Tensor q = Int8Tensor::from_raw(raw);
        CHECK((q.shape == std::vector<size_t>{32, 64}));
        CHECK(q.data.size() == 32 * 64);
        CHECK(q.scale > 0.0f);
        RawTensor deq = q.dequantize();
        CHECK(deq.shape() == raw.shape());
        float mse = 0.0f;
        for (size_t i = 0; i < raw.len(); ++i) mse += (raw.data[i] - deq.data[i]) * (raw.data[i] - deq.data[i]);
        CHECK(std::sqrt(mse / (32.0f * 64.0f)) < 0.05f);
    }
    {  // test_qlinear_from_linear_and_forward (:32-74)
        Linear linear = new_linear(g, 64, 128);
        QLinear ql = QLinear::from_linear(linear);
        CHECK(ql.in_features == 64 && ql.out_features == 128);
        CHECK(ql.qweight.size() == 64 * 128 && ql.scales.size() == 128);
        Tensor x2(randn(g, {8, 64}, 1.0f), false);
        std::vector<float> a = linear_forward(linear, x2);
        Tensor out = ql.forward(x2);
        CHECK((out.shape() == std::vector<size_t>{8, 128}));
        double dot = 0, na = 0, nb = 0;
        for (size_t i = 0; i < a.size(); ++i) {
            dot += (double)a[i] * out.data().data[i];
            na += (double)a[i] * a[i];
            nb += (double)out.data().data[i] * out.data().data[i];
        }
        CHECK(dot / (std::sqrt(na) * std::sqrt(nb)) > 0.995);
        Tensor x3(randn(g, {4, 10, 64}, 1.0f), false);
        CHECK((ql.forward(x3).shape() == std::vector<size_t>{4, 10, 128}));
        CHECK(!ql.forward(x3).requires_grad);
        // error behaviour (:149-162)
        try {
            ql.forward(Tensor(randn(g, {64}, 1.0f), false));
            CHECK(false);
        } catch (const EngineError &e) {
            CHECK(e.kind == EngineError::Kind::InvalidArgument);
        }
        try {
            ql.forward(Tensor(randn(g, {2, 65}, 1.0f), false));
            CHECK(false);
        } catch (const EngineError &e) {
            CHECK(e.kind == EngineError::Kind::ShapeMismatch && e.expected[0] == 64 && e.actual[0] == 65);
        }
        QLinear copy = ql;  // #[derive(Clone)]
        CHECK(copy.forward(x2).data().data == out.data().data);
    }
    {  // test_qlinear_memory_compression (:77-90)
        QLinear ql = QLinear::from_linear(new_linear(g, 256, 512));
        const float fp32_bytes = 256 * 512 * 4 + 512 * 4;
        CHECK(fp32_bytes / (float)ql.memory_bytes() > 3.8f);
    }
    {  // test_qlinear_to_linear_roundtrip (:93-116)
        Linear linear = new_linear(g, 32, 64);
        QLinear ql = QLinear::from_linear(linear);
        Linear rec = ql.to_linear();
        CHECK(rec.in_features == 32 && rec.out_features == 64);
        Tensor x(randn(g, {2, 32}, 1.0f), false);
        Tensor out_q = ql.forward(x);
        std::vector<float> out_rec = linear_forward(rec, x);
        for (size_t i = 0; i < out_rec.size(); ++i) CHECK(std::fabs(out_q.data().data[i] - out_rec[i]) < 1e-4f);
    }
    {  // examples/16_kvcache_and_int8_quantization.rs:105-146
        Linear linear = new_linear(g, 512, 1024);
        QLinear ql = QLinear::from_linear(linear);
        CHECK((512.0f * 1024 * 4 + 1024 * 4) / (float)ql.memory_bytes() > 3.9f);
        Tensor x(randn(g, {16, 512}, 1.0f), false);
        std::vector<float> a = linear_forward(linear, x);
        Tensor b = ql.forward(x);
        double dot = 0, na = 0, nb = 0;
        for (size_t i = 0; i < a.size(); ++i) {
            dot += (double)a[i] * b.data().data[i];
            na += (double)a[i] * a[i];
            nb += (double)b.data().data[i] * b.data().data[i];
        }
        CHECK(dot / (std::sqrt(na) * std::sqrt(nb)) > 0.999);
    }
    std::printf(failures ? "%d check(s) failed\n" : "all reference tests passed\n", failures);
    return failures ? 1 : 0;
}
