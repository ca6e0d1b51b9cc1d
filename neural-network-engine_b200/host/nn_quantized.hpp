// C++ host-side mirror of the reference module nn::quantized (src/nn/quantized.rs) over the
// nne_cuda C ABI.  The reference is Rust; where no Rust toolchain exists this header is the
// compiled-language host side: same type names, public fields, method names, argument meaning
// and error behaviour, so that tests written against it read like the reference's own
// (tests/nn/quantization_tests.rs).  Header-only; link against libnne_cuda.{so,a}.
//
// Boundary types (minimal stand-ins for the reference types the path touches):
//   RawTensor  <- src/tensor/mod.rs:22-27   contiguous f32 data + shape
//   Tensor     <- src/autograd/tensor.rs    data + requires_grad (no autograd here)
//   Linear     <- src/nn/linear.rs:9-14     weight [out,in], optional bias, the two sizes
//   EngineError<- src/error.rs:10-52        the three variants this path can return
#pragma once

#include <cstddef>
#include <cstdint>
#include <memory>
#include <numeric>
#include <optional>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../include/nne_cuda.h"

namespace nne {

struct EngineError : std::runtime_error {
    enum class Kind { InvalidArgument, ShapeMismatch, GpuError };
    Kind kind;
    std::vector<size_t> expected, actual;  // ShapeMismatch only
    EngineError(Kind k, const std::string &msg) : std::runtime_error(msg), kind(k) {}
    static EngineError shape_mismatch(std::vector<size_t> e, std::vector<size_t> a) {
        EngineError err(Kind::ShapeMismatch, "Shape mismatch error");
        err.expected = std::move(e);
        err.actual = std::move(a);
        return err;
    }
};

namespace detail {
inline std::string last_error() {
    char buf[512];
    nne_last_error(buf, sizeof(buf));
    return buf;
}
inline void check(int status) {
    if (status == NNE_OK) return;
    if (status == NNE_ERR_INVALID_ARGUMENT)
        throw EngineError(EngineError::Kind::InvalidArgument, last_error());
    throw EngineError(EngineError::Kind::GpuError, last_error());
}
}  // namespace detail

// Arc<CudaContext>: one per device, shared by the layers on it (src/gpu/layers.rs:12-16).
class CudaContext {
  public:
    explicit CudaContext(int device = 0) { detail::check(nne_cuda_ctx_create(device, &raw_)); }
    ~CudaContext() { nne_cuda_ctx_destroy(raw_); }
    CudaContext(const CudaContext &) = delete;
    CudaContext &operator=(const CudaContext &) = delete;
    nne_ctx *raw() const { return raw_; }
    static std::shared_ptr<CudaContext> global() {
        static std::shared_ptr<CudaContext> ctx = std::make_shared<CudaContext>(0);
        return ctx;
    }

  private:
    nne_ctx *raw_ = nullptr;
};

struct RawTensor {
    std::vector<float> data;
    std::vector<size_t> shape_;
    static RawTensor from_vec(std::vector<float> d, std::vector<size_t> s) { return {std::move(d), std::move(s)}; }
    const std::vector<size_t> &shape() const { return shape_; }
    const float *as_slice() const { return data.data(); }
    size_t len() const { return data.size(); }
};

struct Tensor {
    RawTensor raw;
    bool requires_grad = false;
    Tensor(RawTensor r, bool rg) : raw(std::move(r)), requires_grad(rg) {}
    const std::vector<size_t> &shape() const { return raw.shape_; }
    const RawTensor &data() const { return raw; }
};

struct Linear {
    Tensor weight;
    std::optional<Tensor> bias;
    size_t in_features, out_features;
};

namespace quantized {

// src/nn/quantized.rs:20-73
struct Int8Tensor {
    std::vector<int8_t> data;
    std::vector<size_t> shape;
    float scale = 1.0f;

    static Int8Tensor from_raw(const RawTensor &raw) {
        Int8Tensor t;
        t.data.resize(raw.len());
        t.shape = raw.shape();
        detail::check(nne_quantize_tensor(CudaContext::global()->raw(), raw.as_slice(), raw.len(),
                                          t.data.data(), &t.scale));
        return t;
    }
    RawTensor dequantize() const {
        std::vector<float> out(data.size());
        detail::check(nne_dequantize_rows(CudaContext::global()->raw(), data.data(), &scale, 1,
                                          data.size(), out.data()));
        return RawTensor::from_vec(std::move(out), shape);
    }
    size_t memory_bytes() const { return data.size() + 56; }  // + size_of::<Int8Tensor>() on 64-bit
};

// src/nn/quantized.rs:78-250
class QLinear {
  public:
    std::vector<int8_t> qweight;
    std::vector<float> scales;
    std::optional<std::vector<float>> bias;
    size_t in_features = 0, out_features = 0;

    // QLinear::from_linear (:92-141).  Does not throw: a device failure is kept and thrown as
    // EngineError{GpuError} by the first forward, as the reference's signature is infallible.
    static QLinear from_linear(const Linear &linear) {
        QLinear q;
        q.in_features = linear.in_features;
        q.out_features = linear.out_features;
        const RawTensor &w = linear.weight.data();
        if (w.len() != q.in_features * q.out_features)
            throw std::logic_error("Weight slice length must match out_features * in_features");
        if (linear.bias) q.bias = linear.bias->data().data;
        q.qweight.resize(w.len());
        q.scales.resize(q.out_features);
        try {
            q.ctx_ = CudaContext::global();
            nne_qlinear *h = nullptr;
            detail::check(nne_qlinear_create_from_f32(q.ctx_->raw(), w.as_slice(),
                                                      q.bias ? q.bias->data() : nullptr,
                                                      q.out_features, q.in_features, &h));
            q.dev_.reset(h, nne_qlinear_destroy);
            detail::check(nne_qlinear_download(h, q.qweight.data(), q.scales.data()));
        } catch (const EngineError &e) {
            q.error_ = e.what();
        }
        return q;
    }

    // QLinear::forward_quantized (:146-197)
    Tensor forward_quantized(const Tensor &input) const {
        const auto &in_shape = input.shape();
        const size_t ndim = in_shape.size();
        if (ndim < 2)
            throw EngineError(EngineError::Kind::InvalidArgument,
                              "QLinear forward expects tensor with at least 2 dimensions");
        const size_t in_k = in_shape[ndim - 1];
        if (in_k != in_features) throw EngineError::shape_mismatch({in_features}, {in_k});
        const size_t num_rows = std::accumulate(in_shape.begin(), in_shape.end() - 1, size_t(1),
                                                std::multiplies<size_t>());
        std::vector<size_t> out_shape = in_shape;
        out_shape[ndim - 1] = out_features;
        std::vector<float> out(num_rows * out_features, 0.0f);
        detail::check(nne_qlinear_forward_host(device(), input.data().as_slice(), num_rows, in_k,
                                               out.data()));
        return Tensor(RawTensor::from_vec(std::move(out), std::move(out_shape)), false);
    }
    Tensor forward(const Tensor &input) const { return forward_quantized(input); }  // impl Module
    std::vector<Tensor> parameters() const { return {}; }                            // :245-248

    // QLinear::to_linear (:200-227)
    Linear to_linear() const {
        std::vector<float> w(qweight.size());
        detail::check(nne_dequantize_rows(CudaContext::global()->raw(), qweight.data(), scales.data(),
                                          out_features, in_features, w.data()));
        Linear lin{Tensor(RawTensor::from_vec(std::move(w), {out_features, in_features}), true),
                   std::nullopt, in_features, out_features};
        if (bias) lin.bias = Tensor(RawTensor::from_vec(*bias, {out_features}), true);
        return lin;
    }
    // QLinear::memory_bytes (:230-237)
    size_t memory_bytes() const {
        return qweight.size() + scales.size() * sizeof(float) + (bias ? bias->size() * sizeof(float) : 0);
    }

  private:
    // Built lazily from the public fields when the layer was not made by from_linear
    // (copied, or assembled by hand), so every QLinear value can run.
    nne_qlinear *device() const {
        if (!error_.empty()) throw EngineError(EngineError::Kind::GpuError, error_);
        if (!dev_) {
            ctx_ = CudaContext::global();
            nne_qlinear *h = nullptr;
            detail::check(nne_qlinear_create_from_i8(ctx_->raw(), qweight.data(), scales.data(),
                                                     bias ? bias->data() : nullptr, out_features,
                                                     in_features, &h));
            dev_.reset(h, nne_qlinear_destroy);
        }
        return dev_.get();
    }
    mutable std::shared_ptr<CudaContext> ctx_;
    mutable std::shared_ptr<nne_qlinear> dev_;  // shared by copies: the handle is immutable
    std::string error_;
};

}  // namespace quantized
}  // namespace nne
