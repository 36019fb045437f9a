// C++ host mirror of KORE's quantized-linear operator interface over the C ABI of
// kore_b200.h (header-only, C++17).  Names, argument meaning and error behaviour follow the
// reference's Rust modules, so that code written against them reads the same:
//
//   kore_b200::BitLinear   <- kore_nn::BitLinear   (crates/kore-nn/src/bit_linear.rs:25-288)
//   kore_b200::QuatLinear  <- kore_nn::QuatLinear  (crates/kore-nn/src/quat_linear.rs:27-319)
//   kore_b200::ternary_matmul / quat_matmul / ternary_ternary_matmul / pack_weights_*
//                          <- kore_kernels         (cpu_ternary_matmul.rs:29-240, cpu_quat_matmul.rs:22-214)
//   kore_b200::KoreError   <- kore_core::KoreError (ShapeMismatch, StorageError, UnsupportedDType)
//
// Differences by design: weights are uploaded once into a device-resident handle (the object
// owns it; it is immutable, so const forward from many threads is fine, as Module: Send + Sync),
// activations are quantised per token to int8 on the device, and nothing falls back to a CPU
// path: every failure is an exception carrying the C ABI's status code and message.
#pragma once

#include <cstddef>
#include <cstdint>
#include <cstdio>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "kore_b200.h"

namespace kore_b200 {

class KoreError : public std::runtime_error {
public:
    enum Kind { ShapeMismatch = 1, StorageError = 2, UnsupportedDType = 3, Cuda = 4, Nccl = 5, Timeout = 6,
                BadHandle = 7, InvalidArgument = 8, Unsupported = 9 };
    KoreError(int code, const std::string &what) : std::runtime_error(what), code_(code) {}
    int code() const { return code_; }
    Kind kind() const { return static_cast<Kind>(code_); }

private:
    int code_;
};

inline void check(int rc) {
    if (rc != 0) throw KoreError(rc, kb_last_error());
}

enum class Quantiser { Reference = 0, AbsMean = 1 };

// A tensor shape [d0, ..., in] -> (tokens, in); 1-D input is one token (bit_linear.rs:186-199)
inline std::pair<size_t, size_t> flatten_shape(const std::vector<size_t> &shape) {
    if (shape.empty()) return {0, 0};
    size_t n = 1;
    for (size_t i = 0; i + 1 < shape.size(); ++i) n *= shape[i];
    return {n, shape.back()};
}

class QuantLinear {
public:
    QuantLinear(const QuantLinear &) = delete;
    QuantLinear &operator=(const QuantLinear &) = delete;
    QuantLinear(QuantLinear &&o) noexcept { *this = std::move(o); }
    QuantLinear &operator=(QuantLinear &&o) noexcept {
        if (this != &o) {
            kb_linear_destroy(h_);
            h_ = o.h_; in_ = o.in_; out_ = o.out_; kind_ = o.kind_; has_bias_ = o.has_bias_;
            o.h_ = nullptr;
        }
        return *this;
    }
    ~QuantLinear() { kb_linear_destroy(h_); }

    size_t in_features() const { return in_; }
    size_t out_features() const { return out_; }
    bool has_bias() const { return has_bias_; }
    const kb_linear *handle() const { return h_; }

    // weight_memory_bytes / f32_weight_memory_bytes / compression_ratio (bit_linear.rs:129-143)
    size_t weight_memory_bytes() const {
        size_t m, k, bytes;
        int kind, device;
        check(kb_linear_info(h_, &m, &k, &kind, &device, &bytes));
        return bytes;
    }
    size_t f32_weight_memory_bytes() const { return out_ * in_ * 4; }
    float compression_ratio() const { return (float)f32_weight_memory_bytes() / (float)weight_memory_bytes(); }

    std::vector<uint8_t> packed_weights() const {
        std::vector<uint8_t> p(out_ * (kind_ == KB_TERNARY ? (in_ + 4) / 5 : (in_ + 3) / 4));
        check(kb_linear_packed_weights(h_, p.data(), p.size()));
        return p;
    }
    std::vector<float> scales() const {
        std::vector<float> s(out_);
        check(kb_linear_scales(h_, s.data(), s.size()));
        return s;
    }
    std::vector<float> dequantize_weights() const {
        std::vector<float> w(out_ * in_);
        check(kb_linear_dequantize_weights(h_, w.data(), w.size()));
        return w;
    }

    // Module::forward on host data: x is [.., in] with the given shape, the result is [.., out]
    // (1-D in, 1-D out).  A wrong last dimension is KoreError::ShapeMismatch (bit_linear.rs:179-184).
    std::vector<float> forward(const std::vector<float> &x, const std::vector<size_t> &shape,
                               std::vector<size_t> *out_shape = nullptr) const {
        const auto [n, in_dim] = flatten_shape(shape);
        if (shape.empty() || x.size() != n * in_dim) {
            char msg[128];
            std::snprintf(msg, sizeof msg, "shape mismatch: expected [%zu], got %zu values for the given shape", in_, x.size());
            throw KoreError(KoreError::ShapeMismatch, msg);
        }
        std::vector<float> y(n * out_);
        check(kb_linear_forward_host(h_, x.data(), n, in_dim, y.data()));
        if (out_shape) {
            *out_shape = shape;
            out_shape->back() = out_;
        }
        return y;
    }
    // raw host pointers: x [n, in_dim] -> y [n, out]
    void forward(const float *x, size_t n, size_t in_dim, float *y) const { check(kb_linear_forward_host(h_, x, n, in_dim, y)); }
    // device pointers on a stream (a cudaStream_t passed as void*); returns after enqueueing
    // max(forward(x), 0), the ReLU applied in the kernel epilogue (cuda/ops.rs:828-878 in layer form)
    void forward_relu_device(const float *x_dev, size_t n, float *y_dev, void *stream = nullptr) const {
        check(kb_linear_forward_act(h_, x_dev, n, in_features(), y_dev, 0, KB_ACT_RELU, KB_PATH_AUTO, nullptr, 0, stream));
    }
    void forward_device(const float *x_dev, size_t n, float *y_dev, void *stream = nullptr) const {
        check(kb_linear_forward(h_, x_dev, n, y_dev, stream));
    }

protected:
    QuantLinear() = default;
    void adopt(kb_linear *h, int kind, bool bias) {
        h_ = h;
        kind_ = kind;
        has_bias_ = bias;
        int k2, device;
        size_t bytes;
        check(kb_linear_info(h_, &out_, &in_, &k2, &device, &bytes));
    }
    kb_linear *h_ = nullptr;
    size_t in_ = 0, out_ = 0;
    int kind_ = KB_TERNARY;
    bool has_bias_ = false;
};

class BitLinear : public QuantLinear {
public:
    // BitLinear::new(weight [out, in], bias, threshold) (bit_linear.rs:48-77); quantiser AbsMean is
    // the per-tensor mean|W| ternariser
    static BitLinear create(const float *weight, const float *bias, size_t out_features, size_t in_features,
                            float threshold = 0.3f, Quantiser q = Quantiser::Reference, int device = 0) {
        kb_linear *h = nullptr;
        check(kb_linear_create_from_f32(KB_TERNARY, (int)q, weight, bias, out_features, in_features, threshold, device, &h));
        BitLinear l;
        l.adopt(h, KB_TERNARY, bias != nullptr);
        return l;
    }
    // from packed_weights() [out, ceil(in/5)] and scales() [out] of the reference layer
    static BitLinear from_packed(const std::vector<uint8_t> &packed, const std::vector<float> &scales, const float *bias,
                                 size_t in_features, size_t out_features, int device = 0) {
        kb_linear *h = nullptr;
        check(kb_linear_create_from_ref_packed(KB_TERNARY, packed.data(), packed.size(), scales.data(), scales.size(), bias,
                                               out_features, in_features, device, &h));
        BitLinear l;
        l.adopt(h, KB_TERNARY, bias != nullptr);
        return l;
    }
    std::string to_string() const {  // Display, bit_linear.rs:276-288
        char buf[160];
        std::snprintf(buf, sizeof buf, "BitLinear(in=%zu, out=%zu, bias=%s, compression=%.1fx)", in_, out_,
                      has_bias_ ? "true" : "false", compression_ratio());
        return buf;
    }
};

class QuatLinear : public QuantLinear {
public:
    static QuatLinear create(const float *weight, const float *bias, size_t out_features, size_t in_features, int device = 0) {
        kb_linear *h = nullptr;
        check(kb_linear_create_from_f32(KB_QUATERNARY, KB_QUANT_REFERENCE, weight, bias, out_features, in_features, 0.0f, device, &h));
        QuatLinear l;
        l.adopt(h, KB_QUATERNARY, bias != nullptr);
        return l;
    }
    static QuatLinear from_packed(const std::vector<uint8_t> &packed, const std::vector<float> &scales, const float *bias,
                                  size_t in_features, size_t out_features, int device = 0) {
        kb_linear *h = nullptr;
        check(kb_linear_create_from_ref_packed(KB_QUATERNARY, packed.data(), packed.size(), scales.data(), scales.size(), bias,
                                               out_features, in_features, device, &h));
        QuatLinear l;
        l.adopt(h, KB_QUATERNARY, bias != nullptr);
        return l;
    }
    std::string to_string() const {  // Display, quat_linear.rs:227-238
        char buf[160];
        std::snprintf(buf, sizeof buf, "QuatLinear(in=%zu, out=%zu, bias=%s, compression=%.1fx)", in_, out_,
                      has_bias_ ? "true" : "false", compression_ratio());
        return buf;
    }
};

// ---- kore-kernels shaped free functions: a_packed wire format, b [K,N], result [M,N] ----
// Several layers of one kind, shape and device, each applied to its own single token in ONE launch
// (device pointers: x [count, K] f32 -> y [count, M] f32 on `stream`).  Equivalent, bit for bit, to
// calling forward on every member with its row; the group borrows the members' device memory, so
// it must be destroyed before them.
class LinearGroup {
  public:
    explicit LinearGroup(const std::vector<const QuantLinear *> &members) {
        std::vector<const kb_linear *> hs;
        for (const QuantLinear *m : members) hs.push_back(m ? m->handle() : nullptr);
        check(kb_linear_group_create(hs.data(), hs.size(), &g_));
    }
    LinearGroup(const LinearGroup &) = delete;
    LinearGroup &operator=(const LinearGroup &) = delete;
    ~LinearGroup() { kb_linear_group_destroy(g_); }
    size_t size() const { return kb_linear_group_count(g_); }
    void forward_device(const float *x, size_t ldx, float *y, size_t ldy, kb_stream stream) const {
        check(kb_linear_group_forward(g_, x, ldx, y, ldy, stream));
    }

  private:
    kb_linear_group *g_ = nullptr;
};

inline std::vector<float> ternary_matmul(const std::vector<uint8_t> &a_packed, const std::vector<float> &a_scales,
                                         const std::vector<float> &b, size_t m, size_t n, size_t k) {
    if (b.size() < k * n) throw KoreError(KoreError::StorageError, "b too small");
    std::vector<float> c(m * n);
    check(kb_ternary_matmul(a_packed.data(), a_packed.size(), a_scales.data(), a_scales.size(), b.data(), c.data(), m, n, k));
    return c;
}
inline std::vector<float> quat_matmul(const std::vector<uint8_t> &a_packed, const std::vector<float> &a_scales,
                                      const std::vector<float> &b, size_t m, size_t n, size_t k) {
    if (b.size() < k * n) throw KoreError(KoreError::StorageError, "b too small");
    std::vector<float> c(m * n);
    check(kb_quat_matmul(a_packed.data(), a_packed.size(), a_scales.data(), a_scales.size(), b.data(), c.data(), m, n, k));
    return c;
}
inline std::vector<float> ternary_ternary_matmul(const std::vector<uint8_t> &a_packed, const std::vector<float> &a_scales,
                                                 const std::vector<uint8_t> &b_packed, const std::vector<float> &b_scales,
                                                 size_t m, size_t n, size_t k) {
    if (a_scales.size() < m || b_scales.size() < n) throw KoreError(KoreError::StorageError, "scales too small");
    std::vector<float> c(m * n);
    check(kb_ternary_ternary_matmul(a_packed.data(), a_packed.size(), a_scales.data(), b_packed.data(), b_packed.size(),
                                    b_scales.data(), c.data(), m, n, k));
    return c;
}
inline std::pair<std::vector<uint8_t>, std::vector<float>> pack_weights_ternary(const std::vector<float> &w, size_t m, size_t k,
                                                                                float threshold, int device = 0) {
    if (w.size() < m * k) throw KoreError(KoreError::StorageError, "weights too small");
    std::vector<uint8_t> packed(m * ((k + 4) / 5));
    std::vector<float> scales(m);
    check(kb_pack_weights_ternary(w.data(), m, k, threshold, packed.data(), packed.size(), scales.data(), scales.size(), device));
    return {std::move(packed), std::move(scales)};
}
inline std::pair<std::vector<uint8_t>, std::vector<float>> pack_weights_quaternary(const std::vector<float> &w, size_t m, size_t k,
                                                                                   int device = 0) {
    if (w.size() < m * k) throw KoreError(KoreError::StorageError, "weights too small");
    std::vector<uint8_t> packed(m * ((k + 3) / 4));
    std::vector<float> scales(m);
    check(kb_pack_weights_quaternary(w.data(), m, k, packed.data(), packed.size(), scales.data(), scales.size(), device));
    return {std::move(packed), std::move(scales)};
}

}  // namespace kore_b200
