// b200nn.hpp — header-only C++17 host layer over the C ABI of b200nn.h.
//
// The reference's host side is Rust (`gpu_host::nn`); where no Rust toolchain exists this is the
// compiled-language host mirror: the same type and method names, argument meaning and error
// behaviour as the Rust items each class cites (file:line relative to the reference repository;
// GH = crates/core/gpu-host/src), with RAII in place of Drop and exceptions in place of Result.
// Nothing here computes: every method is one call into libb200nn.so.
#ifndef B200NN_HPP
#define B200NN_HPP

#include <cstdint>
#include <memory>
#include <optional>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "b200nn.h"

namespace b200nn {

// NnError (GH/nn/error.rs:7-29): ShapeMismatch, DimOutOfRange, KernelNotFound, Cuda; the library
// adds Device (a kernel's bounded wait ran out), Arg, Io and MissingTensor (ModelError, GH/model.rs:30-62).
class NnError : public std::runtime_error {
public:
    NnError(int32_t code, const std::string &message) : std::runtime_error(kind_name(code) + ": " + message), code_(code) {}
    int32_t code() const { return code_; }
    static std::string kind_name(int32_t code) {
        switch (code) {
        case B200NN_ERR_SHAPE: return "ShapeMismatch";
        case B200NN_ERR_DIM: return "DimOutOfRange";
        case B200NN_ERR_UNSUPPORTED: return "KernelNotFound";
        case B200NN_ERR_CUDA: return "Cuda";
        case B200NN_ERR_DEVICE: return "Device";
        case B200NN_ERR_ARG: return "Arg";
        case B200NN_ERR_IO: return "Io";
        case B200NN_ERR_MISSING: return "MissingTensor";
        default: return "Error(" + std::to_string(code) + ")";
        }
    }

private:
    int32_t code_;
};

// KernelRegistry (GH/nn/registry.rs:29-147): one per GPU; owns the library context.  The by-name
// kernel lookups and launch-geometry helpers of the reference have no counterpart: kernels are
// linked into the library and choose their own grids.
class KernelRegistry {
public:
    // KernelRegistry::init_default (registry.rs:131-135): device 0.
    static std::shared_ptr<KernelRegistry> init_default() { return std::make_shared<KernelRegistry>(0); }
    explicit KernelRegistry(int device_ordinal) : device_(device_ordinal) {
        const int32_t rc = b200nn_ctx_create(device_ordinal, &ctx_);
        if (rc != B200NN_OK) throw NnError(rc, "no context on CUDA device " + std::to_string(device_ordinal));
    }
    ~KernelRegistry() { if (ctx_) b200nn_ctx_destroy(ctx_); }
    KernelRegistry(const KernelRegistry &) = delete;
    KernelRegistry &operator=(const KernelRegistry &) = delete;

    int device() const { return device_; }
    b200nn_ctx *ctx() const { return ctx_; }
    void synchronize() const { check(b200nn_ctx_synchronize(ctx_)); }
    uint64_t launch_count() const { return b200nn_ctx_launch_count(ctx_); }
    void set_tuning(const char *key, int32_t value) const { check(b200nn_ctx_set_tuning(ctx_, key, value)); }
    // reads and clears the device-side error word
    uint32_t device_error() const {
        uint32_t w = 0;
        check(b200nn_ctx_device_error(ctx_, &w));
        return w;
    }
    // turns a status into the reference's error type, with the library's message for this context
    void check(int32_t rc) const {
        if (rc == B200NN_OK) return;
        const char *m = b200nn_last_error_message(ctx_);
        throw NnError(rc, m ? m : "");
    }

private:
    b200nn_ctx *ctx_ = nullptr;
    int device_ = 0;
};
using Registry = std::shared_ptr<KernelRegistry>;

// GpuTensor (GH/nn/tensor.rs:45-393): f32, row-major, contiguous, on the registry's device.
class GpuTensor {
public:
    GpuTensor() = default;
    GpuTensor(Registry reg, b200nn_tensor *h) : reg_(std::move(reg)), h_(h) {}
    ~GpuTensor() { reset(); }
    GpuTensor(GpuTensor &&o) noexcept : reg_(std::move(o.reg_)), h_(o.h_) { o.h_ = nullptr; }
    GpuTensor &operator=(GpuTensor &&o) noexcept {
        if (this != &o) { reset(); reg_ = std::move(o.reg_); h_ = o.h_; o.h_ = nullptr; }
        return *this;
    }
    GpuTensor(const GpuTensor &) = delete;
    GpuTensor &operator=(const GpuTensor &) = delete;

    // from_host (tensor.rs:83-110): data.size() must equal the product of shape
    static GpuTensor from_host(const std::vector<float> &data, const std::vector<size_t> &shape, const Registry &reg) {
        size_t n = 1;
        for (size_t s : shape) n *= s;
        if (n != data.size())
            throw NnError(B200NN_ERR_SHAPE, "expected " + std::to_string(n) + " elements, got " + std::to_string(data.size()));
        b200nn_tensor *h = nullptr;
        reg->check(b200nn_tensor_from_host(reg->ctx(), data.data(), shape.data(), (int32_t)shape.size(), &h));
        return GpuTensor(reg, h);
    }
    // from_data (tensor.rs:67-77): over f32 values already on the device (copied; the caller keeps its buffer)
    static GpuTensor from_data(const float *dev, const std::vector<size_t> &shape, const Registry &reg) {
        b200nn_tensor *h = nullptr;
        reg->check(b200nn_tensor_from_device(reg->ctx(), dev, shape.data(), (int32_t)shape.size(), &h));
        return GpuTensor(reg, h);
    }
    static GpuTensor zeros(const std::vector<size_t> &shape, const Registry &reg) {
        b200nn_tensor *h = nullptr;
        reg->check(b200nn_tensor_zeros(reg->ctx(), shape.data(), (int32_t)shape.size(), &h));
        return GpuTensor(reg, h);
    }
    std::vector<float> to_host() const {
        std::vector<float> out(numel());
        reg_->check(b200nn_tensor_to_host(h_, out.data(), out.size()));
        return out;
    }
    size_t numel() const { return b200nn_tensor_numel(h_); }
    size_t ndim() const { return (size_t)b200nn_tensor_ndim(h_); }
    std::vector<size_t> shape() const {
        std::vector<size_t> s(ndim());
        reg_->check(b200nn_tensor_shape(h_, s.data(), (int32_t)s.size()));
        return s;
    }
    std::vector<size_t> strides() const {
        const std::vector<size_t> s = shape();
        std::vector<size_t> st(s.size());
        size_t acc = 1;
        for (size_t i = s.size(); i-- > 0;) { st[i] = acc; acc *= s[i]; }
        return st;
    }
    bool is_contiguous() const { return true; }
    size_t size_bytes() const { return numel() * sizeof(float); }
    float *as_ptr() const { return b200nn_tensor_data(h_); } // device pointer
    GpuTensor reshape(const std::vector<size_t> &shape) const {
        b200nn_tensor *h = nullptr;
        reg_->check(b200nn_tensor_reshape(h_, shape.data(), (int32_t)shape.size(), &h));
        return GpuTensor(reg_, h);
    }
    GpuTensor clone_tensor() const {
        b200nn_tensor *h = nullptr;
        reg_->check(b200nn_tensor_clone(h_, &h));
        return GpuTensor(reg_, h);
    }
    GpuTensor transpose(size_t dim0, size_t dim1) const {
        b200nn_tensor *h = nullptr;
        reg_->check(b200nn_tensor_transpose(h_, dim0, dim1, &h));
        return GpuTensor(reg_, h);
    }
    static GpuTensor concat(const std::vector<const GpuTensor *> &tensors, size_t dim) {
        if (tensors.empty()) throw NnError(B200NN_ERR_SHAPE, "concat of an empty list");
        std::vector<const b200nn_tensor *> hs;
        for (const GpuTensor *t : tensors) hs.push_back(t->h_);
        b200nn_tensor *h = nullptr;
        tensors[0]->reg_->check(b200nn_tensor_concat(hs.data(), hs.size(), dim, &h));
        return GpuTensor(tensors[0]->reg_, h);
    }
    std::vector<GpuTensor> split(size_t dim, const std::vector<size_t> &sizes) const {
        std::vector<b200nn_tensor *> hs(sizes.size(), nullptr);
        reg_->check(b200nn_tensor_split(h_, dim, sizes.data(), sizes.size(), hs.data()));
        std::vector<GpuTensor> out;
        for (b200nn_tensor *h : hs) out.emplace_back(reg_, h);
        return out;
    }
    b200nn_tensor *handle() const { return h_; }
    const Registry &registry() const { return reg_; }

private:
    void reset() { if (h_) b200nn_tensor_destroy(h_); h_ = nullptr; }
    Registry reg_;
    b200nn_tensor *h_ = nullptr;
};

// Activation (GH/nn/layers/linear.rs:24-33) and FusedActivation (GH/nn/ops/gemm.rs:803-808).
enum class Activation : int32_t { Gelu = B200NN_ACT_GELU_TANH, Relu = B200NN_ACT_RELU, Silu = B200NN_ACT_SILU, Sigmoid = B200NN_ACT_SIGMOID };
enum class FusedActivation : int32_t { Gelu = B200NN_ACT_GELU_SIGMOID, Relu = B200NN_ACT_RELU };

// Stateless ops (GH/nn/ops/mod.rs:19-37); each takes the registry last, as there.
namespace ops {
inline GpuTensor wrap_(const Registry &reg, int32_t rc, b200nn_tensor *h) {
    reg->check(rc);
    return GpuTensor(reg, h);
}
// ops::layer_norm (ops/norm.rs:14-81)
inline GpuTensor layer_norm(const GpuTensor &x, const GpuTensor &gamma, const GpuTensor &beta, float eps, const Registry &reg) {
    b200nn_tensor *h = nullptr;
    const int32_t rc = b200nn_layer_norm(reg->ctx(), x.handle(), gamma.handle(), beta.handle(), eps, &h);
    return wrap_(reg, rc, h);
}
// ops::layer_norm_residual_dual (ops/norm.rs:248-400): (a + b, LayerNorm(a + b))
inline std::pair<GpuTensor, GpuTensor> layer_norm_residual_dual(const GpuTensor &a, const GpuTensor &b, const GpuTensor &gamma,
                                                                 const GpuTensor &beta, float eps, const Registry &reg) {
    b200nn_tensor *s = nullptr, *n = nullptr;
    reg->check(b200nn_layer_norm_residual_dual(reg->ctx(), a.handle(), b.handle(), gamma.handle(), beta.handle(), eps, &s, &n));
    return {GpuTensor(reg, s), GpuTensor(reg, n)};
}
// ops::layer_norm_residual (ops/norm.rs:88-246): LayerNorm(x + residual); the sum itself is not kept
inline GpuTensor layer_norm_residual(const GpuTensor &x, const GpuTensor &residual, const GpuTensor &gamma, const GpuTensor &beta,
                                     float eps, const Registry &reg) {
    return std::move(layer_norm_residual_dual(x, residual, gamma, beta, eps, reg).second);
}
inline GpuTensor activation_(const GpuTensor &x, int32_t act, const Registry &reg) {
    b200nn_tensor *h = nullptr;
    const int32_t rc = b200nn_activation(reg->ctx(), x.handle(), act, &h);
    return wrap_(reg, rc, h);
}
// ops::gelu / silu / sigmoid / relu (ops/activation.rs).  gelu is the tanh form unless sigmoid_form.
inline GpuTensor gelu(const GpuTensor &x, const Registry &reg, bool sigmoid_form = false) {
    return activation_(x, sigmoid_form ? B200NN_ACT_GELU_SIGMOID : B200NN_ACT_GELU_TANH, reg);
}
inline GpuTensor silu(const GpuTensor &x, const Registry &reg) { return activation_(x, B200NN_ACT_SILU, reg); }
inline GpuTensor sigmoid(const GpuTensor &x, const Registry &reg) { return activation_(x, B200NN_ACT_SIGMOID, reg); }
inline GpuTensor relu(const GpuTensor &x, const Registry &reg) { return activation_(x, B200NN_ACT_RELU, reg); }
// ops::bias_add / elementwise_add (ops/reshape.rs:112-186): in place
inline void bias_add(GpuTensor &data, const GpuTensor &bias, const Registry &reg) {
    reg->check(b200nn_bias_add(reg->ctx(), data.handle(), bias.handle()));
}
inline void elementwise_add(GpuTensor &a, const GpuTensor &b, const Registry &reg) {
    reg->check(b200nn_elementwise_add(reg->ctx(), a.handle(), b.handle()));
}
// ops::elementwise_add_out (ops/reshape.rs:219-290): a + b into a new tensor
inline GpuTensor elementwise_add_out(const GpuTensor &a, const GpuTensor &b, const Registry &reg) {
    if (a.numel() != b.numel())
        throw NnError(B200NN_ERR_SHAPE, "expected same numel, a has " + std::to_string(a.numel()) + ", b has " + std::to_string(b.numel()));
    GpuTensor out = a.clone_tensor();
    elementwise_add(out, b, reg);
    return out;
}
// ops::matmul (ops/gemm.rs:20-212): [M,K] x [K,N]; matmul_v2 / v4 / v4_1 are the same contract
inline GpuTensor matmul(const GpuTensor &a, const GpuTensor &b, const Registry &reg) {
    b200nn_tensor *h = nullptr;
    const int32_t rc = b200nn_matmul(reg->ctx(), a.handle(), b.handle(), &h);
    return wrap_(reg, rc, h);
}
inline GpuTensor matmul_v2(const GpuTensor &a, const GpuTensor &b, const Registry &reg) { return matmul(a, b, reg); }
inline GpuTensor matmul_v4(const GpuTensor &a, const GpuTensor &b, const Registry &reg) { return matmul(a, b, reg); }
inline GpuTensor matmul_v4_1(const GpuTensor &a, const GpuTensor &b, const Registry &reg) { return matmul(a, b, reg); }
// ops::matmul_fused (ops/gemm.rs:814-977): activation(a x b + bias); its GELU is x * sigmoid(1.702 x)
inline GpuTensor matmul_fused(const GpuTensor &a, const GpuTensor &b, const GpuTensor &bias, FusedActivation activation,
                              const Registry &reg) {
    if (a.ndim() != 2 || b.ndim() != 2)
        throw NnError(B200NN_ERR_SHAPE, "expected 2D tensors, actual a.ndim=" + std::to_string(a.ndim()) + ", b.ndim=" + std::to_string(b.ndim()));
    const size_t n = b.shape()[1];
    if (a.shape()[1] != b.shape()[0])
        throw NnError(B200NN_ERR_SHAPE, "expected a.shape[1]=" + std::to_string(a.shape()[1]) + " == b.shape[0], actual b.shape[0]=" + std::to_string(b.shape()[0]));
    if (bias.ndim() != 1 || bias.shape()[0] != n) throw NnError(B200NN_ERR_SHAPE, "expected bias.shape=[" + std::to_string(n) + "]");
    GpuTensor y = matmul(a, b, reg);
    bias_add(y, bias, reg);
    return activation_(y, (int32_t)activation, reg);
}
// ops::int4_matmul (ops/gemm.rs:1186-1266): quantise b [K,N] (host) per group, then a [M,K] x dequant(b)
inline GpuTensor int4_matmul(const GpuTensor &a, const std::vector<float> &b_host, size_t k, size_t n, size_t group, const Registry &reg) {
    if (b_host.size() != k * n) throw NnError(B200NN_ERR_SHAPE, "b must hold k*n values");
    b200nn_tensor *h = nullptr;
    const int32_t rc = b200nn_int4_matmul(reg->ctx(), a.handle(), b_host.data(), k, n, group, &h);
    return wrap_(reg, rc, h);
}
// ops::split_qkv / concat_heads (ops/attention.rs:105-142, 515-549)
struct Qkv { GpuTensor q, k, v; };
inline Qkv split_qkv(const GpuTensor &qkv, size_t seq_len, size_t n_heads, size_t d_head, const Registry &reg) {
    b200nn_tensor *q = nullptr, *k = nullptr, *v = nullptr;
    reg->check(b200nn_split_qkv(reg->ctx(), qkv.handle(), seq_len, n_heads, d_head, &q, &k, &v));
    return Qkv{GpuTensor(reg, q), GpuTensor(reg, k), GpuTensor(reg, v)};
}
inline GpuTensor concat_heads(const GpuTensor &heads, size_t seq_len, size_t n_heads, size_t d_head, const Registry &reg) {
    b200nn_tensor *h = nullptr;
    const int32_t rc = b200nn_concat_heads(reg->ctx(), heads.handle(), seq_len, n_heads, d_head, &h);
    return wrap_(reg, rc, h);
}
// ops::multi_head_flash_attention (ops/attention.rs:151-202; _v3 and _nvrtc are the same contract): q,k,v [H,seq,64]
inline GpuTensor multi_head_flash_attention(const GpuTensor &q, const GpuTensor &k, const GpuTensor &v, size_t seq_len, size_t n_heads,
                                            size_t d_head, bool causal, const Registry &reg) {
    b200nn_tensor *h = nullptr;
    const int32_t rc = b200nn_multi_head_flash_attention(reg->ctx(), q.handle(), k.handle(), v.handle(), seq_len, n_heads, d_head, causal ? 1 : 0, &h);
    return wrap_(reg, rc, h);
}
// ops::scaled_dot_product_attention_kv (ops/attention.rs:557-606): one head, q [q_len,64] against k,v [kv_len,64]
inline GpuTensor scaled_dot_product_attention_kv(const GpuTensor &q, const GpuTensor &k, const GpuTensor &v, bool causal, size_t q_offset,
                                                 const Registry &reg) {
    b200nn_tensor *h = nullptr;
    const int32_t rc = b200nn_attention_kv(reg->ctx(), q.handle(), k.handle(), v.handle(), causal ? 1 : 0, q_offset, &h);
    return wrap_(reg, rc, h);
}
// ops::scaled_dot_product_attention (ops/attention.rs:17-103): one head, q, k, v [seq_len, d_head]
inline GpuTensor scaled_dot_product_attention(const GpuTensor &q, const GpuTensor &k, const GpuTensor &v, bool causal, const Registry &reg) {
    return scaled_dot_product_attention_kv(q, k, v, causal, 0, reg);
}
// host quantiser (ops/quantize.rs:56-162)
struct Int4Quantized { std::vector<uint32_t> packed; std::vector<float> scales; };
inline Int4Quantized quantize_weight_int4(const std::vector<float> &weight_t, size_t k, size_t n, size_t group) {
    if (weight_t.size() != k * n || group == 0) throw NnError(B200NN_ERR_SHAPE, "weight_t must hold k*n values and group be non-zero");
    Int4Quantized q{std::vector<uint32_t>((k / 8) * n), std::vector<float>(((k + group - 1) / group) * n)};
    const int32_t rc = b200nn_quantize_weight_int4(weight_t.data(), k, n, group, q.packed.data(), q.scales.data());
    if (rc != B200NN_OK) throw NnError(rc, "quantize_weight_int4: k must be a multiple of 8");
    return q;
}
inline int32_t unpack_int4(uint32_t packed, int32_t index) { return b200nn_unpack_int4(packed, index); }
}  // namespace ops

// Handle holder shared by the layer and model classes: owns one library object.
template <typename H, void (*Destroy)(H *)>
class Owned {
public:
    Owned() = default;
    Owned(Registry reg, H *h) : reg_(std::move(reg)), h_(h) {}
    ~Owned() { if (h_) Destroy(h_); }
    Owned(Owned &&o) noexcept : reg_(std::move(o.reg_)), h_(o.h_) { o.h_ = nullptr; }
    Owned &operator=(Owned &&o) noexcept {
        if (this != &o) { if (h_) Destroy(h_); reg_ = std::move(o.reg_); h_ = o.h_; o.h_ = nullptr; }
        return *this;
    }
    Owned(const Owned &) = delete;
    Owned &operator=(const Owned &) = delete;
    H *handle() const { return h_; }
    const Registry &registry() const { return reg_; }

protected:
    // rc must be computed before this call is written down: the order in which a call's arguments are
    // evaluated is unspecified, so `out_(f(&t), t)` could read t before f has set it
    GpuTensor out_(int32_t rc, b200nn_tensor *t) const {
        reg_->check(rc);
        return GpuTensor(reg_, t);
    }
    Registry reg_;
    H *h_ = nullptr;
};

// Linear (GH/nn/layers/linear.rs:58-313): weight [out,in] row-major, optional bias [out].
class Linear : public Owned<b200nn_linear, b200nn_linear_destroy> {
public:
    Linear(const std::vector<float> &weight, const std::vector<float> *bias, size_t in_features, size_t out_features, const Registry &reg) {
        if (weight.size() != in_features * out_features)
            throw NnError(B200NN_ERR_SHAPE, "weight: expected " + std::to_string(out_features) + "x" + std::to_string(in_features));
        if (bias && bias->size() != out_features) throw NnError(B200NN_ERR_SHAPE, "bias: expected " + std::to_string(out_features));
        reg_ = reg;
        reg->check(b200nn_linear_create(reg->ctx(), weight.data(), bias ? bias->data() : nullptr, in_features, out_features, &h_));
    }
    GpuTensor forward(const GpuTensor &x) const {
        b200nn_tensor *y = nullptr;
        const int32_t rc = b200nn_linear_forward(h_, x.handle(), &y);
        return out_(rc, y);
    }
    // forward_fused (linear.rs:131-166) with FusedActivation; forward_auto_fused (184-278) with Activation
    GpuTensor forward_fused(const GpuTensor &x, FusedActivation a) const {
        b200nn_tensor *y = nullptr;
        const int32_t rc = b200nn_linear_forward_fused(h_, x.handle(), (int32_t)a, &y);
        return out_(rc, y);
    }
    GpuTensor forward_auto_fused(const GpuTensor &x, Activation a) const {
        b200nn_tensor *y = nullptr;
        const int32_t rc = b200nn_linear_forward_fused(h_, x.handle(), (int32_t)a, &y);
        return out_(rc, y);
    }
};

// Int4Linear (GH/nn/layers/int4_linear.rs:24-147): packed [K/8,N] u32, scales [ceil(K/group),N] f32.
class Int4Linear : public Owned<b200nn_int4_linear, b200nn_int4_linear_destroy> {
public:
    Int4Linear(const std::vector<uint32_t> &packed, const std::vector<float> &scales, const std::vector<float> *bias, size_t in_features,
               size_t out_features, size_t group_size, const Registry &reg) {
        const size_t groups = group_size ? (in_features + group_size - 1) / group_size : 0;
        if (in_features % 8 || packed.size() != in_features / 8 * out_features || scales.size() != groups * out_features)
            throw NnError(B200NN_ERR_SHAPE, "packed must be [K/8,N] and scales [ceil(K/group),N] with K%8==0");
        if (bias && bias->size() != out_features) throw NnError(B200NN_ERR_SHAPE, "bias: expected " + std::to_string(out_features));
        reg_ = reg;
        reg->check(b200nn_int4_linear_create(reg->ctx(), packed.data(), scales.data(), bias ? bias->data() : nullptr, in_features,
                                             out_features, group_size, &h_));
    }
    GpuTensor forward(const GpuTensor &x) const {
        b200nn_tensor *y = nullptr;
        const int32_t rc = b200nn_int4_linear_forward(h_, x.handle(), &y);
        return out_(rc, y);
    }
    size_t memory_bytes() const { return b200nn_int4_linear_memory_bytes(h_); }
};

// LayerNorm (GH/nn/layers/norm.rs:24-55)
class LayerNorm : public Owned<b200nn_layernorm, b200nn_layernorm_destroy> {
public:
    LayerNorm(const std::vector<float> &gamma, const std::vector<float> &beta, float eps, const Registry &reg) : gamma_(gamma), beta_(beta) {
        if (gamma.size() != beta.size() || gamma.empty()) throw NnError(B200NN_ERR_SHAPE, "gamma and beta must have the same non-zero length");
        reg_ = reg;
        reg->check(b200nn_layernorm_create(reg->ctx(), gamma.data(), beta.data(), gamma.size(), eps, &h_));
    }
    GpuTensor forward(const GpuTensor &x) const {
        b200nn_tensor *y = nullptr;
        const int32_t rc = b200nn_layernorm_forward(h_, x.handle(), &y);
        return out_(rc, y);
    }
    GpuTensor gamma() const { return GpuTensor::from_host(gamma_, {gamma_.size()}, reg_); }
    GpuTensor beta() const { return GpuTensor::from_host(beta_, {beta_.size()}, reg_); }

private:
    std::vector<float> gamma_, beta_;
};

// Embedding (GH/nn/layers/embedding.rs:25-93)
class Embedding : public Owned<b200nn_embedding, b200nn_embedding_destroy> {
public:
    Embedding(const std::vector<float> &wte, const std::vector<float> &wpe, size_t vocab_size, size_t max_seq_len, size_t d_model,
              const Registry &reg) {
        if (wte.size() != vocab_size * d_model || wpe.size() != max_seq_len * d_model)
            throw NnError(B200NN_ERR_SHAPE, "wte must be [vocab,d] and wpe [max_seq,d]");
        reg_ = reg;
        reg->check(b200nn_embedding_create(reg->ctx(), wte.data(), wpe.data(), vocab_size, max_seq_len, d_model, &h_));
    }
    GpuTensor forward_tokens(const std::vector<uint32_t> &ids) const { return forward_tokens_with_offset(ids, 0); }
    GpuTensor forward_tokens_with_offset(const std::vector<uint32_t> &ids, size_t pos_offset) const {
        b200nn_tensor *y = nullptr;
        const int32_t rc = b200nn_embedding_forward_tokens(h_, ids.data(), ids.size(), pos_offset, &y);
        return out_(rc, y);
    }
};

// MultiHeadAttention (GH/nn/layers/attention.rs:30-184) and Int4MultiHeadAttention (GH/nn/models/gpt2.rs:1127-1214,
// group_size > 0): qkv_weight [3d,d], out_weight [d,d] in Linear layout.
class MultiHeadAttention : public Owned<b200nn_attention, b200nn_attention_destroy> {
public:
    MultiHeadAttention(const std::vector<float> &qkv_weight, const std::vector<float> &qkv_bias, const std::vector<float> &out_weight,
                       const std::vector<float> &out_bias, size_t n_embd, size_t n_heads, const Registry &reg, size_t group_size = 0)
        : n_heads_(n_heads), d_head_(n_heads ? n_embd / n_heads : 0) {
        if (qkv_weight.size() != 3 * n_embd * n_embd || qkv_bias.size() != 3 * n_embd || out_weight.size() != n_embd * n_embd ||
            out_bias.size() != n_embd)
            throw NnError(B200NN_ERR_SHAPE, "attention weights do not match n_embd");
        reg_ = reg;
        reg->check(group_size ? b200nn_int4_attention_create(reg->ctx(), qkv_weight.data(), qkv_bias.data(), out_weight.data(), out_bias.data(),
                                                             n_embd, n_heads, group_size, &h_)
                              : b200nn_attention_create(reg->ctx(), qkv_weight.data(), qkv_bias.data(), out_weight.data(), out_bias.data(),
                                                        n_embd, n_heads, &h_));
    }
    size_t n_heads() const { return n_heads_; }
    size_t d_head() const { return d_head_; }
    GpuTensor forward_causal(const GpuTensor &x) const {
        b200nn_tensor *y = nullptr;
        const int32_t rc = b200nn_attention_forward_causal(h_, x.handle(), &y);
        return out_(rc, y);
    }
    // forward_cached (attention.rs:133-178): cached_k / cached_v [n_heads][kv_len*d_head]; returns y and
    // appends nothing itself: the new rows [n_heads][new_len*d_head] come back in new_k / new_v
    GpuTensor forward_cached(const GpuTensor &x, const std::vector<float> &cached_k, const std::vector<float> &cached_v, size_t kv_len,
                             std::vector<float> *new_k, std::vector<float> *new_v) const {
        const size_t new_len = x.shape()[0];
        if (cached_k.size() != n_heads_ * kv_len * d_head_ || cached_v.size() != cached_k.size())
            throw NnError(B200NN_ERR_SHAPE, "cached K/V must be [n_heads][kv_len*d_head]");
        new_k->assign(n_heads_ * new_len * d_head_, 0.0f);
        new_v->assign(n_heads_ * new_len * d_head_, 0.0f);
        b200nn_tensor *y = nullptr;
        const int32_t rc = b200nn_attention_forward_cached(h_, x.handle(), kv_len ? cached_k.data() : nullptr, kv_len ? cached_v.data() : nullptr,
                                                    kv_len, &y, new_k->data(), new_v->data());
        return out_(rc, y);
    }

private:
    size_t n_heads_, d_head_;
};

// GELU / SiLU / Sigmoid / ReLU layers (GH/nn/layers/activation.rs:15-96): zero-parameter modules
struct GELU { Registry reg; GpuTensor forward(const GpuTensor &x) const { return ops::gelu(x, reg); } };
struct SiLU { Registry reg; GpuTensor forward(const GpuTensor &x) const { return ops::silu(x, reg); } };
struct Sigmoid { Registry reg; GpuTensor forward(const GpuTensor &x) const { return ops::sigmoid(x, reg); } };
struct ReLU { Registry reg; GpuTensor forward(const GpuTensor &x) const { return ops::relu(x, reg); } };

// Gpt2Config (GH/nn/models/gpt2.rs:20-93)
struct Gpt2Config {
    size_t n_layer = 12, n_embd = 768, n_head = 12, vocab_size = 50257, n_positions = 1024;
    float layer_norm_epsilon = 1e-5f;
    static Gpt2Config small() { return preset_("small"); }
    static Gpt2Config medium() { return preset_("medium"); }
    static Gpt2Config large() { return preset_("large"); }
    static Gpt2Config xl() { return preset_("xl"); }
    size_t head_dim() const { return n_embd / n_head; }
    size_t ffn_dim() const { return 4 * n_embd; }
    b200nn_gpt2_config c() const {
        return b200nn_gpt2_config{(int32_t)n_layer, (int32_t)n_embd, (int32_t)n_head, (int32_t)vocab_size, (int32_t)n_positions, layer_norm_epsilon};
    }
    static Gpt2Config from_c(const b200nn_gpt2_config &c) {
        Gpt2Config g;
        g.n_layer = c.n_layer; g.n_embd = c.n_embd; g.n_head = c.n_head; g.vocab_size = c.vocab_size; g.n_positions = c.n_positions;
        g.layer_norm_epsilon = c.layer_norm_epsilon;
        return g;
    }

private:
    static Gpt2Config preset_(const char *name) {
        b200nn_gpt2_config c;
        const int32_t rc = b200nn_gpt2_config_preset(name, &c);
        if (rc != B200NN_OK) throw NnError(rc, std::string("unknown preset ") + name);
        return from_c(c);
    }
};

// TransformerLayerWeights / Gpt2Weights (GH/model.rs:112-154): host f32, dense weights in the checkpoint's
// Conv1D layout [in,out].
struct TransformerLayerWeights {
    std::vector<float> ln_1_weight, ln_1_bias, c_attn_weight, c_attn_bias, c_proj_weight, c_proj_bias;
    std::vector<float> ln_2_weight, ln_2_bias, mlp_fc_weight, mlp_fc_bias, mlp_proj_weight, mlp_proj_bias;
};
struct Gpt2Weights {
    std::vector<float> wte, wpe, ln_f_weight, ln_f_bias;
    std::vector<TransformerLayerWeights> layers;
};

// SimpleRng (gpt2.rs:1000-1023) and top_k_sample (gpt2.rs:1029-1058)
struct SimpleRng {
    uint64_t state;
    explicit SimpleRng(uint64_t seed) : state(b200nn_simple_rng_new(seed)) {}
    float next_f32() { return b200nn_simple_rng_next_f32(&state); }
};
inline uint32_t top_k_sample(const std::vector<float> &logits, size_t k, float temperature, SimpleRng &rng) {
    uint32_t tok = 0;
    const int32_t rc = b200nn_top_k_sample(logits.data(), logits.size(), k, temperature, &rng.state, &tok);
    if (rc != B200NN_OK) throw NnError(rc, "top_k_sample: empty logits or k = 0");
    return tok;
}

class Gpt2Model;
// KvCache (gpt2.rs:1064-1117): on the device, fp16, one slot per sequence of a batch.
class KvCache : public Owned<b200nn_kvcache, b200nn_kvcache_destroy> {
public:
    KvCache(const Gpt2Model &model, size_t batch, size_t capacity);
    size_t len() const { return b200nn_kvcache_len(h_); }
    bool is_empty() const { return len() == 0; }
    void reset() const { reg_->check(b200nn_kvcache_reset(h_)); }
};

// Gpt2Model (gpt2.rs:293-977) and Int4Gpt2Model (gpt2.rs:1343-1576): one class, the int4 form made by
// from_weights_int4 (what Int4Gpt2Model::from_weights does).
class Gpt2Model : public Owned<b200nn_gpt2, b200nn_gpt2_destroy> {
public:
    // Gpt2Model::from_weights (gpt2.rs:337-404)
    static Gpt2Model from_weights(const Gpt2Weights &w, const Gpt2Config &cfg, const Registry &reg, uint32_t flags = 0) {
        return create_(w, cfg, reg, 0, flags);
    }
    // Int4Gpt2Model::from_weights (gpt2.rs:1356-1436)
    static Gpt2Model from_weights_int4(const Gpt2Weights &w, const Gpt2Config &cfg, size_t group_size, const Registry &reg, uint32_t flags = 0) {
        if (group_size == 0) throw NnError(B200NN_ERR_ARG, "group_size must be non-zero");
        return create_(w, cfg, reg, group_size, flags);
    }
    const Gpt2Config &config() const { return cfg_; }
    size_t group_size() const { return group_; }
    size_t quantized_memory_bytes() const { return b200nn_gpt2_quantized_memory_bytes(h_); }

    // forward (gpt2.rs:481-499): logits [seq_len, vocab] of one sequence
    GpuTensor forward(const std::vector<uint32_t> &token_ids) const {
        b200nn_tensor *y = nullptr;
        const int32_t rc = b200nn_gpt2_forward(h_, token_ids.data(), token_ids.size(), &y);
        return out_(rc, y);
    }
    GpuTensor forward_auto_fused(const std::vector<uint32_t> &token_ids) const { return forward(token_ids); }
    GpuTensor forward_features(const std::vector<uint32_t> &token_ids) const {
        b200nn_tensor *y = nullptr;
        const int32_t rc = b200nn_gpt2_forward_features(h_, token_ids.data(), token_ids.size(), &y);
        return out_(rc, y);
    }
    // forward_cached (gpt2.rs:712-734): ids [batch,new_len] for the cache's batch; logits [batch*new_len, vocab]
    GpuTensor forward_cached(const std::vector<uint32_t> &ids, size_t new_len, KvCache &cache) const {
        b200nn_tensor *y = nullptr;
        const int32_t rc = b200nn_gpt2_forward_cached(h_, ids.data(), new_len, cache.handle(), &y);
        return out_(rc, y);
    }
    // generate / generate_cached (gpt2.rs:672-706, 740-783): greedy; the result holds the prompt and the new tokens
    std::vector<uint32_t> generate(const std::vector<uint32_t> &prompt, size_t max_new_tokens, uint32_t flags = B200NN_STOP_ON_EOS) const {
        std::vector<uint32_t> out(prompt.size() + max_new_tokens);
        size_t n = 0;
        reg_->check(b200nn_gpt2_generate(h_, prompt.data(), prompt.size(), max_new_tokens, flags, out.data(), &n));
        out.resize(n);
        return out;
    }
    std::vector<uint32_t> generate_cached(const std::vector<uint32_t> &prompt, size_t max_new_tokens, uint32_t flags = B200NN_STOP_ON_EOS) const {
        std::vector<uint32_t> out(prompt.size() + max_new_tokens);
        size_t n = 0;
        reg_->check(b200nn_gpt2_generate_cached(h_, prompt.data(), prompt.size(), max_new_tokens, flags, out.data(), &n));
        out.resize(n);
        return out;
    }
    // batched greedy decoding (added axis): prompts [batch,prompt_len] -> tokens [batch,prompt_len+max_new], lengths
    std::vector<uint32_t> generate_batch(const std::vector<uint32_t> &prompts, size_t batch, size_t prompt_len, size_t max_new_tokens,
                                         std::vector<size_t> *lens, uint32_t flags = 0) const {
        if (prompts.size() != batch * prompt_len) throw NnError(B200NN_ERR_SHAPE, "prompts must be [batch,prompt_len]");
        std::vector<uint32_t> out(batch * (prompt_len + max_new_tokens));
        lens->assign(batch, 0);
        reg_->check(b200nn_gpt2_generate_batch(h_, prompts.data(), batch, prompt_len, max_new_tokens, flags, out.data(), lens->data()));
        return out;
    }
    // generate_cached_sampling (gpt2.rs:933-977)
    std::vector<uint32_t> generate_cached_sampling(const std::vector<uint32_t> &prompt, size_t max_new_tokens, size_t top_k, float temperature,
                                                   SimpleRng &rng) const {
        std::vector<uint32_t> out(prompt.size() + max_new_tokens);
        size_t n = 0;
        reg_->check(b200nn_gpt2_generate_cached_sampling(h_, prompt.data(), prompt.size(), max_new_tokens, top_k, temperature, &rng.state,
                                                         out.data(), &n));
        out.resize(n);
        return out;
    }
    // forward_early_exit (gpt2.rs:797-830) -> (logits, blocks run)
    std::pair<GpuTensor, int32_t> forward_early_exit(const std::vector<uint32_t> &token_ids, float threshold) const {
        b200nn_tensor *y = nullptr;
        int32_t used = 0;
        reg_->check(b200nn_gpt2_forward_early_exit(h_, token_ids.data(), token_ids.size(), threshold, &y, &used));
        return {GpuTensor(reg_, y), used};
    }

private:
    static Gpt2Model create_(const Gpt2Weights &w, const Gpt2Config &cfg, const Registry &reg, size_t group, uint32_t flags) {
        if (w.layers.size() != cfg.n_layer) throw NnError(B200NN_ERR_SHAPE, "weights hold " + std::to_string(w.layers.size()) + " layers");
        std::vector<b200nn_gpt2_layer_weights> lw(cfg.n_layer);
        for (size_t i = 0; i < cfg.n_layer; ++i) {
            const TransformerLayerWeights &l = w.layers[i];
            lw[i] = b200nn_gpt2_layer_weights{l.ln_1_weight.data(), l.ln_1_bias.data(), l.c_attn_weight.data(), l.c_attn_bias.data(),
                                              l.c_proj_weight.data(), l.c_proj_bias.data(), l.ln_2_weight.data(), l.ln_2_bias.data(),
                                              l.mlp_fc_weight.data(), l.mlp_fc_bias.data(), l.mlp_proj_weight.data(), l.mlp_proj_bias.data()};
        }
        const b200nn_gpt2_weights cw{w.wte.data(), w.wpe.data(), w.ln_f_weight.data(), w.ln_f_bias.data(), lw.data()};
        const b200nn_gpt2_config cc = cfg.c();
        Gpt2Model m;
        m.reg_ = reg;
        m.cfg_ = cfg;
        m.group_ = group;
        reg->check(group ? b200nn_int4_gpt2_create(reg->ctx(), &cc, &cw, group, flags, &m.h_) : b200nn_gpt2_create(reg->ctx(), &cc, &cw, flags, &m.h_));
        return m;
    }
    Gpt2Config cfg_;
    size_t group_ = 0;
};
using Int4Gpt2Model = Gpt2Model;

inline KvCache::KvCache(const Gpt2Model &model, size_t batch, size_t capacity) {
    reg_ = model.registry();
    reg_->check(b200nn_kvcache_create(model.handle(), batch, capacity, &h_));
}

// TransformerBlock (gpt2.rs:98-289) and Int4TransformerBlock (gpt2.rs:1219-1339, group_size > 0): the twelve
// slices TransformerBlock::new takes, dense weights in Linear layout [out,in].
struct BlockWeights {
    std::vector<float> ln_1_weight, ln_1_bias, attn_qkv_weight, attn_qkv_bias, attn_out_weight, attn_out_bias;
    std::vector<float> ln_2_weight, ln_2_bias, ffn_up_weight, ffn_up_bias, ffn_down_weight, ffn_down_bias;
};
class TransformerBlock : public Owned<b200nn_block, b200nn_block_destroy> {
public:
    TransformerBlock(const BlockWeights &w, const Gpt2Config &cfg, const Registry &reg, size_t group_size = 0, uint32_t flags = 0) {
        const size_t d = cfg.n_embd;
        if (w.attn_qkv_weight.size() != 3 * d * d || w.attn_out_weight.size() != d * d || w.ffn_up_weight.size() != 4 * d * d ||
            w.ffn_down_weight.size() != 4 * d * d || w.ln_1_weight.size() != d || w.ln_2_weight.size() != d)
            throw NnError(B200NN_ERR_SHAPE, "block weights do not match n_embd");
        const b200nn_block_weights cw{w.ln_1_weight.data(), w.ln_1_bias.data(), w.attn_qkv_weight.data(), w.attn_qkv_bias.data(),
                                      w.attn_out_weight.data(), w.attn_out_bias.data(), w.ln_2_weight.data(), w.ln_2_bias.data(),
                                      w.ffn_up_weight.data(), w.ffn_up_bias.data(), w.ffn_down_weight.data(), w.ffn_down_bias.data()};
        const b200nn_gpt2_config cc = cfg.c();
        reg_ = reg;
        reg->check(group_size ? b200nn_int4_block_create(reg->ctx(), &cc, &cw, group_size, flags, &h_)
                              : b200nn_block_create(reg->ctx(), &cc, &cw, flags, &h_));
    }
    // forward / forward_auto_fused (gpt2.rs:172-243, 1299-1339): x [seq_len,d] of one sequence, causal
    GpuTensor forward(const GpuTensor &x) const {
        b200nn_tensor *y = nullptr;
        const int32_t rc = b200nn_block_forward(h_, x.handle(), &y);
        return out_(rc, y);
    }
    GpuTensor forward_auto_fused(const GpuTensor &x) const { return forward(x); }
};
using Int4TransformerBlock = TransformerBlock;

// The batched generate loop in pieces, state resident on the device (no counterpart in the reference, whose
// generate handles one sequence): prefill the prompts, run greedy steps without host synchronisation, read tokens.
class DecodeSession : public Owned<b200nn_session, b200nn_session_destroy> {
public:
    DecodeSession(const Gpt2Model &model, size_t batch, size_t capacity, uint32_t flags = 0) : batch_(batch), capacity_(capacity) {
        reg_ = model.registry();
        reg_->check(b200nn_session_create(model.handle(), batch, capacity, flags, &h_));
    }
    void prefill(const std::vector<uint32_t> &prompts, size_t prompt_len) const {
        if (prompts.size() != batch_ * prompt_len) throw NnError(B200NN_ERR_SHAPE, "prompts must be [batch,prompt_len]");
        reg_->check(b200nn_session_prefill(h_, prompts.data(), prompt_len));
    }
    void step(size_t n_steps) const { reg_->check(b200nn_session_step(h_, n_steps)); }
    size_t position() const { return b200nn_session_position(h_); }
    // tokens generated so far, [batch][generated]
    std::vector<std::vector<uint32_t>> tokens() const {
        std::vector<uint32_t> flat(batch_ * capacity_);
        size_t generated = 0;
        reg_->check(b200nn_session_tokens(h_, flat.data(), capacity_, &generated));
        std::vector<std::vector<uint32_t>> out(batch_);
        for (size_t b = 0; b < batch_; ++b) out[b].assign(flat.begin() + b * capacity_, flat.begin() + b * capacity_ + generated);
        return out;
    }

private:
    size_t batch_, capacity_;
};

}  // namespace b200nn
#endif  // B200NN_HPP
