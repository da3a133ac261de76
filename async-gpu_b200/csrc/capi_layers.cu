// extern "C" surface: stateless ops and the single layers of the `nn` module.
#include <algorithm>
#include <cstring>

#include "model.h"

static inline size_t last_dim(const b200nn_tensor *t) { return t->shape.empty() ? 0 : t->shape.back(); }
static inline size_t lead_rows(const b200nn_tensor *t) { return last_dim(t) ? t->numel / last_dim(t) : 0; }

// ---------------------------------------------------------------------------------------------
// ops
// ---------------------------------------------------------------------------------------------
extern "C" int32_t b200nn_layer_norm(b200nn_ctx *ctx, const b200nn_tensor *x, const b200nn_tensor *gamma,
                                     const b200nn_tensor *beta, float eps, b200nn_tensor **out) {
    if (!ctx || !x || !gamma || !beta || !out) return B200NN_ERR_ARG;
    size_t d = last_dim(x);
    if (gamma->numel != d || beta->numel != d)
        return set_error(ctx, B200NN_ERR_SHAPE, "layer_norm: gamma/beta must have the input's last dimension");
    b200nn_tensor *y = nullptr;
    TRY(tensor_alloc(ctx, x->shape, false, &y));
    int rc = launch_layernorm(ctx, x->data(), nullptr, nullptr, gamma->data(), beta->data(), eps, (int)lead_rows(x),
                              (int)d, y->data(), false);
    if (rc != B200NN_OK) { delete y; return rc; }
    *out = y;
    return B200NN_OK;
}

extern "C" int32_t b200nn_layer_norm_residual_dual(b200nn_ctx *ctx, const b200nn_tensor *a, const b200nn_tensor *b,
                                                   const b200nn_tensor *gamma, const b200nn_tensor *beta, float eps,
                                                   b200nn_tensor **sum_out, b200nn_tensor **norm_out) {
    if (!ctx || !a || !b || !gamma || !beta || !sum_out || !norm_out) return B200NN_ERR_ARG;
    size_t d = last_dim(a);
    if (a->shape != b->shape) return set_error(ctx, B200NN_ERR_SHAPE, "layer_norm_residual: input shapes differ");
    if (gamma->numel != d || beta->numel != d)
        return set_error(ctx, B200NN_ERR_SHAPE, "layer_norm_residual: gamma/beta must have the last dimension");
    b200nn_tensor *s = nullptr, *y = nullptr;
    TRY(tensor_alloc(ctx, a->shape, false, &s));
    int rc = tensor_alloc(ctx, a->shape, false, &y);
    if (rc == B200NN_OK)
        rc = launch_layernorm(ctx, a->data(), b->data(), s->data(), gamma->data(), beta->data(), eps,
                              (int)lead_rows(a), (int)d, y->data(), false);
    if (rc != B200NN_OK) { delete s; delete y; return rc; }
    *sum_out = s;
    *norm_out = y;
    return B200NN_OK;
}

extern "C" int32_t b200nn_activation(b200nn_ctx *ctx, const b200nn_tensor *x, int32_t act, b200nn_tensor **out) {
    if (!ctx || !x || !out) return B200NN_ERR_ARG;
    if (act < B200NN_ACT_NONE || act > B200NN_ACT_SIGMOID) return set_error(ctx, B200NN_ERR_UNSUPPORTED, "unknown activation");
    b200nn_tensor *y = nullptr;
    TRY(tensor_alloc(ctx, x->shape, false, &y));
    int rc = launch_activation(ctx, x->data(), y->data(), x->numel, act);
    if (rc != B200NN_OK) { delete y; return rc; }
    *out = y;
    return B200NN_OK;
}

// ops::matmul (ops/gemm.rs:20-36): [M,K] x [K,N]; b is used where it lies as a [K,N] weight of the f32 FMA kernels.
extern "C" int32_t b200nn_matmul(b200nn_ctx *ctx, const b200nn_tensor *a, const b200nn_tensor *b, b200nn_tensor **out) {
    if (!ctx || !a || !b || !out) return B200NN_ERR_ARG;
    if (a->shape.size() != 2 || b->shape.size() != 2)
        return set_error(ctx, B200NN_ERR_SHAPE, "matmul: expected 2D tensors");
    if (a->shape[1] != b->shape[0])
        return set_error(ctx, B200NN_ERR_SHAPE, "matmul: a is [" + std::to_string(a->shape[0]) + "," + std::to_string(a->shape[1]) +
                                                    "], b is [" + std::to_string(b->shape[0]) + "," + std::to_string(b->shape[1]) + "]");
    const size_t M = a->shape[0], K = a->shape[1], N = b->shape[1];
    b200nn_tensor *y = nullptr;
    TRY(tensor_alloc(ctx, {M, N}, M == 0 || N == 0 || K == 0, &y));
    if (M && N && K) {
        F32Weight w;
        w.K = (int)K;
        w.N = (int)N;
        w.w_kn = b->buf; // shared, not copied; no fp16 copy: the FMA kernels run
        Epilogue e;
        e.out = y->data();
        e.ldo = (int)N;
        int rc = launch_f32_linear(ctx, w, a->data(), false, (int)M, e);
        if (rc != B200NN_OK) { delete y; return rc; }
    }
    *out = y;
    return B200NN_OK;
}

extern "C" int32_t b200nn_bias_add(b200nn_ctx *ctx, b200nn_tensor *data, const b200nn_tensor *bias) {
    if (!ctx || !data || !bias) return B200NN_ERR_ARG;
    if (bias->numel == 0 || last_dim(data) != bias->numel)
        return set_error(ctx, B200NN_ERR_SHAPE, "bias_add: bias length must equal the last dimension");
    return launch_bias_add(ctx, data->data(), bias->data(), data->numel, (int)bias->numel);
}

extern "C" int32_t b200nn_elementwise_add(b200nn_ctx *ctx, b200nn_tensor *a, const b200nn_tensor *b) {
    if (!ctx || !a || !b) return B200NN_ERR_ARG;
    if (a->numel != b->numel) return set_error(ctx, B200NN_ERR_SHAPE, "elementwise_add: element counts differ");
    return launch_add(ctx, a->data(), b->data(), a->numel);
}

extern "C" int32_t b200nn_split_qkv(b200nn_ctx *ctx, const b200nn_tensor *qkv, size_t seq_len, size_t n_heads,
                                    size_t d_head, b200nn_tensor **q, b200nn_tensor **k, b200nn_tensor **v) {
    if (!ctx || !qkv || !q || !k || !v) return B200NN_ERR_ARG;
    if (qkv->numel != seq_len * 3 * n_heads * d_head)
        return set_error(ctx, B200NN_ERR_SHAPE, "split_qkv: expected [seq, 3*n_heads*d_head]");
    b200nn_tensor *t[3] = {nullptr, nullptr, nullptr};
    for (int i = 0; i < 3; ++i) {
        int rc = tensor_alloc(ctx, {n_heads, seq_len, d_head}, false, &t[i]);
        if (rc != B200NN_OK) { for (auto p : t) delete p; return rc; }
    }
    int rc = launch_split_qkv(ctx, qkv->data(), (int)seq_len, (int)n_heads, (int)d_head, t[0]->data(), t[1]->data(),
                              t[2]->data());
    if (rc != B200NN_OK) { for (auto p : t) delete p; return rc; }
    *q = t[0]; *k = t[1]; *v = t[2];
    return B200NN_OK;
}

extern "C" int32_t b200nn_concat_heads(b200nn_ctx *ctx, const b200nn_tensor *heads, size_t seq_len, size_t n_heads,
                                       size_t d_head, b200nn_tensor **out) {
    if (!ctx || !heads || !out) return B200NN_ERR_ARG;
    if (heads->numel != seq_len * n_heads * d_head)
        return set_error(ctx, B200NN_ERR_SHAPE, "concat_heads: expected [n_heads, seq, d_head]");
    b200nn_tensor *y = nullptr;
    TRY(tensor_alloc(ctx, {seq_len, n_heads * d_head}, false, &y));
    int rc = launch_concat_heads(ctx, heads->data(), (int)seq_len, (int)n_heads, (int)d_head, y->data());
    if (rc != B200NN_OK) { delete y; return rc; }
    *out = y;
    return B200NN_OK;
}

// q [H,nq,64], k/v [H,kv_len,64] f32 -> out [H,nq,64]; query i sits at absolute position past+i.
static int attention_op(b200nn_ctx *ctx, const float *q, const float *k, const float *v, size_t H, size_t nq,
                        size_t kv_len, size_t past, b200nn_tensor **out) {
    std::shared_ptr<DevBuf> kc, vc, qrow, orow;
    TRY(dev_alloc(ctx, H * kv_len * 64 * sizeof(__half), &kc));
    TRY(dev_alloc(ctx, H * kv_len * 64 * sizeof(__half), &vc));
    TRY(launch_pack_kv(ctx, k, (int)H, (int)kv_len, (int)kv_len, (__half *)kc->p));
    TRY(launch_pack_kv(ctx, v, (int)H, (int)kv_len, (int)kv_len, (__half *)vc->p));
    // the kernels take token-major rows [nq, H*64]
    TRY(dev_alloc(ctx, nq * H * 64 * 4, &qrow));
    TRY(dev_alloc(ctx, nq * H * 64 * 4, &orow));
    TRY(launch_concat_heads(ctx, q, (int)nq, (int)H, 64, (float *)qrow->p));
    if (nq == 1)
        TRY(launch_decode_attention(ctx, qrow->p, false, (int)(H * 64), (const __half *)kc->p, (const __half *)vc->p, 1,
                                    (int)H, (int)kv_len, nullptr, (int)past, orow->p, false, (int)kv_len));
    else
        TRY(launch_prefill_attention(ctx, qrow->p, false, (int)(H * 64), (const __half *)kc->p, (const __half *)vc->p, 1,
                                     (int)H, (int)kv_len, (int)nq, (int)past, orow->p, false));
    b200nn_tensor *y = nullptr;
    TRY(tensor_alloc(ctx, {H, nq, 64}, false, &y));
    // [nq, H*64] -> [H, nq, 64]: the Q part of split_qkv on a [nq, 3d] view is the same permutation;
    // reuse concat_heads with the roles of seq and heads exchanged
    int rc = launch_concat_heads(ctx, (const float *)orow->p, (int)H, (int)nq, 64, y->data());
    if (rc == B200NN_OK) {
        cudaError_t e = cudaStreamSynchronize(ctx->stream); // temporaries are freed on return
        if (e != cudaSuccess) rc = set_cuda_error(ctx, e, "attention_op");
    }
    if (rc != B200NN_OK) { delete y; return rc; }
    *out = y;
    return B200NN_OK;
}

extern "C" int32_t b200nn_multi_head_flash_attention(b200nn_ctx *ctx, const b200nn_tensor *q, const b200nn_tensor *k,
                                                     const b200nn_tensor *v, size_t seq_len, size_t n_heads,
                                                     size_t d_head, int32_t causal, b200nn_tensor **out) {
    if (!ctx || !q || !k || !v || !out) return B200NN_ERR_ARG;
    if (d_head != 64) return set_error(ctx, B200NN_ERR_UNSUPPORTED, "attention: d_head must be 64");
    if (!causal) return set_error(ctx, B200NN_ERR_UNSUPPORTED, "attention: only the causal form is on this path");
    size_t n = n_heads * seq_len * 64;
    if (q->numel != n || k->numel != n || v->numel != n)
        return set_error(ctx, B200NN_ERR_SHAPE, "attention: expected q,k,v of [n_heads, seq, 64]");
    if (seq_len == 0) return set_error(ctx, B200NN_ERR_SHAPE, "attention: empty sequence");
    return attention_op(ctx, q->data(), k->data(), v->data(), n_heads, seq_len, seq_len, 0, out);
}

extern "C" int32_t b200nn_attention_kv(b200nn_ctx *ctx, const b200nn_tensor *q, const b200nn_tensor *k,
                                       const b200nn_tensor *v, int32_t causal, size_t q_offset, b200nn_tensor **out) {
    if (!ctx || !q || !k || !v || !out) return B200NN_ERR_ARG;
    if (last_dim(q) != 64 || last_dim(k) != 64 || last_dim(v) != 64)
        return set_error(ctx, B200NN_ERR_UNSUPPORTED, "attention_kv: d_head must be 64");
    size_t q_len = lead_rows(q), kv_len = lead_rows(k);
    if (lead_rows(v) != kv_len || q_len == 0 || kv_len == 0)
        return set_error(ctx, B200NN_ERR_SHAPE, "attention_kv: k and v must both be [kv_len, 64]");
    // causal: query i sees keys j <= i + q_offset (compute_transformer.rs:1076-1288); non-causal sees all
    size_t past = causal ? q_offset : kv_len - 1;
    if (causal && q_offset + q_len > kv_len)
        return set_error(ctx, B200NN_ERR_SHAPE, "attention_kv: q_offset + q_len exceeds kv_len");
    if (!causal && q_len != 1)
        return set_error(ctx, B200NN_ERR_UNSUPPORTED, "attention_kv: non-causal form supports one query row");
    b200nn_tensor *y3 = nullptr;
    TRY(attention_op(ctx, q->data(), k->data(), v->data(), 1, q_len, kv_len, past, &y3));
    y3->shape = {q_len, 64};
    *out = y3;
    return B200NN_OK;
}

// ---- batched attention on caller-owned fp16 device buffers ------------------------------------
// The kernels of the model path as stand-alone operations: q and out are token-major rows
// [batch*rows, n_heads*64] fp16, the caches fp16 [batch][n_heads][capacity][64] with the new positions
// already appended.  Stream-ordered on the context's stream; nothing is copied or allocated
// except the decode kernel's split scratch on first use.
extern "C" int32_t b200nn_prefill_attention_f16(b200nn_ctx *ctx, const void *q_dev, const void *k_cache_dev,
                                                const void *v_cache_dev, int32_t batch, int32_t n_heads, int32_t capacity,
                                                int32_t seq_len, int32_t past, void *out_dev) {
    if (!ctx || !q_dev || !k_cache_dev || !v_cache_dev || !out_dev) return B200NN_ERR_ARG;
    if (batch <= 0 || n_heads <= 0 || seq_len <= 0 || past < 0 || past + seq_len > capacity)
        return set_error(ctx, B200NN_ERR_SHAPE, "prefill_attention_f16: need batch, heads, seq_len > 0 and past + seq_len <= capacity");
    if (((uintptr_t)q_dev | (uintptr_t)k_cache_dev | (uintptr_t)v_cache_dev | (uintptr_t)out_dev) & 15)
        return set_error(ctx, B200NN_ERR_ARG, "prefill_attention_f16: buffers must be 16-byte aligned");
    CK(ctx, cudaSetDevice(ctx->device));
    return launch_prefill_attention(ctx, q_dev, true, n_heads * 64, (const __half *)k_cache_dev, (const __half *)v_cache_dev,
                                    batch, n_heads, capacity, seq_len, past, out_dev, true);
}

extern "C" int32_t b200nn_decode_attention_f16(b200nn_ctx *ctx, const void *q_dev, const void *k_cache_dev,
                                               const void *v_cache_dev, int32_t batch, int32_t n_heads, int32_t capacity,
                                               int32_t ctx_len, void *out_dev) {
    if (!ctx || !q_dev || !k_cache_dev || !v_cache_dev || !out_dev) return B200NN_ERR_ARG;
    if (batch <= 0 || n_heads <= 0 || ctx_len <= 0 || ctx_len > capacity)
        return set_error(ctx, B200NN_ERR_SHAPE, "decode_attention_f16: need batch, heads > 0 and 1 <= ctx_len <= capacity");
    if (((uintptr_t)q_dev | (uintptr_t)k_cache_dev | (uintptr_t)v_cache_dev | (uintptr_t)out_dev) & 15)
        return set_error(ctx, B200NN_ERR_ARG, "decode_attention_f16: buffers must be 16-byte aligned");
    CK(ctx, cudaSetDevice(ctx->device));
    return launch_decode_attention(ctx, q_dev, true, n_heads * 64, (const __half *)k_cache_dev, (const __half *)v_cache_dev,
                                   batch, n_heads, capacity, nullptr, ctx_len - 1, out_dev, true, capacity);
}
