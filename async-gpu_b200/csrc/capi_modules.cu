// extern "C" surface: Linear, Int4Linear, LayerNorm, Embedding, MultiHeadAttention, int4_matmul.
#include <algorithm>
#include <cstring>

#include "model.h"

static inline size_t last_dim(const b200nn_tensor *t) { return t->shape.empty() ? 0 : t->shape.back(); }
static inline size_t lead_rows(const b200nn_tensor *t) { return last_dim(t) ? t->numel / last_dim(t) : 0; }

static std::vector<size_t> out_shape(const b200nn_tensor *x, size_t n_out) {
    std::vector<size_t> s = x->shape;
    s.back() = n_out;
    return s;
}

// ---- Linear ---------------------------------------------------------------------------------
extern "C" int32_t b200nn_linear_create(b200nn_ctx *ctx, const float *weight, const float *bias, size_t in_features,
                                        size_t out_features, b200nn_linear **out) {
    if (!ctx || !weight || !out) return B200NN_ERR_ARG;
    auto l = std::unique_ptr<b200nn_linear>(new b200nn_linear());
    l->ctx = ctx;
    l->l.K = (int)in_features;
    l->l.N = (int)out_features;
    TRY(f32_weight_upload(ctx, weight, true, bias, in_features, out_features, &l->l.f)); // [out,in] (linear.rs:58-88)
    *out = l.release();
    return B200NN_OK;
}

extern "C" int32_t b200nn_linear_forward_fused(b200nn_linear *l, const b200nn_tensor *x, int32_t act, b200nn_tensor **y) {
    if (!l || !x || !y) return B200NN_ERR_ARG;
    b200nn_ctx *ctx = l->ctx;
    if (last_dim(x) != (size_t)l->l.K) // linear.rs:284-293
        return set_error(ctx, B200NN_ERR_SHAPE, "Linear: expected last dimension " + std::to_string(l->l.K) + ", got " +
                                                    std::to_string(last_dim(x)));
    if (act < B200NN_ACT_NONE || act > B200NN_ACT_SIGMOID) return set_error(ctx, B200NN_ERR_UNSUPPORTED, "unknown activation");
    b200nn_tensor *o = nullptr;
    TRY(tensor_alloc(ctx, out_shape(x, l->l.N), false, &o));
    Epilogue e;
    e.act = act;
    e.out = o->data();
    e.ldo = l->l.N;
    int rc = linear_forward(ctx, l->l, x->data(), false, (int)lead_rows(x), e);
    if (rc != B200NN_OK) { delete o; return rc; }
    *y = o;
    return B200NN_OK;
}
extern "C" int32_t b200nn_linear_forward(b200nn_linear *l, const b200nn_tensor *x, b200nn_tensor **y) {
    return b200nn_linear_forward_fused(l, x, B200NN_ACT_NONE, y);
}
extern "C" void b200nn_linear_destroy(b200nn_linear *l) { delete l; }

// ---- Int4Linear -----------------------------------------------------------------------------
extern "C" int32_t b200nn_int4_linear_create(b200nn_ctx *ctx, const uint32_t *packed, const float *scales,
                                             const float *bias, size_t in_features, size_t out_features, size_t group,
                                             b200nn_int4_linear **out) {
    if (!ctx || !packed || !scales || !out) return B200NN_ERR_ARG;
    auto l = std::unique_ptr<b200nn_int4_linear>(new b200nn_int4_linear());
    l->ctx = ctx;
    l->l.int4 = true;
    l->l.K = (int)in_features;
    l->l.N = (int)out_features;
    TRY(int4_weight_upload(ctx, packed, scales, bias, in_features, out_features, group, &l->l.q));
    *out = l.release();
    return B200NN_OK;
}

extern "C" int32_t b200nn_int4_linear_forward_dev(b200nn_int4_linear *l, const float *x_dev, size_t m, float *y_dev) {
    if (!l || !x_dev || !y_dev) return B200NN_ERR_ARG;
    b200nn_ctx *ctx = l->ctx;
    Epilogue e;
    e.out = y_dev;
    e.ldo = l->l.N;
    const Int4Weight &w = l->l.q;
    if (w.fast && (int)m > ctx->gemv_max_rows && int4_gemm_tc_supported(w, (int)m)) {
        // tensor-core path consumes fp16 activations
        size_t need = m * (size_t)w.K * sizeof(__half);
        if (!l->xh || l->xh->bytes < need) {
            if (ctx->capturing) return set_error(ctx, B200NN_ERR_UNSUPPORTED, "staging buffer would grow during capture");
            CK(ctx, cudaStreamSynchronize(ctx->stream));
            TRY(dev_alloc(ctx, need, &l->xh));
        }
        TRY(launch_f32_to_half(ctx, x_dev, (__half *)l->xh->p, m * (size_t)w.K));
        return linear_forward(ctx, l->l, l->xh->p, true, (int)m, e);
    }
    return linear_forward(ctx, l->l, x_dev, false, (int)m, e);
}

extern "C" int32_t b200nn_int4_linear_forward(b200nn_int4_linear *l, const b200nn_tensor *x, b200nn_tensor **y) {
    if (!l || !x || !y) return B200NN_ERR_ARG;
    b200nn_ctx *ctx = l->ctx;
    if (last_dim(x) != (size_t)l->l.K) // int4_linear.rs:74-79
        return set_error(ctx, B200NN_ERR_SHAPE, "Int4Linear: expected last dimension " + std::to_string(l->l.K) +
                                                    ", got " + std::to_string(last_dim(x)));
    b200nn_tensor *o = nullptr;
    TRY(tensor_alloc(ctx, out_shape(x, l->l.N), false, &o));
    int rc = b200nn_int4_linear_forward_dev(l, x->data(), lead_rows(x), o->data());
    if (rc != B200NN_OK) { delete o; return rc; }
    *y = o;
    return B200NN_OK;
}

extern "C" int32_t b200nn_int4_linear_forward_host(b200nn_int4_linear *l, const float *x_host, size_t m, float *y_host) {
    if (!l || !x_host || !y_host) return B200NN_ERR_ARG;
    b200nn_ctx *ctx = l->ctx;
    CK(ctx, cudaSetDevice(ctx->device));
    std::shared_ptr<DevBuf> xd, yd;
    TRY(dev_alloc(ctx, m * (size_t)l->l.K * 4, &xd));
    TRY(dev_alloc(ctx, m * (size_t)l->l.N * 4, &yd));
    CK(ctx, cudaMemcpyAsync(xd->p, x_host, m * (size_t)l->l.K * 4, cudaMemcpyHostToDevice, ctx->stream));
    TRY(b200nn_int4_linear_forward_dev(l, (const float *)xd->p, m, (float *)yd->p));
    CK(ctx, cudaMemcpyAsync(y_host, yd->p, m * (size_t)l->l.N * 4, cudaMemcpyDeviceToHost, ctx->stream));
    return stream_sync_check(ctx);
}

extern "C" size_t b200nn_int4_linear_memory_bytes(const b200nn_int4_linear *l) {
    return l ? l->l.q.memory_bytes() : 0; // packed u32 + f32 scales, as int4_linear.rs:136-146 counts
}
extern "C" void b200nn_int4_linear_destroy(b200nn_int4_linear *l) { delete l; }

// ops::int4_matmul (ops/gemm.rs:1186-1266): quantise B on the host on every call, then multiply.
extern "C" int32_t b200nn_int4_matmul(b200nn_ctx *ctx, const b200nn_tensor *a, const float *b_host, size_t k, size_t n,
                                      size_t group, b200nn_tensor **out) {
    if (!ctx || !a || !b_host || !out) return B200NN_ERR_ARG;
    if (last_dim(a) != k) return set_error(ctx, B200NN_ERR_SHAPE, "int4_matmul: A's last dimension must equal K");
    if (k % 8 != 0 || group == 0) return set_error(ctx, B200NN_ERR_SHAPE, "int4_matmul: K must be divisible by 8");
    std::vector<uint32_t> packed((k / 8) * n);
    std::vector<float> scales(((k + group - 1) / group) * n);
    TRY(host_quantize_weight_int4(b_host, k, n, group, packed.data(), scales.data()));
    b200nn_int4_linear *l = nullptr;
    TRY(b200nn_int4_linear_create(ctx, packed.data(), scales.data(), nullptr, k, n, group, &l));
    int rc = b200nn_int4_linear_forward(l, a, out);
    cudaStreamSynchronize(ctx->stream);
    b200nn_int4_linear_destroy(l);
    return rc;
}

// ---- LayerNorm ------------------------------------------------------------------------------
static int upload_f32(b200nn_ctx *ctx, const float *h, size_t n, std::shared_ptr<DevBuf> *out) {
    TRY(dev_alloc(ctx, n * 4, out));
    CK(ctx, cudaMemcpy((*out)->p, h, n * 4, cudaMemcpyHostToDevice));
    return B200NN_OK;
}

extern "C" int32_t b200nn_layernorm_create(b200nn_ctx *ctx, const float *gamma, const float *beta, size_t d, float eps,
                                           b200nn_layernorm **out) {
    if (!ctx || !gamma || !beta || !out || d == 0) return B200NN_ERR_ARG;
    auto ln = std::unique_ptr<b200nn_layernorm>(new b200nn_layernorm());
    ln->ctx = ctx;
    ln->d = d;
    ln->eps = eps;
    TRY(upload_f32(ctx, gamma, d, &ln->gamma));
    TRY(upload_f32(ctx, beta, d, &ln->beta));
    *out = ln.release();
    return B200NN_OK;
}
extern "C" int32_t b200nn_layernorm_forward(b200nn_layernorm *ln, const b200nn_tensor *x, b200nn_tensor **y) {
    if (!ln || !x || !y) return B200NN_ERR_ARG;
    b200nn_ctx *ctx = ln->ctx;
    if (last_dim(x) != ln->d) return set_error(ctx, B200NN_ERR_SHAPE, "LayerNorm: last dimension differs from gamma");
    b200nn_tensor *o = nullptr;
    TRY(tensor_alloc(ctx, x->shape, false, &o));
    int rc = launch_layernorm(ctx, x->data(), nullptr, nullptr, (const float *)ln->gamma->p, (const float *)ln->beta->p,
                              ln->eps, (int)lead_rows(x), (int)ln->d, o->data(), false);
    if (rc != B200NN_OK) { delete o; return rc; }
    *y = o;
    return B200NN_OK;
}
extern "C" void b200nn_layernorm_destroy(b200nn_layernorm *ln) { delete ln; }

// ---- Embedding ------------------------------------------------------------------------------
extern "C" int32_t b200nn_embedding_create(b200nn_ctx *ctx, const float *wte, const float *wpe, size_t vocab,
                                           size_t max_seq, size_t d, b200nn_embedding **out) {
    if (!ctx || !wte || !wpe || !out || !vocab || !max_seq || !d) return B200NN_ERR_ARG;
    auto e = std::unique_ptr<b200nn_embedding>(new b200nn_embedding());
    e->ctx = ctx;
    e->vocab = vocab;
    e->max_seq = max_seq;
    e->d = d;
    TRY(upload_f32(ctx, wte, vocab * d, &e->wte));
    TRY(upload_f32(ctx, wpe, max_seq * d, &e->wpe));
    *out = e.release();
    return B200NN_OK;
}
extern "C" int32_t b200nn_embedding_forward_tokens(b200nn_embedding *e, const uint32_t *ids_host, size_t n,
                                                   size_t pos_offset, b200nn_tensor **out) {
    if (!e || !ids_host || !out) return B200NN_ERR_ARG;
    b200nn_ctx *ctx = e->ctx;
    if (n == 0) return set_error(ctx, B200NN_ERR_SHAPE, "embedding: no tokens");
    if (pos_offset + n > e->max_seq) return set_error(ctx, B200NN_ERR_DIM, "embedding: position exceeds max_seq");
    for (size_t i = 0; i < n; ++i)
        if (ids_host[i] >= e->vocab) return set_error(ctx, B200NN_ERR_DIM, "embedding: token id out of range");
    std::shared_ptr<DevBuf> ids;
    TRY(dev_alloc(ctx, n * 4, &ids));
    CK(ctx, cudaMemcpyAsync(ids->p, ids_host, n * 4, cudaMemcpyHostToDevice, ctx->stream));
    b200nn_tensor *o = nullptr;
    TRY(tensor_alloc(ctx, {n, e->d}, false, &o));
    int rc = launch_embedding(ctx, (const uint32_t *)ids->p, (const float *)e->wte->p, (const float *)e->wpe->p, (int)n,
                              (int)e->d, (int)n, nullptr, (int)pos_offset, (int)e->vocab, (int)e->max_seq, o->data());
    if (rc == B200NN_OK && cudaStreamSynchronize(ctx->stream) != cudaSuccess) rc = B200NN_ERR_CUDA;
    if (rc != B200NN_OK) { delete o; return rc; }
    *out = o;
    return B200NN_OK;
}
extern "C" void b200nn_embedding_destroy(b200nn_embedding *e) { delete e; }

// ---- MultiHeadAttention ---------------------------------------------------------------------
extern "C" int32_t b200nn_attention_create(b200nn_ctx *ctx, const float *qkv_weight, const float *qkv_bias,
                                           const float *out_weight, const float *out_bias, size_t n_embd,
                                           size_t n_heads, b200nn_attention **out) {
    if (!ctx || !qkv_weight || !qkv_bias || !out_weight || !out_bias || !out) return B200NN_ERR_ARG;
    if (n_heads == 0 || n_embd % n_heads != 0 || n_embd / n_heads != 64)
        return set_error(ctx, B200NN_ERR_UNSUPPORTED, "MultiHeadAttention: d_head must be 64");
    auto a = std::unique_ptr<b200nn_attention>(new b200nn_attention());
    a->ctx = ctx;
    a->d = n_embd;
    a->n_heads = n_heads;
    a->qkv.K = (int)n_embd; a->qkv.N = (int)(3 * n_embd);
    a->proj.K = (int)n_embd; a->proj.N = (int)n_embd;
    TRY(f32_weight_upload(ctx, qkv_weight, true, qkv_bias, n_embd, 3 * n_embd, &a->qkv.f));
    TRY(f32_weight_upload(ctx, out_weight, true, out_bias, n_embd, n_embd, &a->proj.f));
    *out = a.release();
    return B200NN_OK;
}

// Int4MultiHeadAttention::new (gpt2.rs:1141-1188): the same layer with both projections quantised at
// construction (weights given [out,in], quantised as [in,out] per group along K).
extern "C" int32_t b200nn_int4_attention_create(b200nn_ctx *ctx, const float *qkv_weight, const float *qkv_bias,
                                                const float *out_weight, const float *out_bias, size_t n_embd,
                                                size_t n_heads, size_t group_size, b200nn_attention **out) {
    if (!ctx || !qkv_weight || !qkv_bias || !out_weight || !out_bias || !out) return B200NN_ERR_ARG;
    if (n_heads == 0 || n_embd % n_heads != 0 || n_embd / n_heads != 64)
        return set_error(ctx, B200NN_ERR_UNSUPPORTED, "Int4MultiHeadAttention: d_head must be 64");
    if (group_size == 0) return set_error(ctx, B200NN_ERR_SHAPE, "group_size must be positive");
    auto a = std::unique_ptr<b200nn_attention>(new b200nn_attention());
    a->ctx = ctx;
    a->d = n_embd;
    a->n_heads = n_heads;
    const float *ws[2] = {qkv_weight, out_weight}, *bs[2] = {qkv_bias, out_bias};
    LinearAny *ls[2] = {&a->qkv, &a->proj};
    for (int i = 0; i < 2; ++i) {
        const size_t K = n_embd, N = i ? n_embd : 3 * n_embd;
        ls[i]->K = (int)K;
        ls[i]->N = (int)N;
        ls[i]->int4 = true;
        std::vector<float> w_kn(K * N);
        for (size_t o = 0; o < N; ++o)
            for (size_t k = 0; k < K; ++k) w_kn[k * N + o] = ws[i][o * K + k];
        std::vector<uint32_t> packed((K / 8) * N);
        std::vector<float> scales(((K + group_size - 1) / group_size) * N);
        int rc = host_quantize_weight_int4(w_kn.data(), K, N, group_size, packed.data(), scales.data());
        if (rc != B200NN_OK) return set_error(ctx, rc, "quantize_weight_int4: K must be divisible by 8");
        TRY(int4_weight_upload(ctx, packed.data(), scales.data(), bs[i], K, N, group_size, &ls[i]->q));
    }
    *out = a.release();
    return B200NN_OK;
}

// x [new_len,d] at positions past..; cache_k/v (optional, host f32 [H][past*64]) precede the new rows.
static int attention_run(b200nn_attention *a, const b200nn_tensor *x, const float *cached_k, const float *cached_v,
                         size_t past, b200nn_tensor **y, float *new_k_out, float *new_v_out) {
    b200nn_ctx *ctx = a->ctx;
    const size_t d = a->d, H = a->n_heads, n = lead_rows(x), cap = past + n;
    if (last_dim(x) != d || n == 0) return set_error(ctx, B200NN_ERR_SHAPE, "MultiHeadAttention: expected [seq, n_embd]");
    std::shared_ptr<DevBuf> kc, vc, q, att, tmp;
    TRY(dev_alloc(ctx, H * cap * 64 * sizeof(__half), &kc));
    TRY(dev_alloc(ctx, H * cap * 64 * sizeof(__half), &vc));
    if (past) {
        TRY(dev_alloc(ctx, H * past * 64 * 4, &tmp));
        CK(ctx, cudaMemcpyAsync(tmp->p, cached_k, H * past * 64 * 4, cudaMemcpyHostToDevice, ctx->stream));
        TRY(launch_pack_kv(ctx, (const float *)tmp->p, (int)H, (int)past, (int)cap, (__half *)kc->p));
        CK(ctx, cudaStreamSynchronize(ctx->stream));
        CK(ctx, cudaMemcpyAsync(tmp->p, cached_v, H * past * 64 * 4, cudaMemcpyHostToDevice, ctx->stream));
        TRY(launch_pack_kv(ctx, (const float *)tmp->p, (int)H, (int)past, (int)cap, (__half *)vc->p));
    }
    TRY(dev_alloc(ctx, n * d * 4, &q));
    TRY(dev_alloc(ctx, n * d * 4, &att));
    // the int4 layer with more rows than the GEMV serves: fp16 activations, tensor-core GEMMs and attention
    const bool half = a->qkv.int4 && (int)n > ctx->gemv_max_rows && int4_gemm_tc_supported(a->qkv.q, (int)n) &&
                      int4_gemm_tc_supported(a->proj.q, (int)n);
    std::shared_ptr<DevBuf> xh;
    const void *xin = x->data();
    if (half) {
        TRY(dev_alloc(ctx, n * d * sizeof(__half), &xh));
        TRY(launch_f32_to_half(ctx, x->data(), (__half *)xh->p, n * d));
        xin = xh->p;
    }
    Epilogue e;
    e.mode = EPI_QKV;
    e.out = q->p;
    e.out_half = half;
    e.ldo = (int)d;
    e.kc = (__half *)kc->p;
    e.vc = (__half *)vc->p;
    e.d_model = (int)d;
    e.n_head = (int)H;
    e.rows_per_seq = (int)n;
    e.cap = (int)cap;
    e.pos_off = (int)past;
    TRY(linear_forward(ctx, a->qkv, xin, half, (int)n, e));
    if (n == 1)
        TRY(launch_decode_attention(ctx, q->p, half, (int)d, (const __half *)kc->p, (const __half *)vc->p, 1, (int)H,
                                    (int)cap, nullptr, (int)past, att->p, half, (int)cap));
    else
        TRY(launch_prefill_attention(ctx, q->p, half, (int)d, (const __half *)kc->p, (const __half *)vc->p, 1, (int)H,
                                     (int)cap, (int)n, (int)past, att->p, half));
    b200nn_tensor *o = nullptr;
    TRY(tensor_alloc(ctx, {n, d}, false, &o));
    Epilogue p;
    p.out = o->data();
    p.ldo = (int)d;
    int rc = linear_forward(ctx, a->proj, att->p, half, (int)n, p);
    if (rc == B200NN_OK && (new_k_out || new_v_out)) {
        // new K,V rows back to the host as f32 [H][n*64] (values as held in the fp16 cache)
        std::shared_ptr<DevBuf> f;
        rc = dev_alloc(ctx, H * cap * 64 * 4, &f);
        for (int which = 0; which < 2 && rc == B200NN_OK; ++which) {
            float *dst = which ? new_v_out : new_k_out;
            if (!dst) continue;
            rc = launch_half_to_f32(ctx, (const __half *)(which ? vc->p : kc->p), (float *)f->p, H * cap * 64);
            if (rc != B200NN_OK) break;
            cudaError_t ce = cudaMemcpy2DAsync(dst, n * 64 * 4, (const float *)f->p + past * 64, cap * 64 * 4, n * 64 * 4,
                                               H, cudaMemcpyDeviceToHost, ctx->stream);
            if (ce == cudaSuccess) ce = cudaStreamSynchronize(ctx->stream);
            if (ce != cudaSuccess) rc = set_cuda_error(ctx, ce, "attention new K/V copy");
        }
    }
    if (rc == B200NN_OK) rc = stream_sync_check(ctx); // new K/V rows went to the host: report a device-side abort
    if (rc != B200NN_OK) { delete o; return rc; }
    *y = o;
    return B200NN_OK;
}

extern "C" int32_t b200nn_attention_forward_causal(b200nn_attention *a, const b200nn_tensor *x, b200nn_tensor **y) {
    if (!a || !x || !y) return B200NN_ERR_ARG;
    return attention_run(a, x, nullptr, nullptr, 0, y, nullptr, nullptr);
}
extern "C" int32_t b200nn_attention_forward_cached(b200nn_attention *a, const b200nn_tensor *x, const float *cached_k,
                                                   const float *cached_v, size_t kv_len, b200nn_tensor **y,
                                                   float *new_k_out, float *new_v_out) {
    if (!a || !x || !y) return B200NN_ERR_ARG;
    if (kv_len && (!cached_k || !cached_v)) return B200NN_ERR_ARG;
    return attention_run(a, x, cached_k, cached_v, kv_len, y, new_k_out, new_v_out);
}
extern "C" void b200nn_attention_destroy(b200nn_attention *a) { delete a; }
