// TransformerBlock / Int4TransformerBlock as public handles (gpt2.rs:98-289, 1219-1339): one pre-LN
// GPT-2 block built from its twelve weight slices, with forward (causal over the given rows) and
// forward_cached (new rows on top of cached K/V handed in and out as host vectors, as the reference's
// per-block cache does).  The block is a one-layer model without embeddings or head, so it runs through
// the same kernels as the models (run_blocks_range).
#include <algorithm>
#include <cstring>

#include "model.h"

struct b200nn_block {
    b200nn_gpt2 m; // cfg.n_layer == 1; wte / wpe / ln_f / lm_head unused
};

namespace {

// Linear layout [out,in] (what TransformerBlock::new takes) -> checkpoint layout [in,out]
std::vector<float> to_in_out(const float *w, size_t out, size_t in) {
    std::vector<float> t(in * out);
    for (size_t o = 0; o < out; ++o)
        for (size_t i = 0; i < in; ++i) t[i * out + o] = w[o * in + i];
    return t;
}

int upload_vec(b200nn_ctx *ctx, const float *h, size_t n, std::shared_ptr<DevBuf> *out) {
    TRY(dev_alloc(ctx, n * sizeof(float), out));
    CK(ctx, cudaMemcpy((*out)->p, h, n * sizeof(float), cudaMemcpyHostToDevice));
    return B200NN_OK;
}

int make_linear(b200nn_ctx *ctx, const float *w_out_in, const float *bias, size_t K, size_t N, bool int4, size_t group,
                LinearAny *out) {
    out->K = (int)K;
    out->N = (int)N;
    out->int4 = int4;
    if (!int4) return f32_weight_upload(ctx, w_out_in, true, bias, K, N, &out->f);
    // Int4TransformerBlock::new quantises the transposed weight [in,out] (gpt2.rs:1248-1262)
    std::vector<float> w_kn = to_in_out(w_out_in, N, K);
    std::vector<uint32_t> packed((K / 8) * N);
    std::vector<float> scales(((K + group - 1) / group) * N);
    int rc = host_quantize_weight_int4(w_kn.data(), K, N, group, packed.data(), scales.data());
    if (rc != B200NN_OK) return set_error(ctx, rc, "quantize_weight_int4: K must be divisible by 8");
    return int4_weight_upload(ctx, packed.data(), scales.data(), bias, K, N, group, &out->q);
}

int block_create(b200nn_ctx *ctx, const b200nn_gpt2_config *cfg, const b200nn_block_weights *w, bool int4, size_t group,
                 uint32_t flags, b200nn_block **out) {
    if (!ctx || !cfg || !w || !out) return B200NN_ERR_ARG;
    const float *all[12] = {w->ln_1_weight, w->ln_1_bias, w->attn_qkv_weight, w->attn_qkv_bias, w->attn_out_weight,
                            w->attn_out_bias, w->ln_2_weight, w->ln_2_bias, w->ffn_up_weight, w->ffn_up_bias,
                            w->ffn_down_weight, w->ffn_down_bias};
    for (const float *p : all)
        if (!p) return set_error(ctx, B200NN_ERR_ARG, "TransformerBlock: null weight slice");
    if (cfg->n_embd <= 0 || cfg->n_head <= 0 || cfg->n_embd % cfg->n_head != 0 || cfg->n_embd / cfg->n_head != 64)
        return set_error(ctx, B200NN_ERR_UNSUPPORTED, "head_dim must be 64 (n_embd / n_head)");
    if (int4 && group == 0) return set_error(ctx, B200NN_ERR_SHAPE, "group_size must be positive");
    CK(ctx, cudaSetDevice(ctx->device));
    auto b = std::unique_ptr<b200nn_block>(new b200nn_block());
    b200nn_gpt2 &m = b->m;
    m.ctx = ctx;
    m.cfg = *cfg;
    m.cfg.n_layer = 1;
    m.flags = flags;
    m.int4 = int4;
    m.group = group;
    const size_t d = cfg->n_embd, ffn = 4 * d;
    m.blocks.resize(1);
    BlockW &bw = m.blocks[0];
    TRY(upload_vec(ctx, w->ln_1_weight, d, &bw.ln1_g));
    TRY(upload_vec(ctx, w->ln_1_bias, d, &bw.ln1_b));
    TRY(upload_vec(ctx, w->ln_2_weight, d, &bw.ln2_g));
    TRY(upload_vec(ctx, w->ln_2_bias, d, &bw.ln2_b));
    TRY(make_linear(ctx, w->attn_qkv_weight, w->attn_qkv_bias, d, 3 * d, int4, group, &bw.qkv));
    TRY(make_linear(ctx, w->attn_out_weight, w->attn_out_bias, d, d, int4, group, &bw.proj));
    TRY(make_linear(ctx, w->ffn_up_weight, w->ffn_up_bias, d, ffn, int4, group, &bw.fc));
    TRY(make_linear(ctx, w->ffn_down_weight, w->ffn_down_bias, ffn, d, int4, group, &bw.fcproj));
    *out = b.release();
    return B200NN_OK;
}

// x [n,d] at positions past..past+n-1 of one sequence; cached_k / cached_v host f32 [H][past*64].
int block_run(b200nn_block *b, const b200nn_tensor *x, const float *cached_k, const float *cached_v, size_t past,
              b200nn_tensor **y, float *new_k_out, float *new_v_out) {
    b200nn_gpt2 *m = &b->m;
    b200nn_ctx *ctx = m->ctx;
    const size_t d = m->cfg.n_embd, H = m->cfg.n_head;
    if (x->shape.size() != 2 || x->shape[1] != d || x->shape[0] == 0)
        return set_error(ctx, B200NN_ERR_SHAPE, "TransformerBlock: expected input [seq_len, n_embd]");
    const size_t n = x->shape[0], cap = past + n;
    if (past && (!cached_k || !cached_v)) return set_error(ctx, B200NN_ERR_ARG, "forward_cached: kv_len > 0 needs cached K and V");
    CK(ctx, cudaSetDevice(ctx->device));
    b200nn_kvcache kv;
    kv.m = m;
    kv.batch = 1;
    kv.cap = cap;
    kv.len = past;
    TRY(dev_alloc(ctx, H * cap * 64 * sizeof(__half), &kv.k));
    TRY(dev_alloc(ctx, H * cap * 64 * sizeof(__half), &kv.v));
    std::shared_ptr<DevBuf> tmp;
    if (past) {
        TRY(dev_alloc(ctx, H * past * 64 * 4, &tmp));
        CK(ctx, cudaMemcpyAsync(tmp->p, cached_k, H * past * 64 * 4, cudaMemcpyHostToDevice, ctx->stream));
        TRY(launch_pack_kv(ctx, (const float *)tmp->p, (int)H, (int)past, (int)cap, (__half *)kv.k->p));
        CK(ctx, cudaStreamSynchronize(ctx->stream));
        CK(ctx, cudaMemcpyAsync(tmp->p, cached_v, H * past * 64 * 4, cudaMemcpyHostToDevice, ctx->stream));
        TRY(launch_pack_kv(ctx, (const float *)tmp->p, (int)H, (int)past, (int)cap, (__half *)kv.v->p));
    }
    Workspace ws;
    ws.rows = n;
    TRY(dev_alloc(ctx, n * d * 4, &ws.x));
    TRY(dev_alloc(ctx, n * d * 4, &ws.ln));
    TRY(dev_alloc(ctx, n * d * 4, &ws.q));
    TRY(dev_alloc(ctx, n * d * 4, &ws.att));
    TRY(dev_alloc(ctx, n * 4 * d * 4, &ws.fc));
    CK(ctx, cudaMemcpyAsync(ws.x->p, x->buf->p, n * d * 4, cudaMemcpyDeviceToDevice, ctx->stream));
    TRY(run_blocks_range(m, ws, kv, 1, (int)n, nullptr, (int)past, model_act_half(m, (int)n), nullptr, 0, 1));
    b200nn_tensor *o = nullptr;
    TRY(tensor_alloc(ctx, {n, d}, false, &o));
    int rc = B200NN_OK;
    cudaError_t e = cudaMemcpyAsync(o->buf->p, ws.x->p, n * d * 4, cudaMemcpyDeviceToDevice, ctx->stream);
    if (e != cudaSuccess) rc = set_cuda_error(ctx, e, "block output copy");
    if (rc == B200NN_OK && (new_k_out || new_v_out)) {
        // the new K,V rows back to the host as f32 [H][n*64] (the values the fp16 cache holds)
        std::shared_ptr<DevBuf> f;
        rc = dev_alloc(ctx, H * cap * 64 * 4, &f);
        for (int which = 0; which < 2 && rc == B200NN_OK; ++which) {
            float *dst = which ? new_v_out : new_k_out;
            if (!dst) continue;
            rc = launch_half_to_f32(ctx, (const __half *)(which ? kv.v->p : kv.k->p), (float *)f->p, H * cap * 64);
            if (rc != B200NN_OK) break;
            e = cudaMemcpy2DAsync(dst, n * 64 * 4, (const float *)f->p + past * 64, cap * 64 * 4, n * 64 * 4, H,
                                  cudaMemcpyDeviceToHost, ctx->stream);
            if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
            if (e != cudaSuccess) rc = set_cuda_error(ctx, e, "block new K/V copy");
        }
    }
    if (rc == B200NN_OK) rc = stream_sync_check(ctx); // the temporaries are released on return
    if (rc != B200NN_OK) {
        delete o;
        return rc;
    }
    *y = o;
    return B200NN_OK;
}

}  // namespace

extern "C" int32_t b200nn_block_create(b200nn_ctx *ctx, const b200nn_gpt2_config *cfg, const b200nn_block_weights *w,
                                       uint32_t flags, b200nn_block **out) {
    return block_create(ctx, cfg, w, false, 0, flags, out);
}

extern "C" int32_t b200nn_int4_block_create(b200nn_ctx *ctx, const b200nn_gpt2_config *cfg, const b200nn_block_weights *w,
                                            size_t group_size, uint32_t flags, b200nn_block **out) {
    return block_create(ctx, cfg, w, true, group_size, flags, out);
}

extern "C" int32_t b200nn_block_forward(b200nn_block *b, const b200nn_tensor *x, b200nn_tensor **y) {
    if (!b || !x || !y) return B200NN_ERR_ARG;
    return block_run(b, x, nullptr, nullptr, 0, y, nullptr, nullptr);
}

extern "C" int32_t b200nn_block_forward_cached(b200nn_block *b, const b200nn_tensor *x, const float *cached_k,
                                               const float *cached_v, size_t kv_len, b200nn_tensor **y, float *new_k_out,
                                               float *new_v_out) {
    if (!b || !x || !y) return B200NN_ERR_ARG;
    return block_run(b, x, cached_k, cached_v, kv_len, y, new_k_out, new_v_out);
}

extern "C" void b200nn_block_destroy(b200nn_block *b) { delete b; }
