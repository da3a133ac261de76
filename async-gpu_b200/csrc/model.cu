// GPT-2 model assembly: weight preparation, transformer blocks, LM head, KV cache, decode session.
// Structure follows crates/core/gpu-host/src/nn/models/gpt2.rs (pre-LN block, gpt2.rs:172-204;
// tied LM head without bias, 391-399; cached forward, 712-734; greedy loops, 672-783).
#include <algorithm>
#include <cstring>

#include "model.h"

int linear_forward(b200nn_ctx *ctx, const LinearAny &l, const void *x, bool x_half, int M, Epilogue epi) {
    if (!epi.ln_stats) epi.bias = l.bias(); // a folded LayerNorm brings its own combined bias
    if (l.int4) return launch_int4_linear(ctx, l.q, x, x_half, M, epi);
    return launch_f32_linear(ctx, l.f, x, x_half, M, epi);
}

static int upload_vec(b200nn_ctx *ctx, const float *h, size_t n, std::shared_ptr<DevBuf> *out) {
    if (!h) return set_error(ctx, B200NN_ERR_ARG, "null weight pointer");
    TRY(dev_alloc(ctx, n * sizeof(float), out));
    CK(ctx, cudaMemcpy((*out)->p, h, n * sizeof(float), cudaMemcpyHostToDevice));
    return B200NN_OK;
}

// Builds one Linear from a checkpoint-layout weight [K,N] (= [in,out]).
// `out_in`: the weight is given in Linear layout [N,K] = [out,in] (what from_generic_weights holds).
static int make_linear(b200nn_ctx *ctx, const float *w_kn, const float *bias, size_t K, size_t N, bool int4,
                       size_t group, LinearAny *out, bool out_in = false) {
    if (!w_kn) return set_error(ctx, B200NN_ERR_ARG, "null weight pointer");
    out->K = (int)K;
    out->N = (int)N;
    out->int4 = int4;
    if (!int4) return f32_weight_upload(ctx, w_kn, out_in, bias, K, N, &out->f);
    std::vector<float> transposed;
    if (out_in) { // the quantiser groups along K per output column of [K,N]
        transposed.resize(K * N);
        for (size_t o = 0; o < N; ++o)
            for (size_t i = 0; i < K; ++i) transposed[i * N + o] = w_kn[o * K + i];
        w_kn = transposed.data();
    }
    std::vector<uint32_t> packed((K / 8) * N);
    std::vector<float> scales(((K + group - 1) / group) * N);
    int rc = host_quantize_weight_int4(w_kn, K, N, group, packed.data(), scales.data());
    if (rc != B200NN_OK) return set_error(ctx, rc, "quantize_weight_int4: K must be divisible by 8");
    return int4_weight_upload(ctx, packed.data(), scales.data(), bias, K, N, group, &out->q);
}

static int model_create(b200nn_ctx *ctx, const b200nn_gpt2_config *cfg, const b200nn_gpt2_weights *w, bool int4,
                        size_t group, uint32_t flags, b200nn_gpt2 **out) {
    if (!ctx || !cfg || !w || !out) return B200NN_ERR_ARG;
    if (cfg->n_layer <= 0 || cfg->n_embd <= 0 || cfg->n_head <= 0 || cfg->vocab_size <= 0 || cfg->n_positions <= 0)
        return set_error(ctx, B200NN_ERR_SHAPE, "Gpt2Config: non-positive dimension");
    if (cfg->n_embd % cfg->n_head != 0 || cfg->n_embd / cfg->n_head != 64)
        return set_error(ctx, B200NN_ERR_UNSUPPORTED, "head_dim must be 64 (n_embd / n_head)");
    if (int4 && group == 0) return set_error(ctx, B200NN_ERR_SHAPE, "group_size must be positive");
    CK(ctx, cudaSetDevice(ctx->device));
    auto m = std::unique_ptr<b200nn_gpt2>(new b200nn_gpt2());
    m->ctx = ctx;
    m->cfg = *cfg;
    m->flags = flags;
    m->int4 = int4;
    m->group = group;
    const size_t d = cfg->n_embd, V = cfg->vocab_size, P = cfg->n_positions, ffn = 4 * d;
    TRY(upload_vec(ctx, w->wte, V * d, &m->wte));
    TRY(upload_vec(ctx, w->wpe, P * d, &m->wpe));
    TRY(upload_vec(ctx, w->ln_f_weight, d, &m->lnf_g));
    TRY(upload_vec(ctx, w->ln_f_bias, d, &m->lnf_b));
    if (!w->layers) return set_error(ctx, B200NN_ERR_ARG, "null layer weights");
    m->blocks.resize(cfg->n_layer);
    for (int l = 0; l < cfg->n_layer; ++l) {
        const b200nn_gpt2_layer_weights &lw = w->layers[l];
        BlockW &b = m->blocks[l];
        TRY(upload_vec(ctx, lw.ln_1_weight, d, &b.ln1_g));
        TRY(upload_vec(ctx, lw.ln_1_bias, d, &b.ln1_b));
        TRY(upload_vec(ctx, lw.ln_2_weight, d, &b.ln2_g));
        TRY(upload_vec(ctx, lw.ln_2_bias, d, &b.ln2_b));
        const bool oi = (flags & B200NN_WEIGHTS_OUT_IN) != 0;
        TRY(make_linear(ctx, lw.c_attn_weight, lw.c_attn_bias, d, 3 * d, int4, group, &b.qkv, oi));
        TRY(make_linear(ctx, lw.c_proj_weight, lw.c_proj_bias, d, d, int4, group, &b.proj, oi));
        TRY(make_linear(ctx, lw.mlp_fc_weight, lw.mlp_fc_bias, d, ffn, int4, group, &b.fc, oi));
        TRY(make_linear(ctx, lw.mlp_proj_weight, lw.mlp_proj_bias, ffn, d, int4, group, &b.fcproj, oi));
    }
    // tied LM head: logits = h * wte^T, i.e. a Linear with weight [K=d, N=V] = wte transposed
    m->lm_head.K = (int)d;
    m->lm_head.N = (int)V;
    if (int4 && (flags & B200NN_QUANT_LM_HEAD)) {
        std::vector<float> wt(d * V);
        for (size_t v = 0; v < V; ++v)
            for (size_t j = 0; j < d; ++j) wt[j * V + v] = w->wte[v * d + j];
        TRY(make_linear(ctx, wt.data(), nullptr, d, V, true, group, &m->lm_head));
    } else {
        m->lm_head.int4 = false;
        TRY(f32_weight_upload(ctx, w->wte, true, nullptr, d, V, &m->lm_head.f));
    }
    *out = m.release();
    return B200NN_OK;
}

extern "C" int32_t b200nn_gpt2_create(b200nn_ctx *ctx, const b200nn_gpt2_config *cfg, const b200nn_gpt2_weights *w,
                                      uint32_t flags, b200nn_gpt2 **out) {
    return model_create(ctx, cfg, w, false, 0, flags, out);
}

extern "C" int32_t b200nn_int4_gpt2_create(b200nn_ctx *ctx, const b200nn_gpt2_config *cfg,
                                           const b200nn_gpt2_weights *w, size_t group_size, uint32_t flags,
                                           b200nn_gpt2 **out) {
    return model_create(ctx, cfg, w, true, group_size, flags, out);
}

extern "C" void b200nn_gpt2_destroy(b200nn_gpt2 *m) { delete m; }

extern "C" int32_t b200nn_gpt2_get_config(const b200nn_gpt2 *m, b200nn_gpt2_config *out) {
    if (!m || !out) return B200NN_ERR_ARG;
    *out = m->cfg;
    return B200NN_OK;
}

extern "C" int32_t b200nn_gpt2_config_preset(const char *name, b200nn_gpt2_config *out) {
    if (!name || !out) return B200NN_ERR_ARG;
    // Gpt2Config::{small,medium,large,xl} (gpt2.rs:36-83)
    struct P { const char *n; int l, d, h; } presets[] = {
        {"small", 12, 768, 12}, {"medium", 24, 1024, 16}, {"large", 36, 1280, 20}, {"xl", 48, 1600, 25}};
    for (auto &p : presets)
        if (!strcmp(name, p.n)) {
            *out = b200nn_gpt2_config{p.l, p.d, p.h, 50257, 1024, 1e-5f};
            return B200NN_OK;
        }
    return B200NN_ERR_UNSUPPORTED;
}

extern "C" size_t b200nn_gpt2_quantized_memory_bytes(const b200nn_gpt2 *m) {
    if (!m || !m->int4) return 0;
    size_t t = 0;
    for (const BlockW &b : m->blocks)
        t += b.qkv.q.memory_bytes() + b.proj.q.memory_bytes() + b.fc.q.memory_bytes() + b.fcproj.q.memory_bytes();
    return t;
}

extern "C" int32_t b200nn_gpt2_get_int4(const b200nn_gpt2 *m, int32_t layer, int32_t which, uint32_t *packed,
                                        float *scales, size_t *k_out, size_t *n_out) {
    if (!m) return B200NN_ERR_ARG;
    const LinearAny *l = nullptr;
    if (layer == -1 && which == 0) l = &m->lm_head;
    else if (layer >= 0 && layer < m->cfg.n_layer) {
        const BlockW &b = m->blocks[layer];
        l = which == 0 ? &b.qkv : which == 1 ? &b.proj : which == 2 ? &b.fc : which == 3 ? &b.fcproj : nullptr;
    }
    if (!l) return set_error(m->ctx, B200NN_ERR_DIM, "get_int4: no such layer / projection");
    if (!l->int4) return set_error(m->ctx, B200NN_ERR_UNSUPPORTED, "get_int4: this projection is f32");
    if (k_out) *k_out = l->K;
    if (n_out) *n_out = l->N;
    if (packed) memcpy(packed, l->q.host_packed.data(), l->q.host_packed.size() * 4);
    if (scales) memcpy(scales, l->q.host_scales.data(), l->q.host_scales.size() * 4);
    return B200NN_OK;
}

// ---------------------------------------------------------------------------------------------
// workspace and forward pieces
// ---------------------------------------------------------------------------------------------
int workspace_alloc(b200nn_gpt2 *m, size_t rows, size_t logit_rows, Workspace *ws) {
    b200nn_ctx *ctx = m->ctx;
    const size_t d = m->cfg.n_embd, V = m->cfg.vocab_size;
    ws->rows = rows;
    ws->logit_rows = logit_rows;
    TRY(dev_alloc(ctx, rows * d * 4, &ws->x));
    TRY(dev_alloc(ctx, rows * d * 4, &ws->ln));
    TRY(dev_alloc(ctx, rows * d * 4, &ws->q));
    TRY(dev_alloc(ctx, rows * d * 4, &ws->att));
    TRY(dev_alloc(ctx, rows * 4 * d * 4, &ws->fc));
    TRY(dev_alloc(ctx, logit_rows * d * 4, &ws->last_x));
    TRY(dev_alloc(ctx, logit_rows * d * 4, &ws->last_ln));
    TRY(dev_alloc(ctx, logit_rows * V * 4, &ws->logits));
    TRY(dev_alloc(ctx, rows * 4, &ws->ids));
    TRY(dev_alloc(ctx, std::max(rows, logit_rows) * 4, &ws->tok));
    ws->amax_entries = (int)((V + 127) / 128) * 4; // one entry per 32 features of the padded width
    TRY(dev_alloc(ctx, std::max<size_t>(1, logit_rows) * ws->amax_entries * 4, &ws->amax_val));
    TRY(dev_alloc(ctx, std::max<size_t>(1, logit_rows) * ws->amax_entries * 4, &ws->amax_idx));
    return B200NN_OK;
}

// Activations between Linears are fp16 when the tensor-core GEMM will consume them.
bool model_act_half(const b200nn_gpt2 *m, int rows) {
    const BlockW &b = m->blocks[0];
    if (!m->int4) // f32 family: fp16 copies of the weights serve more than four rows
        return f16_gemm_tc_supported(m->ctx, b.qkv.f, rows) && f16_gemm_tc_supported(m->ctx, b.proj.f, rows) &&
               f16_gemm_tc_supported(m->ctx, b.fc.f, rows) && f16_gemm_tc_supported(m->ctx, b.fcproj.f, rows);
    if (rows <= m->ctx->gemv_max_rows) return false;
    return int4_gemm_tc_supported(b.qkv.q, rows) && int4_gemm_tc_supported(b.proj.q, rows) &&
           int4_gemm_tc_supported(b.fc.q, rows) && int4_gemm_tc_supported(b.fcproj.q, rows);
}

static inline void prof_mark(b200nn_ctx *ctx, StepProfile *p, int fam) {
    if (!p) return;
    cudaEvent_t e;
    cudaEventCreate(&e);
    cudaEventRecord(e, ctx->stream);
    p->ev.push_back(e);
    p->fam.push_back(fam);
}

// The seven launches of one transformer block, each on its own so that the forward pass (all of them,
// in order) and the per-family timing routine (one family at a time) issue exactly the same launches.
bool model_ln_fold_supported(const b200nn_gpt2 *m, int rows) {
    const int d = m->cfg.n_embd;
    if (!m->int4 || !m->ctx->ln_fold || rows <= m->ctx->gemv_max_rows || d % 8 != 0 || (d + TILE_N - 1) / TILE_N > 32) return false;
    if (!model_act_half(m, rows)) return false;
    const BlockW &b = m->blocks[0];
    for (const LinearAny *l : {&b.qkv, &b.proj, &b.fc, &b.fcproj})
        if (!l->q.fast || int4_via_f16_supported(m->ctx, l->q, rows)) return false;
    return true;
}

int model_prepare_ln_fold(b200nn_gpt2 *m, Workspace *ws) {
    b200nn_ctx *ctx = m->ctx;
    if (!m->ln_fold_ready) {
        for (BlockW &b : m->blocks) {
            TRY(int4_weight_ln_fold(ctx, b.qkv.q, (const float *)b.ln1_g->p, (const float *)b.ln1_b->p, &b.qkv_gsum, &b.qkv_bc));
            TRY(int4_weight_ln_fold(ctx, b.fc.q, (const float *)b.ln2_g->p, (const float *)b.ln2_b->p, &b.fc_gsum, &b.fc_bc));
        }
        m->ln_fold_ready = true;
    }
    ws->ln_nt = (m->cfg.n_embd + TILE_N - 1) / TILE_N;
    return dev_alloc(ctx, (size_t)2 * m->cfg.n_layer * ws->rows * ws->ln_nt * 2 * sizeof(float), &ws->ln_stats);
}

// The consumer side of a folded LayerNorm: statistics slot, weighted column sums and combined bias.
static void fold_consumer(const b200nn_gpt2 *m, const Workspace &ws, int slot, const std::shared_ptr<DevBuf> &gsum,
                          const std::shared_ptr<DevBuf> &bc, Epilogue *e) {
    e->ln_stats = ws.ln_slot(slot);
    e->ln_nt = ws.ln_nt;
    e->ln_gsum = (const float *)gsum->p;
    e->bias = (const float *)bc->p;
    e->ln_eps = m->cfg.layer_norm_epsilon;
    e->ln_inv_d = 1.0f / (float)m->cfg.n_embd;
}
// The producer side: the residual GEMM also writes what the LayerNorm `slot` (scale next_g) will need.
static void fold_producer(const Workspace &ws, int slot, const std::shared_ptr<DevBuf> &next_g, Epilogue *e) {
    e->mode = EPI_RESID_LN;
    e->xg_out = (__half *)ws.ln->p;
    e->next_g = (const float *)next_g->p;
    e->stats_out = ws.ln_slot(slot);
    e->stats_nt = ws.ln_nt;
}

int BlockLaunch::ln1() const {
    if (fold) return B200NN_OK;
    const BlockW &b = m->blocks[l];
    return launch_layernorm(m->ctx, (const float *)ws.x->p, nullptr, nullptr, (const float *)b.ln1_g->p, (const float *)b.ln1_b->p,
                            m->cfg.layer_norm_epsilon, B * S, m->cfg.n_embd, ws.ln->p, act_half);
}
int BlockLaunch::qkv() const {
    const int d = m->cfg.n_embd;
    Epilogue e;
    e.mode = EPI_QKV;
    e.out = ws.q->p;
    e.ldo = d;
    e.out_half = act_half;
    e.kc = kv.kl(l);
    e.vc = kv.vl(l);
    e.d_model = d;
    e.n_head = m->cfg.n_head;
    e.rows_per_seq = S;
    e.cap = (int)kv.cap;
    e.pos_ptr = pos_ptr;
    e.pos_off = pos_off;
    if (fold) fold_consumer(m, ws, 2 * l, m->blocks[l].qkv_gsum, m->blocks[l].qkv_bc, &e);
    return linear_forward(m->ctx, m->blocks[l].qkv, ws.ln->p, act_half, B * S, e);
}
int BlockLaunch::attention() const {
    const int d = m->cfg.n_embd, H = m->cfg.n_head;
    if (S == 1)
        return launch_decode_attention(m->ctx, ws.q->p, act_half, d, kv.kl(l), kv.vl(l), B, H, (int)kv.cap, pos_ptr, pos_off,
                                       ws.att->p, act_half, (int)kv.cap);
    return launch_prefill_attention(m->ctx, ws.q->p, act_half, d, kv.kl(l), kv.vl(l), B, H, (int)kv.cap, S, pos_off, ws.att->p,
                                    act_half);
}
int BlockLaunch::proj() const {
    Epilogue r;
    r.mode = EPI_RESID;
    r.resid = (float *)ws.x->p;
    r.ldo = m->cfg.n_embd;
    if (fold) fold_producer(ws, 2 * l + 1, m->blocks[l].ln2_g, &r);
    return linear_forward(m->ctx, m->blocks[l].proj, ws.att->p, act_half, B * S, r);
}
int BlockLaunch::ln2() const {
    if (fold) return B200NN_OK;
    const BlockW &b = m->blocks[l];
    return launch_layernorm(m->ctx, (const float *)ws.x->p, nullptr, nullptr, (const float *)b.ln2_g->p, (const float *)b.ln2_b->p,
                            m->cfg.layer_norm_epsilon, B * S, m->cfg.n_embd, ws.ln->p, act_half);
}
int BlockLaunch::fc() const {
    Epilogue f;
    f.mode = EPI_STORE;
    f.act = m->act();
    f.out = ws.fc->p;
    f.ldo = 4 * m->cfg.n_embd;
    f.out_half = act_half;
    if (fold) fold_consumer(m, ws, 2 * l + 1, m->blocks[l].fc_gsum, m->blocks[l].fc_bc, &f);
    return linear_forward(m->ctx, m->blocks[l].fc, ws.ln->p, act_half, B * S, f);
}
int BlockLaunch::fcproj() const {
    Epilogue r;
    r.mode = EPI_RESID;
    r.resid = (float *)ws.x->p;
    r.ldo = m->cfg.n_embd;
    // the last block's output goes to the final LayerNorm, which runs as a kernel of its own
    if (fold && l + 1 < m->cfg.n_layer) fold_producer(ws, 2 * l + 2, m->blocks[l + 1].ln1_g, &r);
    return linear_forward(m->ctx, m->blocks[l].fcproj, ws.fc->p, act_half, B * S, r);
}

int run_blocks(b200nn_gpt2 *m, Workspace &ws, b200nn_kvcache &kv, int B, int S, const int *pos_ptr, int pos_off,
               bool act_half, StepProfile *prof, bool fold) {
    return run_blocks_range(m, ws, kv, B, S, pos_ptr, pos_off, act_half, prof, 0, m->cfg.n_layer, fold);
}

int run_blocks_range(b200nn_gpt2 *m, Workspace &ws, b200nn_kvcache &kv, int B, int S, const int *pos_ptr, int pos_off,
                     bool act_half, StepProfile *prof, int layer_begin, int layer_end, bool fold) {
    b200nn_ctx *ctx = m->ctx;
    for (int l = layer_begin; l < layer_end; ++l) {
        const BlockLaunch bl{m, ws, kv, l, B, S, pos_ptr, pos_off, act_half, fold};
        TRY(bl.ln1());
        prof_mark(ctx, prof, B200NN_PROF_LAYERNORM);
        TRY(bl.qkv());
        prof_mark(ctx, prof, B200NN_PROF_LINEAR);
        TRY(bl.attention());
        prof_mark(ctx, prof, B200NN_PROF_ATTENTION);
        TRY(bl.proj());
        prof_mark(ctx, prof, B200NN_PROF_LINEAR);
        TRY(bl.ln2());
        prof_mark(ctx, prof, B200NN_PROF_LAYERNORM);
        TRY(bl.fc());
        prof_mark(ctx, prof, B200NN_PROF_LINEAR);
        TRY(bl.fcproj());
        prof_mark(ctx, prof, B200NN_PROF_LINEAR);
    }
    return B200NN_OK;
}

bool head_act_half(const b200nn_gpt2 *m, int rows, bool act_half) {
    return act_half && (m->lm_head.int4 ? int4_gemm_tc_supported(m->lm_head.q, rows)
                                        : f16_gemm_tc_supported(m->ctx, m->lm_head.f, rows));
}
int launch_head_norm(b200nn_gpt2 *m, Workspace &ws, const float *x, int rows, bool head_half) {
    return launch_layernorm(m->ctx, x, nullptr, nullptr, (const float *)m->lnf_g->p, (const float *)m->lnf_b->p,
                            m->cfg.layer_norm_epsilon, rows, m->cfg.n_embd, ws.last_ln->p, head_half);
}
int launch_head_linear(b200nn_gpt2 *m, Workspace &ws, int rows, bool head_half) {
    Epilogue e;
    e.mode = EPI_STORE;
    e.out = ws.logits->p;
    e.ldo = m->cfg.vocab_size;
    return linear_forward(m->ctx, m->lm_head, ws.last_ln->p, head_half, rows, e);
}

int run_head(b200nn_gpt2 *m, Workspace &ws, const float *x, int rows, bool act_half, StepProfile *prof) {
    b200nn_ctx *ctx = m->ctx;
    const bool head_half = head_act_half(m, rows, act_half);
    TRY(launch_head_norm(m, ws, x, rows, head_half));
    prof_mark(ctx, prof, B200NN_PROF_LAYERNORM);
    TRY(launch_head_linear(m, ws, rows, head_half));
    prof_mark(ctx, prof, B200NN_PROF_LM_HEAD);
    return B200NN_OK;
}

// Which LM-head launches take the greedy pick in their epilogue: the tensor-core GEMMs and the two
// GEMV kernels of an int4 head in the tiled layout, and the fp16 tensor-core GEMM of an f32 head.
static bool head_fuses_pick(const b200nn_gpt2 *m, int rows, bool head_half) {
    if (m->lm_head.int4) return m->lm_head.q.fast && rows < 2048;
    return head_half && f16_gemm_tc_supported(m->ctx, m->lm_head.f, rows);
}

int run_head_pick(b200nn_gpt2 *m, Workspace &ws, const float *x, int rows, bool act_half, bool keep_last, bool tokens_only,
                  uint32_t *tok_out, StepProfile *prof) {
    b200nn_ctx *ctx = m->ctx;
    const int V = m->cfg.vocab_size;
    const bool head_half = head_act_half(m, rows, act_half);
    TRY(launch_head_norm(m, ws, x, rows, head_half));
    prof_mark(ctx, prof, B200NN_PROF_LAYERNORM);
    if (!ctx->fused_argmax || !head_fuses_pick(m, rows, head_half)) {
        TRY(launch_head_linear(m, ws, rows, head_half));
        prof_mark(ctx, prof, B200NN_PROF_LM_HEAD);
        return launch_argmax(ctx, (const float *)ws.logits->p, rows, V, V, keep_last, tok_out);
    }
    Epilogue e;
    e.mode = EPI_STORE;
    e.out = ws.logits->p;
    e.ldo = V;
    e.no_store = tokens_only ? 1 : 0;
    e.amax_val = (float *)ws.amax_val->p;
    e.amax_idx = (int *)ws.amax_idx->p;
    e.amax_entries = ws.amax_entries;
    e.amax_keep_last = keep_last ? 1 : 0;
    TRY(linear_forward(ctx, m->lm_head, ws.last_ln->p, head_half, rows, e));
    prof_mark(ctx, prof, B200NN_PROF_LM_HEAD);
    return launch_argmax_entries(ctx, e.amax_val, e.amax_idx, rows, e.amax_entries, V, keep_last, tok_out);
}
