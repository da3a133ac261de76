// KV cache, full / cached forward, decode session and the greedy generate loops.
#include <algorithm>
#include <cstring>

#include "model.h"

static int kv_init(b200nn_gpt2 *m, size_t batch, size_t cap, b200nn_kvcache *c) {
    if (!batch || !cap) return set_error(m->ctx, B200NN_ERR_SHAPE, "KvCache: batch and capacity must be positive");
    if (cap > (size_t)m->cfg.n_positions)
        return set_error(m->ctx, B200NN_ERR_DIM, "KvCache: capacity exceeds n_positions");
    c->m = m;
    c->batch = batch;
    c->cap = cap;
    c->len = 0;
    size_t bytes = (size_t)m->cfg.n_layer * batch * m->cfg.n_embd * cap * sizeof(__half);
    TRY(dev_alloc(m->ctx, bytes, &c->k));
    TRY(dev_alloc(m->ctx, bytes, &c->v));
    return B200NN_OK;
}

extern "C" int32_t b200nn_kvcache_create(b200nn_gpt2 *m, size_t batch, size_t capacity, b200nn_kvcache **out) {
    if (!m || !out) return B200NN_ERR_ARG;
    auto c = std::unique_ptr<b200nn_kvcache>(new b200nn_kvcache());
    TRY(kv_init(m, batch, capacity, c.get()));
    *out = c.release();
    return B200NN_OK;
}
extern "C" size_t b200nn_kvcache_len(const b200nn_kvcache *c) { return c ? c->len : 0; }
extern "C" int32_t b200nn_kvcache_reset(b200nn_kvcache *c) {
    if (!c) return B200NN_ERR_ARG;
    c->len = 0;
    return B200NN_OK;
}
extern "C" void b200nn_kvcache_destroy(b200nn_kvcache *c) { delete c; }

static int check_ids(b200nn_gpt2 *m, const uint32_t *ids, size_t n) {
    for (size_t i = 0; i < n; ++i)
        if (ids[i] >= (uint32_t)m->cfg.vocab_size)
            return set_error(m->ctx, B200NN_ERR_DIM, "token id out of range for vocab_size");
    return B200NN_OK;
}

// Embeds B sequences of S new tokens each (ids on the host, [B,S]) at positions past.., runs the
// blocks, appends to the cache.  Leaves the residual stream in ws.x.
static int forward_rows(b200nn_gpt2 *m, Workspace &ws, b200nn_kvcache &kv, const uint32_t *ids_host, int B, int S,
                        bool act_half) {
    b200nn_ctx *ctx = m->ctx;
    const int d = m->cfg.n_embd;
    size_t T = (size_t)B * S;
    if (T > ws.rows) return set_error(ctx, B200NN_ERR_SHAPE, "workspace too small");
    if (kv.len + S > kv.cap) return set_error(ctx, B200NN_ERR_DIM, "KV cache capacity exceeded");
    TRY(check_ids(m, ids_host, T));
    CK(ctx, cudaMemcpyAsync(ws.ids->p, ids_host, T * 4, cudaMemcpyHostToDevice, ctx->stream));
    TRY(launch_embedding(ctx, (const uint32_t *)ws.ids->p, (const float *)m->wte->p, (const float *)m->wpe->p, (int)T,
                         d, S, nullptr, (int)kv.len, m->cfg.vocab_size, m->cfg.n_positions, (float *)ws.x->p));
    TRY(run_blocks(m, ws, kv, B, S, nullptr, (int)kv.len, act_half, nullptr));
    kv.len += S;
    return B200NN_OK;
}

// Gpt2Model::forward: one sequence, logits for every position.
extern "C" int32_t b200nn_gpt2_forward(b200nn_gpt2 *m, const uint32_t *ids_host, size_t seq_len,
                                       b200nn_tensor **logits) {
    if (!m || !ids_host || !logits) return B200NN_ERR_ARG;
    b200nn_ctx *ctx = m->ctx;
    if (seq_len == 0 || seq_len > (size_t)m->cfg.n_positions)
        return set_error(ctx, B200NN_ERR_DIM, "forward: seq_len must be in [1, n_positions]");
    CK(ctx, cudaSetDevice(ctx->device));
    b200nn_kvcache kv;
    TRY(kv_init(m, 1, seq_len, &kv));
    Workspace ws;
    TRY(workspace_alloc(m, seq_len, seq_len, &ws));
    bool ah = model_act_half(m, (int)seq_len);
    TRY(forward_rows(m, ws, kv, ids_host, 1, (int)seq_len, ah));
    TRY(run_head(m, ws, (const float *)ws.x->p, (int)seq_len, ah, nullptr));
    b200nn_tensor *t = nullptr;
    TRY(tensor_alloc(ctx, {seq_len, (size_t)m->cfg.vocab_size}, false, &t));
    cudaError_t e = cudaMemcpyAsync(t->buf->p, ws.logits->p, t->numel * 4, cudaMemcpyDeviceToDevice, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) {
        delete t;
        return set_cuda_error(ctx, e, "forward copy");
    }
    *logits = t;
    return B200NN_OK;
}

// Gpt2Model::forward_cached with a batch axis: ids [batch,new_len] -> logits [batch*new_len,vocab].
extern "C" int32_t b200nn_gpt2_forward_cached(b200nn_gpt2 *m, const uint32_t *ids_host, size_t new_len,
                                              b200nn_kvcache *cache, b200nn_tensor **logits) {
    if (!m || !ids_host || !cache || !logits) return B200NN_ERR_ARG;
    b200nn_ctx *ctx = m->ctx;
    if (cache->m != m) return set_error(ctx, B200NN_ERR_ARG, "KvCache belongs to another model");
    if (new_len == 0) return set_error(ctx, B200NN_ERR_SHAPE, "forward_cached: new_len must be positive");
    CK(ctx, cudaSetDevice(ctx->device));
    size_t T = cache->batch * new_len;
    Workspace ws;
    TRY(workspace_alloc(m, T, T, &ws));
    bool ah = model_act_half(m, (int)T);
    TRY(forward_rows(m, ws, *cache, ids_host, (int)cache->batch, (int)new_len, ah));
    TRY(run_head(m, ws, (const float *)ws.x->p, (int)T, ah, nullptr));
    b200nn_tensor *t = nullptr;
    TRY(tensor_alloc(ctx, {T, (size_t)m->cfg.vocab_size}, false, &t));
    cudaError_t e = cudaMemcpyAsync(t->buf->p, ws.logits->p, t->numel * 4, cudaMemcpyDeviceToDevice, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) {
        delete t;
        return set_cuda_error(ctx, e, "forward_cached copy");
    }
    *logits = t;
    return B200NN_OK;
}

// ---------------------------------------------------------------------------------------------
// decode session
// ---------------------------------------------------------------------------------------------
static constexpr size_t PREFILL_ROWS = 16384; // rows per prefill pass (bounds the activation buffers)

extern "C" int32_t b200nn_session_create(b200nn_gpt2 *m, size_t batch, size_t capacity, uint32_t flags,
                                         b200nn_session **out) {
    if (!m || !out) return B200NN_ERR_ARG;
    b200nn_ctx *ctx = m->ctx;
    CK(ctx, cudaSetDevice(ctx->device));
    auto s = std::unique_ptr<b200nn_session>(new b200nn_session());
    s->m = m;
    s->batch = batch;
    s->cap = capacity;
    s->hist_cap = capacity;
    s->flags = flags;
    TRY(kv_init(m, batch, capacity, &s->kv));
    TRY(workspace_alloc(m, batch, batch, &s->ws_step));
    TRY(dev_alloc(ctx, 2 * sizeof(int), &s->counters));
    CK(ctx, cudaMemsetAsync(s->counters->p, 0, 2 * sizeof(int), ctx->stream));
    TRY(dev_alloc(ctx, batch * s->hist_cap * 4, &s->history));
    CK(ctx, cudaMemsetAsync(s->history->p, 0, batch * s->hist_cap * 4, ctx->stream));
    if (model_ln_fold_supported(m, (int)batch)) TRY(model_prepare_ln_fold(m, &s->ws_step));
    if (decode_persistent_supported(m, (int)batch)) {
        TRY(decode_persistent_prepare(s.get()));
        s->persist = true;
    }
    *out = s.release();
    return B200NN_OK;
}

extern "C" void b200nn_session_destroy(b200nn_session *s) {
    if (!s) return;
    if (s->graph) cudaGraphExecDestroy(s->graph);
    delete s;
}

static int set_counters(b200nn_session *s, int position, int step) {
    b200nn_ctx *ctx = s->m->ctx;
    int h[2] = {position, step};
    CK(ctx, cudaMemcpyAsync(s->counters->p, h, sizeof(h), cudaMemcpyHostToDevice, ctx->stream));
    CK(ctx, cudaStreamSynchronize(ctx->stream)); // h is a stack buffer
    return B200NN_OK;
}

extern "C" int32_t b200nn_session_prefill(b200nn_session *s, const uint32_t *prompts_host, size_t prompt_len) {
    if (!s || !prompts_host) return B200NN_ERR_ARG;
    b200nn_gpt2 *m = s->m;
    b200nn_ctx *ctx = m->ctx;
    if (prompt_len == 0 || prompt_len >= s->cap)
        return set_error(ctx, B200NN_ERR_DIM, "prefill: prompt_len must be in [1, capacity)");
    CK(ctx, cudaSetDevice(ctx->device));
    const int d = m->cfg.n_embd;
    size_t seqs_per_pass = std::max<size_t>(1, PREFILL_ROWS / prompt_len);
    seqs_per_pass = std::min(seqs_per_pass, s->batch);
    if (s->ws_prefill.rows < seqs_per_pass * prompt_len || s->ws_prefill.logit_rows < 1) {
        s->ws_prefill = Workspace();
        TRY(workspace_alloc(m, seqs_per_pass * prompt_len, 1, &s->ws_prefill));
    }
    s->kv.len = 0;
    float *last_x = (float *)s->ws_step.last_x->p;
    for (size_t b0 = 0; b0 < s->batch; b0 += seqs_per_pass) {
        size_t nb = std::min(seqs_per_pass, s->batch - b0);
        // a view of the cache that starts at sequence b0
        b200nn_kvcache view;
        view.m = m;
        view.batch = s->batch; // layer stride of the full cache
        view.cap = s->cap;
        view.len = 0;
        view.k = std::make_shared<DevBuf>();
        view.v = std::make_shared<DevBuf>();
        size_t seq_off = b0 * (size_t)m->cfg.n_head * s->cap * 64;
        view.k->p = (__half *)s->kv.k->p + seq_off;
        view.v->p = (__half *)s->kv.v->p + seq_off;
        bool ah = model_act_half(m, (int)(nb * prompt_len));
        int rc = forward_rows(m, s->ws_prefill, view, prompts_host + b0 * prompt_len, (int)nb, (int)prompt_len, ah);
        view.k->p = nullptr; // borrowed pointers: nothing to free
        view.v->p = nullptr;
        TRY(rc);
        TRY(launch_gather_last_rows(ctx, (const float *)s->ws_prefill.x->p, (int)nb, (int)prompt_len, d,
                                    last_x + b0 * d));
    }
    s->kv.len = prompt_len;
    bool ah = model_act_half(m, (int)s->batch);
    TRY(run_head_pick(m, s->ws_step, last_x, (int)s->batch, ah, (s->flags & B200NN_ARGMAX_LAST) != 0,
                      (s->flags & B200NN_TOKENS_ONLY) != 0, (uint32_t *)s->ws_step.tok->p, nullptr));
    TRY(set_counters(s, (int)prompt_len - 1, 0));
    // record: history[0] = first token, step = 1, position = prompt_len
    TRY(launch_record_tokens(ctx, (const uint32_t *)s->ws_step.tok->p, (int)s->batch, (uint32_t *)s->history->p,
                             (int)s->hist_cap, s->step_ptr(), s->pos_ptr()));
    s->position = prompt_len;
    s->steps_done = 1;
    s->prefilled = true;
    return B200NN_OK;
}

// One greedy decode step for every sequence: embed the current tokens at the device-side
// position, run the blocks (K,V appended in the QKV epilogue), LM head, argmax, record.
static int decode_step(b200nn_session *s, StepProfile *prof) {
    b200nn_gpt2 *m = s->m;
    b200nn_ctx *ctx = m->ctx;
    const int B = (int)s->batch, d = m->cfg.n_embd;
    Workspace &ws = s->ws_step;
    bool ah = model_act_half(m, B);
    const bool persistent = s->persist && ctx->persist;
    const bool fold = !persistent && ws.ln_stats && ctx->ln_fold && model_ln_fold_supported(m, B);
    if (fold)
        TRY(launch_embedding_ln(ctx, (const uint32_t *)ws.tok->p, (const float *)m->wte->p, (const float *)m->wpe->p, B, d,
                                s->pos_ptr(), m->cfg.vocab_size, m->cfg.n_positions, (float *)ws.x->p,
                                (const float *)m->blocks[0].ln1_g->p, (__half *)ws.ln->p, ws.ln_slot(0), ws.ln_nt));
    else
        TRY(launch_embedding(ctx, (const uint32_t *)ws.tok->p, (const float *)m->wte->p, (const float *)m->wpe->p, B, d, 1,
                             s->pos_ptr(), 0, m->cfg.vocab_size, m->cfg.n_positions, (float *)ws.x->p));
    if (prof) {
        cudaEvent_t e;
        cudaEventCreate(&e);
        cudaEventRecord(e, ctx->stream);
        prof->ev.push_back(e);
        prof->fam.push_back(B200NN_PROF_EMBED);
    }
    if (persistent) {
        // every transformer block in one cooperative launch; with `prof` its phases are timed inside the
        // kernel and the launch as a whole is booked under the attention family's event slot
        if (prof) CK(ctx, cudaMemsetAsync((char *)s->pd_sync->p + 64, 0, 128, ctx->stream));
        TRY(launch_decode_layers(s, prof != nullptr));
        if (prof) {
            cudaEvent_t e;
            cudaEventCreate(&e);
            cudaEventRecord(e, ctx->stream);
            prof->ev.push_back(e);
            prof->fam.push_back(-1); // split by the in-kernel phase times afterwards
        }
    } else {
        TRY(run_blocks(m, ws, s->kv, B, 1, s->pos_ptr(), 0, ah, prof, fold));
    }
    TRY(run_head_pick(m, ws, (const float *)ws.x->p, B, ah, (s->flags & B200NN_ARGMAX_LAST) != 0,
                      (s->flags & B200NN_TOKENS_ONLY) != 0, (uint32_t *)ws.tok->p, prof));
    TRY(launch_record_tokens(ctx, (const uint32_t *)ws.tok->p, B, (uint32_t *)s->history->p, (int)s->hist_cap,
                             s->step_ptr(), s->pos_ptr()));
    if (prof) {
        cudaEvent_t e;
        cudaEventCreate(&e);
        cudaEventRecord(e, ctx->stream);
        prof->ev.push_back(e);
        prof->fam.push_back(B200NN_PROF_ARGMAX);
    }
    return B200NN_OK;
}

extern "C" int32_t b200nn_session_step(b200nn_session *s, size_t n_steps) {
    if (!s) return B200NN_ERR_ARG;
    b200nn_ctx *ctx = s->m->ctx;
    if (!s->prefilled) return set_error(ctx, B200NN_ERR_ARG, "session_step before prefill");
    if (s->position + n_steps > s->cap) return set_error(ctx, B200NN_ERR_DIM, "session_step: capacity exceeded");
    CK(ctx, cudaSetDevice(ctx->device));
    size_t done = 0;
    if (s->persist && ctx->persist) {
        // a step is six launches (embedding, the persistent kernel, final norm, LM head, argmax, record):
        // nothing to gain from a graph, and the cooperative launch stays an ordinary launch
        for (; done < n_steps; ++done) TRY(decode_step(s, nullptr));
        s->eager_done = true;
        s->position += n_steps;
        s->steps_done += n_steps;
        s->kv.len = s->position;
        return B200NN_OK;
    }
    if (!s->eager_done && n_steps > 0) { // sizes the split scratch before anything is captured
        TRY(decode_step(s, nullptr));
        s->eager_done = true;
        done = 1;
    }
    if (done < n_steps && !s->graph) {
        cudaGraph_t g = nullptr;
        CK(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
        ctx->capturing = true;
        uint64_t launches_before = ctx->launches;
        int rc = decode_step(s, nullptr);
        ctx->capturing = false;
        s->launches_per_step = ctx->launches - launches_before;
        ctx->launches = launches_before; // captured, not launched yet
        cudaError_t e = cudaStreamEndCapture(ctx->stream, &g);
        if (rc != B200NN_OK) {
            if (g) cudaGraphDestroy(g);
            return rc;
        }
        if (e != cudaSuccess) return set_cuda_error(ctx, e, "cudaStreamEndCapture");
        e = cudaGraphInstantiate(&s->graph, g, 0);
        cudaGraphDestroy(g);
        if (e != cudaSuccess) return set_cuda_error(ctx, e, "cudaGraphInstantiate");
    }
    ctx->launches += (uint64_t)(n_steps - done) * s->launches_per_step;
    for (; done < n_steps; ++done) CK(ctx, cudaGraphLaunch(s->graph, ctx->stream));
    s->position += n_steps;
    s->steps_done += n_steps;
    s->kv.len = s->position;
    return B200NN_OK;
}

extern "C" int32_t b200nn_session_rewind(b200nn_session *s, size_t position) {
    if (!s) return B200NN_ERR_ARG;
    b200nn_ctx *ctx = s->m->ctx;
    if (!s->prefilled || position == 0 || position > s->position)
        return set_error(ctx, B200NN_ERR_DIM, "rewind: position must be in [1, current position]");
    size_t back = s->position - position;
    if (back > s->steps_done - 1) return set_error(ctx, B200NN_ERR_DIM, "rewind: before the end of the prompt");
    CK(ctx, cudaSetDevice(ctx->device));
    s->steps_done -= back;
    s->position = position;
    s->kv.len = position;
    return set_counters(s, (int)position, (int)s->steps_done);
}

extern "C" size_t b200nn_session_position(const b200nn_session *s) { return s ? s->position : 0; }

extern "C" int32_t b200nn_session_tokens(b200nn_session *s, uint32_t *out, size_t capacity_per_seq,
                                         size_t *generated) {
    if (!s || !out) return B200NN_ERR_ARG;
    b200nn_ctx *ctx = s->m->ctx;
    CK(ctx, cudaSetDevice(ctx->device));
    size_t n = std::min(s->steps_done, capacity_per_seq);
    CK(ctx, cudaMemcpy2DAsync(out, capacity_per_seq * 4, s->history->p, s->hist_cap * 4, n * 4, s->batch,
                              cudaMemcpyDeviceToHost, ctx->stream));
    TRY(stream_sync_check(ctx));
    if (generated) *generated = n;
    return B200NN_OK;
}

extern "C" int32_t b200nn_session_logits(b200nn_session *s, float *out) {
    if (!s || !out) return B200NN_ERR_ARG;
    b200nn_ctx *ctx = s->m->ctx;
    if (s->flags & B200NN_TOKENS_ONLY)
        return set_error(ctx, B200NN_ERR_UNSUPPORTED, "session_logits: the session was created with B200NN_TOKENS_ONLY");
    CK(ctx, cudaSetDevice(ctx->device));
    CK(ctx, cudaMemcpyAsync(out, s->ws_step.logits->p, s->batch * (size_t)s->m->cfg.vocab_size * 4,
                            cudaMemcpyDeviceToHost, ctx->stream));
    return stream_sync_check(ctx);
}

extern "C" int32_t b200nn_session_profile_step(b200nn_session *s, float *times_ms, uint64_t *linear_bytes) {
    if (!s || !times_ms) return B200NN_ERR_ARG;
    b200nn_gpt2 *m = s->m;
    b200nn_ctx *ctx = m->ctx;
    if (!s->prefilled) return set_error(ctx, B200NN_ERR_ARG, "profile_step before prefill");
    if (s->position + 1 > s->cap) return set_error(ctx, B200NN_ERR_DIM, "profile_step: capacity exceeded");
    CK(ctx, cudaSetDevice(ctx->device));
    StepProfile prof;
    cudaEvent_t e0;
    CK(ctx, cudaEventCreate(&e0));
    CK(ctx, cudaEventRecord(e0, ctx->stream));
    int rc = decode_step(s, &prof);
    cudaStreamSynchronize(ctx->stream);
    for (int i = 0; i < B200NN_PROF_COUNT; ++i) times_ms[i] = 0.0f;
    cudaEvent_t prev = e0;
    for (size_t i = 0; i < prof.ev.size(); ++i) {
        float ms = 0.0f;
        cudaEventElapsedTime(&ms, prev, prof.ev[i]);
        if (prof.fam[i] >= 0) times_ms[prof.fam[i]] += ms;
        else {
            // the persistent kernel: phase kinds LN1, QKV, ATT, PROJ, LN2, FC, ACT, FCPROJ as block 0 saw them
            unsigned long long ns[8] = {};
            cudaMemcpy(ns, (char *)s->pd_sync->p + 64, sizeof(ns), cudaMemcpyDeviceToHost);
            double tot = 0;
            for (int k = 0; k < 8; ++k) tot += (double)ns[k];
            if (tot > 0) {
                times_ms[B200NN_PROF_LAYERNORM] += ms * (float)((ns[0] + ns[4]) / tot);
                times_ms[B200NN_PROF_ATTENTION] += ms * (float)(ns[2] / tot);
                times_ms[B200NN_PROF_LINEAR] += ms * (float)((ns[1] + ns[3] + ns[5] + ns[6] + ns[7]) / tot);
            } else times_ms[B200NN_PROF_LINEAR] += ms;
        }
        prev = prof.ev[i];
    }
    cudaEventDestroy(e0);
    for (cudaEvent_t e : prof.ev) cudaEventDestroy(e);
    TRY(rc);
    s->eager_done = true;
    s->position += 1;
    s->steps_done += 1;
    s->kv.len = s->position;
    if (linear_bytes) {
        // algorithmic bytes of the block Linears in one step: weights + scales + bias, the
        // activations read and the outputs written (LM head reported under its own family)
        bool ah = model_act_half(m, (int)s->batch);
        size_t ab = ah ? 2 : 4, B = s->batch, d = m->cfg.n_embd, t = 0;
        for (const BlockW &b : m->blocks) {
            t += b.qkv.weight_bytes() + B * d * ab + B * 3 * d * 2;       // q + K,V as fp16 / act dtype
            t += b.proj.weight_bytes() + B * d * ab + 2 * B * d * 4;      // residual read + write
            t += b.fc.weight_bytes() + B * d * ab + B * 4 * d * ab;
            t += b.fcproj.weight_bytes() + B * 4 * d * ab + 2 * B * d * 4;
        }
        *linear_bytes = t;
    }
    return B200NN_OK;
}

extern "C" int32_t b200nn_session_time_family(b200nn_session *s, int32_t family, int32_t reps, float *ms_total,
                                              uint64_t *launches) {
    if (!s || !ms_total || reps <= 0) return B200NN_ERR_ARG;
    b200nn_gpt2 *m = s->m;
    b200nn_ctx *ctx = m->ctx;
    if (!s->prefilled) return set_error(ctx, B200NN_ERR_ARG, "time_family before prefill");
    if (family != B200NN_PROF_LAYERNORM && family != B200NN_PROF_LINEAR && family != B200NN_PROF_ATTENTION &&
        family != B200NN_PROF_LM_HEAD)
        return set_error(ctx, B200NN_ERR_UNSUPPORTED, "time_family: family must be layernorm, linear, attention or lm_head");
    if (s->position + 1 > s->cap) return set_error(ctx, B200NN_ERR_DIM, "time_family: capacity exceeded");
    CK(ctx, cudaSetDevice(ctx->device));
    const int B = (int)s->batch;
    const bool ah = model_act_half(m, B);
    const bool fold = s->ws_step.ln_stats && ctx->ln_fold && model_ln_fold_supported(m, B); // as decode_step
    cudaEvent_t e0, e1;
    CK(ctx, cudaEventCreate(&e0));
    CK(ctx, cudaEventCreate(&e1));
    const uint64_t before = ctx->launches;
    uint64_t per_pass = 0;
    int rc = B200NN_OK;
    // the launches of one step that belong to the family, issued directly (the forward pass itself
    // carries no measurement switches)
    auto one_pass = [&]() -> int {
        for (int l = 0; l < m->cfg.n_layer; ++l) {
            const BlockLaunch bl{m, s->ws_step, s->kv, l, B, 1, s->pos_ptr(), 0, ah, fold};
            if (family == B200NN_PROF_LAYERNORM) {
                TRY(bl.ln1());
                TRY(bl.ln2());
            } else if (family == B200NN_PROF_LINEAR) {
                TRY(bl.qkv());
                TRY(bl.proj());
                TRY(bl.fc());
                TRY(bl.fcproj());
            } else if (family == B200NN_PROF_ATTENTION) {
                TRY(bl.attention());
            }
        }
        const bool hh = head_act_half(m, B, ah);
        if (family == B200NN_PROF_LAYERNORM) TRY(launch_head_norm(m, s->ws_step, (const float *)s->ws_step.x->p, B, hh));
        if (family == B200NN_PROF_LM_HEAD) TRY(launch_head_linear(m, s->ws_step, B, hh));
        return B200NN_OK;
    };
    // one untimed pass sizes scratch and warms the instruction cache
    for (int r = -1; r < reps && rc == B200NN_OK; ++r) {
        if (r == 0) cudaEventRecord(e0, ctx->stream);
        rc = one_pass();
        if (r == -1) per_pass = ctx->launches - before;
    }
    cudaEventRecord(e1, ctx->stream);
    cudaError_t ce = cudaStreamSynchronize(ctx->stream);
    float ms = 0.0f;
    cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    TRY(rc);
    if (ce != cudaSuccess) return set_cuda_error(ctx, ce, "time_family");
    *ms_total = ms;
    if (launches) *launches = per_pass * (uint64_t)reps;
    return B200NN_OK;
}

// ---------------------------------------------------------------------------------------------
// greedy generation
// ---------------------------------------------------------------------------------------------
extern "C" int32_t b200nn_gpt2_generate_batch(b200nn_gpt2 *m, const uint32_t *prompts, size_t batch,
                                              size_t prompt_len, size_t max_new, uint32_t flags,
                                              uint32_t *out_tokens, size_t *out_lens) {
    if (!m || !prompts || !out_tokens) return B200NN_ERR_ARG;
    b200nn_ctx *ctx = m->ctx;
    if (batch == 0 || prompt_len == 0) return set_error(ctx, B200NN_ERR_SHAPE, "generate: empty batch or prompt");
    if (prompt_len + max_new > (size_t)m->cfg.n_positions)
        return set_error(ctx, B200NN_ERR_DIM, "generate: prompt_len + max_new exceeds n_positions");
    const size_t stride = prompt_len + max_new;
    for (size_t b = 0; b < batch; ++b) {
        memcpy(out_tokens + b * stride, prompts + b * prompt_len, prompt_len * 4);
        if (out_lens) out_lens[b] = prompt_len;
    }
    if (max_new == 0) return B200NN_OK;
    b200nn_session *s = nullptr;
    TRY(b200nn_session_create(m, batch, stride, flags | B200NN_TOKENS_ONLY, &s)); // greedy tokens are all that is returned
    std::unique_ptr<b200nn_session, void (*)(b200nn_session *)> guard(s, b200nn_session_destroy);
    TRY(b200nn_session_prefill(s, prompts, prompt_len));
    TRY(b200nn_session_step(s, max_new - 1));
    std::vector<uint32_t> gen(batch * max_new);
    size_t n = 0;
    TRY(b200nn_session_tokens(s, gen.data(), max_new, &n));
    for (size_t b = 0; b < batch; ++b) {
        size_t len = n;
        if (flags & B200NN_STOP_ON_EOS) // stop before appending <|endoftext|> (gpt2.rs:698-700)
            for (size_t i = 0; i < n; ++i)
                if (gen[b * max_new + i] == 50256u) { len = i; break; }
        memcpy(out_tokens + b * stride + prompt_len, gen.data() + b * max_new, len * 4);
        if (out_lens) out_lens[b] = prompt_len + len;
    }
    return B200NN_OK;
}

extern "C" int32_t b200nn_gpt2_generate_cached(b200nn_gpt2 *m, const uint32_t *prompt, size_t prompt_len,
                                               size_t max_new, uint32_t flags, uint32_t *out_tokens, size_t *n_out) {
    size_t len = 0;
    int rc = b200nn_gpt2_generate_batch(m, prompt, 1, prompt_len, max_new, flags, out_tokens, &len);
    if (rc == B200NN_OK && n_out) *n_out = len;
    return rc;
}

extern "C" int32_t b200nn_gpt2_generate(b200nn_gpt2 *m, const uint32_t *prompt, size_t prompt_len, size_t max_new,
                                        uint32_t flags, uint32_t *out_tokens, size_t *n_out) {
    return b200nn_gpt2_generate_cached(m, prompt, prompt_len, max_new, flags, out_tokens, n_out);
}
