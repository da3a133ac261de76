// Data-dependent decoding: top-k sampling with temperature and early exit by confidence
// (crates/core/gpu-host/src/nn/models/gpt2.rs:785-1058).
//
// The reference runs these loops on the host with the logits copied back every step (and a full
// sort of the vocabulary per sampled token).  Here the model's work stays on the device and only
// what the host decision needs crosses over: the k best scaled logits with their indices for
// sampling (k x 8 bytes), one confidence value per probed layer for early exit, one token id per
// step.  The sampler itself (softmax over the k candidates, one draw from SimpleRng, cumulative
// search) is the reference's f32 arithmetic on the host, so that with equal candidates the draw is
// the same.
#include <algorithm>
#include <cmath>

#include "device_utils.cuh"
#include "model.h"

// ---------------------------------------------------------------------------------------------
// SimpleRng (gpt2.rs:1000-1023) and top_k_sample (gpt2.rs:1029-1058) on host arrays
// ---------------------------------------------------------------------------------------------
extern "C" uint64_t b200nn_simple_rng_new(uint64_t seed) { return seed ? seed : 0xDEADBEEFCAFE1234ull; }
extern "C" float b200nn_simple_rng_next_f32(uint64_t *state);

// Synthetic tensors a Rust caller can regenerate bit for bit with the reference's own SimpleRng:
// uniforms are next_f32; normals are Box-Muller in f64 on consecutive pairs (u1, u2) of uniforms,
// z0 = sqrt(-2 ln(1 - u1)) cos(2 pi u2), z1 = sqrt(-2 ln(1 - u1)) sin(2 pi u2), scaled by std and cast
// to f32 (1 - u1 lies in (0, 1], so the logarithm is finite); an odd count drops the last z1.
extern "C" int32_t b200nn_simple_rng_fill_uniform(uint64_t *state, size_t n, float *out) {
    if (!state || (!out && n)) return B200NN_ERR_ARG;
    for (size_t i = 0; i < n; ++i) out[i] = b200nn_simple_rng_next_f32(state);
    return B200NN_OK;
}
extern "C" int32_t b200nn_simple_rng_fill_normal(uint64_t *state, size_t n, float std_dev, float *out) {
    if (!state || (!out && n)) return B200NN_ERR_ARG;
    const double two_pi = 6.283185307179586476925286766559;
    for (size_t i = 0; i < n; i += 2) {
        const double u1 = (double)b200nn_simple_rng_next_f32(state), u2 = (double)b200nn_simple_rng_next_f32(state);
        const double r = sqrt(-2.0 * log(1.0 - u1));
        out[i] = (float)(r * cos(two_pi * u2) * (double)std_dev);
        if (i + 1 < n) out[i + 1] = (float)(r * sin(two_pi * u2) * (double)std_dev);
    }
    return B200NN_OK;
}

extern "C" float b200nn_simple_rng_next_f32(uint64_t *state) {
    uint64_t x = *state;
    x ^= x << 13;
    x ^= x >> 7;
    x ^= x << 17;
    *state = x;
    return (float)(x >> 40) / 16777216.0f;
}

namespace {

// Softmax over the candidates (already scaled by 1/temperature, best first), one draw, cumulative
// search: gpt2.rs:1044-1057.  f32 throughout, sums in index order.
uint32_t sample_from_candidates(const float *vals, const uint32_t *idx, size_t k, uint64_t *rng) {
    const float max_val = vals[0];
    std::vector<float> p(k);
    float sum = 0.0f;
    for (size_t i = 0; i < k; ++i) {
        p[i] = expf(vals[i] - max_val);
        sum += p[i];
    }
    const float r = b200nn_simple_rng_next_f32(rng);
    float cum = 0.0f;
    for (size_t i = 0; i < k; ++i) {
        cum += p[i] / sum;
        if (r < cum) return idx[i];
    }
    return idx[k - 1];
}

inline float clamp_temperature(float t) { return t < 1e-8f ? 1e-8f : t; }

}  // namespace

extern "C" int32_t b200nn_top_k_sample(const float *logits, size_t n, size_t k, float temperature, uint64_t *rng_state,
                                       uint32_t *token_out) {
    if (!logits || !rng_state || !token_out || n == 0 || k == 0) return B200NN_ERR_ARG;
    const float temp = clamp_temperature(temperature);
    k = std::min(k, n);
    std::vector<float> scaled(n);
    for (size_t i = 0; i < n; ++i) scaled[i] = logits[i] / temp;
    std::vector<uint32_t> order(n);
    for (size_t i = 0; i < n; ++i) order[i] = (uint32_t)i;
    // the reference's stable descending sort: equal values keep ascending index order
    std::partial_sort(order.begin(), order.begin() + k, order.end(), [&](uint32_t a, uint32_t b) {
        return scaled[a] > scaled[b] || (scaled[a] == scaled[b] && a < b);
    });
    std::vector<float> vals(k);
    for (size_t i = 0; i < k; ++i) vals[i] = scaled[order[i]];
    *token_out = sample_from_candidates(vals.data(), order.data(), k, rng_state);
    return B200NN_OK;
}

// ---------------------------------------------------------------------------------------------
// device kernels
// ---------------------------------------------------------------------------------------------
namespace {

struct Cand {
    float v;
    int i;
};
// order of the reference's sorted list: larger value first, equal values by ascending index
__device__ __forceinline__ bool cand_before(const Cand &a, const Cand &b) { return a.v > b.v || (a.v == b.v && a.i < b.i); }

__device__ __forceinline__ Cand block_best(Cand c, Cand *sm) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Cand t;
        t.v = __shfl_xor_sync(0xffffffffu, c.v, o);
        t.i = __shfl_xor_sync(0xffffffffu, c.i, o);
        if (t.i >= 0 && (c.i < 0 || cand_before(t, c))) c = t;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    __syncthreads();
    if (lane == 0) sm[warp] = c;
    __syncthreads();
    Cand r = sm[0];
    for (int w = 1; w < nw; ++w)
        if (sm[w].i >= 0 && (r.i < 0 || cand_before(sm[w], r))) r = sm[w];
    return r;
}

// One block: writes x/temp for the whole row into `scaled`, then selects the k first entries of the
// row's descending order one after the other (each pass finds the best entry that comes after the
// previous pick in that order).  k passes over an L2-resident row.
__global__ void __launch_bounds__(1024)
topk_scaled_kernel(const float *__restrict__ logits, int n, int k, float temp, float *__restrict__ scaled,
                   float *__restrict__ out_vals, uint32_t *__restrict__ out_idx) {
    __shared__ Cand sm[32];
    for (int i = threadIdx.x; i < n; i += blockDim.x) scaled[i] = logits[i] / temp;
    __syncthreads();
    Cand prev;
    prev.v = INFINITY;
    prev.i = -1;
    for (int r = 0; r < k; ++r) {
        Cand best;
        best.v = -INFINITY;
        best.i = -1;
        for (int i = threadIdx.x; i < n; i += blockDim.x) {
            Cand c;
            c.v = scaled[i];
            c.i = i;
            const bool after_prev = prev.i < 0 || cand_before(prev, c);
            if (after_prev && (best.i < 0 || cand_before(c, best))) best = c;
        }
        best = block_best(best, sm);
        if (threadIdx.x == 0) {
            out_vals[r] = best.v;
            out_idx[r] = (uint32_t)max(best.i, 0);
        }
        prev = best;
        if (best.i < 0) break; // fewer than k comparable entries (NaNs): the rest stays as written
    }
}

// softmax_max_prob (gpt2.rs:980-985): 1 / sum(exp(x - max)) of one row, f32.
__global__ void __launch_bounds__(1024) max_prob_kernel(const float *__restrict__ x, int n, float *__restrict__ out) {
    float m = -INFINITY;
    for (int i = threadIdx.x; i < n; i += blockDim.x) m = fmaxf(m, x[i]);
    __shared__ float sm[32];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) sm[warp] = m;
    __syncthreads();
    m = sm[0];
    for (int w = 1; w < nw; ++w) m = fmaxf(m, sm[w]);
    __syncthreads();
    float s = 0.0f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) s += expf(x[i] - m);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) sm[warp] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.0f;
        for (int w = 0; w < nw; ++w) t += sm[w];
        out[0] = 1.0f / t;
    }
}

// K and V rows of position `pos` set to zero for layers [l0, l1): what the reference appends to
// the caches of the layers an early exit skips (gpt2.rs:897-904).
__global__ void zero_kv_rows_kernel(__half *__restrict__ k, __half *__restrict__ v, size_t layer_stride, int l0, int l1,
                                    int pairs, int cap, int pos) {
    const int total = (l1 - l0) * pairs * 64;
    for (int t = blockIdx.x * blockDim.x + threadIdx.x; t < total; t += gridDim.x * blockDim.x) {
        const int e = t & 63, pr = (t >> 6) % pairs, l = l0 + (t >> 6) / pairs;
        const size_t off = (size_t)l * layer_stride + ((size_t)pr * cap + pos) * 64 + e;
        k[off] = __float2half(0.0f);
        v[off] = __float2half(0.0f);
    }
}

struct CacheGuard { // owns a cache created through the public entry point
    b200nn_kvcache *c = nullptr;
    ~CacheGuard() { b200nn_kvcache_destroy(c); }
};

// Embeds S tokens of one sequence at positions past.. into ws.x.
int embed_one(b200nn_gpt2 *m, Workspace &ws, const uint32_t *ids_host, int S, int past) {
    b200nn_ctx *ctx = m->ctx;
    for (int i = 0; i < S; ++i)
        if (ids_host[i] >= (uint32_t)m->cfg.vocab_size) return set_error(ctx, B200NN_ERR_DIM, "token id out of range for vocab_size");
    CK(ctx, cudaMemcpyAsync(ws.ids->p, ids_host, (size_t)S * 4, cudaMemcpyHostToDevice, ctx->stream));
    CK(ctx, cudaStreamSynchronize(ctx->stream)); // ids_host may be a stack variable of the caller
    return launch_embedding(ctx, (const uint32_t *)ws.ids->p, (const float *)m->wte->p, (const float *)m->wpe->p, S,
                            m->cfg.n_embd, S, nullptr, past, m->cfg.vocab_size, m->cfg.n_positions, (float *)ws.x->p);
}

// Prefill of one prompt through all layers; logits of the last position end up in ws1.logits.
int prefill_one(b200nn_gpt2 *m, b200nn_kvcache &kv, Workspace &ws1, const uint32_t *prompt, int n) {
    b200nn_ctx *ctx = m->ctx;
    Workspace wsp;
    TRY(workspace_alloc(m, (size_t)n, 1, &wsp));
    const bool ah = model_act_half(m, n);
    TRY(embed_one(m, wsp, prompt, n, 0));
    TRY(run_blocks(m, wsp, kv, 1, n, nullptr, 0, ah, nullptr));
    kv.len = (size_t)n;
    TRY(launch_gather_last_rows(ctx, (const float *)wsp.x->p, 1, n, m->cfg.n_embd, (float *)ws1.last_x->p));
    TRY(run_head(m, ws1, (const float *)ws1.last_x->p, 1, model_act_half(m, 1), nullptr));
    CK(ctx, cudaStreamSynchronize(ctx->stream)); // wsp goes out of scope
    return B200NN_OK;
}

// The k best of ws.logits row 0 (scaled by 1/temp) -> host, then the reference's draw.
int sample_row(b200nn_gpt2 *m, Workspace &ws, size_t k, float temp, uint64_t *rng, uint32_t *token) {
    b200nn_ctx *ctx = m->ctx;
    const int V = m->cfg.vocab_size;
    const size_t kk = std::min<size_t>(k, (size_t)V);
    TRY(ensure_scratch(ctx, (size_t)V * 4 + kk * 8 + 64, 0));
    float *scaled = ctx->scratch;
    float *vals_d = scaled + ((V + 3) & ~3);
    uint32_t *idx_d = reinterpret_cast<uint32_t *>(vals_d + kk);
    topk_scaled_kernel<<<1, 1024, 0, ctx->stream>>>((const float *)ws.logits->p, V, (int)kk, temp, scaled, vals_d, idx_d);
    CK_LAUNCH(ctx, "topk_scaled_kernel");
    std::vector<float> vals(kk);
    std::vector<uint32_t> idx(kk);
    CK(ctx, cudaMemcpyAsync(vals.data(), vals_d, kk * 4, cudaMemcpyDeviceToHost, ctx->stream));
    CK(ctx, cudaMemcpyAsync(idx.data(), idx_d, kk * 4, cudaMemcpyDeviceToHost, ctx->stream));
    TRY(stream_sync_check(ctx));
    *token = sample_from_candidates(vals.data(), idx.data(), kk, rng);
    return B200NN_OK;
}

int max_prob_of_row(b200nn_gpt2 *m, const float *row, float *conf_host) {
    b200nn_ctx *ctx = m->ctx;
    TRY(ensure_scratch(ctx, 64, 0));
    max_prob_kernel<<<1, 1024, 0, ctx->stream>>>(row, m->cfg.vocab_size, ctx->scratch);
    CK_LAUNCH(ctx, "max_prob_kernel");
    CK(ctx, cudaMemcpyAsync(conf_host, ctx->scratch, 4, cudaMemcpyDeviceToHost, ctx->stream));
    TRY(stream_sync_check(ctx));
    return B200NN_OK;
}

int argmax_row(b200nn_gpt2 *m, Workspace &ws, uint32_t *token) {
    b200nn_ctx *ctx = m->ctx;
    // the reference's argmax keeps the last of equal maxima (gpt2.rs:991-997)
    TRY(launch_argmax(ctx, (const float *)ws.logits->p, 1, m->cfg.vocab_size, m->cfg.vocab_size, true, (uint32_t *)ws.tok->p));
    CK(ctx, cudaMemcpyAsync(token, ws.tok->p, 4, cudaMemcpyDeviceToHost, ctx->stream));
    TRY(stream_sync_check(ctx));
    return B200NN_OK;
}

}  // namespace

// Gpt2Model::generate_cached_sampling (gpt2.rs:933-977).
extern "C" int32_t b200nn_gpt2_generate_cached_sampling(b200nn_gpt2 *m, const uint32_t *prompt, size_t prompt_len,
                                                        size_t max_new, size_t top_k, float temperature,
                                                        uint64_t *rng_state, uint32_t *out_tokens, size_t *n_out) {
    if (!m || !prompt || !rng_state || !out_tokens || !n_out) return B200NN_ERR_ARG;
    b200nn_ctx *ctx = m->ctx;
    if (prompt_len == 0 || top_k == 0) return set_error(ctx, B200NN_ERR_SHAPE, "sampling: empty prompt or top_k == 0");
    if (prompt_len + max_new > (size_t)m->cfg.n_positions)
        return set_error(ctx, B200NN_ERR_DIM, "sampling: prompt_len + max_new exceeds n_positions");
    CK(ctx, cudaSetDevice(ctx->device));
    const float temp = clamp_temperature(temperature);
    std::copy(prompt, prompt + prompt_len, out_tokens);
    size_t n = prompt_len;
    *n_out = n;
    if (max_new == 0) return B200NN_OK;
    CacheGuard g;
    TRY(b200nn_kvcache_create(m, 1, prompt_len + max_new, &g.c));
    b200nn_kvcache &kv = *g.c;
    Workspace ws;
    TRY(workspace_alloc(m, 1, 1, &ws));
    TRY(prefill_one(m, kv, ws, prompt, (int)prompt_len));
    uint32_t tok = 0;
    TRY(sample_row(m, ws, top_k, temp, rng_state, &tok));
    for (size_t step = 0;; ++step) {
        if (tok == 50256u) break; // stop before appending (gpt2.rs:958-960, 970-972)
        out_tokens[n++] = tok;
        if (step + 1 >= max_new) break;
        TRY(embed_one(m, ws, &tok, 1, (int)kv.len));
        TRY(run_blocks(m, ws, kv, 1, 1, nullptr, (int)kv.len, model_act_half(m, 1), nullptr));
        kv.len += 1;
        TRY(run_head(m, ws, (const float *)ws.x->p, 1, model_act_half(m, 1), nullptr));
        TRY(sample_row(m, ws, top_k, temp, rng_state, &tok));
    }
    *n_out = n;
    return B200NN_OK;
}

// Gpt2Model::forward_early_exit (gpt2.rs:797-830): after every block but the last, LN_f + LM head over
// all positions; if the largest softmax probability at the last position reaches the threshold, those
// logits are returned together with the number of blocks run.
extern "C" int32_t b200nn_gpt2_forward_early_exit(b200nn_gpt2 *m, const uint32_t *ids_host, size_t seq_len,
                                                  float threshold, b200nn_tensor **logits, int32_t *layers_used) {
    if (!m || !ids_host || !logits || !layers_used) return B200NN_ERR_ARG;
    b200nn_ctx *ctx = m->ctx;
    if (seq_len == 0 || seq_len > (size_t)m->cfg.n_positions)
        return set_error(ctx, B200NN_ERR_DIM, "forward_early_exit: seq_len must be in [1, n_positions]");
    CK(ctx, cudaSetDevice(ctx->device));
    const int S = (int)seq_len, L = m->cfg.n_layer, V = m->cfg.vocab_size;
    CacheGuard g;
    TRY(b200nn_kvcache_create(m, 1, seq_len, &g.c));
    Workspace ws;
    TRY(workspace_alloc(m, seq_len, seq_len, &ws));
    const bool ah = model_act_half(m, S);
    TRY(embed_one(m, ws, ids_host, S, 0));
    int used = L;
    bool have_logits = false;
    for (int l = 0; l < L; ++l) {
        TRY(run_blocks_range(m, ws, *g.c, 1, S, nullptr, 0, ah, nullptr, l, l + 1));
        if (l < L - 1) {
            TRY(run_head(m, ws, (const float *)ws.x->p, S, ah, nullptr));
            float conf = 0.0f;
            TRY(max_prob_of_row(m, (const float *)ws.logits->p + (size_t)(S - 1) * V, &conf));
            if (conf >= threshold) {
                used = l + 1;
                have_logits = true;
                break;
            }
        }
    }
    if (!have_logits) TRY(run_head(m, ws, (const float *)ws.x->p, S, ah, nullptr));
    b200nn_tensor *t = nullptr;
    TRY(tensor_alloc(ctx, {seq_len, (size_t)V}, false, &t));
    cudaError_t e = cudaMemcpyAsync(t->buf->p, ws.logits->p, t->numel * 4, cudaMemcpyDeviceToDevice, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) {
        delete t;
        return set_cuda_error(ctx, e, "forward_early_exit copy");
    }
    *logits = t;
    *layers_used = used;
    return B200NN_OK;
}

// Gpt2Model::generate_cached_early_exit (gpt2.rs:837-924): the prefill uses every layer; a decode step
// stops at the first block (but the last) after which the probe's confidence reaches the threshold,
// gives the skipped layers zero K/V rows for that position, and picks the token from the probe.
extern "C" int32_t b200nn_gpt2_generate_cached_early_exit(b200nn_gpt2 *m, const uint32_t *prompt, size_t prompt_len,
                                                          size_t max_new, float threshold, uint32_t *out_tokens,
                                                          size_t *n_out, int32_t *layers_per_step, size_t *n_steps) {
    if (!m || !prompt || !out_tokens || !n_out || !layers_per_step || !n_steps) return B200NN_ERR_ARG;
    b200nn_ctx *ctx = m->ctx;
    if (prompt_len == 0) return set_error(ctx, B200NN_ERR_SHAPE, "early exit: empty prompt");
    if (prompt_len + max_new > (size_t)m->cfg.n_positions)
        return set_error(ctx, B200NN_ERR_DIM, "early exit: prompt_len + max_new exceeds n_positions");
    CK(ctx, cudaSetDevice(ctx->device));
    const int L = m->cfg.n_layer, H = m->cfg.n_head;
    std::copy(prompt, prompt + prompt_len, out_tokens);
    size_t n = prompt_len, steps = 0;
    *n_out = n;
    *n_steps = 0;
    if (max_new == 0) return B200NN_OK;
    CacheGuard g;
    TRY(b200nn_kvcache_create(m, 1, prompt_len + max_new, &g.c));
    b200nn_kvcache &kv = *g.c;
    Workspace ws;
    TRY(workspace_alloc(m, 1, 1, &ws));
    TRY(prefill_one(m, kv, ws, prompt, (int)prompt_len));
    layers_per_step[steps++] = L;
    uint32_t tok = 0;
    TRY(argmax_row(m, ws, &tok));
    const bool ah = model_act_half(m, 1);
    for (size_t step = 0;; ++step) {
        if (tok == 50256u) break;
        out_tokens[n++] = tok;
        if (step + 1 >= max_new) break;
        const int pos = (int)kv.len;
        TRY(embed_one(m, ws, &tok, 1, pos));
        int used = L;
        bool have_logits = false;
        for (int l = 0; l < L; ++l) {
            TRY(run_blocks_range(m, ws, kv, 1, 1, nullptr, pos, ah, nullptr, l, l + 1));
            if (l < L - 1) {
                TRY(run_head(m, ws, (const float *)ws.x->p, 1, ah, nullptr));
                float conf = 0.0f;
                TRY(max_prob_of_row(m, (const float *)ws.logits->p, &conf));
                if (conf >= threshold) {
                    zero_kv_rows_kernel<<<std::max(1, std::min(64, (L - l - 1) * H)), 256, 0, ctx->stream>>>(
                        static_cast<__half *>(kv.k->p), static_cast<__half *>(kv.v->p), kv.layer_stride(), l + 1, L, H,
                        (int)kv.cap, pos);
                    CK_LAUNCH(ctx, "zero_kv_rows_kernel");
                    used = l + 1;
                    have_logits = true;
                    break;
                }
            }
        }
        kv.len += 1;
        layers_per_step[steps++] = used;
        if (!have_logits) TRY(run_head(m, ws, (const float *)ws.x->p, 1, ah, nullptr));
        TRY(argmax_row(m, ws, &tok));
    }
    *n_out = n;
    *n_steps = steps;
    return B200NN_OK;
}

// ---------------------------------------------------------------------------------------------
// forward_features, embedding_table, forward_profiled (gpt2.rs:529-590)
// ---------------------------------------------------------------------------------------------

// Gpt2Model::forward_features (gpt2.rs:570-581): the hidden states after every block and the final
// LayerNorm, [seq_len, n_embd] f32, for callers that bring their own head.
extern "C" int32_t b200nn_gpt2_forward_features(b200nn_gpt2 *m, const uint32_t *ids_host, size_t seq_len,
                                                b200nn_tensor **features) {
    if (!m || !ids_host || !features) return B200NN_ERR_ARG;
    b200nn_ctx *ctx = m->ctx;
    if (seq_len == 0 || seq_len > (size_t)m->cfg.n_positions)
        return set_error(ctx, B200NN_ERR_DIM, "forward_features: seq_len must be in [1, n_positions]");
    CK(ctx, cudaSetDevice(ctx->device));
    const int S = (int)seq_len, d = m->cfg.n_embd;
    CacheGuard g;
    TRY(b200nn_kvcache_create(m, 1, seq_len, &g.c));
    Workspace ws;
    TRY(workspace_alloc(m, seq_len, 1, &ws));
    TRY(embed_one(m, ws, ids_host, S, 0));
    TRY(run_blocks(m, ws, *g.c, 1, S, nullptr, 0, model_act_half(m, S), nullptr));
    b200nn_tensor *t = nullptr;
    TRY(tensor_alloc(ctx, {seq_len, (size_t)d}, false, &t));
    int rc = launch_layernorm(ctx, (const float *)ws.x->p, nullptr, nullptr, (const float *)m->lnf_g->p,
                              (const float *)m->lnf_b->p, m->cfg.layer_norm_epsilon, S, d, t->buf->p, false);
    cudaError_t e = rc == B200NN_OK ? cudaStreamSynchronize(ctx->stream) : cudaSuccess;
    if (rc != B200NN_OK || e != cudaSuccess) {
        delete t;
        return rc != B200NN_OK ? rc : set_cuda_error(ctx, e, "forward_features");
    }
    *features = t;
    return B200NN_OK;
}

// Gpt2Model::embedding_table (gpt2.rs:584-586): the token and position tables as tensors sharing the
// model's device buffers ([vocab, n_embd] and [n_positions, n_embd]); destroy them like any tensor.
extern "C" int32_t b200nn_gpt2_embedding_table(b200nn_gpt2 *m, b200nn_tensor **wte, b200nn_tensor **wpe) {
    if (!m || !wte || !wpe) return B200NN_ERR_ARG;
    const size_t d = (size_t)m->cfg.n_embd;
    auto view = [&](const std::shared_ptr<DevBuf> &buf, size_t rows) {
        auto *t = new b200nn_tensor();
        t->ctx = m->ctx;
        t->buf = buf;
        t->shape = {rows, d};
        t->numel = rows * d;
        return t;
    };
    *wte = view(m->wte, (size_t)m->cfg.vocab_size);
    *wpe = view(m->wpe, (size_t)m->cfg.n_positions);
    return B200NN_OK;
}

// Gpt2Model::forward_profiled (gpt2.rs:529-568): forward with the device time of every component,
// in the reference's order: embedding, block_0 .. block_{L-1}, ln_f, lm_head (CUDA events on the
// context's stream instead of the reference's host clock around synchronisations).
extern "C" int32_t b200nn_gpt2_forward_profiled(b200nn_gpt2 *m, const uint32_t *ids_host, size_t seq_len,
                                                b200nn_tensor **logits, float *times_ms, int32_t capacity,
                                                int32_t *n_times) {
    if (!m || !ids_host || !logits || !times_ms || !n_times) return B200NN_ERR_ARG;
    b200nn_ctx *ctx = m->ctx;
    const int L = m->cfg.n_layer, S = (int)seq_len, V = m->cfg.vocab_size;
    if (seq_len == 0 || seq_len > (size_t)m->cfg.n_positions)
        return set_error(ctx, B200NN_ERR_DIM, "forward_profiled: seq_len must be in [1, n_positions]");
    if (capacity < L + 3) return set_error(ctx, B200NN_ERR_SHAPE, "forward_profiled: times_ms needs n_layer + 3 entries");
    CK(ctx, cudaSetDevice(ctx->device));
    CacheGuard g;
    TRY(b200nn_kvcache_create(m, 1, seq_len, &g.c));
    Workspace ws;
    TRY(workspace_alloc(m, seq_len, seq_len, &ws));
    const bool ah = model_act_half(m, S);
    std::vector<cudaEvent_t> ev((size_t)L + 4);
    for (auto &e : ev) CK(ctx, cudaEventCreate(&e));
    auto cleanup = [&]() { for (auto &e : ev) cudaEventDestroy(e); };
    int rc = B200NN_OK;
    size_t k = 0;
    auto mark = [&]() { cudaEventRecord(ev[k++], ctx->stream); };
    mark();
    rc = embed_one(m, ws, ids_host, S, 0);
    mark();
    for (int l = 0; l < L && rc == B200NN_OK; ++l) {
        rc = run_blocks_range(m, ws, *g.c, 1, S, nullptr, 0, ah, nullptr, l, l + 1);
        mark();
    }
    StepProfile head; // run_head marks after the final LayerNorm and after the LM head
    if (rc == B200NN_OK) rc = run_head(m, ws, (const float *)ws.x->p, S, ah, &head);
    b200nn_tensor *t = nullptr;
    if (rc == B200NN_OK) rc = tensor_alloc(ctx, {seq_len, (size_t)V}, false, &t);
    if (rc == B200NN_OK) {
        cudaError_t e = cudaMemcpyAsync(t->buf->p, ws.logits->p, t->numel * 4, cudaMemcpyDeviceToDevice, ctx->stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
        if (e != cudaSuccess) rc = set_cuda_error(ctx, e, "forward_profiled copy");
    }
    if (rc == B200NN_OK && head.ev.size() == 2) {
        for (int i = 0; i < L + 1; ++i) cudaEventElapsedTime(&times_ms[i], ev[i], ev[i + 1]);
        cudaEventElapsedTime(&times_ms[L + 1], ev[L + 1], head.ev[0]);
        cudaEventElapsedTime(&times_ms[L + 2], head.ev[0], head.ev[1]);
        *n_times = L + 3;
    } else if (rc == B200NN_OK) {
        rc = set_error(ctx, B200NN_ERR_CUDA, "forward_profiled: missing head events");
    }
    for (auto &e : head.ev) cudaEventDestroy(e);
    cleanup();
    if (rc != B200NN_OK) {
        delete t;
        return rc;
    }
    *logits = t;
    return B200NN_OK;
}

// Gpt2Model::forward_diagnostic (gpt2.rs:595-667): forward of one sequence that also reports the values
// the reference prints to stderr: the first four hidden values after the embedding (position 0 and the
// last position), after block 0 and after the last block (last position, with the count of non-finite
// values of the whole hidden state), after the final LayerNorm, and the five best tokens of the last
// position.  The reference hard-codes "block 11"; here it is the model's last block.
extern "C" int32_t b200nn_gpt2_forward_diagnostic(b200nn_gpt2 *m, const uint32_t *ids_host, size_t seq_len,
                                                  b200nn_tensor **logits, b200nn_gpt2_diagnostic *diag) {
    if (!m || !ids_host || !logits || !diag) return B200NN_ERR_ARG;
    b200nn_ctx *ctx = m->ctx;
    const int L = m->cfg.n_layer, S = (int)seq_len, V = m->cfg.vocab_size, d = m->cfg.n_embd;
    if (seq_len == 0 || seq_len > (size_t)m->cfg.n_positions)
        return set_error(ctx, B200NN_ERR_DIM, "forward_diagnostic: seq_len must be in [1, n_positions]");
    CK(ctx, cudaSetDevice(ctx->device));
    memset(diag, 0, sizeof(*diag));
    CacheGuard g;
    TRY(b200nn_kvcache_create(m, 1, seq_len, &g.c));
    Workspace ws;
    TRY(workspace_alloc(m, seq_len, seq_len, &ws));
    const bool ah = model_act_half(m, S);
    std::vector<float> h((size_t)S * d);
    auto fetch = [&](const void *src) -> int {
        CK(ctx, cudaMemcpyAsync(h.data(), src, h.size() * 4, cudaMemcpyDeviceToHost, ctx->stream));
        return stream_sync_check(ctx);
    };
    auto count_bad = [&]() {
        int32_t n = 0;
        for (float v : h) n += !std::isfinite(v);
        return n;
    };
    const size_t last = (size_t)(S - 1) * d;
    TRY(embed_one(m, ws, ids_host, S, 0));
    TRY(fetch(ws.x->p));
    for (int i = 0; i < 4 && i < d; ++i) {
        diag->embedding_first[i] = h[i];
        diag->embedding_last[i] = h[last + i];
    }
    for (int l = 0; l < L; ++l) {
        TRY(run_blocks_range(m, ws, *g.c, 1, S, nullptr, 0, ah, nullptr, l, l + 1));
        if (l == 0 || l == L - 1) {
            TRY(fetch(ws.x->p));
            float *dst = l == 0 ? diag->block0_last : diag->final_block_last;
            for (int i = 0; i < 4 && i < d; ++i) dst[i] = h[last + i];
            (l == 0 ? diag->block0_nonfinite : diag->final_block_nonfinite) = count_bad();
            if (L == 1) {
                memcpy(diag->final_block_last, diag->block0_last, sizeof(diag->block0_last));
                diag->final_block_nonfinite = diag->block0_nonfinite;
            }
        }
    }
    // final LayerNorm in f32 for the report, then the regular head
    std::shared_ptr<DevBuf> lnf;
    TRY(dev_alloc(ctx, h.size() * 4, &lnf));
    TRY(launch_layernorm(ctx, (const float *)ws.x->p, nullptr, nullptr, (const float *)m->lnf_g->p, (const float *)m->lnf_b->p,
                         m->cfg.layer_norm_epsilon, S, d, lnf->p, false));
    TRY(fetch(lnf->p));
    for (int i = 0; i < 4 && i < d; ++i) diag->ln_f_last[i] = h[last + i];
    TRY(run_head(m, ws, (const float *)ws.x->p, S, ah, nullptr));
    b200nn_tensor *t = nullptr;
    TRY(tensor_alloc(ctx, {seq_len, (size_t)V}, false, &t));
    std::vector<float> row((size_t)V);
    cudaError_t e = cudaMemcpyAsync(t->buf->p, ws.logits->p, t->numel * 4, cudaMemcpyDeviceToDevice, ctx->stream);
    if (e == cudaSuccess)
        e = cudaMemcpyAsync(row.data(), (const float *)ws.logits->p + (size_t)(S - 1) * V, (size_t)V * 4, cudaMemcpyDeviceToHost,
                            ctx->stream);
    int rc = e == cudaSuccess ? stream_sync_check(ctx) : set_cuda_error(ctx, e, "forward_diagnostic copy");
    if (rc != B200NN_OK) {
        delete t;
        return rc;
    }
    // stable descending order, as the reference's sort_by on (index, value) pairs
    std::vector<int> idx((size_t)V);
    for (int i = 0; i < V; ++i) idx[i] = i;
    const int k = std::min(5, V);
    std::stable_sort(idx.begin(), idx.end(), [&](int a, int b) { return row[a] > row[b]; });
    for (int i = 0; i < k; ++i) {
        diag->top_tokens[i] = (uint32_t)idx[i];
        diag->top_scores[i] = row[idx[i]];
    }
    diag->n_top = k;
    *logits = t;
    return B200NN_OK;
}
