// Model-level structures: layers, GPT-2 model, KV cache, decode session.
#pragma once
#include "common.h"

struct LinearAny {
    bool int4 = false;
    Int4Weight q;
    F32Weight f;
    int K = 0, N = 0;
    const float *bias() const {
        const std::shared_ptr<DevBuf> &b = int4 ? q.bias : f.bias;
        return b ? static_cast<const float *>(b->p) : nullptr;
    }
    // algorithmic bytes of the weight side (nibbles + fp16 scales, or f32 weights) plus bias
    size_t weight_bytes() const {
        if (int4) return (size_t)K * N / 2 + (size_t)q.n_groups * N * 2 + (q.bias ? (size_t)N * 4 : 0);
        return (size_t)K * N * 4 + (f.bias ? (size_t)N * 4 : 0);
    }
};
int linear_forward(b200nn_ctx *ctx, const LinearAny &l, const void *x, bool x_half, int M, Epilogue epi);

struct b200nn_linear {
    b200nn_ctx *ctx;
    LinearAny l;
};
struct b200nn_int4_linear {
    b200nn_ctx *ctx;
    LinearAny l;
    std::shared_ptr<DevBuf> xh; // fp16 staging of the input when the tensor-core path is taken
};
struct b200nn_layernorm {
    b200nn_ctx *ctx;
    std::shared_ptr<DevBuf> gamma, beta;
    size_t d;
    float eps;
};
struct b200nn_embedding {
    b200nn_ctx *ctx;
    std::shared_ptr<DevBuf> wte, wpe;
    size_t vocab, max_seq, d;
};
struct b200nn_attention {
    b200nn_ctx *ctx;
    LinearAny qkv, proj;
    size_t d, n_heads;
};

struct BlockW {
    std::shared_ptr<DevBuf> ln1_g, ln1_b, ln2_g, ln2_b;
    LinearAny qkv, proj, fc, fcproj;
    // ln_1 folded into the q/k/v Linear and ln_2 into the MLP's first Linear (int4_weight_ln_fold);
    // built by model_prepare_ln_fold on first use
    std::shared_ptr<DevBuf> qkv_gsum, qkv_bc, fc_gsum, fc_bc;
};

struct b200nn_gpt2 {
    b200nn_ctx *ctx = nullptr;
    b200nn_gpt2_config cfg{};
    uint32_t flags = 0;
    bool int4 = false;
    size_t group = 0;
    std::shared_ptr<DevBuf> wte, wpe, lnf_g, lnf_b;
    std::vector<BlockW> blocks;
    LinearAny lm_head;
    bool ln_fold_ready = false;
    int act() const { return (flags & B200NN_GELU_SIGMOID) ? B200NN_ACT_GELU_SIGMOID : B200NN_ACT_GELU_TANH; }
};

struct b200nn_kvcache {
    b200nn_gpt2 *m = nullptr;
    size_t batch = 0, cap = 0, len = 0;
    std::shared_ptr<DevBuf> k, v; // [layer][seq][head][cap][64] fp16
    size_t layer_stride() const { return batch * (size_t)m->cfg.n_head * cap * 64; }
    __half *kl(int l) const { return static_cast<__half *>(k->p) + (size_t)l * layer_stride(); }
    __half *vl(int l) const { return static_cast<__half *>(v->p) + (size_t)l * layer_stride(); }
};

// Activation buffers for up to `rows` token rows.
struct Workspace {
    size_t rows = 0, logit_rows = 0;
    std::shared_ptr<DevBuf> x, ln, q, att, fc, last_x, last_ln, logits, ids, tok;
    std::shared_ptr<DevBuf> amax_val, amax_idx; // [logit_rows][entries]: partial greedy picks of the LM head's epilogue
    int amax_entries = 0;
    // folded LayerNorms: f32 [2 * n_layer][rows][ln_nt][2] partial (sum, sum of squares) of every row of the
    // residual stream as it enters each LayerNorm (absent unless the workspace serves folded decode steps)
    std::shared_ptr<DevBuf> ln_stats;
    int ln_nt = 0;
    float *ln_slot(int i) const { return static_cast<float *>(ln_stats->p) + (size_t)i * rows * ln_nt * 2; }
};
int workspace_alloc(b200nn_gpt2 *m, size_t rows, size_t logit_rows, Workspace *ws);

struct StepProfile {
    std::vector<cudaEvent_t> ev;
    std::vector<int> fam;
};

// Runs the transformer blocks over T = B*S rows already embedded in ws.x.  Row t belongs to
// sequence t/S at position pos(t) = *pos_ptr + pos_off + t%S; K and V go straight into `kv`.
int run_blocks(b200nn_gpt2 *m, Workspace &ws, b200nn_kvcache &kv, int B, int S, const int *pos_ptr, int pos_off,
               bool act_half, StepProfile *prof, bool fold = false);
// Whether decode steps over `rows` rows can run with the block LayerNorms folded into the GEMMs (int4
// weights in the tiled layout, every Linear on the tensor-core GEMM), and the one-time preparation of the
// per-Linear vectors and the workspace's statistics buffer.
bool model_ln_fold_supported(const b200nn_gpt2 *m, int rows);
int model_prepare_ln_fold(b200nn_gpt2 *m, Workspace *ws);
// The same for blocks [layer_begin, layer_end) only (data-dependent depth: early exit).
int run_blocks_range(b200nn_gpt2 *m, Workspace &ws, b200nn_kvcache &kv, int B, int S, const int *pos_ptr, int pos_off,
                     bool act_half, StepProfile *prof, int layer_begin, int layer_end, bool fold = false);
// The launches of transformer block `l` over B*S rows (arguments as run_blocks), one at a time.
struct BlockLaunch {
    b200nn_gpt2 *m;
    Workspace &ws;
    b200nn_kvcache &kv;
    int l, B, S;
    const int *pos_ptr;
    int pos_off;
    bool act_half;
    bool fold = false; // block LayerNorms folded into the GEMMs around them: ln1() and ln2() launch nothing
    int ln1() const, qkv() const, attention() const, proj() const, ln2() const, fc() const, fcproj() const;
};
bool head_act_half(const b200nn_gpt2 *m, int rows, bool act_half);
int launch_head_norm(b200nn_gpt2 *m, Workspace &ws, const float *x, int rows, bool head_half);
int launch_head_linear(b200nn_gpt2 *m, Workspace &ws, int rows, bool head_half);
// Final LayerNorm + LM head + greedy pick of every row -> tok_out [rows] (and ws.logits unless
// tokens_only): the pick is taken in the LM head's epilogue when the kernel that runs it supports that,
// else by argmax_kernel over the logits.
int run_head_pick(b200nn_gpt2 *m, Workspace &ws, const float *x, int rows, bool act_half, bool keep_last, bool tokens_only,
                  uint32_t *tok_out, StepProfile *prof);
// Final LayerNorm + LM head over `rows` rows of `x` -> ws.logits [rows, vocab].
int run_head(b200nn_gpt2 *m, Workspace &ws, const float *x, int rows, bool act_half, StepProfile *prof);
bool model_act_half(const b200nn_gpt2 *m, int rows);

struct b200nn_session {
    b200nn_gpt2 *m = nullptr;
    size_t batch = 0, cap = 0, hist_cap = 0;
    uint32_t flags = 0;
    b200nn_kvcache kv;
    Workspace ws_step, ws_prefill;
    std::shared_ptr<DevBuf> counters; // int[2]: {position, step}
    std::shared_ptr<DevBuf> history;  // u32 [batch][hist_cap]
    size_t position = 0, steps_done = 0;
    bool prefilled = false, eager_done = false;
    cudaGraphExec_t graph = nullptr;
    uint64_t launches_per_step = 0; // kernels in one captured decode step
    // persistent decode (decode_persistent.cu): per-layer pointer table, f32 accumulators of the q/k/v and
    // MLP hidden GEMMs (zero at rest), grid counter + per-phase nanoseconds
    bool persist = false;
    std::shared_ptr<DevBuf> pd_layers, pd_qkv_acc, pd_fc_acc, pd_sync;
    int *pos_ptr() const { return static_cast<int *>(counters->p); }
    int *step_ptr() const { return static_cast<int *>(counters->p) + 1; }
};

// All transformer blocks of an int4 decode step as one persistent cooperative kernel.
bool decode_persistent_supported(const b200nn_gpt2 *m, int rows);
int decode_persistent_prepare(b200nn_session *s);
int launch_decode_layers(b200nn_session *s, bool profile);
