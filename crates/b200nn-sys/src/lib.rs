//! Raw bindings to `libb200nn` (see `include/b200nn.h`, which names the `gpu_host::nn` item every
//! function replaces).  One `extern "C"` declaration per exported symbol, nothing else: the safe
//! wrappers (`KernelRegistry`, `GpuTensor`, `Linear`, `Int4Linear`, `LayerNorm`, `Embedding`,
//! `MultiHeadAttention`, `TransformerBlock`, `Gpt2Model`, `Int4Gpt2Model`, `KvCache`) live in the crate
//! above this one and map the status codes back to `NnError`.
//!
//! Not compiled on the machine this repository was developed on (no Rust toolchain there);
//! `tests/test_capi_cpu.py` checks that the functions declared here are exactly the header's.
#![allow(non_camel_case_types)]

use core::ffi::{c_char, c_void};

/// Status codes (`B200NN_*`); 1-4 mirror `NnError`'s variants (nn/error.rs:7-29).
pub const B200NN_OK: i32 = 0;
pub const B200NN_ERR_SHAPE: i32 = 1;
pub const B200NN_ERR_DIM: i32 = 2;
pub const B200NN_ERR_UNSUPPORTED: i32 = 3;
pub const B200NN_ERR_CUDA: i32 = 4;
pub const B200NN_ERR_DEVICE: i32 = 5;
pub const B200NN_ERR_ARG: i32 = 6;
pub const B200NN_ERR_IO: i32 = 7;
pub const B200NN_ERR_MISSING: i32 = 8;

/// `Activation` (nn/layers/linear.rs:24-33).
pub const B200NN_ACT_NONE: i32 = 0;
pub const B200NN_ACT_GELU_TANH: i32 = 1;
pub const B200NN_ACT_GELU_SIGMOID: i32 = 2;
pub const B200NN_ACT_RELU: i32 = 3;
pub const B200NN_ACT_SILU: i32 = 4;
pub const B200NN_ACT_SIGMOID: i32 = 5;

/// Model / generation flags.
pub const B200NN_GELU_SIGMOID: u32 = 1 << 0;
pub const B200NN_QUANT_LM_HEAD: u32 = 1 << 1;
pub const B200NN_ARGMAX_LAST: u32 = 1 << 2;
pub const B200NN_STOP_ON_EOS: u32 = 1 << 3;
pub const B200NN_TOKENS_ONLY: u32 = 1 << 4;
pub const B200NN_WEIGHTS_OUT_IN: u32 = 1 << 5;

/// Kernel families of `b200nn_session_profile_step` / `b200nn_session_time_family`.
pub const B200NN_PROF_EMBED: i32 = 0;
pub const B200NN_PROF_LAYERNORM: i32 = 1;
pub const B200NN_PROF_LINEAR: i32 = 2;
pub const B200NN_PROF_ATTENTION: i32 = 3;
pub const B200NN_PROF_LM_HEAD: i32 = 4;
pub const B200NN_PROF_ARGMAX: i32 = 5;
pub const B200NN_PROF_COUNT: i32 = 6;

macro_rules! opaque {
    ($($name:ident),* $(,)?) => {
        $(
            #[repr(C)]
            pub struct $name {
                _private: [u8; 0],
            }
        )*
    };
}
opaque!(
    b200nn_ctx,
    b200nn_tensor,
    b200nn_linear,
    b200nn_int4_linear,
    b200nn_layernorm,
    b200nn_embedding,
    b200nn_attention,
    b200nn_gpt2,
    b200nn_kvcache,
    b200nn_session,
    b200nn_block,
    b200nn_safetensors,
    b200nn_bpe,
);

/// `Gpt2Config` (nn/models/gpt2.rs:20-34).
#[repr(C)]
#[derive(Clone, Copy, Debug, PartialEq)]
pub struct b200nn_gpt2_config {
    pub n_layer: i32,
    pub n_embd: i32,
    pub n_head: i32,
    pub vocab_size: i32,
    pub n_positions: i32,
    pub layer_norm_epsilon: f32,
}

/// `TransformerLayerWeights` (model.rs:112-139): host f32, dense weights in Conv1D layout [in,out].
#[repr(C)]
#[derive(Clone, Copy)]
pub struct b200nn_gpt2_layer_weights {
    pub ln_1_weight: *const f32,
    pub ln_1_bias: *const f32,
    pub c_attn_weight: *const f32,
    pub c_attn_bias: *const f32,
    pub c_proj_weight: *const f32,
    pub c_proj_bias: *const f32,
    pub ln_2_weight: *const f32,
    pub ln_2_bias: *const f32,
    pub mlp_fc_weight: *const f32,
    pub mlp_fc_bias: *const f32,
    pub mlp_proj_weight: *const f32,
    pub mlp_proj_bias: *const f32,
}

/// `Gpt2Weights` (model.rs:141-154).
#[repr(C)]
#[derive(Clone, Copy)]
pub struct b200nn_gpt2_weights {
    pub wte: *const f32,
    pub wpe: *const f32,
    pub ln_f_weight: *const f32,
    pub ln_f_bias: *const f32,
    pub layers: *const b200nn_gpt2_layer_weights,
}

/// The twelve slices of `TransformerBlock::new` (gpt2.rs:120-135), dense weights in Linear layout [out,in].
#[repr(C)]
#[derive(Clone, Copy)]
pub struct b200nn_block_weights {
    pub ln_1_weight: *const f32,
    pub ln_1_bias: *const f32,
    pub attn_qkv_weight: *const f32,
    pub attn_qkv_bias: *const f32,
    pub attn_out_weight: *const f32,
    pub attn_out_bias: *const f32,
    pub ln_2_weight: *const f32,
    pub ln_2_bias: *const f32,
    pub ffn_up_weight: *const f32,
    pub ffn_up_bias: *const f32,
    pub ffn_down_weight: *const f32,
    pub ffn_down_bias: *const f32,
}

/// What `Gpt2Model::forward_diagnostic` (gpt2.rs:595-667) prints, as values.
#[repr(C)]
#[derive(Clone, Copy, Debug, Default)]
pub struct b200nn_gpt2_diagnostic {
    pub embedding_first: [f32; 4],
    pub embedding_last: [f32; 4],
    pub block0_last: [f32; 4],
    pub final_block_last: [f32; 4],
    pub block0_nonfinite: i32,
    pub final_block_nonfinite: i32,
    pub ln_f_last: [f32; 4],
    pub top_tokens: [u32; 5],
    pub top_scores: [f32; 5],
    pub n_top: i32,
}

#[link(name = "b200nn")]
extern "C" {
    pub fn b200nn_version() -> *const c_char;
    pub fn b200nn_ctx_create(device_ordinal: i32, out: *mut *mut b200nn_ctx) -> i32;
    pub fn b200nn_ctx_destroy(ctx: *mut b200nn_ctx);
    pub fn b200nn_ctx_synchronize(ctx: *mut b200nn_ctx) -> i32;
    pub fn b200nn_ctx_trim(ctx: *mut b200nn_ctx) -> i32;
    pub fn b200nn_ctx_stream(ctx: *mut b200nn_ctx) -> *mut c_void;
    pub fn b200nn_last_error_message(ctx: *mut b200nn_ctx) -> *const c_char;
    pub fn b200nn_last_cuda_error(ctx: *mut b200nn_ctx) -> i32;
    pub fn b200nn_ctx_device_error(ctx: *mut b200nn_ctx, word_out: *mut u32) -> i32;
    pub fn b200nn_ctx_launch_count(ctx: *mut b200nn_ctx) -> u64;
    pub fn b200nn_ctx_set_gemv_max_rows(ctx: *mut b200nn_ctx, rows: i32) -> i32;
    pub fn b200nn_ctx_set_tuning(ctx: *mut b200nn_ctx, key: *const c_char, value: i32) -> i32;
    pub fn b200nn_ctx_read_trace(ctx: *mut b200nn_ctx, out256: *mut i64) -> i32;
    pub fn b200nn_ctx_read_persist_trace(ctx: *mut b200nn_ctx, out: *mut u64, capacity: usize) -> i32;
    pub fn b200nn_tensor_from_host(
        ctx: *mut b200nn_ctx,
        host: *const f32,
        shape: *const usize,
        ndim: i32,
        out: *mut *mut b200nn_tensor,
    ) -> i32;
    pub fn b200nn_tensor_from_device(
        ctx: *mut b200nn_ctx,
        dev: *const f32,
        shape: *const usize,
        ndim: i32,
        out: *mut *mut b200nn_tensor,
    ) -> i32;
    pub fn b200nn_tensor_zeros(
        ctx: *mut b200nn_ctx,
        shape: *const usize,
        ndim: i32,
        out: *mut *mut b200nn_tensor,
    ) -> i32;
    pub fn b200nn_tensor_to_host(t: *const b200nn_tensor, host: *mut f32, capacity_elems: usize) -> i32;
    pub fn b200nn_tensor_ndim(t: *const b200nn_tensor) -> i32;
    pub fn b200nn_tensor_numel(t: *const b200nn_tensor) -> usize;
    pub fn b200nn_tensor_shape(t: *const b200nn_tensor, shape_out: *mut usize, capacity: i32) -> i32;
    pub fn b200nn_tensor_reshape(
        t: *const b200nn_tensor,
        shape: *const usize,
        ndim: i32,
        out: *mut *mut b200nn_tensor,
    ) -> i32;
    pub fn b200nn_tensor_clone(t: *const b200nn_tensor, out: *mut *mut b200nn_tensor) -> i32;
    pub fn b200nn_tensor_transpose(
        t: *const b200nn_tensor,
        dim0: usize,
        dim1: usize,
        out: *mut *mut b200nn_tensor,
    ) -> i32;
    pub fn b200nn_tensor_concat(
        tensors: *const *const b200nn_tensor,
        count: usize,
        dim: usize,
        out: *mut *mut b200nn_tensor,
    ) -> i32;
    pub fn b200nn_tensor_split(
        t: *const b200nn_tensor,
        dim: usize,
        sizes: *const usize,
        count: usize,
        outs: *mut *mut b200nn_tensor,
    ) -> i32;
    pub fn b200nn_tensor_data(t: *mut b200nn_tensor) -> *mut f32;
    pub fn b200nn_tensor_destroy(t: *mut b200nn_tensor);
    pub fn b200nn_quantize_weight_int4(
        weight_t: *const f32,
        k: usize,
        n: usize,
        group: usize,
        packed: *mut u32,
        scales: *mut f32,
    ) -> i32;
    pub fn b200nn_quantize_int4_per_group(
        data: *const f32,
        len: usize,
        group: usize,
        packed: *mut u32,
        scales: *mut f32,
    ) -> i32;
    pub fn b200nn_unpack_int4(packed: u32, index: i32) -> i32;
    pub fn b200nn_pack_int8_to_u32(values: *const i8, n: usize, packed: *mut u32) -> i32;
    pub fn b200nn_quantize_int8_per_tensor(data: *const f32, n: usize, q: *mut i8, scale: *mut f32) -> i32;
    pub fn b200nn_layer_norm(
        ctx: *mut b200nn_ctx,
        x: *const b200nn_tensor,
        gamma: *const b200nn_tensor,
        beta: *const b200nn_tensor,
        eps: f32,
        out: *mut *mut b200nn_tensor,
    ) -> i32;
    pub fn b200nn_layer_norm_residual_dual(
        ctx: *mut b200nn_ctx,
        a: *const b200nn_tensor,
        b: *const b200nn_tensor,
        gamma: *const b200nn_tensor,
        beta: *const b200nn_tensor,
        eps: f32,
        sum_out: *mut *mut b200nn_tensor,
        norm_out: *mut *mut b200nn_tensor,
    ) -> i32;
    pub fn b200nn_activation(
        ctx: *mut b200nn_ctx,
        x: *const b200nn_tensor,
        act: i32,
        out: *mut *mut b200nn_tensor,
    ) -> i32;
    pub fn b200nn_bias_add(ctx: *mut b200nn_ctx, data: *mut b200nn_tensor, bias: *const b200nn_tensor) -> i32;
    pub fn b200nn_elementwise_add(
        ctx: *mut b200nn_ctx,
        a: *mut b200nn_tensor,
        b: *const b200nn_tensor,
    ) -> i32;
    pub fn b200nn_split_qkv(
        ctx: *mut b200nn_ctx,
        qkv: *const b200nn_tensor,
        seq_len: usize,
        n_heads: usize,
        d_head: usize,
        q: *mut *mut b200nn_tensor,
        k: *mut *mut b200nn_tensor,
        v: *mut *mut b200nn_tensor,
    ) -> i32;
    pub fn b200nn_concat_heads(
        ctx: *mut b200nn_ctx,
        heads: *const b200nn_tensor,
        seq_len: usize,
        n_heads: usize,
        d_head: usize,
        out: *mut *mut b200nn_tensor,
    ) -> i32;
    pub fn b200nn_multi_head_flash_attention(
        ctx: *mut b200nn_ctx,
        q: *const b200nn_tensor,
        k: *const b200nn_tensor,
        v: *const b200nn_tensor,
        seq_len: usize,
        n_heads: usize,
        d_head: usize,
        causal: i32,
        out: *mut *mut b200nn_tensor,
    ) -> i32;
    pub fn b200nn_attention_kv(
        ctx: *mut b200nn_ctx,
        q: *const b200nn_tensor,
        k: *const b200nn_tensor,
        v: *const b200nn_tensor,
        causal: i32,
        q_offset: usize,
        out: *mut *mut b200nn_tensor,
    ) -> i32;
    pub fn b200nn_matmul(
        ctx: *mut b200nn_ctx,
        a: *const b200nn_tensor,
        b: *const b200nn_tensor,
        out: *mut *mut b200nn_tensor,
    ) -> i32;
    pub fn b200nn_int4_matmul(
        ctx: *mut b200nn_ctx,
        a: *const b200nn_tensor,
        b_host: *const f32,
        k: usize,
        n: usize,
        group: usize,
        out: *mut *mut b200nn_tensor,
    ) -> i32;
    pub fn b200nn_linear_create(
        ctx: *mut b200nn_ctx,
        weight: *const f32,
        bias: *const f32,
        in_features: usize,
        out_features: usize,
        out: *mut *mut b200nn_linear,
    ) -> i32;
    pub fn b200nn_linear_forward(
        l: *mut b200nn_linear,
        x: *const b200nn_tensor,
        y: *mut *mut b200nn_tensor,
    ) -> i32;
    pub fn b200nn_linear_forward_fused(
        l: *mut b200nn_linear,
        x: *const b200nn_tensor,
        act: i32,
        y: *mut *mut b200nn_tensor,
    ) -> i32;
    pub fn b200nn_linear_destroy(l: *mut b200nn_linear);
    pub fn b200nn_int4_linear_create(
        ctx: *mut b200nn_ctx,
        packed: *const u32,
        scales: *const f32,
        bias: *const f32,
        in_features: usize,
        out_features: usize,
        group: usize,
        out: *mut *mut b200nn_int4_linear,
    ) -> i32;
    pub fn b200nn_int4_linear_forward(
        l: *mut b200nn_int4_linear,
        x: *const b200nn_tensor,
        y: *mut *mut b200nn_tensor,
    ) -> i32;
    pub fn b200nn_int4_linear_forward_dev(
        l: *mut b200nn_int4_linear,
        x_dev: *const f32,
        m: usize,
        y_dev: *mut f32,
    ) -> i32;
    pub fn b200nn_int4_linear_forward_host(
        l: *mut b200nn_int4_linear,
        x_host: *const f32,
        m: usize,
        y_host: *mut f32,
    ) -> i32;
    pub fn b200nn_int4_linear_memory_bytes(l: *const b200nn_int4_linear) -> usize;
    pub fn b200nn_int4_linear_destroy(l: *mut b200nn_int4_linear);
    pub fn b200nn_layernorm_create(
        ctx: *mut b200nn_ctx,
        gamma: *const f32,
        beta: *const f32,
        d: usize,
        eps: f32,
        out: *mut *mut b200nn_layernorm,
    ) -> i32;
    pub fn b200nn_layernorm_forward(
        ln: *mut b200nn_layernorm,
        x: *const b200nn_tensor,
        y: *mut *mut b200nn_tensor,
    ) -> i32;
    pub fn b200nn_layernorm_destroy(ln: *mut b200nn_layernorm);
    pub fn b200nn_embedding_create(
        ctx: *mut b200nn_ctx,
        wte: *const f32,
        wpe: *const f32,
        vocab: usize,
        max_seq: usize,
        d: usize,
        out: *mut *mut b200nn_embedding,
    ) -> i32;
    pub fn b200nn_embedding_forward_tokens(
        e: *mut b200nn_embedding,
        ids_host: *const u32,
        n: usize,
        pos_offset: usize,
        out: *mut *mut b200nn_tensor,
    ) -> i32;
    pub fn b200nn_embedding_destroy(e: *mut b200nn_embedding);
    pub fn b200nn_attention_create(
        ctx: *mut b200nn_ctx,
        qkv_weight: *const f32,
        qkv_bias: *const f32,
        out_weight: *const f32,
        out_bias: *const f32,
        n_embd: usize,
        n_heads: usize,
        out: *mut *mut b200nn_attention,
    ) -> i32;
    pub fn b200nn_int4_attention_create(
        ctx: *mut b200nn_ctx,
        qkv_weight: *const f32,
        qkv_bias: *const f32,
        out_weight: *const f32,
        out_bias: *const f32,
        n_embd: usize,
        n_heads: usize,
        group_size: usize,
        out: *mut *mut b200nn_attention,
    ) -> i32;
    pub fn b200nn_attention_forward_causal(
        a: *mut b200nn_attention,
        x: *const b200nn_tensor,
        y: *mut *mut b200nn_tensor,
    ) -> i32;
    pub fn b200nn_attention_forward_cached(
        a: *mut b200nn_attention,
        x: *const b200nn_tensor,
        cached_k: *const f32,
        cached_v: *const f32,
        kv_len: usize,
        y: *mut *mut b200nn_tensor,
        new_k_out: *mut f32,
        new_v_out: *mut f32,
    ) -> i32;
    pub fn b200nn_attention_destroy(a: *mut b200nn_attention);
    pub fn b200nn_gpt2_config_preset(name: *const c_char, out: *mut b200nn_gpt2_config) -> i32;
    pub fn b200nn_gpt2_create(
        ctx: *mut b200nn_ctx,
        cfg: *const b200nn_gpt2_config,
        w: *const b200nn_gpt2_weights,
        flags: u32,
        out: *mut *mut b200nn_gpt2,
    ) -> i32;
    pub fn b200nn_int4_gpt2_create(
        ctx: *mut b200nn_ctx,
        cfg: *const b200nn_gpt2_config,
        w: *const b200nn_gpt2_weights,
        group_size: usize,
        flags: u32,
        out: *mut *mut b200nn_gpt2,
    ) -> i32;
    pub fn b200nn_gpt2_destroy(m: *mut b200nn_gpt2);
    pub fn b200nn_gpt2_get_config(m: *const b200nn_gpt2, out: *mut b200nn_gpt2_config) -> i32;
    pub fn b200nn_gpt2_quantized_memory_bytes(m: *const b200nn_gpt2) -> usize;
    pub fn b200nn_gpt2_get_int4(
        m: *const b200nn_gpt2,
        layer: i32,
        which: i32,
        packed: *mut u32,
        scales: *mut f32,
        k_out: *mut usize,
        n_out: *mut usize,
    ) -> i32;
    pub fn b200nn_block_create(
        ctx: *mut b200nn_ctx,
        cfg: *const b200nn_gpt2_config,
        w: *const b200nn_block_weights,
        flags: u32,
        out: *mut *mut b200nn_block,
    ) -> i32;
    pub fn b200nn_int4_block_create(
        ctx: *mut b200nn_ctx,
        cfg: *const b200nn_gpt2_config,
        w: *const b200nn_block_weights,
        group_size: usize,
        flags: u32,
        out: *mut *mut b200nn_block,
    ) -> i32;
    pub fn b200nn_block_forward(
        b: *mut b200nn_block,
        x: *const b200nn_tensor,
        y: *mut *mut b200nn_tensor,
    ) -> i32;
    pub fn b200nn_block_forward_cached(
        b: *mut b200nn_block,
        x: *const b200nn_tensor,
        cached_k: *const f32,
        cached_v: *const f32,
        kv_len: usize,
        y: *mut *mut b200nn_tensor,
        new_k_out: *mut f32,
        new_v_out: *mut f32,
    ) -> i32;
    pub fn b200nn_block_destroy(b: *mut b200nn_block);
    pub fn b200nn_gpt2_forward(
        m: *mut b200nn_gpt2,
        ids_host: *const u32,
        seq_len: usize,
        logits: *mut *mut b200nn_tensor,
    ) -> i32;
    pub fn b200nn_kvcache_create(
        m: *mut b200nn_gpt2,
        batch: usize,
        capacity: usize,
        out: *mut *mut b200nn_kvcache,
    ) -> i32;
    pub fn b200nn_kvcache_len(c: *const b200nn_kvcache) -> usize;
    pub fn b200nn_kvcache_reset(c: *mut b200nn_kvcache) -> i32;
    pub fn b200nn_kvcache_destroy(c: *mut b200nn_kvcache);
    pub fn b200nn_gpt2_forward_cached(
        m: *mut b200nn_gpt2,
        ids_host: *const u32,
        new_len: usize,
        cache: *mut b200nn_kvcache,
        logits: *mut *mut b200nn_tensor,
    ) -> i32;
    pub fn b200nn_gpt2_generate(
        m: *mut b200nn_gpt2,
        prompt: *const u32,
        prompt_len: usize,
        max_new: usize,
        flags: u32,
        out_tokens: *mut u32,
        n_out: *mut usize,
    ) -> i32;
    pub fn b200nn_gpt2_generate_cached(
        m: *mut b200nn_gpt2,
        prompt: *const u32,
        prompt_len: usize,
        max_new: usize,
        flags: u32,
        out_tokens: *mut u32,
        n_out: *mut usize,
    ) -> i32;
    pub fn b200nn_gpt2_generate_batch(
        m: *mut b200nn_gpt2,
        prompts: *const u32,
        batch: usize,
        prompt_len: usize,
        max_new: usize,
        flags: u32,
        out_tokens: *mut u32,
        out_lens: *mut usize,
    ) -> i32;
    pub fn b200nn_gpt2_forward_features(
        m: *mut b200nn_gpt2,
        ids_host: *const u32,
        seq_len: usize,
        features: *mut *mut b200nn_tensor,
    ) -> i32;
    pub fn b200nn_gpt2_embedding_table(
        m: *mut b200nn_gpt2,
        wte: *mut *mut b200nn_tensor,
        wpe: *mut *mut b200nn_tensor,
    ) -> i32;
    pub fn b200nn_gpt2_forward_diagnostic(
        m: *mut b200nn_gpt2,
        ids_host: *const u32,
        seq_len: usize,
        logits: *mut *mut b200nn_tensor,
        diag: *mut b200nn_gpt2_diagnostic,
    ) -> i32;
    pub fn b200nn_gpt2_forward_profiled(
        m: *mut b200nn_gpt2,
        ids_host: *const u32,
        seq_len: usize,
        logits: *mut *mut b200nn_tensor,
        times_ms: *mut f32,
        capacity: i32,
        n_times: *mut i32,
    ) -> i32;
    pub fn b200nn_simple_rng_new(seed: u64) -> u64;
    pub fn b200nn_simple_rng_next_f32(state: *mut u64) -> f32;
    pub fn b200nn_simple_rng_fill_uniform(state: *mut u64, n: usize, out: *mut f32) -> i32;
    pub fn b200nn_simple_rng_fill_normal(state: *mut u64, n: usize, std_dev: f32, out: *mut f32) -> i32;
    pub fn b200nn_top_k_sample(
        logits: *const f32,
        n: usize,
        k: usize,
        temperature: f32,
        rng_state: *mut u64,
        token_out: *mut u32,
    ) -> i32;
    pub fn b200nn_gpt2_generate_cached_sampling(
        m: *mut b200nn_gpt2,
        prompt: *const u32,
        prompt_len: usize,
        max_new: usize,
        top_k: usize,
        temperature: f32,
        rng_state: *mut u64,
        out_tokens: *mut u32,
        n_out: *mut usize,
    ) -> i32;
    pub fn b200nn_gpt2_forward_early_exit(
        m: *mut b200nn_gpt2,
        ids_host: *const u32,
        seq_len: usize,
        threshold: f32,
        logits: *mut *mut b200nn_tensor,
        layers_used: *mut i32,
    ) -> i32;
    pub fn b200nn_gpt2_generate_cached_early_exit(
        m: *mut b200nn_gpt2,
        prompt: *const u32,
        prompt_len: usize,
        max_new: usize,
        threshold: f32,
        out_tokens: *mut u32,
        n_out: *mut usize,
        layers_per_step: *mut i32,
        n_steps: *mut usize,
    ) -> i32;
    pub fn b200nn_session_create(
        m: *mut b200nn_gpt2,
        batch: usize,
        capacity: usize,
        flags: u32,
        out: *mut *mut b200nn_session,
    ) -> i32;
    pub fn b200nn_session_prefill(s: *mut b200nn_session, prompts_host: *const u32, prompt_len: usize) -> i32;
    pub fn b200nn_session_step(s: *mut b200nn_session, n_steps: usize) -> i32;
    pub fn b200nn_session_rewind(s: *mut b200nn_session, position: usize) -> i32;
    pub fn b200nn_session_position(s: *const b200nn_session) -> usize;
    pub fn b200nn_session_tokens(
        s: *mut b200nn_session,
        out: *mut u32,
        capacity_per_seq: usize,
        generated: *mut usize,
    ) -> i32;
    pub fn b200nn_session_logits(s: *mut b200nn_session, out: *mut f32) -> i32;
    pub fn b200nn_session_profile_step(
        s: *mut b200nn_session,
        times_ms: *mut f32,
        linear_bytes: *mut u64,
    ) -> i32;
    pub fn b200nn_session_time_family(
        s: *mut b200nn_session,
        family: i32,
        reps: i32,
        ms_total: *mut f32,
        launches: *mut u64,
    ) -> i32;
    pub fn b200nn_session_destroy(s: *mut b200nn_session);
    pub fn b200nn_safetensors_open(path: *const c_char, out: *mut *mut b200nn_safetensors) -> i32;
    pub fn b200nn_safetensors_close(st: *mut b200nn_safetensors);
    pub fn b200nn_safetensors_count(st: *const b200nn_safetensors) -> i32;
    pub fn b200nn_safetensors_info(
        st: *const b200nn_safetensors,
        index: i32,
        name: *mut *const c_char,
        dtype: *mut *const c_char,
        shape_out: *mut usize,
        shape_capacity: i32,
        ndim: *mut i32,
        nbytes: *mut usize,
    ) -> i32;
    pub fn b200nn_safetensors_find(st: *const b200nn_safetensors, name: *const c_char) -> i32;
    pub fn b200nn_safetensors_read(
        st: *const b200nn_safetensors,
        index: i32,
        out: *mut c_void,
        capacity_bytes: usize,
    ) -> i32;
    pub fn b200nn_safetensors_last_error() -> *const c_char;
    pub fn b200nn_gpt2_load_safetensors(
        ctx: *mut b200nn_ctx,
        path: *const c_char,
        cfg: *const b200nn_gpt2_config,
        int4_group: usize,
        flags: u32,
        out: *mut *mut b200nn_gpt2,
    ) -> i32;
    pub fn b200nn_bpe_load(path: *const c_char, endoftext_id: u32, out: *mut *mut b200nn_bpe) -> i32;
    pub fn b200nn_bpe_create(
        token_bytes: *const u8,
        token_offsets: *const usize,
        ranks: *const u32,
        n_tokens: usize,
        endoftext_id: u32,
        out: *mut *mut b200nn_bpe,
    ) -> i32;
    pub fn b200nn_bpe_destroy(t: *mut b200nn_bpe);
    pub fn b200nn_bpe_vocab_size(t: *const b200nn_bpe) -> usize;
    pub fn b200nn_bpe_encode(
        t: *const b200nn_bpe,
        text: *const u8,
        n: usize,
        out: *mut u32,
        capacity: usize,
        n_out: *mut usize,
    ) -> i32;
    pub fn b200nn_bpe_encode_piece(
        t: *const b200nn_bpe,
        piece: *const u8,
        n: usize,
        out: *mut u32,
        capacity: usize,
        n_out: *mut usize,
    ) -> i32;
    pub fn b200nn_bpe_decode(
        t: *const b200nn_bpe,
        ids: *const u32,
        n: usize,
        out: *mut u8,
        capacity: usize,
        n_out: *mut usize,
    ) -> i32;
    pub fn b200nn_bpe_last_error() -> *const c_char;
    pub fn b200nn_prefill_attention_f16(
        ctx: *mut b200nn_ctx,
        q_dev: *const c_void,
        k_cache_dev: *const c_void,
        v_cache_dev: *const c_void,
        batch: i32,
        n_heads: i32,
        capacity: i32,
        seq_len: i32,
        past: i32,
        out_dev: *mut c_void,
    ) -> i32;
    pub fn b200nn_decode_attention_f16(
        ctx: *mut b200nn_ctx,
        q_dev: *const c_void,
        k_cache_dev: *const c_void,
        v_cache_dev: *const c_void,
        batch: i32,
        n_heads: i32,
        capacity: i32,
        ctx_len: i32,
        out_dev: *mut c_void,
    ) -> i32;
    pub fn b200nn_decode_attention_noalloc(
        device: i32,
        stream: *mut c_void,
        q_dev: *const f32,
        k_cache_dev: *const c_void,
        v_cache_dev: *const c_void,
        batch: i32,
        n_heads: i32,
        capacity: i32,
        ctx_len: i32,
        out_dev: *mut f32,
    ) -> i32;
    pub fn b200nn_noalloc_last_error() -> *const c_char;
}
