/*
 * b200nn — C ABI of the B200-native GPT-2 inference path that stands in for
 * async-gpu's `gpu_host::nn` module (Linear / Int4Linear / LayerNorm / causal
 * attention with KV cache / GELU MLP / Gpt2Model forward + generate).
 *
 * The reference has no FFI for this path: its boundary is the Rust `nn` API,
 * which reaches kernels by name through `KernelRegistry` and launches them with
 * cudarc.  Each entry point below names the Rust item it replaces
 * (file:line relative to the reference repository; GH = crates/core/gpu-host/src).
 * A Rust `-sys` crate binds these symbols one to one.
 *
 * Conventions
 *   - Plain pointers and sizes only.  "host" pointers are ordinary host memory,
 *     "dev" pointers are CUDA device memory of the context's device.
 *   - Every function that can fail returns an int32 status (B200NN_*); the text
 *     of the last failure is kept per context (b200nn_last_error_message).
 *   - All tensors a caller can see are f32, row-major, contiguous, as in the
 *     reference (GH/nn/tensor.rs:45-60).  fp16 / int4 exist only inside the library.
 *   - One context per GPU, used from one host thread at a time; work is ordered on
 *     the context's stream.  Functions returning host data synchronise that stream.
 *   - There is no CPU fallback: without a CUDA device every compute entry point
 *     fails with B200NN_ERR_CUDA.
 */
#ifndef B200NN_H
#define B200NN_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define B200NN_API __attribute__((visibility("default")))
#else
#define B200NN_API
#endif

/* Status codes; 1-4 mirror NnError's variants (GH/nn/error.rs:7-29). */
enum {
    B200NN_OK = 0,
    B200NN_ERR_SHAPE = 1,       /* NnError::ShapeMismatch                      */
    B200NN_ERR_DIM = 2,         /* NnError::DimOutOfRange                      */
    B200NN_ERR_UNSUPPORTED = 3, /* NnError::KernelNotFound / unsupported shape */
    B200NN_ERR_CUDA = 4,        /* NnError::Cuda                               */
    B200NN_ERR_DEVICE = 5,      /* a kernel's bounded wait ran out             */
    B200NN_ERR_ARG = 6,         /* null handle / invalid argument              */
    B200NN_ERR_IO = 7,          /* ModelError::Io / ::SafeTensor (GH/model.rs:30-62): unreadable or malformed file */
    B200NN_ERR_MISSING = 8      /* ModelError::MissingTensor                   */
};

/* Activation selector (GH/nn/layers/linear.rs:24-33 `Activation`). */
/* Activation (layers/linear.rs:24-33): Gelu (tanh form, or the sigmoid form of gelu_forward_v2), Relu, Silu, Sigmoid */
enum { B200NN_ACT_NONE = 0, B200NN_ACT_GELU_TANH = 1, B200NN_ACT_GELU_SIGMOID = 2, B200NN_ACT_RELU = 3, B200NN_ACT_SILU = 4,
       B200NN_ACT_SIGMOID = 5 };

/* Model / generation flags. */
enum {
    B200NN_GELU_SIGMOID = 1u << 0,   /* x*sigmoid(1.702x) (compute_transformer.rs:1473) instead of tanh */
    B200NN_QUANT_LM_HEAD = 1u << 1,  /* int4 models: quantise the tied LM head as well               */
    B200NN_ARGMAX_LAST = 1u << 2,    /* keep the last maximum on ties (GH/nn/models/gpt2.rs:991-997)  */
    B200NN_STOP_ON_EOS = 1u << 3,    /* stop before appending token 50256 (gpt2.rs:698-700)          */
    B200NN_TOKENS_ONLY = 1u << 4,    /* decode sessions: the step's logits are not written to memory (the greedy
                                        pick is taken in the LM head's epilogue); b200nn_session_logits fails */
    B200NN_WEIGHTS_OUT_IN = 1u << 5  /* model creation: the four Linear weights of every block are given in Linear
                                        layout [out,in], as Gpt2Model::from_generic_weights holds them after the
                                        generic loader's Conv1D transposes (gpt2.rs:410-476, 1436-1500;
                                        model_generic.rs:222-277), instead of checkpoint layout [in,out] */
};

typedef struct b200nn_ctx b200nn_ctx;
typedef struct b200nn_tensor b200nn_tensor;
typedef struct b200nn_linear b200nn_linear;
typedef struct b200nn_int4_linear b200nn_int4_linear;
typedef struct b200nn_layernorm b200nn_layernorm;
typedef struct b200nn_embedding b200nn_embedding;
typedef struct b200nn_attention b200nn_attention;
typedef struct b200nn_gpt2 b200nn_gpt2;
typedef struct b200nn_kvcache b200nn_kvcache;
typedef struct b200nn_session b200nn_session;
typedef struct b200nn_block b200nn_block;

/* ---- context: KernelRegistry::init_default (GH/nn/registry.rs:131-135) --------------------- */
B200NN_API const char *b200nn_version(void);
B200NN_API int32_t b200nn_ctx_create(int32_t device_ordinal, b200nn_ctx **out);
B200NN_API void b200nn_ctx_destroy(b200nn_ctx *ctx);
B200NN_API int32_t b200nn_ctx_synchronize(b200nn_ctx *ctx);
/* Device blocks released by tensors, workspaces and KV caches are kept by the context for reuse
 * (up to 64 GB; an allocation failure also releases them).  This hands them back to the driver.
 * The reference frees eagerly through cudarc's Drop; there is nothing to replace. */
B200NN_API int32_t b200nn_ctx_trim(b200nn_ctx *ctx);
/* cudaStream_t of the context, for callers that record their own events on it. */
B200NN_API void *b200nn_ctx_stream(b200nn_ctx *ctx);
B200NN_API const char *b200nn_last_error_message(b200nn_ctx *ctx);
B200NN_API int32_t b200nn_last_cuda_error(b200nn_ctx *ctx);
/* Reads and clears the device-side error word (non-zero after a bounded wait gave up). */
B200NN_API int32_t b200nn_ctx_device_error(b200nn_ctx *ctx, uint32_t *word_out);
/* Number of kernels this library has launched on the context since creation. */
B200NN_API uint64_t b200nn_ctx_launch_count(b200nn_ctx *ctx);
/* Linear layers with at most this many input rows take the CUDA-core GEMV; more rows take the
 * tcgen05 GEMM.  Negative restores the default. */
B200NN_API int32_t b200nn_ctx_set_gemv_max_rows(b200nn_ctx *ctx, int32_t rows);
/* Tuning overrides of the tensor-core GEMM's launch policy, for measurements: "tc_mb" (cap of the
 * token-tile width: 16..256, 0 = default), "tc_splits" (K splits, 0 = automatic), "tc_min_kb"
 * (fewest 64-wide K blocks per split; 0 = default: 2 up to 64 rows, else 3), "tc_min_kb_cluster" (the same for splits that run as
 * a cluster; default 6, measured best among 3, 4, 6, 8), "gemv_max_rows", "pdl" (programmatic dependent launch on/off),
 * "attn_tc" (0 = run fp16 prefill attention on the CUDA cores instead of the tensor cores),
 * "attn_stream" (0 = never use the TMA-fed decode-attention kernel), "attn_stream_min10" (tenths of
 * a (sequence, head) pair per warp of its grid from which it is used; default 20), "attn_stream_wide_min10" (the same for
 * its 16-warp block shape; default 25, 0 = never), "kv_prefetch_mb" (KV-cache
 * megabytes that kernel asks into L2 before its dependency wait), "attn_split_items" (items it
 * hands out as two halves at the end of the grid; 0 = none), "attn_blocks_per_sm" (blocks per SM the
 * split-context decode attention aims for when it splits the context of few pairs; default 4, measured
 * best: 8 and more cost 0.2 ms per GPT-2 XL step at 32 sequences through the merge of the partials).
 * "f32_tc" selects how an f32 Linear (linear.rs:283-313) multiplies more than four rows: 2 (default;
 * negative restores it) fp16 activations times the weight held as fp16 hi + lo on the tensor cores,
 * f32 accumulation (the weight enters with about 22 bits, the activations with fp16's 11); 1 the
 * weight rounded to fp16 only (half the tensor work, weight error 2^-11 relative); 0 the f32 FMA
 * kernels for every row count (the reference's arithmetic).
 * "tc_persistent" (default 1): the fp16 GEMM runs as one persistent block per SM from two 256-row
 * tiles per SM on; 0 = always one tile per block.  "int4_via_f16" (default 1): an int4 Linear over
 * such a pass of at least 2048 rows writes its weight out once as fp16 and uses that GEMM; 0 = the
 * int4 GEMM for every row count.
 * "fused_argmax" (default 1): greedy decode steps take the token inside the LM head's epilogue (one
 * (maximum, index) entry per 32 logits, a second small kernel per row); 0 = a separate pass over the
 * stored logits.  Same tokens either way.
 * "ln_rows_min" (default 1024): a LayerNorm over at least this many rows (no residual input, width a
 * multiple of 4 up to 2048) runs as one warp per row instead of one block per row.
 * "ln_fold" (default 0): decode steps of an int4 model with more than gemv_max_rows sequences run without
 * LayerNorm kernels inside the blocks: the residual GEMMs write fp16(x * scale) and per-tile row sums,
 * the q/k/v and MLP GEMMs normalise in their epilogue.  Measured slower than the kernels it removes
 * (the residual GEMMs then need complete sums, i.e. cluster splits); sessions read it when created.
 * "persist" (default 0): decode steps of an int4 model run all transformer blocks as one cooperative
 * kernel (decode sessions whose shape it supports).  Measured slower than the per-op CUDA graph.
 * Its aids: "persist_min_rows" / "persist_max_rows" (batch range it is used for), "persist_prefetch_mb",
 * "persist_wait_kcycles" (limit of its device-wide waits in thousands of SM cycles; default about one
 * second), "persist_fault_phase" (test aid: one block skips its arrival in that phase, so that the
 * bounded wait runs out and B200NN_ERR_DEVICE is reported; nothing hangs), "persist_trace" /
 * "trace" (stamp buffers for b200nn_ctx_read_persist_trace / b200nn_ctx_read_trace). */
B200NN_API int32_t b200nn_ctx_set_tuning(b200nn_ctx *ctx, const char *key, int32_t value);
/* Measurement aid: after set_tuning("trace", 1) the first block of the next tensor-core GEMM
 * writes SM-clock stamps of its pipeline events into a 256-slot buffer; this copies it out. */
B200NN_API int32_t b200nn_ctx_read_trace(b200nn_ctx *ctx, long long *out256);
/* Measurement aid of the persistent decode kernel (one cooperative launch for all transformer blocks
 * of an int4 decode step; tuning keys "persist" 0/1, "persist_min_rows", "persist_max_rows",
 * "persist_prefetch_mb", "persist_wait_kcycles" = bound of its grid-wide waits in thousands of SM
 * clocks, "persist_fault_phase" = test hook: block 0 leaves out its arrival after that phase so that
 * every bounded wait runs out and the step reports B200NN_ERR_DEVICE).  After
 * set_tuning("persist_trace", 1) each block stamps the global timer when the inputs of a phase are
 * ready and when it arrives at the phase's end, for the first 32 phases of a launch; this copies
 * out [block][32][2] nanosecond stamps (capacity in 64-bit words).  No counterpart in the reference. */
B200NN_API int32_t b200nn_ctx_read_persist_trace(b200nn_ctx *ctx, unsigned long long *out, size_t capacity);

/* ---- GpuTensor (GH/nn/tensor.rs:45-110, 201-221, 270) -------------------------------------- */
B200NN_API int32_t b200nn_tensor_from_host(b200nn_ctx *ctx, const float *host, const size_t *shape, int32_t ndim,
                                           b200nn_tensor **out);
B200NN_API int32_t b200nn_tensor_zeros(b200nn_ctx *ctx, const size_t *shape, int32_t ndim, b200nn_tensor **out);
/* GpuTensor::from_data (tensor.rs:67-77): a tensor over data that is already on this context's device.
 * The reference takes ownership of the caller's device slice; a foreign allocation cannot change owner
 * across this boundary, so the numel f32 values at dev are copied (device to device, on the context's
 * stream, complete on return) and the caller keeps its buffer. */
B200NN_API int32_t b200nn_tensor_from_device(b200nn_ctx *ctx, const float *dev, const size_t *shape, int32_t ndim,
                                             b200nn_tensor **out);
B200NN_API int32_t b200nn_tensor_to_host(const b200nn_tensor *t, float *host, size_t capacity_elems);
B200NN_API int32_t b200nn_tensor_ndim(const b200nn_tensor *t);
B200NN_API size_t b200nn_tensor_numel(const b200nn_tensor *t);
B200NN_API int32_t b200nn_tensor_shape(const b200nn_tensor *t, size_t *shape_out, int32_t capacity);
B200NN_API int32_t b200nn_tensor_reshape(const b200nn_tensor *t, const size_t *shape, int32_t ndim, b200nn_tensor **out);
B200NN_API int32_t b200nn_tensor_clone(const b200nn_tensor *t, b200nn_tensor **out);
/* GpuTensor::transpose(dim0, dim1), GpuTensor::concat(tensors, dim), GpuTensor::split(dim, sizes)
 * (tensor.rs:227-393; the reference goes through the host, these stay on the device).  Errors as there:
 * B200NN_ERR_DIM for a dimension out of range, B200NN_ERR_SHAPE for an empty list, mismatched shapes or
 * sizes that do not add up.  split writes `count` new tensors into outs. */
B200NN_API int32_t b200nn_tensor_transpose(const b200nn_tensor *t, size_t dim0, size_t dim1, b200nn_tensor **out);
B200NN_API int32_t b200nn_tensor_concat(const b200nn_tensor *const *tensors, size_t count, size_t dim, b200nn_tensor **out);
B200NN_API int32_t b200nn_tensor_split(const b200nn_tensor *t, size_t dim, const size_t *sizes, size_t count,
                                       b200nn_tensor **outs);
B200NN_API float *b200nn_tensor_data(b200nn_tensor *t); /* device pointer */
B200NN_API void b200nn_tensor_destroy(b200nn_tensor *t);

/* ---- host quantiser (GH/nn/ops/quantize.rs:56-162) ----------------------------------------- */
/* weight_t [K,N] row-major -> packed [K/8,N] u32 (nibble i of a word = k index 8*kp+i, value+8),
 * scales [ceil(K/group),N] f32.  K%8 != 0 returns B200NN_ERR_SHAPE (the reference asserts). */
B200NN_API int32_t b200nn_quantize_weight_int4(const float *weight_t, size_t k, size_t n, size_t group,
                                               uint32_t *packed, float *scales);
B200NN_API int32_t b200nn_quantize_int4_per_group(const float *data, size_t len, size_t group, uint32_t *packed,
                                                  float *scales);
B200NN_API int32_t b200nn_unpack_int4(uint32_t packed, int32_t index);
B200NN_API int32_t b200nn_pack_int8_to_u32(const int8_t *values, size_t n, uint32_t *packed);
B200NN_API int32_t b200nn_quantize_int8_per_tensor(const float *data, size_t n, int8_t *q, float *scale);

/* ---- stateless ops (GH/nn/ops/mod.rs:19-37) ------------------------------------------------- */
/* ops::layer_norm (ops/norm.rs:14-81). gamma/beta: tensors of [d]. */
B200NN_API int32_t b200nn_layer_norm(b200nn_ctx *ctx, const b200nn_tensor *x, const b200nn_tensor *gamma,
                                     const b200nn_tensor *beta, float eps, b200nn_tensor **out);
/* ops::layer_norm_residual_dual (ops/norm.rs:248-400): sum=a+b, norm=LN(sum); both returned. */
B200NN_API int32_t b200nn_layer_norm_residual_dual(b200nn_ctx *ctx, const b200nn_tensor *a, const b200nn_tensor *b,
                                                   const b200nn_tensor *gamma, const b200nn_tensor *beta, float eps,
                                                   b200nn_tensor **sum_out, b200nn_tensor **norm_out);
/* ops::gelu (ops/activation.rs:14-16) and the other Activation kinds; `act` is B200NN_ACT_*. */
B200NN_API int32_t b200nn_activation(b200nn_ctx *ctx, const b200nn_tensor *x, int32_t act, b200nn_tensor **out);
/* ops::bias_add (ops/reshape.rs:112-156): data[i] += bias[i % n_cols], in place. */
B200NN_API int32_t b200nn_bias_add(b200nn_ctx *ctx, b200nn_tensor *data, const b200nn_tensor *bias);
/* ops::elementwise_add (ops/reshape.rs:166-186): a += b, in place. */
B200NN_API int32_t b200nn_elementwise_add(b200nn_ctx *ctx, b200nn_tensor *a, const b200nn_tensor *b);
/* ops::split_qkv / ops::concat_heads (ops/attention.rs:105-142, 515-549). */
B200NN_API int32_t b200nn_split_qkv(b200nn_ctx *ctx, const b200nn_tensor *qkv, size_t seq_len, size_t n_heads,
                                    size_t d_head, b200nn_tensor **q, b200nn_tensor **k, b200nn_tensor **v);
B200NN_API int32_t b200nn_concat_heads(b200nn_ctx *ctx, const b200nn_tensor *heads, size_t seq_len, size_t n_heads,
                                       size_t d_head, b200nn_tensor **out);
/* ops::multi_head_flash_attention (ops/attention.rs:151-202): q,k,v [H,seq,64] -> [H,seq,64]. */
B200NN_API int32_t b200nn_multi_head_flash_attention(b200nn_ctx *ctx, const b200nn_tensor *q, const b200nn_tensor *k,
                                                     const b200nn_tensor *v, size_t seq_len, size_t n_heads,
                                                     size_t d_head, int32_t causal, b200nn_tensor **out);
/* ops::scaled_dot_product_attention_kv (ops/attention.rs:557-606): one head, q [q_len,64] against
 * k,v [kv_len,64], causal with q_offset. */
B200NN_API int32_t b200nn_attention_kv(b200nn_ctx *ctx, const b200nn_tensor *q, const b200nn_tensor *k,
                                       const b200nn_tensor *v, int32_t causal, size_t q_offset, b200nn_tensor **out);
/* ops::int4_matmul (ops/gemm.rs:1186-1266): quantise B [K,N] on the host, then A[M,K] x dequant(B). */
/* ops::matmul (ops/gemm.rs:20-212): a [M,K] x b [K,N] -> [M,N], both device tensors, f32 FMA arithmetic
 * (the weights of a Linear are better held by b200nn_linear_create, which keeps them in kernel layouts). */
B200NN_API int32_t b200nn_matmul(b200nn_ctx *ctx, const b200nn_tensor *a, const b200nn_tensor *b, b200nn_tensor **out);
B200NN_API int32_t b200nn_int4_matmul(b200nn_ctx *ctx, const b200nn_tensor *a, const float *b_host, size_t k, size_t n,
                                      size_t group, b200nn_tensor **out);

/* ---- Linear (GH/nn/layers/linear.rs:58-88, 131-166, 283-313) -------------------------------- */
/* weight [out,in] row-major host f32, bias [out] or NULL. */
B200NN_API int32_t b200nn_linear_create(b200nn_ctx *ctx, const float *weight, const float *bias, size_t in_features,
                                        size_t out_features, b200nn_linear **out);
B200NN_API int32_t b200nn_linear_forward(b200nn_linear *l, const b200nn_tensor *x, b200nn_tensor **y);
B200NN_API int32_t b200nn_linear_forward_fused(b200nn_linear *l, const b200nn_tensor *x, int32_t act, b200nn_tensor **y);
B200NN_API void b200nn_linear_destroy(b200nn_linear *l);

/* ---- Int4Linear (GH/nn/layers/int4_linear.rs:40-147) ---------------------------------------- */
/* packed [K/8,N] u32, scales [ceil(K/group),N] f32 (rounded to fp16 inside), bias [N] or NULL. */
B200NN_API int32_t b200nn_int4_linear_create(b200nn_ctx *ctx, const uint32_t *packed, const float *scales,
                                             const float *bias, size_t in_features, size_t out_features, size_t group,
                                             b200nn_int4_linear **out);
B200NN_API int32_t b200nn_int4_linear_forward(b200nn_int4_linear *l, const b200nn_tensor *x, b200nn_tensor **y);
/* Same computation on caller-owned buffers.  _dev: x [m,K], y [m,N] device f32, enqueued on the
 * context stream, no synchronisation.  _host: pageable or pinned host buffers; copies in, runs,
 * copies out and synchronises. */
B200NN_API int32_t b200nn_int4_linear_forward_dev(b200nn_int4_linear *l, const float *x_dev, size_t m, float *y_dev);
B200NN_API int32_t b200nn_int4_linear_forward_host(b200nn_int4_linear *l, const float *x_host, size_t m, float *y_host);
B200NN_API size_t b200nn_int4_linear_memory_bytes(const b200nn_int4_linear *l); /* int4_linear.rs:136-146 */
B200NN_API void b200nn_int4_linear_destroy(b200nn_int4_linear *l);

/* ---- LayerNorm (GH/nn/layers/norm.rs:24-55) -------------------------------------------------- */
B200NN_API int32_t b200nn_layernorm_create(b200nn_ctx *ctx, const float *gamma, const float *beta, size_t d, float eps,
                                           b200nn_layernorm **out);
B200NN_API int32_t b200nn_layernorm_forward(b200nn_layernorm *ln, const b200nn_tensor *x, b200nn_tensor **y);
B200NN_API void b200nn_layernorm_destroy(b200nn_layernorm *ln);

/* ---- Embedding (GH/nn/layers/embedding.rs:25-93) --------------------------------------------- */
B200NN_API int32_t b200nn_embedding_create(b200nn_ctx *ctx, const float *wte, const float *wpe, size_t vocab,
                                           size_t max_seq, size_t d, b200nn_embedding **out);
/* forward_tokens_with_offset: out[p,:] = wte[ids[p],:] + wpe[offset+p,:]; ids are host u32. */
B200NN_API int32_t b200nn_embedding_forward_tokens(b200nn_embedding *e, const uint32_t *ids_host, size_t n,
                                                   size_t pos_offset, b200nn_tensor **out);
B200NN_API void b200nn_embedding_destroy(b200nn_embedding *e);

/* ---- MultiHeadAttention (GH/nn/layers/attention.rs:30-184) ----------------------------------- */
/* qkv_weight [3d,d], qkv_bias [3d], out_weight [d,d], out_bias [d] (Linear layout [out,in]). */
B200NN_API int32_t b200nn_attention_create(b200nn_ctx *ctx, const float *qkv_weight, const float *qkv_bias,
                                           const float *out_weight, const float *out_bias, size_t n_embd,
                                           size_t n_heads, b200nn_attention **out);
/* Int4MultiHeadAttention::new (gpt2.rs:1141-1188): the same layer with both projections quantised to int4 at
 * construction (weights given [out,in]; quantised per group of `group_size` along the input dimension).
 * forward_causal / forward_cached / destroy are those of b200nn_attention. */
B200NN_API int32_t b200nn_int4_attention_create(b200nn_ctx *ctx, const float *qkv_weight, const float *qkv_bias,
                                                const float *out_weight, const float *out_bias, size_t n_embd,
                                                size_t n_heads, size_t group_size, b200nn_attention **out);
B200NN_API int32_t b200nn_attention_forward_causal(b200nn_attention *a, const b200nn_tensor *x, b200nn_tensor **y);
/* forward_cached: x [new_len,d]; cached_k/cached_v host f32 [n_heads][kv_len*d_head] flattened head
 * after head; returns y and the new K,V rows [n_heads][new_len*d_head] in host buffers. */
B200NN_API int32_t b200nn_attention_forward_cached(b200nn_attention *a, const b200nn_tensor *x, const float *cached_k,
                                                   const float *cached_v, size_t kv_len, b200nn_tensor **y,
                                                   float *new_k_out, float *new_v_out);
B200NN_API void b200nn_attention_destroy(b200nn_attention *a);

/* ---- GPT-2 models (GH/nn/models/gpt2.rs) ------------------------------------------------------ */
/* Gpt2Config (gpt2.rs:20-93). */
typedef struct {
    int32_t n_layer, n_embd, n_head, vocab_size, n_positions;
    float layer_norm_epsilon;
} b200nn_gpt2_config;
B200NN_API int32_t b200nn_gpt2_config_preset(const char *name /* small|medium|large|xl */, b200nn_gpt2_config *out);

/* Gpt2Weights / TransformerLayerWeights (GH/model.rs:112-154): host f32, dense weights in the
 * checkpoint's Conv1D layout [in,out]. */
typedef struct {
    const float *ln_1_weight, *ln_1_bias;
    const float *c_attn_weight /* [d,3d] */, *c_attn_bias;
    const float *c_proj_weight /* [d,d] */, *c_proj_bias;
    const float *ln_2_weight, *ln_2_bias;
    const float *mlp_fc_weight /* [d,4d] */, *mlp_fc_bias;
    const float *mlp_proj_weight /* [4d,d] */, *mlp_proj_bias;
} b200nn_gpt2_layer_weights;
typedef struct {
    const float *wte /* [vocab,d] */, *wpe /* [n_positions,d] */;
    const float *ln_f_weight, *ln_f_bias;
    const b200nn_gpt2_layer_weights *layers; /* n_layer entries */
} b200nn_gpt2_weights;

/* Gpt2Model::from_weights (gpt2.rs:337-404): f32 weights. */
B200NN_API int32_t b200nn_gpt2_create(b200nn_ctx *ctx, const b200nn_gpt2_config *cfg, const b200nn_gpt2_weights *w,
                                      uint32_t flags, b200nn_gpt2 **out);
/* Int4Gpt2Model::from_weights (gpt2.rs:1356-1436): quantises every block Linear on the host with
 * the rule of quantize.rs:102-153 (scales then rounded to fp16); embeddings and LayerNorm stay f32;
 * the LM head stays f32 unless B200NN_QUANT_LM_HEAD. */
B200NN_API int32_t b200nn_int4_gpt2_create(b200nn_ctx *ctx, const b200nn_gpt2_config *cfg, const b200nn_gpt2_weights *w,
                                           size_t group_size, uint32_t flags, b200nn_gpt2 **out);
B200NN_API void b200nn_gpt2_destroy(b200nn_gpt2 *m);
B200NN_API int32_t b200nn_gpt2_get_config(const b200nn_gpt2 *m, b200nn_gpt2_config *out);
/* Int4Gpt2Model::quantized_memory_bytes (gpt2.rs:1563-1576); 0 for an f32 model. */
B200NN_API size_t b200nn_gpt2_quantized_memory_bytes(const b200nn_gpt2 *m);
/* Read back the int4 data the model holds for one block Linear (which: 0 c_attn, 1 c_proj, 2 mlp.c_fc,
 * 3 mlp.c_proj; layer -1 with which 0 = the LM head), in the reference layout: packed [K/8,N], scales
 * [ceil(K/g),N] (already fp16-rounded).  Lets a checker run the same nibbles through its own math. */
B200NN_API int32_t b200nn_gpt2_get_int4(const b200nn_gpt2 *m, int32_t layer, int32_t which, uint32_t *packed,
                                        float *scales, size_t *k_out, size_t *n_out);

/* ---- TransformerBlock / Int4TransformerBlock (gpt2.rs:98-289, 1219-1339) ---------------------------
 * One pre-LN block: x += Attn(LN1(x)); x += W2.GELU(W1.LN2(x)+b1)+b2.  The twelve slices are what
 * TransformerBlock::new takes (gpt2.rs:120-135), dense weights in Linear layout [out,in]:
 * attn_qkv_weight [3d,d], attn_out_weight [d,d], ffn_up_weight [4d,d], ffn_down_weight [d,4d]. */
typedef struct {
    const float *ln_1_weight, *ln_1_bias;
    const float *attn_qkv_weight, *attn_qkv_bias;
    const float *attn_out_weight, *attn_out_bias;
    const float *ln_2_weight, *ln_2_bias;
    const float *ffn_up_weight, *ffn_up_bias;
    const float *ffn_down_weight, *ffn_down_bias;
} b200nn_block_weights;
/* TransformerBlock::new (gpt2.rs:120-170); cfg gives n_embd, n_head and layer_norm_epsilon; flags as
 * for the models (B200NN_GELU_SIGMOID). */
B200NN_API int32_t b200nn_block_create(b200nn_ctx *ctx, const b200nn_gpt2_config *cfg, const b200nn_block_weights *w,
                                       uint32_t flags, b200nn_block **out);
/* Int4TransformerBlock::new (gpt2.rs:1232-1296) with Int4MultiHeadAttention::new (1141-1188): every
 * dense weight is transposed to [in,out] and quantised with quantize_weight_int4 (scales rounded to fp16). */
B200NN_API int32_t b200nn_int4_block_create(b200nn_ctx *ctx, const b200nn_gpt2_config *cfg, const b200nn_block_weights *w,
                                            size_t group_size, uint32_t flags, b200nn_block **out);
/* TransformerBlock::forward / forward_auto_fused, Int4TransformerBlock::forward (gpt2.rs:172-243,
 * 1299-1339): x [seq_len,d] of one sequence, causal attention over its rows -> [seq_len,d].  The fused
 * epilogues are always on, so forward_auto_fused is this call. */
B200NN_API int32_t b200nn_block_forward(b200nn_block *b, const b200nn_tensor *x, b200nn_tensor **y);
/* TransformerBlock::forward_cached (gpt2.rs:249-288): x [new_len,d] at positions kv_len..; cached_k /
 * cached_v host f32 [n_head][kv_len*64] (NULL when kv_len is 0); returns y and, when the pointers are
 * given, the new K,V rows [n_head][new_len*64] (the values the fp16 cache holds). */
B200NN_API int32_t b200nn_block_forward_cached(b200nn_block *b, const b200nn_tensor *x, const float *cached_k,
                                               const float *cached_v, size_t kv_len, b200nn_tensor **y, float *new_k_out,
                                               float *new_v_out);
B200NN_API void b200nn_block_destroy(b200nn_block *b);

/* Gpt2Model::forward / Int4Gpt2Model::forward (gpt2.rs:481-499, 1522-1533): one sequence of host
 * token ids -> logits [seq_len,vocab] for every position. */
B200NN_API int32_t b200nn_gpt2_forward(b200nn_gpt2 *m, const uint32_t *ids_host, size_t seq_len, b200nn_tensor **logits);

/* KvCache (gpt2.rs:1064-1117), device resident, fp16, with a batch axis added:
 * [layer][sequence][head][capacity][64] for K and V. */
B200NN_API int32_t b200nn_kvcache_create(b200nn_gpt2 *m, size_t batch, size_t capacity, b200nn_kvcache **out);
B200NN_API size_t b200nn_kvcache_len(const b200nn_kvcache *c);
B200NN_API int32_t b200nn_kvcache_reset(b200nn_kvcache *c);
B200NN_API void b200nn_kvcache_destroy(b200nn_kvcache *c);
/* Gpt2Model::forward_cached (gpt2.rs:712-734): ids_host is [batch,new_len] (batch = the cache's);
 * appends to the cache and returns logits [batch*new_len,vocab]. */
B200NN_API int32_t b200nn_gpt2_forward_cached(b200nn_gpt2 *m, const uint32_t *ids_host, size_t new_len,
                                              b200nn_kvcache *cache, b200nn_tensor **logits);

/* Gpt2Model::generate / generate_cached, Int4Gpt2Model::generate (gpt2.rs:672-706, 740-783,
 * 1536-1560): greedy decoding of one sequence.  out_tokens holds prompt_len+max_new entries;
 * *n_out = prompt + generated count.  Both run KV-cached on the device (same tokens as the
 * reference's uncached loop, which recomputes the same positions). */
B200NN_API int32_t b200nn_gpt2_generate(b200nn_gpt2 *m, const uint32_t *prompt, size_t prompt_len, size_t max_new,
                                        uint32_t flags, uint32_t *out_tokens, size_t *n_out);
B200NN_API int32_t b200nn_gpt2_generate_cached(b200nn_gpt2 *m, const uint32_t *prompt, size_t prompt_len,
                                               size_t max_new, uint32_t flags, uint32_t *out_tokens, size_t *n_out);
/* Batched greedy decoding (added axis; batch=1 equals the call above): prompts [batch,prompt_len]
 * host u32 -> out_tokens [batch,prompt_len+max_new], out_lens [batch]. */
B200NN_API int32_t b200nn_gpt2_generate_batch(b200nn_gpt2 *m, const uint32_t *prompts, size_t batch, size_t prompt_len,
                                              size_t max_new, uint32_t flags, uint32_t *out_tokens, size_t *out_lens);

/* Gpt2Model::forward_features (gpt2.rs:570-581): hidden states after every block and the final
 * LayerNorm, [seq_len, n_embd] f32, for callers that bring their own head (LoRA, retrieval). */
B200NN_API int32_t b200nn_gpt2_forward_features(b200nn_gpt2 *m, const uint32_t *ids_host, size_t seq_len,
                                                b200nn_tensor **features);
/* Gpt2Model::embedding_table (gpt2.rs:584-586): wte [vocab,n_embd] and wpe [n_positions,n_embd] as
 * tensors that share the model's device buffers; destroy them with b200nn_tensor_destroy. */
B200NN_API int32_t b200nn_gpt2_embedding_table(b200nn_gpt2 *m, b200nn_tensor **wte, b200nn_tensor **wpe);
/* Gpt2Model::forward_diagnostic (gpt2.rs:595-667): forward of one sequence plus the values the
 * reference prints to stderr while it runs, returned instead of printed: the first four hidden values
 * after the embedding (position 0 and the last position), after block 0 and after the last block (last
 * position; with the number of NaN/Inf values in the whole hidden state), after the final LayerNorm
 * (last position), and the five highest logits of the last position with their token ids. */
typedef struct {
    float embedding_first[4], embedding_last[4];
    float block0_last[4], final_block_last[4];
    int32_t block0_nonfinite, final_block_nonfinite;
    float ln_f_last[4];
    uint32_t top_tokens[5];
    float top_scores[5];
    int32_t n_top;
} b200nn_gpt2_diagnostic;
B200NN_API int32_t b200nn_gpt2_forward_diagnostic(b200nn_gpt2 *m, const uint32_t *ids_host, size_t seq_len,
                                                  b200nn_tensor **logits, b200nn_gpt2_diagnostic *diag);
/* Gpt2Model::forward_profiled (gpt2.rs:529-568): forward plus the device time in milliseconds of
 * every component in the reference's order: embedding, block_0 .. block_{L-1}, ln_f, lm_head
 * (n_layer + 3 values; `capacity` is the length of times_ms). */
B200NN_API int32_t b200nn_gpt2_forward_profiled(b200nn_gpt2 *m, const uint32_t *ids_host, size_t seq_len,
                                                b200nn_tensor **logits, float *times_ms, int32_t capacity,
                                                int32_t *n_times);

/* ---- data-dependent decoding (gpt2.rs:785-1058) ------------------------------------------------ */
/* SimpleRng (gpt2.rs:1000-1023): xorshift64; the state is a plain u64 the caller keeps.  _new maps
 * seed 0 to the reference's fixed non-zero constant; _next_f32 advances the state and returns
 * (state >> 40) / 2^24 in [0,1). */
B200NN_API uint64_t b200nn_simple_rng_new(uint64_t seed);
B200NN_API float b200nn_simple_rng_next_f32(uint64_t *state);
/* Seeded synthetic tensors from the reference's own generator, so that a Rust caller holding only
 * SimpleRng (gpt2.rs:1000-1023) can regenerate them bit for bit: n uniforms in [0,1) (next_f32), or n
 * normals N(0, std_dev) by Box-Muller in f64 on consecutive pairs of uniforms (u1, u2):
 * sqrt(-2 ln(1-u1)) cos(2 pi u2), then sqrt(-2 ln(1-u1)) sin(2 pi u2), each times std_dev, cast to f32.
 * No counterpart in the reference (it has no synthetic-weight generator). */
B200NN_API int32_t b200nn_simple_rng_fill_uniform(uint64_t *state, size_t n, float *out);
B200NN_API int32_t b200nn_simple_rng_fill_normal(uint64_t *state, size_t n, float std_dev, float *out);
/* top_k_sample (gpt2.rs:1029-1058) on a host logits vector: logits / max(temperature, 1e-8), the k
 * largest in the order of a stable descending sort, f32 softmax over them, one draw, cumulative search. */
B200NN_API int32_t b200nn_top_k_sample(const float *logits, size_t n, size_t k, float temperature, uint64_t *rng_state,
                                       uint32_t *token_out);
/* Gpt2Model::generate_cached_sampling (gpt2.rs:933-977): KV-cached decoding of one sequence, every
 * token drawn with top_k_sample; stops before appending token 50256.  The k candidates are selected
 * on the device; the draw is the host code above.  out_tokens holds prompt_len+max_new entries. */
B200NN_API int32_t b200nn_gpt2_generate_cached_sampling(b200nn_gpt2 *m, const uint32_t *prompt, size_t prompt_len,
                                                        size_t max_new, size_t top_k, float temperature,
                                                        uint64_t *rng_state, uint32_t *out_tokens, size_t *n_out);
/* Gpt2Model::forward_early_exit (gpt2.rs:797-830): returns the logits [seq_len,vocab] of the first
 * block (probed through LN_f + LM head after every block but the last) at which the largest softmax
 * probability of the last position reaches `threshold`, and the number of blocks run (1..n_layer). */
B200NN_API int32_t b200nn_gpt2_forward_early_exit(b200nn_gpt2 *m, const uint32_t *ids_host, size_t seq_len,
                                                  float threshold, b200nn_tensor **logits, int32_t *layers_used);
/* Gpt2Model::generate_cached_early_exit (gpt2.rs:837-924): greedy (last maximum on ties), prefill with
 * every layer, each decode step with as many blocks as the probe's confidence asks for; the skipped
 * layers get zero K/V rows for that position.  layers_per_step holds 1+max_new entries (the prefill
 * first); *n_steps is how many were written. */
B200NN_API int32_t b200nn_gpt2_generate_cached_early_exit(b200nn_gpt2 *m, const uint32_t *prompt, size_t prompt_len,
                                                          size_t max_new, float threshold, uint32_t *out_tokens,
                                                          size_t *n_out, int32_t *layers_per_step, size_t *n_steps);

/* ---- decode session: the batched generate loop in pieces, state resident on the device -------- */
/* A session owns a KV cache for `batch` sequences of up to `capacity` positions plus the step
 * buffers.  prefill() runs the prompts and picks the first token; step() runs n greedy decode
 * steps, feeding each sequence's token back on the device, without host synchronisation. */
B200NN_API int32_t b200nn_session_create(b200nn_gpt2 *m, size_t batch, size_t capacity, uint32_t flags,
                                         b200nn_session **out);
B200NN_API int32_t b200nn_session_prefill(b200nn_session *s, const uint32_t *prompts_host, size_t prompt_len);
B200NN_API int32_t b200nn_session_step(b200nn_session *s, size_t n_steps);
/* Move the position counter back (keeps the cache contents): lets a benchmark time the same
 * context window repeatedly. */
B200NN_API int32_t b200nn_session_rewind(b200nn_session *s, size_t position);
B200NN_API size_t b200nn_session_position(const b200nn_session *s);
/* Tokens generated so far, [batch,generated] host u32 (synchronises). */
B200NN_API int32_t b200nn_session_tokens(b200nn_session *s, uint32_t *out, size_t capacity_per_seq, size_t *generated);
/* Logits of the most recent step, [batch,vocab] host f32 (synchronises). */
B200NN_API int32_t b200nn_session_logits(b200nn_session *s, float *out);
/* Per-kernel-family device time of ONE decode step at the current position, measured with CUDA
 * events around each launch (Gpt2Model::forward_profiled, gpt2.rs:529-568).  times_ms has
 * B200NN_PROF_COUNT entries. */
enum {
    B200NN_PROF_EMBED = 0, B200NN_PROF_LAYERNORM, B200NN_PROF_LINEAR, B200NN_PROF_ATTENTION,
    B200NN_PROF_LM_HEAD, B200NN_PROF_ARGMAX, B200NN_PROF_COUNT
};
B200NN_API int32_t b200nn_session_profile_step(b200nn_session *s, float *times_ms, uint64_t *linear_bytes);
/* Device time of ONE kernel family in isolation: launches only that family's kernels of a decode
 * step (e.g. the decode-attention launch of every layer) `reps` times back to back at the current
 * position, between two CUDA events on the context's stream.  *ms_total is the elapsed time,
 * *launches the number of kernels it covers.  The activations are left in an arbitrary state:
 * call prefill() again before decoding on. */
B200NN_API int32_t b200nn_session_time_family(b200nn_session *s, int32_t family, int32_t reps, float *ms_total,
                                              uint64_t *launches);
B200NN_API void b200nn_session_destroy(b200nn_session *s);

/* ---- checkpoints: the safetensors container and the GPT-2 loader (GH/model.rs) ------------------ */
/* The reference reads checkpoints with the `safetensors` crate; these entry points read the same
 * public format (8-byte little-endian header length, JSON header, raw little-endian data) on the
 * host.  open() parses and validates the header only; tensors are listed sorted by name as
 * list_tensors does (model.rs:201-221) and read on demand.  Host-only: no context needed; the text
 * of the calling thread's last failure comes from b200nn_safetensors_last_error(). */
typedef struct b200nn_safetensors b200nn_safetensors;
B200NN_API int32_t b200nn_safetensors_open(const char *path, b200nn_safetensors **out);
B200NN_API void b200nn_safetensors_close(b200nn_safetensors *st);
B200NN_API int32_t b200nn_safetensors_count(const b200nn_safetensors *st);
/* TensorInfo (model.rs:186-198): name, dtype string ("F32", "U32", ...), shape, size in bytes.  The
 * strings stay valid until close(). */
B200NN_API int32_t b200nn_safetensors_info(const b200nn_safetensors *st, int32_t index, const char **name,
                                           const char **dtype, size_t *shape_out, int32_t shape_capacity, int32_t *ndim,
                                           size_t *nbytes);
B200NN_API int32_t b200nn_safetensors_find(const b200nn_safetensors *st, const char *name); /* index or -1 */
/* Raw bytes of one tensor (load_all_tensors, model.rs:388-397, is this over every F32 tensor). */
B200NN_API int32_t b200nn_safetensors_read(const b200nn_safetensors *st, int32_t index, void *out, size_t capacity_bytes);
B200NN_API const char *b200nn_safetensors_last_error(void);
/* load_gpt2_weights (model.rs:308-386) followed by Gpt2Model::from_weights / Int4Gpt2Model::from_weights:
 * Hugging Face key names (wte.weight, wpe.weight, ln_f.*, h.{i}.ln_1.*, h.{i}.attn.c_attn.*,
 * h.{i}.attn.c_proj.*, h.{i}.ln_2.*, h.{i}.mlp.c_fc.*, h.{i}.mlp.c_proj.*), every tensor F32 with
 * exactly the shape the configuration implies (Conv1D weights [in,out]); a missing tensor returns
 * B200NN_ERR_MISSING, another dtype B200NN_ERR_UNSUPPORTED, another shape B200NN_ERR_SHAPE.  The
 * reference's loader is fixed to GPT-2 Small; here cfg may be any GPT-2 shape, or NULL to read it
 * off the file (vocab, width and positions from wte / wpe, layers counted, heads = width / 64).
 * int4_group 0 builds the f32 model, otherwise the int4 model quantised with that group size. */
B200NN_API int32_t b200nn_gpt2_load_safetensors(b200nn_ctx *ctx, const char *path, const b200nn_gpt2_config *cfg,
                                                size_t int4_group, uint32_t flags, b200nn_gpt2 **out);

/* ---- Gpt2Tokenizer (crates/core/gpu-host/src/tokenizer.rs:34-62) ---------------------------------
 * Host code.  The reference wraps tiktoken-rs' r50k_base; here the byte-level BPE is implemented over a
 * vocabulary given at run time: a file in tiktoken's format (one "base64(token bytes) rank" per
 * line, as r50k_base.tiktoken is published) or a table in memory.  `endoftext_id` is the id of the
 * special token <|endoftext|> (50256 for GPT-2; tokenizer.rs:10-11).  Every single byte must be a
 * token.  b200nn_bpe_encode = Gpt2Tokenizer::encode (encode_with_special_tokens), b200nn_bpe_decode =
 * ::decode (returns raw bytes; the caller checks UTF-8), b200nn_bpe_vocab_size = ::vocab_size.
 * b200nn_bpe_encode_piece merges one already-split piece (for hosts that split with their own Unicode
 * tables; the library's splitter is exact for ASCII and approximates \p{L} / \p{N} by block beyond).
 * Buffers too small return B200NN_ERR_SHAPE with the needed length in *n_out. */
typedef struct b200nn_bpe b200nn_bpe;
B200NN_API int32_t b200nn_bpe_load(const char *path, uint32_t endoftext_id, b200nn_bpe **out);
/* token i = token_bytes[token_offsets[i] .. token_offsets[i+1]) with rank ranks[i] */
B200NN_API int32_t b200nn_bpe_create(const uint8_t *token_bytes, const size_t *token_offsets, const uint32_t *ranks,
                                     size_t n_tokens, uint32_t endoftext_id, b200nn_bpe **out);
B200NN_API void b200nn_bpe_destroy(b200nn_bpe *t);
B200NN_API size_t b200nn_bpe_vocab_size(const b200nn_bpe *t);
B200NN_API int32_t b200nn_bpe_encode(const b200nn_bpe *t, const uint8_t *text, size_t n, uint32_t *out, size_t capacity,
                                     size_t *n_out);
B200NN_API int32_t b200nn_bpe_encode_piece(const b200nn_bpe *t, const uint8_t *piece, size_t n, uint32_t *out,
                                           size_t capacity, size_t *n_out);
B200NN_API int32_t b200nn_bpe_decode(const b200nn_bpe *t, const uint32_t *ids, size_t n, uint8_t *out, size_t capacity,
                                     size_t *n_out);
B200NN_API const char *b200nn_bpe_last_error(void);

/* ---- batched attention on caller-owned fp16 device buffers ----------------------------------------
 * The model path's attention kernels as stand-alone, stream-ordered operations (what
 * ops::multi_head_flash_attention / flash_attention_kv, ops/attention.rs:151-202, 557-606, are to the
 * reference's layers), with the batch axis and the fp16 cache layout of this library:
 *   q_dev, out_dev              fp16 [batch*rows, n_heads*64], token-major (rows = seq_len, or 1 for decode)
 *   k_cache_dev, v_cache_dev    fp16 [batch][n_heads][capacity][64], new positions already appended
 * prefill: row i of a sequence sits at position past+i and attends to positions 0..past+i (tcgen05
 * kernel); decode: one query per sequence against positions 0..ctx_len-1.  All buffers 16-byte aligned. */
B200NN_API int32_t b200nn_prefill_attention_f16(b200nn_ctx *ctx, const void *q_dev, const void *k_cache_dev,
                                                const void *v_cache_dev, int32_t batch, int32_t n_heads, int32_t capacity,
                                                int32_t seq_len, int32_t past, void *out_dev);
B200NN_API int32_t b200nn_decode_attention_f16(b200nn_ctx *ctx, const void *q_dev, const void *k_cache_dev,
                                               const void *v_cache_dev, int32_t batch, int32_t n_heads, int32_t capacity,
                                               int32_t ctx_len, void *out_dev);

/* ---- decode attention without any allocation ----------------------------------------------------
 * This entry point has no counterpart in the reference.  It is for callers that cannot let the
 * library call cudaMalloc: a host that has handed out its whole device-memory budget, or code that
 * runs where an allocation would synchronise the device (inside a latency-critical loop).
 * It needs no context: the caller passes the device ordinal, its own
 * stream (NULL = default stream), and device buffers it owns:
 *   q_dev   [batch, n_heads*64] f32    one query row per sequence
 *   k_cache_dev, v_cache_dev  fp16 [batch][n_heads][capacity][64], positions [0, ctx_len) filled;
 *                             both 16-byte aligned (rows are read with 16-byte loads; a misaligned
 *                             pointer returns B200NN_ERR_ARG instead of faulting on the device)
 *   out_dev [batch, n_heads*64] f32
 * and gets softmax(q.K^T/8).V per (sequence, head) over the first ctx_len positions, computed by
 * the same kernel as the regular decode path.  The kernel's split-context scratch is a fixed
 * array inside the library image (about 4.2 MB per GPU, held until the process exits), so
 * batch*n_heads must not exceed 4096; larger requests return B200NN_ERR_SHAPE.  The first call on
 * a device looks up the array's device address; make that call before capturing a stream.  All
 * calls share the array: calls that overlap on the GPU (different streams) race.  No cudaMalloc,
 * cudaFree or allocating library routine is called.  b200nn_noalloc_last_error() gives the text of
 * the calling thread's last failure. */
B200NN_API int32_t b200nn_decode_attention_noalloc(int32_t device, void *stream, const float *q_dev,
                                                   const void *k_cache_dev, const void *v_cache_dev, int32_t batch,
                                                   int32_t n_heads, int32_t capacity, int32_t ctx_len, float *out_dev);
B200NN_API const char *b200nn_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* B200NN_H */
