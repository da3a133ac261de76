// Internal declarations shared by the translation units of libb200nn.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "b200nn.h"

// Device blocks released by tensors, workspaces and KV caches are kept for reuse instead of going
// back to the driver: cudaMalloc / cudaFree of a multi-gigabyte KV cache cost tens of milliseconds
// and synchronise the device, which a generate call per request cannot afford.  Shared between the
// context and its buffers so that a buffer may outlive the context (it then frees directly).
struct DevPool {
    std::mutex mu;
    std::multimap<size_t, void *> free_blocks; // by size
    size_t held_bytes = 0;
    bool alive = true;                          // false once the context is gone
    static constexpr size_t MAX_HELD = (size_t)64 << 30;
};

// ---------------------------------------------------------------------------------------------
// context
// ---------------------------------------------------------------------------------------------
struct DevBuf;
struct b200nn_ctx {
    int device = 0;
    std::shared_ptr<DevPool> pool = std::make_shared<DevPool>();
    cudaStream_t stream = nullptr;
    std::string last_error;
    int last_cuda = 0;
    int sm_count = 148;
    int gemv_max_rows = 2;       // rows at or below this take the CUDA-core GEMV
    int ln_rows_min = 1024;      // LayerNorm of at least this many rows (no residual) takes the warp-per-row kernel
    int ln_fold = 0;             // 1: decode steps of int4 models fold each block LayerNorm into the GEMMs around it (measured slower than the LayerNorm kernels: the residual GEMMs then need complete sums, i.e. cluster splits)
    int fused_argmax = 1;        // greedy decode steps take the argmax in the LM head's epilogue (0: separate kernel)
    uint64_t launches = 0;       // kernels launched by this library
    uint32_t *dev_err = nullptr; // device error word (bounded waits report here)
    uint32_t *host_err = nullptr; // pinned landing place of that word for stream_sync_check
    // split-K / split-KV scratch, grown on demand outside stream capture
    float *scratch = nullptr;
    size_t scratch_bytes = 0;
    unsigned *counters = nullptr; // arrival counters, self-resetting, zeroed at allocation
    size_t n_counters = 0;
    std::vector<void *> retired;  // outgrown scratch / counter blocks, freed with the context
    void *encode_tiled = nullptr; // cuTensorMapEncodeTiled, resolved through the runtime
    int tc_mb = 0, tc_splits = 0; // tensor-core GEMM tuning overrides (0 = automatic)
    int tc_min_kb_cluster = 6;    // the same for splits that run as a cluster (their partial tiles cross shared memory)
    int tc_min_kb = 0;            // fewest 64-wide K blocks a K split of the residual epilogue may get; 0 = by row count:
                                  // 2 up to 64 rows, 3 above (GPT-2 XL step, ms with 2 / 3: 32 rows 1.717 / 1.723,
                                  // 48 rows 2.164 / 2.202, 64 rows 2.433 / 2.475, 96 rows 3.099 / 3.085, 128 rows
                                  // 3.404 / 3.399; 4 is slower everywhere below 256 rows, where nothing splits)
    long long *trace = nullptr;  // optional device buffer for in-kernel time stamps (measurement aid)
    int attn_tc = 1;              // prefill attention with fp16 q and output runs on the tensor cores
    int attn_stream = 1;          // decode attention over many (sequence, head) pairs uses the TMA-fed kernel
    int attn_stream_min10 = 20;   // ... when there are at least this many tenths of a pair per warp of its grid
                                  // (measured: 2.7 pairs per warp 9 % faster than the split kernel, 1.35 pairs 13 % slower)
    int attn_stream_wide_min10 = 25; // ... and its 16-warp shape from this many tenths of a pair per warp of that grid (0 = never;
                                  // GPT-2 XL, ms of attention per step with 16 / 8 warps: 256 sequences 2.49–2.52 / 2.61, 224: 2.36 / 2.33, 192: 2.11 / 2.05)
    int attn_split_items = 0;    // items the streaming decode attention hands out as two halves at the end
    int attn_blocks_per_sm = 4;  // blocks per SM the split-context decode attention aims for when it splits the context
    int kv_prefetch_mb = 64;     // KV-cache bytes the streaming decode attention asks into L2 before its wait
    int pdl = 1;                  // launch the decode-step kernels with programmatic dependent launch
    int f32_tc = 2;               // f32 Linears of more than four rows on the tensor cores: 0 off (f32 FMA kernels),
                                  // 1 weight rounded to fp16, 2 weight as fp16 hi + lo (two products per K block)
    std::shared_ptr<DevBuf> xh;   // fp16 copy of an f32 activation handed to such a Linear
    int tc_persistent = 1;        // the plain fp16 GEMM runs one persistent block per SM from two 256-row tiles per SM on
    int int4_via_f16 = 1;         // int4 Linears with that many tiles dequantise the weight to fp16 once and use that GEMM
    std::shared_ptr<DevBuf> wh;   // the dequantised weight, [N,K] fp16, one Linear at a time
    bool capturing = false;      // true while a decode step is being captured into a graph
    // one persistent kernel for all transformer blocks of an int4 decode step (decode_persistent.cu)
    int persist = 0;              // 1: decode steps of persist_min_rows..persist_max_rows rows take it (opt-in: measured
                                  // slower than one kernel per operation on GPT-2 XL at every batch size, see decode_persistent.cu)
    int persist_min_rows = 3, persist_max_rows = 256; // decode batches (rows) that take it
    int persist_prefetch_mb = 48; // KV-cache megabytes per layer it asks into L2 ahead of the attention phase
    long long persist_wait_cycles = 0; // bound of its grid-wide waits in SM clocks (0: about a second)
    void *persist_trace = nullptr; // optional stamp buffer [148][32][2] u64 (measurement aid, "persist_trace")
    int persist_fault_phase = -1; // test hook: block 0 leaves out its arrival after this phase, so the bounded
                                  // waits of every other block run out (-1: never)
};

int set_error(b200nn_ctx *ctx, int code, const std::string &msg);
int set_cuda_error(b200nn_ctx *ctx, cudaError_t e, const char *what);
int ensure_scratch(b200nn_ctx *ctx, size_t bytes, size_t counters);
int stream_sync_check(b200nn_ctx *ctx); // stream synchronise + device error word -> B200NN_ERR_DEVICE

#define CK(ctx, call)                                                     \
    do {                                                                  \
        cudaError_t _e = (call);                                          \
        if (_e != cudaSuccess) return set_cuda_error((ctx), _e, #call);   \
    } while (0)

#define CK_LAUNCH(ctx, name)                                              \
    do {                                                                  \
        (ctx)->launches++;                                                \
        cudaError_t _e = cudaPeekAtLastError();                           \
        if (_e != cudaSuccess) return set_cuda_error((ctx), _e, name);    \
    } while (0)

// Every kernel of the library asks for the largest shared-memory carve-out, so that consecutive
// kernels of a decode step never make the SMs re-partition L1 / shared memory between launches
// (the tensor-core GEMM needs ~100-180 KB of shared memory; a kernel that prefers L1 before or after
// it costs a reconfiguration of several microseconds).  Call once per kernel function.
template <typename Kernel>
inline void prefer_max_smem(Kernel kern) {
    cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
}
#define PREFER_SMEM_ONCE(kern)                    \
    do {                                          \
        static bool _done[16] = {};               \
        int _dev = 0;                             \
        cudaGetDevice(&_dev);                     \
        if (!_done[_dev & 15]) {                  \
            prefer_max_smem(kern);                \
            _done[_dev & 15] = true;              \
        }                                         \
    } while (0)

// Launch with programmatic dependent launch allowed: the kernel may start while its predecessor
// on the stream is still running and must execute pdl_wait() (griddepcontrol.wait) before it reads
// or writes anything the predecessor touches.  Only kernels that do so are launched this way.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(b200nn_ctx *ctx, void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem,
                              Args &&...args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

#define TRY(expr)                       \
    do {                                \
        int _rc = (expr);               \
        if (_rc != B200NN_OK) return _rc; \
    } while (0)

struct DevBuf {
    void *p = nullptr;
    size_t bytes = 0;
    int device = 0;
    size_t block_bytes = 0;        // size of the underlying allocation (>= bytes)
    std::shared_ptr<DevPool> pool; // where the block goes when the buffer dies
    ~DevBuf();
};
int dev_alloc(b200nn_ctx *ctx, size_t bytes, std::shared_ptr<DevBuf> *out);
void pool_trim(b200nn_ctx *ctx); // returns every kept block to the driver

struct b200nn_tensor {
    b200nn_ctx *ctx = nullptr;
    std::shared_ptr<DevBuf> buf;
    std::vector<size_t> shape;
    size_t numel = 0;
    float *data() const { return static_cast<float *>(buf->p); }
};
int tensor_alloc(b200nn_ctx *ctx, const std::vector<size_t> &shape, bool zero, b200nn_tensor **out);

// ---------------------------------------------------------------------------------------------
// weights in kernel layouts
// ---------------------------------------------------------------------------------------------
static constexpr int TILE_N = 128;   // output features per weight tile
static constexpr int TILE_K = 64;    // reduction elements per weight tile
static constexpr int TILE_BYTES = TILE_N * TILE_K / 2; // 4096

// Int4 weight of a Linear y = x * dequant(W) (+bias); reference layout packed [K/8,N], scales
// [ceil(K/g),N] (int4_linear.rs:18-33).  `tiled` is the layout the fast kernels stream:
//   tile (nt, kb) at byte (nt*k_blocks + kb)*4096, holding rows n = nt*128 .. +127 and
//   k = kb*64 .. +63 as [plane 2][row 128][16 bytes]; plane p of a row carries words j = 4p..4p+3,
//   word j = k indices 8j..8j+7 of the block with nibble positions 0..7 holding
//   k offsets 0,2,4,6,1,3,5,7 (so that (w & 0x000f000f) yields the half2 pair (k0,k1), etc.).
//   Rows n >= N are stored as nibble 8 (value 0).
// `scales_h` is [n_groups][n_pad] fp16.  Shapes that do not fit (K%64, group%64) keep the
// reference layout in `ref_packed`/`ref_scales` and run on the one-thread-per-output kernel.
struct Int4Weight {
    int K = 0, N = 0, group = 0;
    int n_tiles = 0, k_blocks = 0, n_pad = 0, n_groups = 0;
    bool fast = false;
    std::shared_ptr<DevBuf> tiled, scales_h, bias, ref_packed, ref_scales;
    std::vector<uint32_t> host_packed; // reference-layout copies for read-back
    std::vector<float> host_scales;    // fp16-rounded values
    size_t memory_bytes() const { return host_packed.size() * 4 + host_scales.size() * 4; }
};
int int4_weight_upload(b200nn_ctx *ctx, const uint32_t *packed, const float *scales, const float *bias, size_t K,
                       size_t N, size_t group, Int4Weight *out);
// The two per-feature vectors a Linear needs to take a LayerNorm (scale g, shift beta, both [K] on the
// device) in through its epilogue (see Epilogue): gsum[n] = sum_k g_k w_kn and
// bc[n] = sum_k beta_k w_kn + bias[n], with w the dequantised weight as the kernels see it
// (fp16(nibble * fp16 scale)); accumulated in f64.
int int4_weight_ln_fold(b200nn_ctx *ctx, const Int4Weight &w, const float *g_dev, const float *beta_dev,
                        std::shared_ptr<DevBuf> *gsum, std::shared_ptr<DevBuf> *bc);

// f32 weight of a Linear, stored [K,N] (= [in,out]) row-major on the device.
// w_nk_h: the same weight rounded to fp16 and stored [N,K] (K contiguous), the operand of the
// tensor-core GEMM that serves more than four rows; absent when a value does not fit fp16's range.
struct F32Weight {
    int K = 0, N = 0;
    std::shared_ptr<DevBuf> w_kn, bias, w_nk_h;
};
// weight given as [out,in] (Linear layout) or [in,out] (checkpoint layout)
int f32_weight_upload(b200nn_ctx *ctx, const float *w, bool is_out_in, const float *bias, size_t K, size_t N,
                      F32Weight *out);

// ---------------------------------------------------------------------------------------------
// epilogue shared by every Linear kernel
// ---------------------------------------------------------------------------------------------
enum { EPI_STORE = 0, EPI_RESID = 1, EPI_QKV = 2, EPI_RESID_LN = 3 };

struct Epilogue {
    int mode = EPI_STORE;
    int act = B200NN_ACT_NONE;
    int out_half = 0;          // out is __half* instead of float*
    const float *bias = nullptr;
    void *out = nullptr;       // [M, ldo]
    int ldo = 0;
    float *resid = nullptr;    // EPI_RESID: resid[m*ldo+n] += value (f32, in place)
    // EPI_QKV: columns [0,d) -> out (q), [d,2d) -> K cache, [2d,3d) -> V cache
    __half *kc = nullptr, *vc = nullptr; // this layer's cache, [seq][head][cap][64]
    int d_model = 0, n_head = 0, rows_per_seq = 1, cap = 0;
    const int *pos_ptr = nullptr; // optional device scalar added to pos_off
    int pos_off = 0;
    // Greedy pick fused into the epilogue (LM head): per output row and per group of 32 consecutive
    // features the largest finished value and its feature index go to amax_val / amax_idx
    // [row][amax_entries]; a second, tiny kernel reduces the entries of a row (launch_argmax_entries).
    // Ties keep the lowest index, or the highest with amax_keep_last.  no_store: do not write `out`.
    float *amax_val = nullptr;
    int *amax_idx = nullptr;
    int amax_entries = 0, amax_keep_last = 0, no_store = 0;
    // LayerNorm folded into the GEMMs on either side of it (decode steps of the int4 models), so that no
    // LayerNorm kernel runs between them.  With LN(x) = (x - mean) * rstd * g + b,
    //     LN(x) . W = rstd * ((x * g) . W - mean * sum_k g_k W_kn) + sum_k b_k W_kn :
    // producer (mode EPI_RESID_LN, a residual GEMM whose block holds complete sums): x_new = resid + value
    //   is written back (f32), xg_out = fp16(x_new * next_g) is what the next GEMM multiplies, and the
    //   row's (sum x_new, sum x_new^2) over the 128 features of feature tile t goes to
    //   stats_out[(row * stats_nt + t) * 2 + 0..1] (every tile writes its own slot: no zeroing, no atomics);
    // consumer (ln_stats set): finished value = rstd * (acc - mean * ln_gsum[n]) + bias[n], where mean and
    //   rstd come from the ln_nt (<= 32) partial sums of the row and `bias` already holds
    //   sum_k b_k W_kn + the Linear's own bias.
    const float *ln_stats = nullptr, *ln_gsum = nullptr;
    int ln_nt = 0, stats_nt = 0;
    float ln_eps = 0.0f, ln_inv_d = 0.0f;
    __half *xg_out = nullptr;
    const float *next_g = nullptr;
    float *stats_out = nullptr;
};

// ---------------------------------------------------------------------------------------------
// kernel launchers (each in its own translation unit)
// ---------------------------------------------------------------------------------------------
// x: [M,K] f32 or fp16 (x_half).  Dispatches GEMV / tensor-core GEMM / generic kernel.
int launch_int4_linear(b200nn_ctx *ctx, const Int4Weight &w, const void *x, bool x_half, int M, const Epilogue &epi);
int launch_int4_gemv(b200nn_ctx *ctx, const Int4Weight &w, const void *x, bool x_half, int M, const Epilogue &epi);
int launch_int4_naive(b200nn_ctx *ctx, const Int4Weight &w, const void *x, bool x_half, int M, const Epilogue &epi);
bool int4_gemm_tc_supported(const Int4Weight &w, int M);
int launch_int4_gemm_tc(b200nn_ctx *ctx, const Int4Weight &w, const __half *x, int M, const Epilogue &epi);
int launch_f32_linear(b200nn_ctx *ctx, const F32Weight &w, const void *x, bool x_half, int M, const Epilogue &epi);
bool f16_gemm_tc_supported(const b200nn_ctx *ctx, const F32Weight &w, int M);
int launch_f16_gemm_tc(b200nn_ctx *ctx, const F32Weight &w, const __half *x, int M, const Epilogue &epi);
bool int4_via_f16_supported(const b200nn_ctx *ctx, const Int4Weight &w, int M);
int launch_int4_via_f16(b200nn_ctx *ctx, const Int4Weight &w, const __half *x, int M, const Epilogue &epi);

int launch_layernorm(b200nn_ctx *ctx, const float *x, const float *res_in, float *sum_out, const float *gamma,
                     const float *beta, float eps, int rows, int d, void *out, bool out_half);
// launch_embedding that also prepares the first LayerNorm for folding: xg = fp16(out * g) and each row's
// (sum, sum of squares) in partial 0 of stats [n_rows][stats_nt][2] (the other partials zero).
int launch_embedding_ln(b200nn_ctx *ctx, const uint32_t *ids, const float *wte, const float *wpe, int n_rows, int d,
                        const int *pos_ptr, int vocab, int n_positions, float *out, const float *g, __half *xg,
                        float *stats, int stats_nt);
int launch_embedding(b200nn_ctx *ctx, const uint32_t *ids, const float *wte, const float *wpe, int n_rows, int d,
                     int rows_per_seq, const int *pos_ptr, int pos_off, int vocab, int n_positions, float *out);
int launch_activation(b200nn_ctx *ctx, const float *x, float *y, size_t n, int act);
int launch_bias_add(b200nn_ctx *ctx, float *data, const float *bias, size_t total, int n_cols);
int launch_add(b200nn_ctx *ctx, float *a, const float *b, size_t n);
int launch_split_qkv(b200nn_ctx *ctx, const float *qkv, int seq, int H, int dh, float *q, float *k, float *v);
int launch_concat_heads(b200nn_ctx *ctx, const float *heads, int seq, int H, int dh, float *out);
int launch_tensor_transpose(b200nn_ctx *ctx, const float *in, float *out, const std::vector<size_t> &shape, int dim0, int dim1);
int launch_f32_to_half(b200nn_ctx *ctx, const float *x, __half *y, size_t n);
int launch_half_to_f32(b200nn_ctx *ctx, const __half *x, float *y, size_t n);
// rows of `src` ([n_seq*rows_per_seq, d]) at index rows_per_seq-1 of each sequence -> dst [n_seq, d]
int launch_gather_last_rows(b200nn_ctx *ctx, const float *src, int n_seq, int rows_per_seq, int d, float *dst);
// logits [rows, ld] -> token per row; appends to history[row*hist_cap + *hist_len_ptr]; finished mask
int launch_argmax(b200nn_ctx *ctx, const float *logits, int rows, int vocab, int ld, bool keep_last,
                  uint32_t *tok_out);
// second stage of the fused greedy pick: entries [rows][n_entries] (value, index) -> token per row
int launch_argmax_entries(b200nn_ctx *ctx, const float *val, const int *idx, int rows, int n_entries, int vocab,
                          bool keep_last, uint32_t *tok_out);
int launch_record_tokens(b200nn_ctx *ctx, const uint32_t *tok, int rows, uint32_t *history, int hist_cap,
                         int *step_ptr, int *pos_ptr);

// Decode attention: one query row per sequence against the fp16 cache (new position already
// appended).  q [B, d] f32/half with leading dimension ldq; out [B, d] f32/half.
int launch_decode_attention(b200nn_ctx *ctx, const void *q, bool q_half, int ldq, const __half *kc,
                            const __half *vc, int B, int H, int cap, const int *pos_ptr, int pos_off, void *out,
                            bool out_half, int max_ctx_hint);
// Prefill attention: S query rows per sequence at absolute positions past..past+S-1, causal.
int launch_prefill_attention(b200nn_ctx *ctx, const void *q, bool q_half, int ldq, const __half *kc,
                             const __half *vc, int B, int H, int cap, int S, int past, void *out, bool out_half);
// The tensor-core form of the above for fp16 q and output (ldq a multiple of 8 halves).
int launch_prefill_attention_tc(b200nn_ctx *ctx, const __half *q, int ldq, const __half *kc, const __half *vc, int B, int H,
                                int cap, int S, int past, __half *out);
// f32 [H,len,64] (public op layout) -> fp16 cache layout [1][H][cap][64]
int launch_pack_kv(b200nn_ctx *ctx, const float *src, int H, int len, int cap, __half *dst);

// host quantiser (quantize.cpp)
int host_quantize_weight_int4(const float *weight_t, size_t k, size_t n, size_t group, uint32_t *packed,
                              float *scales);
float host_f16_round(float v);
