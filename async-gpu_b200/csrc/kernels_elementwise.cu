// Small fused kernels of the GPT-2 path: LayerNorm (+residual), embedding gather, activations,
// bias / residual adds, head split / concat, dtype conversion, greedy argmax.
#include "device_utils.cuh"

// ---------------------------------------------------------------------------------------------
// LayerNorm: gamma*(x-mean)/sqrt(var+eps)+beta, biased variance (cpu_ref.rs:27-54).  One block per
// row; the row lives in registers between the mean pass and the variance pass, so the input is
// read once and the variance is the two-pass form (no E[x^2]-mean^2 cancellation).
// Optional residual: s = x + res_in is normalised and also written to sum_out
// (ops/norm.rs:248-400 `layer_norm_residual_dual`).
// ---------------------------------------------------------------------------------------------
template <int VPT, typename TOut>
__global__ void __launch_bounds__(256) layernorm_kernel(const float *__restrict__ x, const float *__restrict__ res_in,
                                                        float *__restrict__ sum_out, const float *__restrict__ gamma,
                                                        const float *__restrict__ beta, float eps, int d,
                                                        TOut *__restrict__ out) {
    __shared__ float red[32];
    const int row = blockIdx.x, tid = threadIdx.x;
    pdl_trigger();
    // scale and shift are constants: fetched before the wait on the previous kernel, not after the
    // two reductions where their latency would sit at the end of the block's critical path
    float g[VPT], bt[VPT];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        int j = tid + i * 256;
        g[i] = (j < d) ? gamma[j] : 0.0f;
        bt[i] = (j < d) ? beta[j] : 0.0f;
    }
    pdl_wait();
    const float *xr = x + (size_t)row * d;
    const float *rr = res_in ? res_in + (size_t)row * d : nullptr;
    float v[VPT];
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        int j = tid + i * 256;
        float t = 0.0f;
        if (j < d) {
            t = xr[j];
            if (rr) t += rr[j];
            if (sum_out) sum_out[(size_t)row * d + j] = t;
        }
        v[i] = t;
        s += t;
    }
    float mean = block_sum(s, red) / (float)d;
    float q = 0.0f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        int j = tid + i * 256;
        float t = (j < d) ? v[i] - mean : 0.0f;
        q += t * t;
    }
    float var = block_sum(q, red) / (float)d;
    float inv_std = rsqrtf(var + eps);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        int j = tid + i * 256;
        if (j < d) {
            float y = (v[i] - mean) * inv_std * g[i] + bt[i];
            if constexpr (sizeof(TOut) == 2)
                out[(size_t)row * d + j] = __float2half_rn(y);
            else
                out[(size_t)row * d + j] = y;
        }
    }
}

// The same for many rows (prefill passes): one warp per row, eight rows per block at a time, blocks
// walking the rows.  The row sits in the warp's registers (NV float4 per lane), both reductions are
// shuffles, nothing waits on a block barrier, and scale / shift come from shared memory; 16-byte loads and
// 8-byte (fp16) or 16-byte (f32) stores, all coalesced.  d a multiple of 4, at most 128 * NV.
template <int NV, typename TOut>
__global__ void __launch_bounds__(256) layernorm_rows_kernel(const float *__restrict__ x, const float *__restrict__ gamma,
                                                             const float *__restrict__ beta, float eps, int rows, int d,
                                                             TOut *__restrict__ out) {
    extern __shared__ float4 gb[]; // [d/4] scale, then [d/4] shift
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, d4 = d >> 2;
    pdl_trigger();
    for (int i = threadIdx.x; i < d4; i += 256) {
        gb[i] = reinterpret_cast<const float4 *>(gamma)[i];
        gb[d4 + i] = reinterpret_cast<const float4 *>(beta)[i];
    }
    __syncthreads();
    pdl_wait();
    const float inv_d = 1.0f / (float)d;
    for (int row = blockIdx.x * 8 + warp; row < rows; row += gridDim.x * 8) {
        const float4 *xr = reinterpret_cast<const float4 *>(x + (size_t)row * d);
        float4 v[NV];
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int c = lane + 32 * i;
            v[i] = c < d4 ? __ldcs(xr + c) : make_float4(0.f, 0.f, 0.f, 0.f);
            s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
        }
        const float mean = warp_sum(s) * inv_d;
        float q = 0.0f;
#pragma unroll
        for (int i = 0; i < NV; ++i)
            if (lane + 32 * i < d4) {
                const float a = v[i].x - mean, b = v[i].y - mean, c = v[i].z - mean, e = v[i].w - mean;
                q += (a * a + b * b) + (c * c + e * e);
            }
        const float inv_std = rsqrtf(warp_sum(q) * inv_d + eps);
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int c = lane + 32 * i;
            if (c < d4) {
                const float4 g = gb[c], b = gb[d4 + c];
                float4 y;
                y.x = (v[i].x - mean) * inv_std * g.x + b.x;
                y.y = (v[i].y - mean) * inv_std * g.y + b.y;
                y.z = (v[i].z - mean) * inv_std * g.z + b.z;
                y.w = (v[i].w - mean) * inv_std * g.w + b.w;
                if constexpr (sizeof(TOut) == 2) {
                    __half2 lo = __floats2half2_rn(y.x, y.y), hi = __floats2half2_rn(y.z, y.w);
                    reinterpret_cast<uint2 *>(out + (size_t)row * d)[c] =
                        make_uint2(*reinterpret_cast<uint32_t *>(&lo), *reinterpret_cast<uint32_t *>(&hi));
                } else {
                    reinterpret_cast<float4 *>(out + (size_t)row * d)[c] = y;
                }
            }
        }
    }
}

template <int NV>
static void launch_layernorm_rows(b200nn_ctx *ctx, const float *x, const float *gamma, const float *beta, float eps, int rows,
                                  int d, void *out, bool out_half) {
    const int grid = std::min((rows + 7) / 8, 8 * ctx->sm_count);
    const size_t smem = (size_t)d * 2 * sizeof(float);
    PREFER_SMEM_ONCE((layernorm_rows_kernel<NV, __half>));
    PREFER_SMEM_ONCE((layernorm_rows_kernel<NV, float>));
    if (out_half)
        launch_pdl(ctx, layernorm_rows_kernel<NV, __half>, dim3(grid), dim3(256), smem, x, gamma, beta, eps, rows, d, (__half *)out);
    else
        launch_pdl(ctx, layernorm_rows_kernel<NV, float>, dim3(grid), dim3(256), smem, x, gamma, beta, eps, rows, d, (float *)out);
}

int launch_layernorm(b200nn_ctx *ctx, const float *x, const float *res_in, float *sum_out, const float *gamma,
                     const float *beta, float eps, int rows, int d, void *out, bool out_half) {
    if (rows <= 0) return B200NN_OK;
    if (d > 256 * 32) return set_error(ctx, B200NN_ERR_UNSUPPORTED, "layer_norm: d > 8192");
    // many rows without a residual (prefill passes): a warp per row
    if (rows >= ctx->ln_rows_min && !res_in && !sum_out && d % 4 == 0 && d <= 2048 && !((uintptr_t)x & 15) && !((uintptr_t)out & 15) &&
        !((uintptr_t)gamma & 15) && !((uintptr_t)beta & 15)) {
        const int nv = (d / 4 + 31) / 32;
        if (nv <= 6) launch_layernorm_rows<6>(ctx, x, gamma, beta, eps, rows, d, out, out_half);
        else if (nv <= 8) launch_layernorm_rows<8>(ctx, x, gamma, beta, eps, rows, d, out, out_half);
        else if (nv <= 10) launch_layernorm_rows<10>(ctx, x, gamma, beta, eps, rows, d, out, out_half);
        else if (nv <= 13) launch_layernorm_rows<13>(ctx, x, gamma, beta, eps, rows, d, out, out_half);
        else launch_layernorm_rows<16>(ctx, x, gamma, beta, eps, rows, d, out, out_half);
        CK_LAUNCH(ctx, "layernorm_rows_kernel");
        return B200NN_OK;
    }
#define LN_LAUNCH(V)                                                                                              \
    do {                                                                                                          \
        PREFER_SMEM_ONCE((layernorm_kernel<V, __half>));                                                          \
        PREFER_SMEM_ONCE((layernorm_kernel<V, float>));                                                           \
        if (out_half)                                                                                             \
            launch_pdl(ctx, layernorm_kernel<V, __half>, dim3(rows), dim3(256), 0, x, res_in, sum_out, gamma,    \
                       beta, eps, d, (__half *)out);                                                             \
        else                                                                                                      \
            launch_pdl(ctx, layernorm_kernel<V, float>, dim3(rows), dim3(256), 0, x, res_in, sum_out, gamma,     \
                       beta, eps, d, (float *)out);                                                              \
    } while (0)
    int vpt = (d + 255) / 256;
    if (vpt <= 4) LN_LAUNCH(4);
    else if (vpt <= 8) LN_LAUNCH(8);
    else if (vpt <= 16) LN_LAUNCH(16);
    else LN_LAUNCH(32);
#undef LN_LAUNCH
    CK_LAUNCH(ctx, "layernorm_kernel");
    return B200NN_OK;
}

// ---------------------------------------------------------------------------------------------
// Embedding: out[r,:] = wte[ids[r],:] + wpe[pos(r),:], pos(r) = *pos_ptr + pos_off + r % rows_per_seq
// (layers/embedding.rs:59-93 computes the offset form on the host; here it is one gather).
// ---------------------------------------------------------------------------------------------
__global__ void embedding_kernel(const uint32_t *__restrict__ ids, const float *__restrict__ wte,
                                 const float *__restrict__ wpe, int d, int rows_per_seq, const int *pos_ptr,
                                 int pos_off, int vocab, int n_positions, float *__restrict__ out) {
    int r = blockIdx.x;
    pdl_trigger();
    pdl_wait();
    uint32_t tok = ids[r];
    if (tok >= (uint32_t)vocab) tok = vocab - 1; // ids are validated on the host; never read out of range
    int pos = (pos_ptr ? *pos_ptr : 0) + pos_off + r % rows_per_seq;
    if (pos >= n_positions) pos = n_positions - 1;
    const float *a = wte + (size_t)tok * d, *b = wpe + (size_t)pos * d;
    for (int j = threadIdx.x; j < d; j += blockDim.x) out[(size_t)r * d + j] = a[j] + b[j];
}

int launch_embedding(b200nn_ctx *ctx, const uint32_t *ids, const float *wte, const float *wpe, int n_rows, int d,
                     int rows_per_seq, const int *pos_ptr, int pos_off, int vocab, int n_positions, float *out) {
    if (n_rows <= 0) return B200NN_OK;
    PREFER_SMEM_ONCE(embedding_kernel);
    launch_pdl(ctx, embedding_kernel, dim3(n_rows), dim3(256), 0, ids, wte, wpe, d, rows_per_seq, pos_ptr, pos_off, vocab,
               n_positions, out);
    CK_LAUNCH(ctx, "embedding_kernel");
    return B200NN_OK;
}

// The decode-step embedding when the first LayerNorm is folded into the q/k/v GEMM (see Epilogue): one
// row per block at position *pos_ptr.
__global__ void __launch_bounds__(256) embedding_ln_kernel(const uint32_t *__restrict__ ids, const float *__restrict__ wte,
                                                           const float *__restrict__ wpe, int d, const int *pos_ptr, int vocab,
                                                           int n_positions, float *__restrict__ out,
                                                           const float *__restrict__ g, __half *__restrict__ xg,
                                                           float *__restrict__ stats, int stats_nt) {
    __shared__ float red[32];
    const int r = blockIdx.x;
    pdl_trigger();
    pdl_wait();
    uint32_t tok = ids[r];
    if (tok >= (uint32_t)vocab) tok = vocab - 1;
    int pos = *pos_ptr;
    if (pos >= n_positions) pos = n_positions - 1;
    const float *a = wte + (size_t)tok * d, *b = wpe + (size_t)pos * d;
    float s1 = 0.0f, s2 = 0.0f;
    for (int j = threadIdx.x; j < d; j += blockDim.x) {
        const float v = a[j] + b[j];
        out[(size_t)r * d + j] = v;
        xg[(size_t)r * d + j] = __float2half_rn(v * g[j]);
        s1 += v;
        s2 += v * v;
    }
    s1 = block_sum(s1, red);
    s2 = block_sum(s2, red);
    for (int t = threadIdx.x; t < stats_nt; t += blockDim.x)
        reinterpret_cast<float2 *>(stats)[(size_t)r * stats_nt + t] = t == 0 ? make_float2(s1, s2) : make_float2(0.f, 0.f);
}

int launch_embedding_ln(b200nn_ctx *ctx, const uint32_t *ids, const float *wte, const float *wpe, int n_rows, int d,
                        const int *pos_ptr, int vocab, int n_positions, float *out, const float *g, __half *xg,
                        float *stats, int stats_nt) {
    if (n_rows <= 0) return B200NN_OK;
    PREFER_SMEM_ONCE(embedding_ln_kernel);
    launch_pdl(ctx, embedding_ln_kernel, dim3(n_rows), dim3(256), 0, ids, wte, wpe, d, pos_ptr, vocab, n_positions, out, g, xg,
               stats, stats_nt);
    CK_LAUNCH(ctx, "embedding_ln_kernel");
    return B200NN_OK;
}

// ---------------------------------------------------------------------------------------------
// element-wise ops (ops/activation.rs, ops/reshape.rs:112-186)
// ---------------------------------------------------------------------------------------------
__global__ void activation_kernel(const float *__restrict__ x, float *__restrict__ y, size_t n, int act) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x, st = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += st) y[i] = apply_act(x[i], act);
}
__global__ void bias_add_kernel(float *__restrict__ data, const float *__restrict__ bias, size_t total, int n_cols) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x, st = (size_t)gridDim.x * blockDim.x;
    for (; i < total; i += st) data[i] += bias[i % n_cols];
}
__global__ void add_kernel(float *__restrict__ a, const float *__restrict__ b, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x, st = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += st) a[i] += b[i];
}
__global__ void f32_to_half_kernel(const float *__restrict__ x, __half *__restrict__ y, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x, st = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += st) y[i] = __float2half_rn(x[i]);
}
__global__ void half_to_f32_kernel(const __half *__restrict__ x, float *__restrict__ y, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x, st = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += st) y[i] = __half2float(x[i]);
}

static inline int grid_for(b200nn_ctx *ctx, size_t n, int block) {
    size_t g = (n + block - 1) / block;
    size_t cap = (size_t)ctx->sm_count * 16;
    return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

int launch_activation(b200nn_ctx *ctx, const float *x, float *y, size_t n, int act) {
    if (!n) return B200NN_OK;
    PREFER_SMEM_ONCE(activation_kernel);
    activation_kernel<<<grid_for(ctx, n, 256), 256, 0, ctx->stream>>>(x, y, n, act);
    CK_LAUNCH(ctx, "activation_kernel");
    return B200NN_OK;
}
int launch_bias_add(b200nn_ctx *ctx, float *data, const float *bias, size_t total, int n_cols) {
    if (!total) return B200NN_OK;
    PREFER_SMEM_ONCE(bias_add_kernel);
    bias_add_kernel<<<grid_for(ctx, total, 256), 256, 0, ctx->stream>>>(data, bias, total, n_cols);
    CK_LAUNCH(ctx, "bias_add_kernel");
    return B200NN_OK;
}
int launch_add(b200nn_ctx *ctx, float *a, const float *b, size_t n) {
    if (!n) return B200NN_OK;
    PREFER_SMEM_ONCE(add_kernel);
    add_kernel<<<grid_for(ctx, n, 256), 256, 0, ctx->stream>>>(a, b, n);
    CK_LAUNCH(ctx, "add_kernel");
    return B200NN_OK;
}
int launch_f32_to_half(b200nn_ctx *ctx, const float *x, __half *y, size_t n) {
    if (!n) return B200NN_OK;
    PREFER_SMEM_ONCE(f32_to_half_kernel);
    f32_to_half_kernel<<<grid_for(ctx, n, 256), 256, 0, ctx->stream>>>(x, y, n);
    CK_LAUNCH(ctx, "f32_to_half_kernel");
    return B200NN_OK;
}
int launch_half_to_f32(b200nn_ctx *ctx, const __half *x, float *y, size_t n) {
    if (!n) return B200NN_OK;
    PREFER_SMEM_ONCE(half_to_f32_kernel);
    half_to_f32_kernel<<<grid_for(ctx, n, 256), 256, 0, ctx->stream>>>(x, y, n);
    CK_LAUNCH(ctx, "half_to_f32_kernel");
    return B200NN_OK;
}

// ---------------------------------------------------------------------------------------------
// split_qkv / concat_heads (ops/attention.rs:105-142, 515-549): [seq,3d] <-> Q,K,V [H,seq,dh]
// with Q columns [0,d), K [d,2d), V [2d,3d), head h at h*dh.
// ---------------------------------------------------------------------------------------------
__global__ void split_qkv_kernel(const float *__restrict__ qkv, int seq, int H, int dh, float *__restrict__ q,
                                 float *__restrict__ k, float *__restrict__ v) {
    size_t total = (size_t)H * seq * dh;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x, st = (size_t)gridDim.x * blockDim.x;
    int d = H * dh;
    for (; i < total; i += st) {
        int e = i % dh;
        int s = (i / dh) % seq;
        int h = i / ((size_t)dh * seq);
        const float *row = qkv + (size_t)s * 3 * d + h * dh + e;
        q[i] = row[0];
        k[i] = row[d];
        v[i] = row[2 * d];
    }
}
__global__ void concat_heads_kernel(const float *__restrict__ heads, int seq, int H, int dh, float *__restrict__ out) {
    size_t total = (size_t)H * seq * dh;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x, st = (size_t)gridDim.x * blockDim.x;
    for (; i < total; i += st) {
        int e = i % dh;
        int h = (i / dh) % H;
        int s = i / ((size_t)dh * H);
        out[i] = heads[((size_t)h * seq + s) * dh + e];
    }
}
int launch_split_qkv(b200nn_ctx *ctx, const float *qkv, int seq, int H, int dh, float *q, float *k, float *v) {
    size_t n = (size_t)seq * H * dh;
    if (!n) return B200NN_OK;
    PREFER_SMEM_ONCE(split_qkv_kernel);
    split_qkv_kernel<<<grid_for(ctx, n, 256), 256, 0, ctx->stream>>>(qkv, seq, H, dh, q, k, v);
    CK_LAUNCH(ctx, "split_qkv_kernel");
    return B200NN_OK;
}
int launch_concat_heads(b200nn_ctx *ctx, const float *heads, int seq, int H, int dh, float *out) {
    size_t n = (size_t)seq * H * dh;
    if (!n) return B200NN_OK;
    PREFER_SMEM_ONCE(concat_heads_kernel);
    concat_heads_kernel<<<grid_for(ctx, n, 256), 256, 0, ctx->stream>>>(heads, seq, H, dh, out);
    CK_LAUNCH(ctx, "concat_heads_kernel");
    return B200NN_OK;
}

__global__ void gather_last_rows_kernel(const float *__restrict__ src, int rows_per_seq, int d, float *__restrict__ dst) {
    int b = blockIdx.x;
    const float *s = src + ((size_t)b * rows_per_seq + rows_per_seq - 1) * d;
    for (int j = threadIdx.x; j < d; j += blockDim.x) dst[(size_t)b * d + j] = s[j];
}
int launch_gather_last_rows(b200nn_ctx *ctx, const float *src, int n_seq, int rows_per_seq, int d, float *dst) {
    if (n_seq <= 0) return B200NN_OK;
    PREFER_SMEM_ONCE(gather_last_rows_kernel);
    gather_last_rows_kernel<<<n_seq, 256, 0, ctx->stream>>>(src, rows_per_seq, d, dst);
    CK_LAUNCH(ctx, "gather_last_rows_kernel");
    return B200NN_OK;
}

// f32 [H,len,64] -> fp16 [H,cap,64]
__global__ void pack_kv_kernel(const float *__restrict__ src, int len, int cap, size_t total, __half *__restrict__ dst) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x, st = (size_t)gridDim.x * blockDim.x;
    for (; i < total; i += st) {
        int e = i & 63;
        size_t r = i >> 6;
        int s = r % len;
        int h = r / len;
        dst[((size_t)h * cap + s) * 64 + e] = __float2half_rn(src[i]);
    }
}
int launch_pack_kv(b200nn_ctx *ctx, const float *src, int H, int len, int cap, __half *dst) {
    size_t n = (size_t)H * len * 64;
    if (!n) return B200NN_OK;
    PREFER_SMEM_ONCE(pack_kv_kernel);
    pack_kv_kernel<<<grid_for(ctx, n, 256), 256, 0, ctx->stream>>>(src, len, cap, n, dst);
    CK_LAUNCH(ctx, "pack_kv_kernel");
    return B200NN_OK;
}

// ---------------------------------------------------------------------------------------------
// Greedy argmax over logits [rows, ld] restricted to [0, vocab).  keep_last=false keeps the first
// maximum (the CPU f64 reference, tests_inference.rs:4504-4515); keep_last=true keeps the last
// (Rust max_by, models/gpt2.rs:991-997).
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(1024) argmax_kernel(const float *__restrict__ logits, int vocab, int ld,
                                                      int keep_last, uint32_t *__restrict__ tok_out) {
    __shared__ float sv[32];
    __shared__ int si[32];
    pdl_trigger();
    pdl_wait();
    const float *row = logits + (size_t)blockIdx.x * ld;
    float best = -INFINITY;
    int bi = keep_last ? -1 : 0x7fffffff;
    for (int j = threadIdx.x; j < vocab; j += blockDim.x) {
        float v = row[j];
        if (v > best || (v == best && (keep_last ? j > bi : j < bi))) {
            best = v;
            bi = j;
        }
    }
    auto better = [&](float v, int i, float bv, int bidx) {
        return v > bv || (v == bv && (keep_last ? i > bidx : i < bidx));
    };
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, best, o);
        int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (better(ov, oi, best, bi)) { best = ov; bi = oi; }
    }
    int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    if (lane == 0) { sv[w] = best; si[w] = bi; }
    __syncthreads();
    if (w == 0) {
        int nw = blockDim.x >> 5;
        best = lane < nw ? sv[lane] : -INFINITY;
        bi = lane < nw ? si[lane] : (keep_last ? -1 : 0x7fffffff);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            float ov = __shfl_xor_sync(0xffffffffu, best, o);
            int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (better(ov, oi, best, bi)) { best = ov; bi = oi; }
        }
        if (lane == 0) tok_out[blockIdx.x] = (bi < 0 || bi >= vocab) ? 0u : (uint32_t)bi;
    }
}
int launch_argmax(b200nn_ctx *ctx, const float *logits, int rows, int vocab, int ld, bool keep_last,
                  uint32_t *tok_out) {
    if (rows <= 0) return B200NN_OK;
    PREFER_SMEM_ONCE(argmax_kernel);
    launch_pdl(ctx, argmax_kernel, dim3(rows), dim3(1024), 0, logits, vocab, ld, keep_last ? 1 : 0, tok_out);
    CK_LAUNCH(ctx, "argmax_kernel");
    return B200NN_OK;
}

// Second stage of the greedy pick fused into the LM head's epilogue: the (value, index) entries of a
// row, one per 32 features, reduced with the same tie rule as argmax_kernel (same token, bit for bit:
// a maximum does not depend on the order it is taken in).
__global__ void __launch_bounds__(256) argmax_entries_kernel(const float *__restrict__ val, const int *__restrict__ idx,
                                                            int n_entries, int vocab, int keep_last,
                                                            uint32_t *__restrict__ tok_out) {
    __shared__ float sv[8];
    __shared__ int si[8];
    pdl_trigger();
    pdl_wait();
    const float *rv = val + (size_t)blockIdx.x * n_entries;
    const int *ri = idx + (size_t)blockIdx.x * n_entries;
    float best = -INFINITY;
    int bi = keep_last ? -1 : 0x7fffffff;
    for (int j = threadIdx.x; j < n_entries; j += blockDim.x) amax_merge(best, bi, rv[j], ri[j], keep_last);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        amax_merge(best, bi, ov, oi, keep_last);
    }
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    if (lane == 0) { sv[w] = best; si[w] = bi; }
    __syncthreads();
    if (w == 0) {
        best = lane < 8 ? sv[lane] : -INFINITY;
        bi = lane < 8 ? si[lane] : (keep_last ? -1 : 0x7fffffff);
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            amax_merge(best, bi, ov, oi, keep_last);
        }
        if (lane == 0) tok_out[blockIdx.x] = (bi < 0 || bi >= vocab) ? 0u : (uint32_t)bi;
    }
}
int launch_argmax_entries(b200nn_ctx *ctx, const float *val, const int *idx, int rows, int n_entries, int vocab,
                          bool keep_last, uint32_t *tok_out) {
    if (rows <= 0) return B200NN_OK;
    PREFER_SMEM_ONCE(argmax_entries_kernel);
    launch_pdl(ctx, argmax_entries_kernel, dim3(rows), dim3(256), 0, val, idx, n_entries, vocab, keep_last ? 1 : 0, tok_out);
    CK_LAUNCH(ctx, "argmax_entries_kernel");
    return B200NN_OK;
}

// Appends this step's token of every sequence to the history and advances the step / position
// counters that the next step's kernels read (single block, so the increment is ordered).
__global__ void record_tokens_kernel(const uint32_t *__restrict__ tok, int rows, uint32_t *__restrict__ history,
                                     int hist_cap, int *step_ptr, int *pos_ptr) {
    pdl_trigger();
    pdl_wait();
    int step = *step_ptr;
    for (int r = threadIdx.x; r < rows; r += blockDim.x)
        if (step < hist_cap) history[(size_t)r * hist_cap + step] = tok[r];
    __syncthreads();
    if (threadIdx.x == 0) {
        *step_ptr = step + 1;
        if (pos_ptr) *pos_ptr += 1;
    }
}
int launch_record_tokens(b200nn_ctx *ctx, const uint32_t *tok, int rows, uint32_t *history, int hist_cap,
                         int *step_ptr, int *pos_ptr) {
    PREFER_SMEM_ONCE(record_tokens_kernel);
    launch_pdl(ctx, record_tokens_kernel, dim3(1), dim3(256), 0, tok, rows, history, hist_cap, step_ptr, pos_ptr);
    CK_LAUNCH(ctx, "record_tokens_kernel");
    return B200NN_OK;
}


// ---------------------------------------------------------------------------------------------
// GpuTensor::transpose (tensor.rs:227-268): out[..., i, ..., j, ...] = in[..., j, ..., i, ...] for any two
// dimensions of a contiguous tensor of up to 8 dimensions.  The reference goes through the host; here each
// thread walks from its output index to the input index over the swapped strides.
// ---------------------------------------------------------------------------------------------
struct TransposeDims {
    int ndim;
    unsigned long long out_stride[8], src_stride[8]; // src strides already swapped
};
__global__ void tensor_transpose_kernel(const float *__restrict__ in, float *__restrict__ out, size_t n, TransposeDims td) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    size_t rem = i, src = 0;
    for (int d = 0; d < td.ndim; ++d) {
        const size_t idx = rem / td.out_stride[d];
        rem -= idx * td.out_stride[d];
        src += idx * td.src_stride[d];
    }
    out[i] = in[src];
}

int launch_tensor_transpose(b200nn_ctx *ctx, const float *in, float *out, const std::vector<size_t> &shape, int dim0, int dim1) {
    const int nd = (int)shape.size();
    if (nd > 8) return set_error(ctx, B200NN_ERR_UNSUPPORTED, "transpose: more than 8 dimensions");
    std::vector<size_t> stride(nd, 1), oshape(shape);
    for (int d = nd - 2; d >= 0; --d) stride[d] = stride[d + 1] * shape[d + 1];
    std::swap(oshape[dim0], oshape[dim1]);
    std::swap(stride[dim0], stride[dim1]);
    TransposeDims td;
    td.ndim = nd;
    size_t n = 1, os = 1;
    for (int d = nd - 1; d >= 0; --d) {
        td.out_stride[d] = os;
        os *= oshape[d];
        td.src_stride[d] = stride[d];
        n *= shape[d];
    }
    if (n == 0) return B200NN_OK;
    tensor_transpose_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(in, out, n, td);
    CK_LAUNCH(ctx, "tensor_transpose_kernel");
    return B200NN_OK;
}
