// Context, device buffers, tensors, host-side quantiser and the upload / re-tiling of weights.
#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstring>
#include <thread>

#include "common.h"

// ---------------------------------------------------------------------------------------------
// errors
// ---------------------------------------------------------------------------------------------
int set_error(b200nn_ctx *ctx, int code, const std::string &msg) {
    if (ctx) ctx->last_error = msg;
    return code;
}

int set_cuda_error(b200nn_ctx *ctx, cudaError_t e, const char *what) {
    if (ctx) {
        ctx->last_cuda = (int)e;
        ctx->last_error = std::string("CUDA error ") + cudaGetErrorName(e) + " (" + cudaGetErrorString(e) + ") at " + what;
    }
    return B200NN_ERR_CUDA;
}

// Waits for the context's stream and brings the device error word back in the same step.  A kernel
// whose bounded wait ran out leaves its output unwritten and a code in that word: the call that hands
// results to the host then fails with B200NN_ERR_DEVICE instead of returning stale data.  The word is
// cleared so that the context stays usable.
int stream_sync_check(b200nn_ctx *ctx) {
    if (!ctx->host_err) CK(ctx, cudaMallocHost((void **)&ctx->host_err, sizeof(uint32_t)));
    *ctx->host_err = 0;
    CK(ctx, cudaMemcpyAsync(ctx->host_err, ctx->dev_err, sizeof(uint32_t), cudaMemcpyDeviceToHost, ctx->stream));
    CK(ctx, cudaStreamSynchronize(ctx->stream));
    const uint32_t w = *ctx->host_err;
    if (!w) return B200NN_OK;
    CK(ctx, cudaMemsetAsync(ctx->dev_err, 0, sizeof(uint32_t), ctx->stream));
    char msg[96];
    snprintf(msg, sizeof(msg), "a kernel's bounded wait ran out (device error word 0x%x); results were not written", w);
    return set_error(ctx, B200NN_ERR_DEVICE, msg);
}

static void free_on_device(void *p, int device) {
    int cur = -1;
    cudaGetDevice(&cur);
    if (cur != device) cudaSetDevice(device);
    cudaFree(p);
    if (cur >= 0 && cur != device) cudaSetDevice(cur);
}

DevBuf::~DevBuf() {
    if (!p) return;
    if (pool) {
        std::lock_guard<std::mutex> g(pool->mu);
        if (pool->alive && pool->held_bytes + block_bytes <= DevPool::MAX_HELD) {
            pool->free_blocks.emplace(block_bytes, p);
            pool->held_bytes += block_bytes;
            return;
        }
    }
    free_on_device(p, device);
}

void pool_trim(b200nn_ctx *ctx) {
    std::lock_guard<std::mutex> g(ctx->pool->mu);
    for (auto &kv : ctx->pool->free_blocks) free_on_device(kv.second, ctx->device);
    ctx->pool->free_blocks.clear();
    ctx->pool->held_bytes = 0;
}

// A kept block is reused when it is at least as large as the request and at most a quarter
// larger.  All of the library's device work runs on the context's stream, so a reused block is
// ordered after its previous owner's kernels there; synchronous copies from the host are not
// stream-ordered, hence the synchronise on reuse (the stream is idle at that point in practice).
int dev_alloc(b200nn_ctx *ctx, size_t bytes, std::shared_ptr<DevBuf> *out) {
    auto b = std::make_shared<DevBuf>();
    b->device = ctx->device;
    b->bytes = bytes;
    b->pool = ctx->pool;
    const size_t want = bytes ? (bytes + 255) & ~(size_t)255 : 256;
    CK(ctx, cudaSetDevice(ctx->device));
    {
        std::lock_guard<std::mutex> g(ctx->pool->mu);
        auto it = ctx->pool->free_blocks.lower_bound(want);
        if (it != ctx->pool->free_blocks.end() && it->first <= want + want / 4) {
            b->p = it->second;
            b->block_bytes = it->first;
            ctx->pool->held_bytes -= it->first;
            ctx->pool->free_blocks.erase(it);
        }
    }
    if (b->p) {
        if (!ctx->capturing) CK(ctx, cudaStreamSynchronize(ctx->stream));
        *out = b;
        return B200NN_OK;
    }
    cudaError_t e = cudaMalloc(&b->p, want);
    if (e == cudaErrorMemoryAllocation) { // give the kept blocks back and try once more
        cudaGetLastError();
        pool_trim(ctx);
        e = cudaMalloc(&b->p, want);
    }
    if (e != cudaSuccess) {
        b->p = nullptr;
        return set_cuda_error(ctx, e, "cudaMalloc");
    }
    b->block_bytes = want;
    *out = b;
    return B200NN_OK;
}

int tensor_alloc(b200nn_ctx *ctx, const std::vector<size_t> &shape, bool zero, b200nn_tensor **out) {
    size_t n = 1;
    for (size_t s : shape) n *= s;
    auto *t = new b200nn_tensor();
    t->ctx = ctx;
    t->shape = shape;
    t->numel = n;
    int rc = dev_alloc(ctx, n * sizeof(float), &t->buf);
    if (rc != B200NN_OK) {
        delete t;
        return rc;
    }
    if (zero && n) {
        cudaError_t e = cudaMemsetAsync(t->buf->p, 0, n * sizeof(float), ctx->stream);
        if (e != cudaSuccess) {
            delete t;
            return set_cuda_error(ctx, e, "cudaMemsetAsync");
        }
    }
    *out = t;
    return B200NN_OK;
}

// Split-K / split-KV scratch.  Grown only outside graph capture; a captured step must have been
// run once eagerly (which sizes the scratch) before it is captured.
int ensure_scratch(b200nn_ctx *ctx, size_t bytes, size_t counters) {
    if (bytes > ctx->scratch_bytes) {
        if (ctx->capturing) return set_error(ctx, B200NN_ERR_UNSUPPORTED, "scratch would grow during graph capture");
        CK(ctx, cudaStreamSynchronize(ctx->stream));
        // a captured decode step may still name the old block: it stays allocated until the context goes
        if (ctx->scratch) ctx->retired.push_back(ctx->scratch);
        ctx->scratch = nullptr;
        size_t nb = std::max(bytes, (size_t)8 << 20);
        CK(ctx, cudaMalloc(&ctx->scratch, nb));
        ctx->scratch_bytes = nb;
    }
    if (counters > ctx->n_counters) {
        if (ctx->capturing) return set_error(ctx, B200NN_ERR_UNSUPPORTED, "counters would grow during graph capture");
        CK(ctx, cudaStreamSynchronize(ctx->stream));
        if (ctx->counters) ctx->retired.push_back(ctx->counters);
        ctx->counters = nullptr;
        size_t nc = std::max(counters, (size_t)65536);
        CK(ctx, cudaMalloc(&ctx->counters, nc * sizeof(unsigned)));
        CK(ctx, cudaMemset(ctx->counters, 0, nc * sizeof(unsigned)));
        ctx->n_counters = nc;
    }
    return B200NN_OK;
}

// ---------------------------------------------------------------------------------------------
// host quantiser: crates/core/gpu-host/src/nn/ops/quantize.rs
// ---------------------------------------------------------------------------------------------
float host_f16_round(float v) { return __half2float(__float2half_rn(v)); }

template <typename F>
static void parallel_for(size_t n, F f) {
    unsigned hw = std::thread::hardware_concurrency();
    size_t nt = std::min<size_t>(hw ? hw : 4, 64);
    if (n < 256 || nt <= 1) {
        f(0, n);
        return;
    }
    std::vector<std::thread> th;
    size_t per = (n + nt - 1) / nt;
    for (size_t t = 0; t < nt; ++t) {
        size_t a = t * per, b = std::min(n, a + per);
        if (a >= b) break;
        th.emplace_back([=] { f(a, b); });
    }
    for (auto &t : th) t.join();
}

static inline uint32_t quant_nibble(float v, float inv_scale) {
    // quantize.rs:144-145: round half away from zero (Rust f32::round), clamp to [-8,7], store +8.
    int q = (int)std::round(v * inv_scale);
    q = std::max(-8, std::min(7, q));
    return (uint32_t)(q + 8) & 0xFu;
}

// quantize.rs:102-153.
int host_quantize_weight_int4(const float *weight_t, size_t k, size_t n, size_t group, uint32_t *packed,
                              float *scales) {
    if (k % 8 != 0 || group == 0) return B200NN_ERR_SHAPE;
    size_t k_packed = k / 8, n_groups = (k + group - 1) / group;
    parallel_for(n, [=](size_t c0, size_t c1) {
        for (size_t col = c0; col < c1; ++col) {
            for (size_t g = 0; g < n_groups; ++g) {
                size_t s = g * group, e = std::min(k, s + group);
                float max_abs = 0.0f;
                for (size_t ki = s; ki < e; ++ki) max_abs = std::max(max_abs, std::fabs(weight_t[ki * n + col]));
                scales[g * n + col] = (max_abs < 1e-12f) ? 1.0f : max_abs / 7.0f;
            }
            for (size_t kp = 0; kp < k_packed; ++kp) {
                uint32_t word = 0;
                for (unsigned bit = 0; bit < 8; ++bit) {
                    size_t ki = kp * 8 + bit;
                    float inv = 1.0f / scales[(ki / group) * n + col];
                    word |= quant_nibble(weight_t[ki * n + col], inv) << (bit * 4);
                }
                packed[kp * n + col] = word;
            }
        }
    });
    return B200NN_OK;
}

// ---------------------------------------------------------------------------------------------
// weight upload
// ---------------------------------------------------------------------------------------------
static int upload(b200nn_ctx *ctx, const void *host, size_t bytes, std::shared_ptr<DevBuf> *out) {
    TRY(dev_alloc(ctx, bytes, out));
    if (bytes) CK(ctx, cudaMemcpy((*out)->p, host, bytes, cudaMemcpyHostToDevice));
    return B200NN_OK;
}

int int4_weight_upload(b200nn_ctx *ctx, const uint32_t *packed, const float *scales, const float *bias, size_t K,
                       size_t N, size_t group, Int4Weight *w) {
    if (K == 0 || N == 0 || K % 8 != 0 || group == 0)
        return set_error(ctx, B200NN_ERR_SHAPE, "Int4Linear: K must be a positive multiple of 8 and group > 0");
    w->K = (int)K;
    w->N = (int)N;
    w->group = (int)group;
    w->n_groups = (int)((K + group - 1) / group);
    w->n_tiles = (int)((N + TILE_N - 1) / TILE_N);
    w->n_pad = w->n_tiles * TILE_N;
    w->k_blocks = (int)(K / TILE_K);
    w->fast = (K % TILE_K == 0) && (group % TILE_K == 0);
    w->host_packed.assign(packed, packed + (K / 8) * N);
    w->host_scales.resize((size_t)w->n_groups * N);
    for (size_t i = 0; i < w->host_scales.size(); ++i) w->host_scales[i] = host_f16_round(scales[i]);
    if (bias) TRY(upload(ctx, bias, N * sizeof(float), &w->bias));
    if (!w->fast) {
        TRY(upload(ctx, w->host_packed.data(), w->host_packed.size() * 4, &w->ref_packed));
        TRY(upload(ctx, w->host_scales.data(), w->host_scales.size() * 4, &w->ref_scales));
        return B200NN_OK;
    }
    // re-tile: see the layout comment on Int4Weight
    size_t tile_bytes = (size_t)w->n_tiles * w->k_blocks * TILE_BYTES;
    std::vector<uint32_t> tiled(tile_bytes / 4);
    const int k_blocks = w->k_blocks;
    const uint32_t *hp = w->host_packed.data();
    uint32_t *tp = tiled.data();
    parallel_for((size_t)w->n_tiles, [=](size_t t0, size_t t1) {
        for (size_t nt = t0; nt < t1; ++nt)
            for (int kb = 0; kb < k_blocks; ++kb) {
                uint32_t *tile = tp + (nt * k_blocks + kb) * (TILE_BYTES / 4);
                for (int r = 0; r < TILE_N; ++r) {
                    size_t n = nt * TILE_N + r;
                    for (int j = 0; j < 8; ++j) {
                        uint32_t ref = (n < N) ? hp[((size_t)kb * 8 + j) * N + n] : 0x88888888u;
                        uint32_t o = 0;
                        static const int src[8] = {0, 2, 4, 6, 1, 3, 5, 7};
                        for (int i = 0; i < 8; ++i) o |= ((ref >> (4 * src[i])) & 0xFu) << (4 * i);
                        tile[(j >> 2) * 512 + r * 4 + (j & 3)] = o;
                    }
                }
            }
    });
    std::vector<__half> sh((size_t)w->n_groups * w->n_pad, __float2half_rn(0.0f));
    for (int g = 0; g < w->n_groups; ++g)
        for (size_t n = 0; n < N; ++n) sh[(size_t)g * w->n_pad + n] = __float2half_rn(w->host_scales[(size_t)g * N + n]);
    TRY(upload(ctx, tiled.data(), tile_bytes, &w->tiled));
    TRY(upload(ctx, sh.data(), sh.size() * sizeof(__half), &w->scales_h));
    return B200NN_OK;
}

int int4_weight_ln_fold(b200nn_ctx *ctx, const Int4Weight &w, const float *g_dev, const float *beta_dev,
                        std::shared_ptr<DevBuf> *gsum, std::shared_ptr<DevBuf> *bc) {
    const size_t K = w.K, N = w.N, group = w.group;
    std::vector<float> g(K), beta(K), bias(N, 0.0f);
    CK(ctx, cudaMemcpy(g.data(), g_dev, K * 4, cudaMemcpyDeviceToHost));
    CK(ctx, cudaMemcpy(beta.data(), beta_dev, K * 4, cudaMemcpyDeviceToHost));
    if (w.bias) CK(ctx, cudaMemcpy(bias.data(), w.bias->p, N * 4, cudaMemcpyDeviceToHost));
    std::vector<float> gs(N), cs(N);
    const uint32_t *hp = w.host_packed.data();
    const float *hs = w.host_scales.data(); // already fp16 values
    const float *gp = g.data(), *bp = beta.data(), *biasp = bias.data();
    float *gsp = gs.data(), *csp = cs.data();
    parallel_for(N, [=](size_t n0, size_t n1) {
        const size_t cnt = n1 - n0;
        std::vector<double> ag(cnt, 0.0), ab(cnt, 0.0);
        for (size_t kp = 0; kp < K / 8; ++kp) {
            const float *sc = hs + ((kp * 8) / group) * N;
            for (size_t n = n0; n < n1; ++n) {
                const uint32_t word = hp[kp * N + n];
                double sg = 0.0, sb = 0.0;
                for (unsigned bit = 0; bit < 8; ++bit) {
                    const float wv = host_f16_round((float)((int)((word >> (4 * bit)) & 0xFu) - 8) * sc[n]);
                    sg += (double)gp[kp * 8 + bit] * wv;
                    sb += (double)bp[kp * 8 + bit] * wv;
                }
                ag[n - n0] += sg;
                ab[n - n0] += sb;
            }
        }
        for (size_t n = n0; n < n1; ++n) {
            gsp[n] = (float)ag[n - n0];
            csp[n] = (float)(ab[n - n0] + (double)biasp[n]);
        }
    });
    TRY(upload(ctx, gs.data(), N * 4, gsum));
    TRY(upload(ctx, cs.data(), N * 4, bc));
    return B200NN_OK;
}

int f32_weight_upload(b200nn_ctx *ctx, const float *wsrc, bool is_out_in, const float *bias, size_t K, size_t N,
                      F32Weight *w) {
    if (K == 0 || N == 0) return set_error(ctx, B200NN_ERR_SHAPE, "Linear: empty weight");
    w->K = (int)K;
    w->N = (int)N;
    if (is_out_in) { // [N,K] -> [K,N]
        std::vector<float> t(K * N);
        float *tp = t.data();
        parallel_for(N, [=](size_t n0, size_t n1) {
            for (size_t n = n0; n < n1; ++n)
                for (size_t k = 0; k < K; ++k) tp[k * N + n] = wsrc[n * K + k];
        });
        TRY(upload(ctx, t.data(), K * N * sizeof(float), &w->w_kn));
    } else {
        TRY(upload(ctx, wsrc, K * N * sizeof(float), &w->w_kn));
    }
    if (bias) TRY(upload(ctx, bias, N * sizeof(float), &w->bias));
    // fp16 representation for the tensor-core GEMM (rows > 4): hi[N,K] = the weight rounded to fp16,
    // then lo[N,K] = the rounded remainder w - hi.  Skipped when a value would overflow fp16 or the
    // row stride would not be a multiple of 16 bytes.
    w->w_nk_h.reset();
    if (K % 8 == 0) {
        std::vector<__half> h(2 * K * N);
        __half *hp = h.data(), *lp = h.data() + K * N;
        std::atomic<int> too_large{0};
        parallel_for(N, [&, hp, lp](size_t n0, size_t n1) {
            bool big = false;
            for (size_t n = n0; n < n1; ++n)
                for (size_t k = 0; k < K; ++k) {
                    const float v = is_out_in ? wsrc[n * K + k] : wsrc[k * N + n];
                    big |= !(fabsf(v) <= 65504.0f);
                    const __half hi = __float2half_rn(v);
                    hp[n * K + k] = hi;
                    lp[n * K + k] = __float2half_rn(v - __half2float(hi));
                }
            if (big) too_large.store(1);
        });
        if (!too_large.load()) TRY(upload(ctx, h.data(), h.size() * sizeof(__half), &w->w_nk_h));
    }
    return B200NN_OK;
}
