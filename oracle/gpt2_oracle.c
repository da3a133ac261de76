/*
 * CPU oracle for the GPT-2 `nn` inference path of async-gpu.
 *
 * TEST INFRASTRUCTURE ONLY.  This file restates, in plain C, the algorithms the
 * reference project uses for this path, so that the CUDA library can be checked
 * against them.  It is never linked into, loaded by, or called from the product
 * library; only the test-suite, the smoke check and the benchmark's CPU-baseline
 * leg use it.
 *
 * Parity status: PINNED against the reference's own known-answer tests for the
 * quantiser / packer (crates/core/gpu-host/src/nn/ops/quantize.rs:169-268), the
 * CPU reference helpers (crates/core/gpu-host/src/nn/test_utils.rs:225-285) and
 * the arithmetic-pattern layer tests (layers/linear.rs:388-464,
 * layers/norm.rs:159-188); the vectors are restated in tests/golden/.  The
 * reference's real-weight goldens (.research/golden/*.golden) need GPT-2
 * checkpoint files that are not available offline and are not replayed.
 *
 * The reference itself is Rust (nightly + nvptx64) and cannot be compiled with
 * the C/C++ toolchain, so there is no oracle/_ref build of it.
 *
 * Every function cites the reference file:line it follows (paths relative to
 * the reference repository root).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------- */
/* helpers                                                                   */
/* ------------------------------------------------------------------------- */

/* Rust f32::round(): half away from zero (quantize.rs:80 uses `.round()`). */
static inline float round_half_away(float v) { return roundf(v); }

/* IEEE binary16 round trip (round-to-nearest-even), used to model an fp16 KV
 * cache and fp16 group scales. */
static inline float f16_round(float v) { return (float)(_Float16)v; }

ORC_API float orc_f16_round(float v) { return f16_round(v); }

ORC_API void orc_f16_round_array(const float *in, size_t n, float *out) {
    for (size_t i = 0; i < n; ++i) out[i] = f16_round(in[i]);
}

ORC_API int orc_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

ORC_API void orc_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* ------------------------------------------------------------------------- */
/* quantisation: crates/core/gpu-host/src/nn/ops/quantize.rs                 */
/* ------------------------------------------------------------------------- */

/* quantize.rs:5-18 — symmetric per-tensor int8. */
ORC_API void orc_quantize_int8_per_tensor(const float *data, size_t n, int8_t *q, float *scale_out) {
    float max_abs = 0.0f;
    for (size_t i = 0; i < n; ++i) max_abs = fmaxf(max_abs, fabsf(data[i]));
    float scale = (max_abs < 1e-12f) ? 1.0f : max_abs / 127.0f;
    float inv = 1.0f / scale;
    for (size_t i = 0; i < n; ++i) {
        float r = round_half_away(data[i] * inv);
        if (r < -128.0f) r = -128.0f;
        if (r > 127.0f) r = 127.0f;
        q[i] = (int8_t)r;
    }
    *scale_out = scale;
}

/* quantize.rs:23-32 — four int8 per u32, little-endian byte order, zero padded.
 * `packed` holds ceil(n/4) words. */
ORC_API void orc_pack_int8_to_u32(const int8_t *values, size_t n, uint32_t *packed) {
    size_t n_u32 = (n + 3) / 4;
    memset(packed, 0, n_u32 * sizeof(uint32_t));
    for (size_t i = 0; i < n; ++i)
        packed[i / 4] |= ((uint32_t)(uint8_t)values[i]) << ((i % 4) * 8);
}

static inline uint32_t quant_nibble(float v, float inv_scale) {
    /* quantize.rs:80-81 / 144-145: round, cast to i32, clamp to [-8,7], +8. */
    int q = (int)round_half_away(v * inv_scale);
    if (q < -8) q = -8;
    if (q > 7) q = 7;
    return (uint32_t)(q + 8) & 0xFu;
}

/* quantize.rs:56-89 — flat vector, groups of `group` consecutive elements.
 * packed: len/8 words; scales: ceil(len/group). */
ORC_API void orc_quantize_int4_per_group(const float *data, size_t len, size_t group,
                                         uint32_t *packed, float *scales) {
    size_t n_groups = (len + group - 1) / group;
    memset(packed, 0, (len / 8) * sizeof(uint32_t));
    for (size_t g = 0; g < n_groups; ++g) {
        size_t start = g * group, end = start + group;
        if (end > len) end = len;
        float max_abs = 0.0f;
        for (size_t i = start; i < end; ++i) max_abs = fmaxf(max_abs, fabsf(data[i]));
        float scale = (max_abs < 1e-12f) ? 1.0f : max_abs / 7.0f;
        scales[g] = scale;
        float inv = 1.0f / scale;
        for (size_t idx = start; idx < end; ++idx)
            packed[idx / 8] |= quant_nibble(data[idx], inv) << ((idx % 8) * 4);
    }
}

/* quantize.rs:102-153 — weight_t is [K,N] row-major; groups run along K per
 * column; packed is [K/8,N] (nibble i of a word = k index 8*kp+i), scales
 * [ceil(K/group),N].  Returns -1 if K%8 != 0 (the reference asserts). */
ORC_API int orc_quantize_weight_int4(const float *weight_t, size_t k, size_t n, size_t group,
                                     uint32_t *packed, float *scales) {
    if (k % 8 != 0 || group == 0) return -1;
    size_t k_packed = k / 8, n_groups = (k + group - 1) / group;
#pragma omp parallel for schedule(static)
    for (size_t col = 0; col < n; ++col) {
        for (size_t g = 0; g < n_groups; ++g) {
            size_t s = g * group, e = s + group;
            if (e > k) e = k;
            float max_abs = 0.0f;
            for (size_t ki = s; ki < e; ++ki) max_abs = fmaxf(max_abs, fabsf(weight_t[ki * n + col]));
            scales[g * n + col] = (max_abs < 1e-12f) ? 1.0f : max_abs / 7.0f;
        }
        for (size_t kp = 0; kp < k_packed; ++kp) {
            uint32_t word = 0;
            for (unsigned bit = 0; bit < 8; ++bit) {
                size_t ki = kp * 8 + bit;
                float scale = scales[(ki / group) * n + col];
                float inv = 1.0f / scale;
                word |= quant_nibble(weight_t[ki * n + col], inv) << (bit * 4);
            }
            packed[kp * n + col] = word;
        }
    }
    return 0;
}

/* quantize.rs:158-162. */
ORC_API int orc_unpack_int4(uint32_t packed, int index) {
    return (int)((packed >> (index * 4)) & 0xFu) - 8;
}

/* Dequantised weight matrix [K,N] f32: w = (nibble-8) * scale, the value the
 * reference kernel forms in f32 (compute_gemm.rs:2882-2886). */
ORC_API void orc_dequant_weight_int4(const uint32_t *packed, const float *scales, size_t k, size_t n,
                                     size_t group, float *w_out) {
#pragma omp parallel for schedule(static)
    for (size_t ki = 0; ki < k; ++ki) {
        const uint32_t *prow = packed + (ki / 8) * n;
        const float *srow = scales + (ki / group) * n;
        unsigned sh = (unsigned)(ki % 8) * 4;
        for (size_t col = 0; col < n; ++col) {
            int q = (int)((prow[col] >> sh) & 0xFu) - 8;
            w_out[ki * n + col] = (float)q * srow[col];
        }
    }
}

/* ------------------------------------------------------------------------- */
/* int4 linear: crates/kernel/gpu-kernel-compute/src/compute_gemm.rs:2849-2910 */
/* ------------------------------------------------------------------------- */

/* Exactly the reference kernel's arithmetic: f32 dequant, one fma.rn.f32 per
 * k in ascending order, bias added afterwards in f32 (the separate bias_add
 * kernel, compute_transformer.rs:1354-1387). */
ORC_API void orc_int4_linear_f32(const float *a, const uint32_t *packed, const float *scales,
                                 const float *bias, size_t m, size_t n, size_t k, size_t group,
                                 float *c) {
#pragma omp parallel for schedule(static)
    for (size_t col = 0; col < n; ++col) {
        for (size_t row = 0; row < m; ++row) {
            float acc = 0.0f;
            for (size_t kp = 0; kp < k / 8; ++kp) {
                uint32_t w = packed[kp * n + col];
                for (unsigned bit = 0; bit < 8; ++bit) {
                    size_t ki = kp * 8 + bit;
                    int q = (int)((w >> (bit * 4)) & 0xFu) - 8;
                    float wf = (float)q * scales[(ki / group) * n + col];
                    acc = fmaf(a[row * k + ki], wf, acc);
                }
            }
            c[row * n + col] = bias ? acc + bias[col] : acc;
        }
    }
}

/* Same weights, f64 accumulation: the high-precision answer the GPU result is
 * compared with (tolerances are stated in the tests). */
ORC_API void orc_int4_linear_f64(const float *a, const uint32_t *packed, const float *scales,
                                 const float *bias, size_t m, size_t n, size_t k, size_t group,
                                 float *c) {
#pragma omp parallel for schedule(static)
    for (size_t col = 0; col < n; ++col) {
        for (size_t row = 0; row < m; ++row) {
            double acc = 0.0;
            for (size_t ki = 0; ki < k; ++ki) {
                uint32_t w = packed[(ki / 8) * n + col];
                int q = (int)((w >> ((ki % 8) * 4)) & 0xFu) - 8;
                float wf = (float)q * scales[(ki / group) * n + col];
                acc += (double)a[row * k + ki] * (double)wf;
            }
            if (bias) acc += (double)bias[col];
            c[row * n + col] = (float)acc;
        }
    }
}

/* ------------------------------------------------------------------------- */
/* crates/core/gpu-host/src/nn/cpu_ref.rs                                    */
/* ------------------------------------------------------------------------- */

/* cpu_ref.rs:9-21 — C[m,n] = A[m,k] * B[k,n], f64 accumulate in ascending p.
 * The loop nest is reordered (i,p,j) for speed; each C element still receives
 * its products in ascending p, so the result is bit-identical. */
ORC_API void orc_matmul_f64(const float *a, const float *b, size_t m, size_t k, size_t n, float *c) {
#pragma omp parallel
    {
        double *acc = (double *)malloc(n * sizeof(double));
#pragma omp for schedule(static)
        for (size_t i = 0; i < m; ++i) {
            for (size_t j = 0; j < n; ++j) acc[j] = 0.0;
            for (size_t p = 0; p < k; ++p) {
                double av = (double)a[i * k + p];
                const float *brow = b + p * n;
                for (size_t j = 0; j < n; ++j) acc[j] += av * (double)brow[j];
            }
            for (size_t j = 0; j < n; ++j) c[i * n + j] = (float)acc[j];
        }
        free(acc);
    }
}

/* cpu_ref.rs:27-54 — biased variance, eps inside the root. */
ORC_API void orc_layer_norm_f64(const float *input, const float *gamma, const float *beta,
                                size_t rows, size_t d, float eps, float *out) {
    for (size_t i = 0; i < rows; ++i) {
        const float *row = input + i * d;
        double mean = 0.0;
        for (size_t j = 0; j < d; ++j) mean += (double)row[j];
        mean /= (double)d;
        double var = 0.0;
        for (size_t j = 0; j < d; ++j) {
            double diff = (double)row[j] - mean;
            var += diff * diff;
        }
        var /= (double)d;
        double inv_std = 1.0 / sqrt(var + (double)eps);
        for (size_t j = 0; j < d; ++j) {
            double norm = ((double)row[j] - mean) * inv_std;
            out[i * d + j] = (float)(norm * (double)gamma[j] + (double)beta[j]);
        }
    }
}

/* cpu_ref.rs:111-125. */
ORC_API void orc_softmax_f64(const float *input, size_t rows, size_t cols, float *out) {
    for (size_t i = 0; i < rows; ++i) {
        const float *row = input + i * cols;
        double mx = -INFINITY;
        for (size_t j = 0; j < cols; ++j) mx = fmax(mx, (double)row[j]);
        double sum = 0.0;
        for (size_t j = 0; j < cols; ++j) sum += exp((double)row[j] - mx);
        for (size_t j = 0; j < cols; ++j) out[i * cols + j] = (float)(exp((double)row[j] - mx) / sum);
    }
}

/* cpu_ref.rs:130-165 — single head, causal, scores and probabilities rounded to
 * f32 between the stages exactly as the reference does. */
ORC_API void orc_attention_f64(const float *q, const float *k, const float *v, size_t seq, size_t d,
                               float *out) {
    double scale = 1.0 / sqrt((double)d);
    float *scores = (float *)malloc(seq * seq * sizeof(float));
    float *probs = (float *)malloc(seq * seq * sizeof(float));
    for (size_t i = 0; i < seq; ++i)
        for (size_t j = 0; j < seq; ++j) {
            double dot = 0.0;
            for (size_t p = 0; p < d; ++p) dot += (double)q[i * d + p] * (double)k[j * d + p];
            scores[i * seq + j] = (j > i) ? -INFINITY : (float)(dot * scale);
        }
    orc_softmax_f64(scores, seq, seq, probs);
    for (size_t i = 0; i < seq; ++i)
        for (size_t j = 0; j < d; ++j) {
            double sum = 0.0;
            for (size_t p = 0; p < seq; ++p) sum += (double)probs[i * seq + p] * (double)v[p * d + j];
            out[i * d + j] = (float)sum;
        }
    free(scores);
    free(probs);
}

/* ------------------------------------------------------------------------- */
/* activations                                                               */
/* ------------------------------------------------------------------------- */

/* tanh GELU: crates/test/gpu-test-harness/src/tests_inference.rs:3680-3685. */
ORC_API double orc_gelu_tanh(double x) {
    const double sqrt_2_over_pi = 0.7978845608028654;
    const double coeff = 0.044715;
    double inner = sqrt_2_over_pi * (x + coeff * x * x * x);
    return x * 0.5 * (1.0 + tanh(inner));
}

/* sigmoid GELU x*sigmoid(1.702x): crates/kernel/gpu-kernel-compute/src/
 * compute_transformer.rs:1486-1504 (the default `nn` GELU kernel). */
ORC_API double orc_gelu_sigmoid(double x) { return x / (1.0 + exp(-1.702 * x)); }

/* ------------------------------------------------------------------------- */
/* full model: crates/test/gpu-test-harness/src/tests_inference.rs:3577-4554 */
/* ------------------------------------------------------------------------- */

enum {
    ORC_GELU_SIGMOID = 1u << 0, /* default is tanh (the CPU f64 reference)           */
    ORC_KV_FP16 = 1u << 1,      /* round K and V to binary16 before they are used     */
    ORC_ARGMAX_LAST = 1u << 2,  /* Rust max_by keeps the last maximum (gpt2.rs:991)   */
    ORC_STOP_ON_EOS = 1u << 3,  /* stop before appending token 50256 (gpt2.rs:698)    */
};

typedef struct {
    int32_t n_layer, n_embd, n_head, vocab_size, n_positions;
    float layer_norm_epsilon;
} orc_config;

typedef struct {
    const float *ln1_g, *ln1_b, *attn_w, *attn_b, *proj_w, *proj_b;
    const float *ln2_g, *ln2_b, *fc_w, *fc_b, *fcproj_w, *fcproj_b;
} orc_layer;

/* Weights are BORROWED pointers in the checkpoint (Conv1D) layout the reference
 * loader produces (crates/core/gpu-host/src/model.rs:121-154): every dense
 * weight is [in,out] row-major.  wte is [vocab,d], wpe is [n_positions,d].
 * lm_head, when non-NULL, is a [d,vocab] matrix that replaces the tied wte
 * head (used when the head has been int4-quantised and dequantised again). */
typedef struct orc_model {
    orc_config cfg;
    const float *wte, *wpe, *lnf_g, *lnf_b, *lm_head;
    orc_layer *layers;
} orc_model;

ORC_API orc_model *orc_model_create(const orc_config *cfg, const float *wte, const float *wpe,
                                    const float *lnf_g, const float *lnf_b) {
    orc_model *m = (orc_model *)calloc(1, sizeof(orc_model));
    m->cfg = *cfg;
    m->wte = wte;
    m->wpe = wpe;
    m->lnf_g = lnf_g;
    m->lnf_b = lnf_b;
    m->layers = (orc_layer *)calloc((size_t)cfg->n_layer, sizeof(orc_layer));
    return m;
}

ORC_API void orc_model_set_layer(orc_model *m, int layer, const float *ln1_g, const float *ln1_b,
                                 const float *attn_w, const float *attn_b, const float *proj_w,
                                 const float *proj_b, const float *ln2_g, const float *ln2_b,
                                 const float *fc_w, const float *fc_b, const float *fcproj_w,
                                 const float *fcproj_b) {
    orc_layer *l = &m->layers[layer];
    l->ln1_g = ln1_g; l->ln1_b = ln1_b; l->attn_w = attn_w; l->attn_b = attn_b;
    l->proj_w = proj_w; l->proj_b = proj_b; l->ln2_g = ln2_g; l->ln2_b = ln2_b;
    l->fc_w = fc_w; l->fc_b = fc_b; l->fcproj_w = fcproj_w; l->fcproj_b = fcproj_b;
}

ORC_API void orc_model_set_lm_head(orc_model *m, const float *lm_head_d_by_vocab) {
    m->lm_head = lm_head_d_by_vocab;
}

ORC_API void orc_model_destroy(orc_model *m) {
    if (!m) return;
    free(m->layers);
    free(m);
}

/* tests_inference.rs:3639-3652 (all-f64 LayerNorm). */
static void ln_d(const double *in, const float *g, const float *b, size_t rows, size_t d, double eps,
                 double *out) {
    for (size_t s = 0; s < rows; ++s) {
        const double *row = in + s * d;
        double mean = 0.0;
        for (size_t j = 0; j < d; ++j) mean += row[j];
        mean /= (double)d;
        double var = 0.0;
        for (size_t j = 0; j < d; ++j) var += (row[j] - mean) * (row[j] - mean);
        var /= (double)d;
        double inv_std = 1.0 / sqrt(var + eps);
        for (size_t j = 0; j < d; ++j) out[s * d + j] = (row[j] - mean) * inv_std * (double)g[j] + (double)b[j];
    }
}

/* tests_inference.rs:3655-3677 — C = A[m,k] * B[k,n] + bias, all f64, products
 * added in ascending k per output element. */
static void mm_bias_d(const double *a, const float *b, const float *bias, size_t m, size_t k, size_t n,
                      double *c) {
    const size_t JB = 512;
    size_t nblk = (n + JB - 1) / JB;
#pragma omp parallel for schedule(dynamic, 1)
    for (size_t jb = 0; jb < nblk; ++jb) {
        size_t j0 = jb * JB, j1 = j0 + JB;
        if (j1 > n) j1 = n;
        for (size_t i = 0; i < m; ++i)
            for (size_t j = j0; j < j1; ++j) c[i * n + j] = 0.0;
        for (size_t p = 0; p < k; ++p) {
            const float *brow = b + p * n;
            for (size_t i = 0; i < m; ++i) {
                double av = a[i * k + p];
                double *crow = c + i * n;
                for (size_t j = j0; j < j1; ++j) crow[j] += av * (double)brow[j];
            }
        }
        if (bias)
            for (size_t i = 0; i < m; ++i)
                for (size_t j = j0; j < j1; ++j) c[i * n + j] += (double)bias[j];
    }
}

/* Logits of one hidden row against the head.  Tied head: wte[v,:] . h
 * (tests_inference.rs:3966-3973); explicit head: column v of [d,vocab]. */
static void lm_head_row(const orc_model *m, const double *h, double *logits) {
    size_t d = (size_t)m->cfg.n_embd, V = (size_t)m->cfg.vocab_size;
    if (m->lm_head) {
        mm_bias_d(h, m->lm_head, NULL, 1, d, V, logits);
    } else {
#pragma omp parallel for schedule(static)
        for (size_t v = 0; v < V; ++v) {
            double dot = 0.0;
            const float *w = m->wte + v * d;
            for (size_t j = 0; j < d; ++j) dot += h[j] * (double)w[j];
            logits[v] = dot;
        }
    }
}

/* Greedy pick.  First maximum: tests_inference.rs:4504-4515 (`dot > best`).
 * Last maximum: gpt2.rs:991-997 (Rust max_by returns the last of equal maxima). */
static uint32_t argmax_d(const double *x, size_t n, int last) {
    double best = -INFINITY;
    uint32_t bi = 0;
    for (size_t i = 0; i < n; ++i) {
        if (last ? (x[i] >= best) : (x[i] > best)) {
            best = x[i];
            bi = (uint32_t)i;
        }
    }
    return bi;
}

/* One transformer block over `nq` new rows whose absolute positions start at
 * `past`; K and V for positions [0,past) are read from the caches, the new ones
 * are appended.  kc/vc: [n_head][cap][dh] f64.  With past==0 and nq==seq this
 * is the full causal forward of tests_inference.rs:3734-3850. */
static void block_forward(const orc_model *m, const orc_layer *L, double *hidden, size_t nq,
                          size_t past, double *kc, double *vc, size_t cap, uint32_t flags) {
    size_t d = (size_t)m->cfg.n_embd, H = (size_t)m->cfg.n_head, dh = d / H, ffn = 4 * d;
    double eps = (double)m->cfg.layer_norm_epsilon;
    double *ln = (double *)malloc(nq * d * sizeof(double));
    double *qkv = (double *)malloc(nq * 3 * d * sizeof(double));
    double *ac = (double *)malloc(nq * d * sizeof(double));
    double *tmp = (double *)malloc(nq * d * sizeof(double));
    double *fh = (double *)malloc(nq * ffn * sizeof(double));

    ln_d(hidden, L->ln1_g, L->ln1_b, nq, d, eps, ln);
    mm_bias_d(ln, L->attn_w, L->attn_b, nq, d, 3 * d, qkv);

    /* append K,V: column blocks [d,2d) and [2d,3d), head h at h*dh
     * (tests_inference.rs:3771-3776). */
    for (size_t s = 0; s < nq; ++s)
        for (size_t h = 0; h < H; ++h)
            for (size_t e = 0; e < dh; ++e) {
                double kv = qkv[s * 3 * d + d + h * dh + e];
                double vv = qkv[s * 3 * d + 2 * d + h * dh + e];
                if (flags & ORC_KV_FP16) {
                    kv = (double)f16_round((float)kv);
                    vv = (double)f16_round((float)vv);
                }
                kc[(h * cap + past + s) * dh + e] = kv;
                vc[(h * cap + past + s) * dh + e] = vv;
            }

    double scale = 1.0 / sqrt((double)dh);
#pragma omp parallel for schedule(dynamic, 1) collapse(2)
    for (size_t h = 0; h < H; ++h)
        for (size_t i = 0; i < nq; ++i) {
            size_t kv_len = past + i + 1; /* causal: j <= absolute position */
            double *sc = (double *)malloc(kv_len * sizeof(double));
            const double *q = qkv + i * 3 * d + h * dh;
            double mx = -INFINITY;
            for (size_t j = 0; j < kv_len; ++j) {
                const double *kr = kc + (h * cap + j) * dh;
                double dot = 0.0;
                for (size_t e = 0; e < dh; ++e) dot += q[e] * kr[e];
                sc[j] = dot * scale;
                if (sc[j] > mx) mx = sc[j];
            }
            double sum = 0.0;
            for (size_t j = 0; j < kv_len; ++j) {
                sc[j] = exp(sc[j] - mx);
                sum += sc[j];
            }
            for (size_t j = 0; j < kv_len; ++j) sc[j] /= sum;
            for (size_t e = 0; e < dh; ++e) {
                double o = 0.0;
                for (size_t j = 0; j < kv_len; ++j) o += sc[j] * vc[(h * cap + j) * dh + e];
                ac[i * d + h * dh + e] = o;
            }
            free(sc);
        }

    mm_bias_d(ac, L->proj_w, L->proj_b, nq, d, d, tmp);
    for (size_t i = 0; i < nq * d; ++i) hidden[i] += tmp[i];

    ln_d(hidden, L->ln2_g, L->ln2_b, nq, d, eps, ln);
    mm_bias_d(ln, L->fc_w, L->fc_b, nq, d, ffn, fh);
    if (flags & ORC_GELU_SIGMOID)
        for (size_t i = 0; i < nq * ffn; ++i) fh[i] = orc_gelu_sigmoid(fh[i]);
    else
        for (size_t i = 0; i < nq * ffn; ++i) fh[i] = orc_gelu_tanh(fh[i]);
    mm_bias_d(fh, L->fcproj_w, L->fcproj_b, nq, ffn, d, tmp);
    for (size_t i = 0; i < nq * d; ++i) hidden[i] += tmp[i];

    free(ln); free(qkv); free(ac); free(tmp); free(fh);
}

/* One transformer block on its own (TransformerBlock::forward / forward_cached, gpt2.rs:172-288), for
 * checking a block handle in isolation: layer `layer` of `m` over `nq` rows x [nq,d] at positions
 * past..; kc / vc f32 [n_head][cap][dh] hold the cached rows [0,past) on entry and the new rows as
 * well on return; out [nq,d]. */
ORC_API void orc_block_forward(const orc_model *m, int layer, const float *x, size_t nq, size_t past, float *kc,
                               float *vc, size_t cap, uint32_t flags, float *out) {
    size_t d = (size_t)m->cfg.n_embd, H = (size_t)m->cfg.n_head, dh = d / H, nkv = H * cap * dh;
    double *h = (double *)malloc(nq * d * sizeof(double));
    double *kd = (double *)malloc(nkv * sizeof(double)), *vd = (double *)malloc(nkv * sizeof(double));
    for (size_t i = 0; i < nq * d; ++i) h[i] = (double)x[i];
    for (size_t i = 0; i < nkv; ++i) { kd[i] = (double)kc[i]; vd[i] = (double)vc[i]; }
    block_forward(m, &m->layers[layer], h, nq, past, kd, vd, cap, flags);
    for (size_t i = 0; i < nq * d; ++i) out[i] = (float)h[i];
    for (size_t i = 0; i < nkv; ++i) { kc[i] = (float)kd[i]; vc[i] = (float)vd[i]; }
    free(h); free(kd); free(vd);
}

typedef struct {
    double *k, *v; /* [n_layer][n_head][cap][dh] */
    size_t cap, len;
} orc_kv;

static void embed(const orc_model *m, const uint32_t *tok, size_t n, size_t pos0, double *h) {
    size_t d = (size_t)m->cfg.n_embd;
    /* tests_inference.rs:3617-3624; position offset as gpt2.rs:718-721. */
    for (size_t p = 0; p < n; ++p)
        for (size_t j = 0; j < d; ++j)
            h[p * d + j] = (double)m->wte[(size_t)tok[p] * d + j] + (double)m->wpe[(pos0 + p) * d + j];
}

/* Run `n` new tokens through the model on top of `kv`; writes logits for the
 * rows in [first_logit_row, n) to `logits` ([rows,vocab] f64) if non-NULL. */
static void forward_rows(const orc_model *m, const uint32_t *tok, size_t n, orc_kv *kv,
                         size_t first_logit_row, double *logits, uint32_t flags) {
    size_t d = (size_t)m->cfg.n_embd, H = (size_t)m->cfg.n_head, dh = d / H, V = (size_t)m->cfg.vocab_size;
    double *h = (double *)malloc(n * d * sizeof(double));
    double *lnf = (double *)malloc(n * d * sizeof(double));
    embed(m, tok, n, kv->len, h);
    size_t per_layer = H * kv->cap * dh;
    for (int l = 0; l < m->cfg.n_layer; ++l)
        block_forward(m, &m->layers[l], h, n, kv->len, kv->k + (size_t)l * per_layer,
                      kv->v + (size_t)l * per_layer, kv->cap, flags);
    kv->len += n;
    ln_d(h, m->lnf_g, m->lnf_b, n, d, (double)m->cfg.layer_norm_epsilon, lnf);
    if (logits)
        for (size_t r = first_logit_row; r < n; ++r) lm_head_row(m, lnf + r * d, logits + (r - first_logit_row) * V);
    free(h);
    free(lnf);
}

static int kv_alloc(const orc_model *m, size_t cap, orc_kv *kv) {
    size_t d = (size_t)m->cfg.n_embd;
    size_t total = (size_t)m->cfg.n_layer * cap * d;
    kv->k = (double *)malloc(total * sizeof(double));
    kv->v = (double *)malloc(total * sizeof(double));
    kv->cap = cap;
    kv->len = 0;
    return (kv->k && kv->v) ? 0 : -1;
}

static void kv_free(orc_kv *kv) {
    free(kv->k);
    free(kv->v);
}

/* Full causal forward over one sequence; logits for every position, [seq,vocab]
 * as f32 (the reference model returns all rows, gpt2.rs:481-499).  With
 * last_only != 0 only the final row is produced ([vocab]). */
ORC_API int orc_forward(const orc_model *m, const uint32_t *tokens, int32_t seq, int32_t last_only,
                        uint32_t flags, float *logits_out) {
    if (seq <= 0 || seq > m->cfg.n_positions) return -1;
    size_t V = (size_t)m->cfg.vocab_size, n = (size_t)seq;
    orc_kv kv;
    if (kv_alloc(m, n, &kv)) return -2;
    size_t first = last_only ? n - 1 : 0, rows = n - first;
    double *lg = (double *)malloc(rows * V * sizeof(double));
    forward_rows(m, tokens, n, &kv, first, lg, flags);
    for (size_t i = 0; i < rows * V; ++i) logits_out[i] = (float)lg[i];
    free(lg);
    kv_free(&kv);
    return 0;
}

/* Greedy generation WITHOUT a cache: every step re-runs the whole sequence,
 * as the CPU f64 reference (tests_inference.rs:4393-4540) and the model's
 * `generate` (gpt2.rs:672-706) do.  out_tokens must hold prompt_len+max_new
 * entries; returns the total token count (prompt + generated), or <0 on error.
 * step_logits, if non-NULL, receives the last-row logits of every step,
 * [max_new, vocab] f32. */
ORC_API int orc_generate(const orc_model *m, const uint32_t *prompt, int32_t prompt_len, int32_t max_new,
                         uint32_t flags, uint32_t *out_tokens, float *step_logits) {
    size_t V = (size_t)m->cfg.vocab_size;
    if (prompt_len <= 0 || prompt_len + max_new > m->cfg.n_positions) return -1;
    memcpy(out_tokens, prompt, (size_t)prompt_len * sizeof(uint32_t));
    int n = prompt_len;
    double *lg = (double *)malloc(V * sizeof(double));
    for (int step = 0; step < max_new; ++step) {
        orc_kv kv;
        if (kv_alloc(m, (size_t)n, &kv)) { free(lg); return -2; }
        forward_rows(m, out_tokens, (size_t)n, &kv, (size_t)n - 1, lg, flags);
        kv_free(&kv);
        if (step_logits)
            for (size_t i = 0; i < V; ++i) step_logits[(size_t)step * V + i] = (float)lg[i];
        uint32_t t = argmax_d(lg, V, (flags & ORC_ARGMAX_LAST) != 0);
        if ((flags & ORC_STOP_ON_EOS) && t == 50256u) break;
        out_tokens[n++] = t;
    }
    free(lg);
    return n;
}

/* Greedy generation WITH a KV cache (semantics of gpt2.rs:740-783: prefill the
 * prompt, then one token per step).  Mathematically the same sequence of
 * operations per position as orc_generate; used where the uncached form is too
 * slow, and as the timed CPU baseline. */
ORC_API int orc_generate_cached(const orc_model *m, const uint32_t *prompt, int32_t prompt_len,
                                int32_t max_new, uint32_t flags, uint32_t *out_tokens,
                                float *step_logits) {
    size_t V = (size_t)m->cfg.vocab_size;
    if (prompt_len <= 0 || prompt_len + max_new > m->cfg.n_positions) return -1;
    memcpy(out_tokens, prompt, (size_t)prompt_len * sizeof(uint32_t));
    int n = prompt_len;
    orc_kv kv;
    if (kv_alloc(m, (size_t)(prompt_len + max_new), &kv)) return -2;
    double *lg = (double *)malloc(V * sizeof(double));
    for (int step = 0; step < max_new; ++step) {
        if (step == 0)
            forward_rows(m, out_tokens, (size_t)n, &kv, (size_t)n - 1, lg, flags);
        else
            forward_rows(m, out_tokens + n - 1, 1, &kv, 0, lg, flags);
        if (step_logits)
            for (size_t i = 0; i < V; ++i) step_logits[(size_t)step * V + i] = (float)lg[i];
        uint32_t t = argmax_d(lg, V, (flags & ORC_ARGMAX_LAST) != 0);
        if ((flags & ORC_STOP_ON_EOS) && t == 50256u) break;
        out_tokens[n++] = t;
    }
    free(lg);
    kv_free(&kv);
    return n;
}

/* Timed-baseline helper: prefill `prompt_len` tokens, then run `steps` decode
 * steps feeding the greedy token back, for one sequence; returns seconds spent
 * in the decode steps only (prefill excluded) through *decode_seconds. */
ORC_API int orc_time_decode(const orc_model *m, const uint32_t *prompt, int32_t prompt_len, int32_t steps,
                            uint32_t flags, double *decode_seconds, uint32_t *out_tokens) {
    size_t V = (size_t)m->cfg.vocab_size;
    if (prompt_len <= 0 || prompt_len + steps + 1 > m->cfg.n_positions) return -1;
    orc_kv kv;
    if (kv_alloc(m, (size_t)(prompt_len + steps + 1), &kv)) return -2;
    double *lg = (double *)malloc(V * sizeof(double));
    forward_rows(m, prompt, (size_t)prompt_len, &kv, (size_t)prompt_len - 1, lg, flags);
    uint32_t t = argmax_d(lg, V, 0);
    double t0 = 0.0, t1 = 0.0;
#ifdef _OPENMP
    t0 = omp_get_wtime();
#endif
    for (int s = 0; s < steps; ++s) {
        if (out_tokens) out_tokens[s] = t;
        forward_rows(m, &t, 1, &kv, 0, lg, flags);
        t = argmax_d(lg, V, 0);
    }
#ifdef _OPENMP
    t1 = omp_get_wtime();
#endif
    *decode_seconds = t1 - t0;
    free(lg);
    kv_free(&kv);
    return 0;
}

/* Multi-head causal attention over new queries with an optional past, f64:
 * q [nq,H*dh] (row stride q_stride), kc/vc [H][kv_len][dh] already containing
 * the new positions; out [nq,H*dh].  Query i sits at absolute position
 * past+i.  Used to check the attention kernels in isolation
 * (layers/attention.rs:112-184 semantics: causal with q_offset = past). */
ORC_API void orc_mha_f64(const float *q, size_t q_stride, const float *kc, const float *vc, size_t H,
                         size_t dh, size_t nq, size_t past, size_t cap, float *out) {
    double scale = 1.0 / sqrt((double)dh);
#pragma omp parallel for schedule(dynamic, 1) collapse(2)
    for (size_t h = 0; h < H; ++h)
        for (size_t i = 0; i < nq; ++i) {
            size_t kv_len = past + i + 1;
            double *sc = (double *)malloc(kv_len * sizeof(double));
            double mx = -INFINITY;
            for (size_t j = 0; j < kv_len; ++j) {
                double dot = 0.0;
                for (size_t e = 0; e < dh; ++e)
                    dot += (double)q[i * q_stride + h * dh + e] * (double)kc[(h * cap + j) * dh + e];
                sc[j] = dot * scale;
                if (sc[j] > mx) mx = sc[j];
            }
            double sum = 0.0;
            for (size_t j = 0; j < kv_len; ++j) { sc[j] = exp(sc[j] - mx); sum += sc[j]; }
            for (size_t e = 0; e < dh; ++e) {
                double o = 0.0;
                for (size_t j = 0; j < kv_len; ++j) o += (sc[j] / sum) * (double)vc[(h * cap + j) * dh + e];
                out[i * H * dh + h * dh + e] = (float)o;
            }
            free(sc);
        }
}

/* ------------------------------------------------------------------------- */
/* Data-dependent decoding: sampling and early exit (gpt2.rs:785-1058)        */
/* ------------------------------------------------------------------------- */

/* SimpleRng (gpt2.rs:1000-1023): xorshift64, seed 0 replaced by a fixed constant. */
ORC_API uint64_t orc_rng_new(uint64_t seed) { return seed ? seed : 0xDEADBEEFCAFE1234ull; }
ORC_API float orc_rng_next_f32(uint64_t *s) {
    uint64_t x = *s;
    x ^= x << 13;
    x ^= x >> 7;
    x ^= x << 17;
    *s = x;
    return (float)(x >> 40) / (float)(1ull << 24);
}

typedef struct { float v; uint32_t i; } orc_cand;
/* the order a stable descending sort by value leaves: equal values by ascending index */
static int cand_cmp(const void *a, const void *b) {
    const orc_cand *x = (const orc_cand *)a, *y = (const orc_cand *)b;
    if (x->v > y->v) return -1;
    if (x->v < y->v) return 1;
    return (x->i > y->i) - (x->i < y->i);
}

/* top_k_sample (gpt2.rs:1029-1058), f32 as there.  *margin, if non-NULL, receives how far the draw
 * was from the nearest boundary of the cumulative distribution it fell between (a small margin means
 * that logits differing in the last bits may pick a neighbouring token). */
ORC_API uint32_t orc_top_k_sample(const float *logits, size_t n, size_t k, float temperature, uint64_t *rng,
                                  float *margin) {
    float temp = temperature < 1e-8f ? 1e-8f : temperature;
    orc_cand *c = (orc_cand *)malloc(n * sizeof(orc_cand));
    for (size_t i = 0; i < n; ++i) { c[i].v = logits[i] / temp; c[i].i = (uint32_t)i; }
    qsort(c, n, sizeof(orc_cand), cand_cmp);
    if (k > n) k = n;
    float max_val = c[0].v, sum = 0.0f;
    float *p = (float *)malloc(k * sizeof(float));
    for (size_t i = 0; i < k; ++i) { p[i] = expf(c[i].v - max_val); sum += p[i]; }
    float r = orc_rng_next_f32(rng), cum = 0.0f, prev = 0.0f;
    uint32_t pick = c[k - 1].i;
    float mg = 1.0f;
    for (size_t i = 0; i < k; ++i) {
        prev = cum;
        cum += p[i] / sum;
        if (r < cum) {
            pick = c[i].i;
            mg = fminf(r - prev, cum - r);
            if (i == 0) mg = cum - r;
            break;
        }
    }
    if (margin) *margin = mg;
    free(p);
    free(c);
    return pick;
}

/* softmax_max_prob (gpt2.rs:980-985): 1 / sum exp(x - max), f32, summed in index order. */
ORC_API float orc_softmax_max_prob(const float *x, size_t n) {
    float mx = -INFINITY, s = 0.0f;
    for (size_t i = 0; i < n; ++i) if (x[i] > mx) mx = x[i];
    for (size_t i = 0; i < n; ++i) s += expf(x[i] - mx);
    return 1.0f / s;
}

static void logits_row_f32(const orc_model *m, const double *h_row, double *lnf, double *lg, float *out) {
    size_t d = (size_t)m->cfg.n_embd, V = (size_t)m->cfg.vocab_size;
    ln_d(h_row, m->lnf_g, m->lnf_b, 1, d, (double)m->cfg.layer_norm_epsilon, lnf);
    lm_head_row(m, lnf, lg);
    for (size_t i = 0; i < V; ++i) out[i] = (float)lg[i];
}

/* generate_cached_sampling (gpt2.rs:933-977).  step_logits [max_new,vocab] f32 and margins [max_new]
 * are optional. */
ORC_API int orc_generate_cached_sampling(const orc_model *m, const uint32_t *prompt, int32_t prompt_len,
                                         int32_t max_new, int32_t top_k, float temperature, uint64_t *rng,
                                         uint32_t flags, uint32_t *out_tokens, float *step_logits, float *margins) {
    size_t V = (size_t)m->cfg.vocab_size;
    if (prompt_len <= 0 || prompt_len + max_new > m->cfg.n_positions || top_k <= 0) return -1;
    memcpy(out_tokens, prompt, (size_t)prompt_len * sizeof(uint32_t));
    int n = prompt_len;
    orc_kv kv;
    if (kv_alloc(m, (size_t)(prompt_len + max_new), &kv)) return -2;
    double *lg = (double *)malloc(V * sizeof(double));
    float *lf = (float *)malloc(V * sizeof(float));
    for (int step = 0; step < max_new; ++step) {
        if (step == 0)
            forward_rows(m, out_tokens, (size_t)n, &kv, (size_t)n - 1, lg, flags);
        else
            forward_rows(m, out_tokens + n - 1, 1, &kv, 0, lg, flags);
        for (size_t i = 0; i < V; ++i) lf[i] = (float)lg[i];
        if (step_logits) memcpy(step_logits + (size_t)step * V, lf, V * sizeof(float));
        float mg = 0.0f;
        uint32_t t = orc_top_k_sample(lf, V, (size_t)top_k, temperature, rng, &mg);
        if (margins) margins[step] = mg;
        if (t == 50256u) break;
        out_tokens[n++] = t;
    }
    free(lg);
    free(lf);
    kv_free(&kv);
    return n;
}

/* forward_early_exit (gpt2.rs:797-830): logits [seq,vocab] f32 of the exit layer; *layers_used in
 * 1..n_layer; confidences [n_layer-1] (optional) receives the probe value after every block reached. */
ORC_API int orc_forward_early_exit(const orc_model *m, const uint32_t *tokens, int32_t seq, float threshold,
                                   uint32_t flags, float *logits_out, int32_t *layers_used, float *confidences) {
    if (seq <= 0 || seq > m->cfg.n_positions) return -1;
    size_t d = (size_t)m->cfg.n_embd, H = (size_t)m->cfg.n_head, dh = d / H, V = (size_t)m->cfg.vocab_size, n = (size_t)seq;
    int L = m->cfg.n_layer;
    orc_kv kv;
    if (kv_alloc(m, n, &kv)) return -2;
    double *h = (double *)malloc(n * d * sizeof(double));
    double *lnf = (double *)malloc(d * sizeof(double));
    double *lg = (double *)malloc(V * sizeof(double));
    embed(m, tokens, n, 0, h);
    size_t per_layer = H * kv.cap * dh;
    int used = L;
    for (int l = 0; l < L; ++l) {
        block_forward(m, &m->layers[l], h, n, 0, kv.k + (size_t)l * per_layer, kv.v + (size_t)l * per_layer, kv.cap, flags);
        if (l < L - 1) {
            logits_row_f32(m, h + (n - 1) * d, lnf, lg, logits_out + (n - 1) * V);
            float conf = orc_softmax_max_prob(logits_out + (n - 1) * V, V);
            if (confidences) confidences[l] = conf;
            if (conf >= threshold) { used = l + 1; break; }
        }
    }
    for (size_t r = 0; r < n; ++r) logits_row_f32(m, h + r * d, lnf, lg, logits_out + r * V);
    *layers_used = used;
    free(h); free(lnf); free(lg);
    kv_free(&kv);
    return 0;
}

/* generate_cached_early_exit (gpt2.rs:837-924).  layers_per_step holds 1+max_new entries; returns the
 * token count, *n_steps the entries written.  min_gap (optional) receives the smallest distance
 * |confidence - threshold| met, so that a caller can tell a robust run from a borderline one. */
ORC_API int orc_generate_cached_early_exit(const orc_model *m, const uint32_t *prompt, int32_t prompt_len,
                                           int32_t max_new, float threshold, uint32_t flags, uint32_t *out_tokens,
                                           int32_t *layers_per_step, int32_t *n_steps, float *step_logits,
                                           float *min_gap) {
    size_t d = (size_t)m->cfg.n_embd, H = (size_t)m->cfg.n_head, dh = d / H, V = (size_t)m->cfg.vocab_size;
    int L = m->cfg.n_layer;
    if (prompt_len <= 0 || prompt_len + max_new > m->cfg.n_positions) return -1;
    memcpy(out_tokens, prompt, (size_t)prompt_len * sizeof(uint32_t));
    int n = prompt_len, steps = 0;
    float gap = INFINITY;
    *n_steps = 0;
    if (max_new <= 0) return n;
    orc_kv kv;
    if (kv_alloc(m, (size_t)(prompt_len + max_new), &kv)) return -2;
    size_t per_layer = H * kv.cap * dh;
    double *lg = (double *)malloc(V * sizeof(double));
    double *lnf = (double *)malloc(d * sizeof(double));
    double *h = (double *)malloc(d * sizeof(double));
    float *lf = (float *)malloc(V * sizeof(float));
    forward_rows(m, out_tokens, (size_t)n, &kv, (size_t)n - 1, lg, flags);
    layers_per_step[steps++] = L;
    for (int step = 0;; ++step) {
        if (step_logits && step < max_new)
            for (size_t i = 0; i < V; ++i) step_logits[(size_t)step * V + i] = (float)lg[i];
        uint32_t t = argmax_d(lg, V, 1); /* the model's argmax keeps the last maximum (gpt2.rs:991-997) */
        if (t == 50256u) break;
        out_tokens[n++] = t;
        if (step + 1 >= max_new) break;
        size_t pos = kv.len;
        embed(m, &t, 1, pos, h);
        int used = L;
        for (int l = 0; l < L; ++l) {
            block_forward(m, &m->layers[l], h, 1, pos, kv.k + (size_t)l * per_layer, kv.v + (size_t)l * per_layer, kv.cap, flags);
            if (l < L - 1) {
                logits_row_f32(m, h, lnf, lg, lf);
                float conf = orc_softmax_max_prob(lf, V);
                if (fabsf(conf - threshold) < gap) gap = fabsf(conf - threshold);
                if (conf >= threshold) {
                    for (int j = l + 1; j < L; ++j) /* zero K/V rows for the skipped layers (gpt2.rs:897-904) */
                        for (size_t hh = 0; hh < H; ++hh) {
                            memset(kv.k + (size_t)j * per_layer + (hh * kv.cap + pos) * dh, 0, dh * sizeof(double));
                            memset(kv.v + (size_t)j * per_layer + (hh * kv.cap + pos) * dh, 0, dh * sizeof(double));
                        }
                    used = l + 1;
                    break;
                }
            }
        }
        kv.len += 1;
        layers_per_step[steps++] = used;
        ln_d(h, m->lnf_g, m->lnf_b, 1, d, (double)m->cfg.layer_norm_epsilon, lnf);
        lm_head_row(m, lnf, lg);
    }
    *n_steps = steps;
    if (min_gap) *min_gap = gap;
    free(lg); free(lnf); free(h); free(lf);
    kv_free(&kv);
    return n;
}
