// Exercises the C++ host layer (include/b200nn.hpp) the way the reference's Rust tests use `gpu_host::nn`:
// construct through the reference's names, run, compare with plain host arithmetic.
// Exit codes: 0 all checks passed, 1 a check failed, 3 no CUDA device (the library refuses to run: no CPU fallback).
#include <cmath>
#include <cstdio>
#include <string>
#include <vector>

#include "b200nn.hpp"

using namespace b200nn;

static int g_checks = 0, g_failed = 0;
#define CHECK(cond, what)                                                        \
    do {                                                                         \
        ++g_checks;                                                              \
        if (!(cond)) { ++g_failed; std::printf("FAILED: %s (line %d)\n", what, __LINE__); } \
    } while (0)

static std::vector<float> normal(uint64_t seed, size_t n, float std_dev) {
    uint64_t st = b200nn_simple_rng_new(seed);
    std::vector<float> v(n);
    b200nn_simple_rng_fill_normal(&st, n, std_dev, v.data());
    return v;
}

static double max_abs_diff(const std::vector<float> &a, const std::vector<double> &b) {
    double m = 0;
    for (size_t i = 0; i < a.size(); ++i) m = std::fmax(m, std::fabs((double)a[i] - b[i]));
    return m;
}

template <typename F>
static bool throws_code(int32_t code, F f) {
    try { f(); } catch (const NnError &e) { return e.code() == code; }
    return false;
}

static Gpt2Weights tiny_weights(const Gpt2Config &c, uint64_t seed) {
    Gpt2Weights w;
    const size_t d = c.n_embd;
    w.wte = normal(seed + 1, c.vocab_size * d, 0.08f);
    w.wpe = normal(seed + 2, c.n_positions * d, 0.02f);
    w.ln_f_weight.assign(d, 1.0f);
    w.ln_f_bias = normal(seed + 3, d, 0.02f);
    for (size_t l = 0; l < c.n_layer; ++l) {
        TransformerLayerWeights t;
        const uint64_t s = seed + 1000 * (l + 1);
        t.ln_1_weight.assign(d, 1.0f);
        t.ln_1_bias = normal(s + 1, d, 0.02f);
        t.c_attn_weight = normal(s + 2, d * 3 * d, 0.08f);
        t.c_attn_bias = normal(s + 3, 3 * d, 0.02f);
        t.c_proj_weight = normal(s + 4, d * d, 0.08f);
        t.c_proj_bias = normal(s + 5, d, 0.02f);
        t.ln_2_weight.assign(d, 1.0f);
        t.ln_2_bias = normal(s + 6, d, 0.02f);
        t.mlp_fc_weight = normal(s + 7, d * 4 * d, 0.08f);
        t.mlp_fc_bias = normal(s + 8, 4 * d, 0.02f);
        t.mlp_proj_weight = normal(s + 9, 4 * d * d, 0.08f);
        t.mlp_proj_bias = normal(s + 10, d, 0.02f);
        w.layers.push_back(std::move(t));
    }
    return w;
}

int main() {
    Registry reg;
    try {
        reg = KernelRegistry::init_default();
    } catch (const NnError &e) {
        std::printf("NO_DEVICE: %s\n", e.what());
        return e.code() == B200NN_ERR_CUDA ? 3 : 1;
    }

    // ---- GpuTensor -------------------------------------------------------------------------
    std::vector<float> a(24);
    for (size_t i = 0; i < a.size(); ++i) a[i] = 0.5f * (float)i;
    GpuTensor t = GpuTensor::from_host(a, {2, 3, 4}, reg);
    CHECK(t.numel() == 24 && t.ndim() == 3 && t.shape() == std::vector<size_t>({2, 3, 4}), "shape");
    CHECK(t.strides() == std::vector<size_t>({12, 4, 1}) && t.size_bytes() == 96, "strides");
    CHECK(t.to_host() == a && t.reshape({6, 4}).to_host() == a && t.clone_tensor().to_host() == a, "round trip");
    CHECK(GpuTensor::from_data(t.as_ptr(), {24}, reg).to_host() == a, "from_data");
    GpuTensor tr = t.reshape({6, 4}).transpose(0, 1);
    CHECK(tr.shape() == std::vector<size_t>({4, 6}) && tr.to_host()[1] == a[4], "transpose");
    std::vector<GpuTensor> parts = t.reshape({6, 4}).split(0, {2, 4});
    CHECK(parts.size() == 2 && parts[1].shape()[0] == 4, "split");
    CHECK(GpuTensor::concat({&parts[0], &parts[1]}, 0).to_host() == a, "concat");
    CHECK(throws_code(B200NN_ERR_SHAPE, [&] { GpuTensor::from_host(a, {5, 5}, reg); }), "from_host size error");
    CHECK(throws_code(B200NN_ERR_DIM, [&] { t.transpose(0, 7); }), "transpose dim error");

    // ---- Linear, LayerNorm, matmul_fused ---------------------------------------------------
    const size_t M = 3, K = 40, N = 24;
    std::vector<float> x = normal(11, M * K, 1.0f), w = normal(12, N * K, 0.2f), b = normal(13, N, 0.5f);
    GpuTensor tx = GpuTensor::from_host(x, {M, K}, reg);
    std::vector<double> ref(M * N);
    for (size_t m = 0; m < M; ++m)
        for (size_t n = 0; n < N; ++n) {
            double s = b[n];
            for (size_t k = 0; k < K; ++k) s += (double)x[m * K + k] * w[n * K + k];
            ref[m * N + n] = s;
        }
    Linear lin(w, &b, K, N, reg);
    CHECK(max_abs_diff(lin.forward(tx).to_host(), ref) < 1e-4, "Linear::forward");
    std::vector<double> ref_relu = ref;
    for (double &v : ref_relu) v = v > 0 ? v : 0;
    CHECK(max_abs_diff(lin.forward_auto_fused(tx, Activation::Relu).to_host(), ref_relu) < 1e-4, "Linear::forward_auto_fused");
    std::vector<float> wt(K * N);
    for (size_t k = 0; k < K; ++k)
        for (size_t n = 0; n < N; ++n) wt[k * N + n] = w[n * K + k];
    GpuTensor twt = GpuTensor::from_host(wt, {K, N}, reg), tb = GpuTensor::from_host(b, {N}, reg);
    CHECK(max_abs_diff(ops::matmul_fused(tx, twt, tb, FusedActivation::Relu, reg).to_host(), ref_relu) < 1e-4, "ops::matmul_fused");
    CHECK(throws_code(B200NN_ERR_SHAPE, [&] { ops::matmul_fused(tx, tx, tb, FusedActivation::Relu, reg); }), "matmul_fused shape error");
    std::vector<float> g = normal(14, K, 1.0f), be = normal(15, K, 1.0f);
    LayerNorm ln(g, be, 1e-5f, reg);
    std::vector<double> ref_ln(M * K);
    for (size_t m = 0; m < M; ++m) {
        double mean = 0, var = 0;
        for (size_t k = 0; k < K; ++k) mean += x[m * K + k];
        mean /= K;
        for (size_t k = 0; k < K; ++k) var += (x[m * K + k] - mean) * (x[m * K + k] - mean);
        var /= K;
        for (size_t k = 0; k < K; ++k) ref_ln[m * K + k] = (x[m * K + k] - mean) / std::sqrt(var + 1e-5) * g[k] + be[k];
    }
    CHECK(max_abs_diff(ln.forward(tx).to_host(), ref_ln) < 1e-4, "LayerNorm::forward");
    CHECK(ln.gamma().to_host() == g && ln.beta().to_host() == be, "LayerNorm::gamma / beta");

    // ---- Int4Linear against the host dequantisation of the same nibbles --------------------------
    const size_t K4 = 256, N4 = 48, G = 128;
    std::vector<float> w4 = normal(21, K4 * N4, 0.05f), x4 = normal(22, 2 * K4, 1.0f);
    ops::Int4Quantized q = ops::quantize_weight_int4(w4, K4, N4, G);
    Int4Linear l4(q.packed, q.scales, nullptr, K4, N4, G, reg);
    std::vector<double> ref4(2 * N4, 0.0);
    for (size_t m = 0; m < 2; ++m)
        for (size_t n = 0; n < N4; ++n)
            for (size_t k = 0; k < K4; ++k) {
                const int32_t nib = ops::unpack_int4(q.packed[(k / 8) * N4 + n], (int32_t)(k % 8));
                ref4[m * N4 + n] += (double)x4[m * K4 + k] * nib * q.scales[(k / G) * N4 + n];
            }
    // the library rounds the scales to fp16: allow that (2^-11 relative) on sums of this size
    CHECK(max_abs_diff(l4.forward(GpuTensor::from_host(x4, {2, K4}, reg)).to_host(), ref4) < 5e-3, "Int4Linear::forward");
    CHECK(l4.memory_bytes() > 0, "Int4Linear::memory_bytes");

    // ---- Gpt2Model / Int4Gpt2Model / KvCache ----------------------------------------------------
    Gpt2Config cfg;
    cfg.n_layer = 2; cfg.n_embd = 128; cfg.n_head = 2; cfg.vocab_size = 97; cfg.n_positions = 32;
    CHECK(cfg.head_dim() == 64 && cfg.ffn_dim() == 512 && Gpt2Config::xl().n_embd == 1600 && Gpt2Config::small().n_layer == 12, "Gpt2Config");
    Gpt2Weights gw = tiny_weights(cfg, 20260101);
    Gpt2Model model = Gpt2Model::from_weights(gw, cfg, reg);
    std::vector<uint32_t> prompt = {5, 17, 3, 96, 42, 8};
    GpuTensor logits = model.forward(prompt);
    CHECK(logits.shape() == std::vector<size_t>({prompt.size(), cfg.vocab_size}), "forward shape");
    std::vector<float> lg = logits.to_host();
    bool finite = true;
    for (float v : lg) finite = finite && std::isfinite(v);
    CHECK(finite, "forward finite");
    KvCache cache(model, 1, 32);
    CHECK(cache.is_empty(), "KvCache::is_empty");
    std::vector<float> lc = model.forward_cached(prompt, prompt.size(), cache).to_host();
    CHECK(cache.len() == prompt.size(), "KvCache::len");
    double dmax = 0;
    for (size_t i = 0; i < lg.size(); ++i) dmax = std::fmax(dmax, std::fabs((double)lg[i] - lc[i]));
    CHECK(dmax < 1e-2, "forward_cached == forward");
    std::vector<uint32_t> g1 = model.generate(prompt, 8, 0), g2 = model.generate_cached(prompt, 8, 0);
    CHECK(g1.size() == prompt.size() + 8 && g1 == g2, "generate == generate_cached");
    // the first generated token is the argmax of forward's last row
    size_t best = 0;
    for (size_t v = 1; v < cfg.vocab_size; ++v)
        if (lg[(prompt.size() - 1) * cfg.vocab_size + v] > lg[(prompt.size() - 1) * cfg.vocab_size + best]) best = v;
    CHECK(g1[prompt.size()] == best, "greedy pick");
    SimpleRng r1(7), r2(7);
    CHECK(model.generate_cached_sampling(prompt, 6, 5, 0.8f, r1) == model.generate_cached_sampling(prompt, 6, 5, 0.8f, r2), "sampling is seeded");
    CHECK(model.forward_early_exit(prompt, 2.0f).second == (int32_t)cfg.n_layer, "forward_early_exit never confident");

    Int4Gpt2Model m4 = Gpt2Model::from_weights_int4(gw, cfg, 128, reg);
    CHECK(m4.group_size() == 128 && m4.quantized_memory_bytes() > 0 && model.quantized_memory_bytes() == 0, "quantized_memory_bytes");
    std::vector<uint32_t> p2 = prompt;
    p2.insert(p2.end(), {1, 2, 3, 4, 5, 6});
    std::vector<size_t> lens;
    std::vector<uint32_t> both = m4.generate_batch(p2, 2, 6, 5, &lens);
    std::vector<uint32_t> first = m4.generate(prompt, 5, 0);
    CHECK(lens.size() == 2 && lens[0] == 11 && std::vector<uint32_t>(both.begin(), both.begin() + 11) == first, "generate_batch row 0 == generate");
    CHECK(throws_code(B200NN_ERR_DIM, [&] { std::vector<uint32_t> far(40, 1); model.forward(far); }), "forward beyond n_positions");
    // ---- DecodeSession: the batched loop in pieces == generate_batch --------------------------------
    DecodeSession sess(m4, 2, 16);
    sess.prefill(p2, 6);
    sess.step(4);
    std::vector<std::vector<uint32_t>> st = sess.tokens();
    CHECK(sess.position() == 6 + 4 && st.size() == 2 && st[0].size() == 5, "DecodeSession position / token count");
    CHECK(st[0] == std::vector<uint32_t>(both.begin() + 6, both.begin() + 11) &&
              st[1] == std::vector<uint32_t>(both.begin() + 11 + 6, both.begin() + 22),
          "DecodeSession tokens == generate_batch");

    // ---- TransformerBlock == its parts composed through the layer classes --------------------------
    const size_t d = 128;
    BlockWeights bw;
    bw.ln_1_weight = normal(31, d, 0.1f); for (float &v : bw.ln_1_weight) v += 1.0f;
    bw.ln_1_bias = normal(32, d, 0.05f);
    bw.attn_qkv_weight = normal(33, 3 * d * d, 0.06f); bw.attn_qkv_bias = normal(34, 3 * d, 0.02f);
    bw.attn_out_weight = normal(35, d * d, 0.06f);     bw.attn_out_bias = normal(36, d, 0.02f);
    bw.ln_2_weight = normal(37, d, 0.1f); for (float &v : bw.ln_2_weight) v += 1.0f;
    bw.ln_2_bias = normal(38, d, 0.05f);
    bw.ffn_up_weight = normal(39, 4 * d * d, 0.06f);   bw.ffn_up_bias = normal(40, 4 * d, 0.02f);
    bw.ffn_down_weight = normal(41, 4 * d * d, 0.06f); bw.ffn_down_bias = normal(42, d, 0.02f);
    Gpt2Config bc = cfg;
    TransformerBlock block(bw, bc, reg);
    GpuTensor bx = GpuTensor::from_host(normal(43, 3 * d, 1.0f), {3, d}, reg);
    std::vector<float> by = block.forward(bx).to_host();
    LayerNorm ln1(bw.ln_1_weight, bw.ln_1_bias, bc.layer_norm_epsilon, reg), ln2(bw.ln_2_weight, bw.ln_2_bias, bc.layer_norm_epsilon, reg);
    MultiHeadAttention mha(bw.attn_qkv_weight, bw.attn_qkv_bias, bw.attn_out_weight, bw.attn_out_bias, d, bc.n_head, reg);
    Linear up(bw.ffn_up_weight, &bw.ffn_up_bias, d, 4 * d, reg), down(bw.ffn_down_weight, &bw.ffn_down_bias, 4 * d, d, reg);
    GpuTensor res1 = ops::elementwise_add_out(bx, mha.forward_causal(ln1.forward(bx)), reg);
    GpuTensor res2 = ops::elementwise_add_out(res1, down.forward(up.forward_auto_fused(ln2.forward(res1), Activation::Gelu)), reg);
    std::vector<float> composed = res2.to_host();
    double bmax = 0;
    for (size_t i = 0; i < by.size(); ++i) bmax = std::fmax(bmax, std::fabs((double)by[i] - composed[i]));
    CHECK(by.size() == 3 * d && bmax < 5e-3, "TransformerBlock::forward == LN, attention, MLP composed");
    Int4TransformerBlock block4(bw, bc, reg, 128);
    std::vector<float> by4 = block4.forward(bx).to_host();
    double b4max = 0;
    for (size_t i = 0; i < by4.size(); ++i) b4max = std::fmax(b4max, std::fabs((double)by4[i] - by[i]));
    CHECK(b4max > 0 && b4max < 0.5, "Int4TransformerBlock::forward close to the f32 block");

    CHECK(reg->device_error() == 0, "device error word");

    std::printf("%s %d checks, %d failed\n", g_failed ? "FAILED" : "OK", g_checks, g_failed);
    return g_failed ? 1 : 0;
}
