"""CPU tests: the C oracle against the reference's known-answer vectors, against an independent
numpy implementation, and against the committed golden fixtures."""
import json
import os

import numpy as np
import pytest

import np_ref
from oracle import oracle

HERE = os.path.dirname(os.path.abspath(__file__))
KATS = json.load(open(os.path.join(HERE, "golden", "reference_kats.json")))


def _formula(expr, n, **env):
    return np.array([eval(expr, {}, dict(i=i, **env)) for i in range(n)], dtype=np.float32)


# ---- reference known-answer vectors ---------------------------------------------------------
def test_pack_int8_kat():
    for c in KATS["pack_int8_to_u32"]:
        assert oracle.pack_int8_to_u32(c["values"]).tolist() == c["packed"]


def test_quantize_int8_kat():
    for c in KATS["quantize_int8_per_tensor"]:
        q, s = oracle.quantize_int8_per_tensor(c["data"])
        assert abs(s - c["scale"]) < c["scale_tol"]
        assert q[: len(c["q_prefix"])].tolist() == c["q_prefix"]


def test_int4_per_group_kat():
    for c in KATS["quantize_int4_per_group"]:
        packed, scales = oracle.quantize_int4_per_group(c["data"], c["group"])
        assert packed.size == c["n_packed"] and scales.size == c["n_scales"]
        for i, x in enumerate(c["data"]):
            assert abs(oracle.unpack_int4(packed[0], i) * scales[0] - x) < scales[0] + 1e-6


def test_quantize_weight_int4_kat():
    for c in KATS["quantize_weight_int4"]:
        k, n, g = c["k"], c["n"], c["group"]
        w = _formula(c["weight_formula"], k * n)
        packed, scales = oracle.quantize_weight_int4(w, k, n, g)
        assert packed.size == c["n_packed"] and scales.size == c["n_scales"]
        for col in range(n):
            for ki in range(k):
                q = oracle.unpack_int4(packed[ki // 8, col], ki % 8)
                assert abs(q * scales[ki // g, col] - w[ki * n + col]) < scales[ki // g, col] + 1e-6


def test_unpack_int4_kat():
    for c in KATS["unpack_int4"]:
        word = 0
        for i, v in enumerate(c["values"]):
            word |= ((v + 8) & 0xF) << (4 * i)
        assert [oracle.unpack_int4(word, i) for i in range(8)] == c["values"]


def test_cpu_ref_kats():
    mm, sm, att = KATS["cpu_ref"]
    np.testing.assert_allclose(oracle.matmul(mm["a"], mm["b"], 2, 2, 2).ravel(), mm["c"], atol=1e-6)
    out = oracle.softmax(sm["input"], sm["rows"], sm["cols"]).reshape(sm["rows"], sm["cols"])
    assert np.all(np.abs(out.sum(1) - 1.0) < sm["row_sum_tol"])
    seq, d = att["seq"], att["d"]
    q = _formula(att["q_formula"], seq * d)
    v = _formula(att["v_formula"], seq * d)
    o = oracle.attention(q, q, v, seq, d)
    np.testing.assert_allclose(o[0], v[:d], atol=1e-6)


def test_gelu_kat():
    for x, y in KATS["gelu_tanh"]["points"]:
        assert abs(oracle.lib().orc_gelu_tanh(x) - y) < KATS["gelu_tanh"]["tol"]


def test_reference_pattern_linear_and_layernorm():
    lin1, lin2, ln = KATS["patterns"]
    for c in (lin1, lin2):
        b, k, n = c["batch"], c["in"], c["out"]
        w = _formula(c["weight_formula"], n * k).reshape(n, k)  # [out,in]
        bias = _formula(c["bias_formula"], n)
        x = _formula(c["input_formula"], b * k).reshape(b, k)
        got = oracle.matmul(x, np.ascontiguousarray(w.T), b, k, n) + bias
        ref = x.astype(np.float64) @ w.astype(np.float64).T + bias
        assert np.abs(got - ref).max() < 1e-5
    b, d = ln["batch"], ln["d"]
    g = _formula(ln["gamma_formula"], d)
    be = _formula(ln["beta_formula"], d)
    x = _formula(ln["input_formula"], b * d, batch=b, d=d).reshape(b, d)
    got = oracle.layer_norm(x, g, be, ln["eps"])
    assert np.abs(got - np_ref.layer_norm(x, g, be, ln["eps"])).max() < 1e-6


# ---- oracle vs independent numpy --------------------------------------------------------------
@pytest.mark.parametrize("k,n,group", [(8, 4, 128), (64, 24, 32), (256, 40, 128), (192, 17, 128)])
def test_quantizer_matches_numpy(k, n, group):
    rng = np.random.default_rng(k * 1000 + n)
    w = (rng.standard_normal((k, n)) * 0.02).astype(np.float32)
    w[:, 0] = 0.0  # all-zero group -> scale 1.0 branch
    p1, s1 = oracle.quantize_weight_int4(w, k, n, group)
    p2, s2 = np_ref.quantize_weight_int4(w, k, n, group)
    assert np.array_equal(p1, p2) and np.array_equal(s1, s2)
    assert np.all(s1[:, 0] == 1.0)
    np.testing.assert_array_equal(oracle.dequant_weight_int4(p1, s1, k, n, group), np_ref.dequant(p1, s1, k, n, group))


def test_rounding_is_half_away_from_zero():
    # scale = 7/7 = 1: 0.5 -> 1, -0.5 -> -1, 2.5 -> 3, -2.5 -> -3 (Rust f32::round), clamp at -8 / 7
    data = np.array([7.0, 0.5, -0.5, 2.5, -2.5, 1.5, -7.0, 0.0], dtype=np.float32)
    packed, scales = oracle.quantize_int4_per_group(data, 128)
    assert scales[0] == 1.0
    assert [oracle.unpack_int4(packed[0], i) for i in range(8)] == [7, 1, -1, 3, -3, 2, -7, 0]


@pytest.mark.parametrize("m,k,n", [(1, 64, 16), (3, 128, 40), (5, 192, 9)])
def test_int4_linear_variants(m, k, n):
    from b200nn import synth
    packed, scales, x, q = synth.int4_linear_case(7 + m, m, k, n, 128)
    bias = np.linspace(-1, 1, n).astype(np.float32)
    ref = x.astype(np.float64) @ (q * np.repeat(scales, 128, 0)[:k].astype(np.float64)) + bias
    y64 = oracle.int4_linear(x, packed, scales, bias, m, n, k, 128, f64=True)
    y32 = oracle.int4_linear(x, packed, scales, bias, m, n, k, 128, f64=False)
    assert np.abs(y64 - ref).max() < 1e-5
    assert np.abs(y32 - ref).max() < 1e-4


TINY = dict(n_layer=2, n_embd=128, n_head=2, vocab_size=211, n_positions=32, layer_norm_epsilon=1e-5)


def _tiny_weights(seed=5):
    from b200nn import synth
    from b200nn.gpt2 import Gpt2Config
    return synth.gpt2_weights(Gpt2Config(**TINY), base_seed=seed, std=0.08, random_ln=True)


@pytest.mark.parametrize("flags,gelu,kvh", [(0, "tanh", False), (oracle.GELU_SIGMOID, "sigmoid", False),
                                            (oracle.KV_FP16, "tanh", True)])
def test_model_forward_matches_numpy(flags, gelu, kvh):
    w = _tiny_weights()
    toks = np.array([3, 17, 200, 5, 5, 99, 0, 42, 7], dtype=np.uint32)
    got = oracle.Model(TINY, w).forward(toks, flags=flags)
    ref = np_ref.gpt2_forward(TINY, w, toks, gelu=gelu, kv_fp16=kvh)
    assert np.abs(got - ref).max() < 2e-5


def test_cached_generation_equals_uncached():
    # the reference's pass criterion for its KV cache: same tokens as the uncached loop
    # (crates/test/gpu-test-harness/src/tests_inference.rs:6166-6177)
    w = _tiny_weights(11)
    m = oracle.Model(TINY, w)
    prompt = np.array([1, 2, 3, 4, 5], dtype=np.uint32)
    a, la = m.generate(prompt, 12, want_logits=True)
    b, lb = m.generate_cached(prompt, 12, want_logits=True)
    assert np.array_equal(a, b)
    assert np.abs(la - lb).max() < 1e-5
    assert a.size == prompt.size + 12


def test_eos_and_argmax_rules():
    w = _tiny_weights(3)
    # make token 50256 unreachable in the tiny vocab: EOS flag must not change anything
    m = oracle.Model(TINY, w)
    prompt = np.array([9, 8, 7], dtype=np.uint32)
    a, _ = m.generate_cached(prompt, 6)
    b, _ = m.generate_cached(prompt, 6, flags=oracle.STOP_ON_EOS | oracle.ARGMAX_LAST)
    assert np.array_equal(a, b)  # no ties in generic position, no EOS in a 211-token vocabulary


def test_lm_head_override_matches_tied():
    w = _tiny_weights(4)
    toks = np.array([4, 5, 6, 7], dtype=np.uint32)
    tied = oracle.Model(TINY, w).forward(toks)
    w2 = dict(w)
    w2["lm_head"] = np.ascontiguousarray(w["wte"].T)
    assert np.abs(oracle.Model(TINY, w2).forward(toks) - tied).max() < 1e-6


def test_mha_matches_model_attention():
    rng = np.random.default_rng(0)
    H, dh, past, nq = 3, 64, 5, 4
    cap = past + nq
    q = rng.standard_normal((nq, H * dh)).astype(np.float32)
    kc = rng.standard_normal((H, cap, dh)).astype(np.float32)
    vc = rng.standard_normal((H, cap, dh)).astype(np.float32)
    got = oracle.mha(q, kc, vc, H, dh, nq, past, cap)
    for h in range(H):
        for i in range(nq):
            s = kc[h, : past + i + 1].astype(np.float64) @ q[i, h * dh:(h + 1) * dh].astype(np.float64) / 8.0
            p = np.exp(s - s.max())
            p /= p.sum()
            ref = p @ vc[h, : past + i + 1].astype(np.float64)
            assert np.abs(got[i, h * dh:(h + 1) * dh] - ref).max() < 1e-5


# ---- committed golden fixtures -----------------------------------------------------------------
def test_golden_fixture():
    path = os.path.join(HERE, "golden", "tiny_gpt2_golden.npz")
    g = np.load(path)
    w = _tiny_weights(int(g["seed"]))
    m = oracle.Model(TINY, w)
    np.testing.assert_allclose(m.forward(g["tokens"]), g["logits"], atol=1e-6)
    toks, _ = m.generate_cached(g["tokens"][:5], 8)
    assert np.array_equal(toks, g["generated"])
    p, s = oracle.quantize_weight_int4(w["h.0.mlp.c_fc.weight"], 128, 512, 128)
    assert np.array_equal(p, g["fc_packed"]) and np.array_equal(s, g["fc_scales"])
    # data-dependent decoding
    rng = oracle.SimpleRng(7)
    assert np.array_equal(np.array([rng.next_f32() for _ in range(8)], np.float32), g["rng_draws"])
    sampled, _, _ = m.generate_cached_sampling(g["tokens"][:5], 10, 20, 0.8, oracle.SimpleRng(2026))
    assert np.array_equal(sampled, g["sampled"])
    np.testing.assert_allclose(m.forward_early_exit(g["tokens"], 2.0)[2], g["probe_conf"], rtol=1e-5)
    toks, layers, _, _ = m.generate_cached_early_exit(g["tokens"][:5], 10, float(g["ee_threshold"]))
    assert np.array_equal(toks, g["ee_tokens"]) and np.array_equal(layers, g["ee_layers"])


def test_sampling_and_early_exit_reduce_to_greedy():
    """Limits of the dynamic loops (gpt2.rs:785-977): k = 1 samples the maximum; a threshold nothing
    reaches runs every layer and equals the cached greedy loop with the model's last-maximum tie rule;
    threshold 0 leaves after the first block at every decode step, the prefill excepted."""
    from b200nn import synth
    w = _tiny_weights(33)
    m = oracle.Model(TINY, w)
    prompt = synth.token_ids(5, (6,), TINY["vocab_size"])
    greedy, _ = m.generate_cached(prompt, 9)
    k1, _, _ = m.generate_cached_sampling(prompt, 9, 1, 0.7, oracle.SimpleRng(3))
    assert np.array_equal(k1, greedy)
    never, layers, _, _ = m.generate_cached_early_exit(prompt, 9, 2.0)
    assert np.array_equal(never, m.generate_cached(prompt, 9, flags=oracle.ARGMAX_LAST)[0])
    assert layers.tolist() == [TINY["n_layer"]] * 9
    _, always, _, _ = m.generate_cached_early_exit(prompt, 9, 0.0)
    assert always.tolist() == [TINY["n_layer"]] + [1] * 8
    full = m.forward(prompt)
    lg, used, conf = m.forward_early_exit(prompt, 2.0)
    assert used == TINY["n_layer"] and np.allclose(lg, full, atol=1e-6) and conf.size == TINY["n_layer"] - 1
    lg0, used0, _ = m.forward_early_exit(prompt, 0.0)
    assert used0 == 1 and not np.allclose(lg0, full, atol=1e-3)
    assert oracle.softmax_max_prob(lg0[-1]) == pytest.approx(conf[0], rel=1e-5)
