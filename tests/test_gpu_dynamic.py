"""GPU parity of the data-dependent decoding entry points (gpt2.rs:785-1058: top-k sampling, early exit
by confidence) against the oracle's restatement on identical seeded weights, prompts and RNG seeds.
Draws and exit decisions are compared exactly wherever the oracle reports that the decision was not
borderline (a draw within 3e-3 of a boundary of the cumulative distribution or a k-th/k+1-th logit gap
below 3e-3, a confidence within 2 % of the threshold, a top-2 logit gap below 1e-3)."""
import numpy as np
import pytest

import b200nn
import np_ref
from b200nn import Gpt2Config, Gpt2Model, Int4Gpt2Model, SimpleRng, synth
from oracle import oracle

pytestmark = pytest.mark.gpu


def _mini(n_layer=4, d=128, vocab=331, npos=64):
    return Gpt2Config(n_layer=n_layer, n_embd=d, n_head=d // 64, vocab_size=vocab, n_positions=npos)


def _models(reg, int4, seed, **kw):
    cfg = _mini(**kw)
    w = synth.gpt2_weights(cfg, base_seed=seed, std=0.1, random_ln=True)
    if not int4:  # the device KV cache is fp16 for both model families: the oracle rounds K and V alike
        return cfg, Gpt2Model.from_weights(w, cfg, reg), oracle.Model(cfg.as_dict(), w), oracle.KV_FP16
    m = Int4Gpt2Model.from_weights(w, cfg, reg)
    w2 = dict(w)
    for i in range(cfg.n_layer):
        for which, nm in enumerate(["attn.c_attn.weight", "attn.c_proj.weight", "mlp.c_fc.weight", "mlp.c_proj.weight"]):
            p, s, K, N = m.get_int4(i, which)
            w2[f"h.{i}.{nm}"] = oracle.dequant_weight_int4(p, s, K, N, m.group_size())
    return cfg, m, oracle.Model(cfg.as_dict(), w2), oracle.KV_FP16


@pytest.mark.parametrize("int4", [False, True])
def test_generate_cached_sampling(reg, int4):
    cfg, m, om, oflags = _models(reg, int4, 101)
    prompt = synth.token_ids(21, (9,), cfg.vocab_size)
    for seed, k, temp in [(1, 40, 1.0), (2, 5, 0.7), (12345, 331, 1.3), (7, 1, 1.0)]:
        got = m.generate_cached_sampling(prompt, 14, k, temp, SimpleRng(seed))
        ref, lg, margin = om.generate_cached_sampling(prompt, 14, k, temp, oracle.SimpleRng(seed), flags=oflags)
        assert np.array_equal(got[:9], prompt)
        for i in range(9, min(len(got), len(ref))):
            if got[i] != ref[i]:
                row = np.sort(lg[i - 9] / np.float32(max(temp, 1e-8)))[::-1]
                kth_gap = row[k - 1] - row[k] if k < row.size else 1.0
                assert margin[i - 9] < 3e-3 or kth_gap < 3e-3, (seed, i, margin[i - 9], kth_gap)
                break
        else:
            assert len(got) == len(ref)
    # k = 1 is greedy decoding
    assert np.array_equal(m.generate_cached_sampling(prompt, 10, 1, 1.0, SimpleRng(3)), m.generate_cached(prompt, 10, flags=0))
    # one draw per generated token
    r = SimpleRng(77)
    out = m.generate_cached_sampling(prompt, 6, 10, 1.0, r)
    r2 = SimpleRng(77)
    for _ in range(len(out) - 9):
        r2.next_f32()
    assert r.state.value == r2.state.value
    with pytest.raises(b200nn.NnError):
        m.generate_cached_sampling(prompt, 6, 0, 1.0, SimpleRng(1))
    with pytest.raises(b200nn.NnError):
        m.generate_cached_sampling(prompt, 60, 5, 1.0, SimpleRng(1))  # beyond n_positions
    assert reg.device_error() == 0


def test_sampling_stops_before_eos(reg):
    cfg = Gpt2Config(n_layer=1, n_embd=64, n_head=1, vocab_size=50257, n_positions=32)
    w = synth.gpt2_weights(cfg, base_seed=71, std=0.02)
    w["wte"] = np.array(w["wte"], np.float32).reshape(50257, 64).copy()
    prompt = np.array([5, 6, 7], dtype=np.uint32)
    lg = oracle.Model(cfg.as_dict(), w).generate_cached(prompt, 2, want_logits=True)[1]
    target = int(np.argmax(lg[1]))
    w["wte"][50256] = w["wte"][target] * 1.5  # EOS beats `target` at the second generated token
    m = Gpt2Model.from_weights(w, cfg, reg)
    got = m.generate_cached_sampling(prompt, 6, 1, 1.0, SimpleRng(5))
    ref = oracle.Model(cfg.as_dict(), w).generate_cached(prompt, 6, flags=oracle.STOP_ON_EOS)[0]
    assert np.array_equal(got, ref) and 50256 not in got.tolist() and len(got) < 9


def test_forward_features_embedding_table_and_profiled(reg):
    """forward_features (gpt2.rs:570-581), embedding_table (584-586), forward_profiled (529-568)."""
    cfg = _mini(n_layer=3)
    w = synth.gpt2_weights(cfg, base_seed=107, std=0.1, random_ln=True)
    m = Gpt2Model.from_weights(w, cfg, reg)
    toks = synth.token_ids(24, (13,), cfg.vocab_size)
    logits = m.forward(toks).to_host()
    wte_t, wpe_t = m.embedding_table()
    wte = np.asarray(w["wte"], np.float32).reshape(cfg.vocab_size, cfg.n_embd)
    assert wte_t.shape() == (cfg.vocab_size, cfg.n_embd) and np.array_equal(wte_t.to_host(), wte)
    assert np.array_equal(wpe_t.to_host(), np.asarray(w["wpe"], np.float32).reshape(cfg.n_positions, cfg.n_embd))
    feats = m.forward_features(toks)
    assert feats.shape() == (13, cfg.n_embd)
    # the tied LM head applied by hand to the features gives the model's logits
    # (the model's head multiplies fp16 copies of both operands for more than four rows)
    by_hand = feats.to_host().astype(np.float64) @ wte.astype(np.float64).T
    assert np.abs(by_hand - logits).max() < 2e-2 and np_ref.rel_rms(logits, by_hand) < 5e-4
    # and the features are the oracle's last hidden state: check through the oracle's logits
    ref = oracle.Model(cfg.as_dict(), w).forward(toks, flags=oracle.KV_FP16)
    assert np.abs(by_hand - ref).max() < 2e-2 and np_ref.rel_rms(by_hand.astype(np.float32), ref) < 1e-3
    lg, timings = m.forward_profiled(toks)
    assert [n for n, _ in timings] == ["embedding", "block_0", "block_1", "block_2", "ln_f", "lm_head"]
    assert all(t > 0 for _, t in timings)
    # run to run the residual GEMMs add their K splits in a different order: last bits move
    assert np.abs(lg.to_host() - logits).max() < 2e-3
    assert np.abs(m.forward_auto_fused(toks).to_host() - logits).max() < 2e-3
    with pytest.raises(b200nn.NnError):
        m.forward_features(np.zeros(cfg.n_positions + 1, np.uint32))
    del wte_t, wpe_t  # views on the model's buffers: the model stays usable
    assert np.abs(m.forward(toks).to_host() - logits).max() < 2e-3


@pytest.mark.parametrize("int4", [False, True])
def test_forward_early_exit(reg, int4):
    cfg, m, om, oflags = _models(reg, int4, 103)
    toks = synth.token_ids(22, (17,), cfg.vocab_size)
    _, _, conf = om.forward_early_exit(toks, 2.0, flags=oflags)  # never exits: every probe's confidence
    assert np.isfinite(conf).all() and conf.size == cfg.n_layer - 1
    cases = [(0.0, 1), (2.0, cfg.n_layer)]
    for layer in range(1, cfg.n_layer):
        # block `layer` is the first to qualify for thresholds in (max of the earlier probes, its own probe]
        lo = float(conf[: layer - 1].max()) if layer > 1 else 0.0
        hi = float(conf[layer - 1])
        if hi - lo > 0.05 * hi:  # wide enough that f32-vs-f64 logits cannot move the decision
            cases.append(((hi + lo) / 2, layer))
    assert len(cases) >= 3
    for th, want in cases:
        ref, used, _ = om.forward_early_exit(toks, th, flags=oflags)
        assert used == want
        t, got_used = m.forward_early_exit(toks, th)
        assert got_used == used, (th, conf)
        got = t.to_host()
        assert np.abs(got - ref).max() < 2e-2 and np_ref.rel_rms(got, ref) < 1e-3
    full = m.forward(toks).to_host()
    # the residual GEMMs add their K splits in arrival order, so two runs differ in the last bits, which
    # the fp16 activations downstream then round differently
    assert np.abs(m.forward_early_exit(toks, 2.0)[0].to_host() - full).max() < 2e-3


@pytest.mark.parametrize("int4", [False, True])
def test_generate_cached_early_exit(reg, int4):
    cfg, m, om, oflags = _models(reg, int4, 105)
    prompt = synth.token_ids(23, (8,), cfg.vocab_size)
    # thresholds: never exit, always exit after the first block, and one in between taken from the
    # confidences the oracle meets (retried until no decision of the run is borderline)
    _, layers_never, _, _ = om.generate_cached_early_exit(prompt, 12, 2.0, flags=oflags)
    assert set(layers_never.tolist()) == {cfg.n_layer}
    conf = om.forward_early_exit(prompt, 2.0, flags=oflags)[2]  # the scale of this model's confidences
    mids = [float(np.median(conf)) * f for f in (1.0, 0.8, 1.25, 0.6, 1.6, 0.4, 2.5)]
    tested_mid = False
    for th in [2.0, 0.0] + mids:
        ref, ref_layers, lg, gap = om.generate_cached_early_exit(prompt, 12, th, flags=oflags)
        if th in mids and (gap < 0.02 * th or len(set(ref_layers[1:].tolist())) < 2 or tested_mid):
            continue
        tested_mid = tested_mid or th in mids
        got, got_layers = m.generate_cached_early_exit(prompt, 12, th)
        assert np.array_equal(got_layers, ref_layers), (th, got_layers, ref_layers)
        assert got_layers[0] == cfg.n_layer  # the prefill always runs every layer
        for i in range(8, min(len(got), len(ref))):
            if got[i] != ref[i]:
                row = np.sort(lg[i - 8])[::-1]
                assert row[0] - row[1] < 1e-3, (th, i)
                break
        else:
            assert len(got) == len(ref)
        if th == 0.0:
            assert set(got_layers[1:].tolist()) == {1}
    assert tested_mid, "no threshold gave a run with mixed depths: widen the list"
    # never exiting is the model's own cached greedy decoding (last maximum on ties)
    assert np.array_equal(m.generate_cached_early_exit(prompt, 12, 2.0)[0],
                          m.generate_cached(prompt, 12, flags=b200nn.ARGMAX_LAST))
    assert reg.device_error() == 0
