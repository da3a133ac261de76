"""GPU parity tests of the GPT-2 models (f32 and int4) against the f64 oracle on identical seeded
weights and token ids.  Tolerance is the path's: logits within 2e-2 max-abs and 1e-3 relative RMS;
greedy tokens identical except where the oracle's top-2 logit gap is below 1e-3."""
import numpy as np
import pytest

import b200nn
import np_ref
from b200nn import DecodeSession, Gpt2Config, Gpt2Model, Int4Gpt2Model, KvCache, synth
from oracle import oracle

pytestmark = pytest.mark.gpu

MAX_ABS, REL_RMS, TIE_GAP = 2e-2, 1e-3, 1e-3


@pytest.fixture
def one_k_split(reg):
    """Tests that compare two runs token for token: without K splits the residual GEMMs add in one fixed
    order (with splits the order of their `red.add` partials differs from run to run in the last bit, which
    can flip a near-tie)."""
    reg.set_tuning("tc_splits", 1)
    yield
    reg.set_tuning("tc_splits", 0)


def _mini(n_layer=2, d=128, vocab=331, npos=64):
    return Gpt2Config(n_layer=n_layer, n_embd=d, n_head=d // 64, vocab_size=vocab, n_positions=npos)


def _check_logits(got, ref):
    assert got.shape == ref.shape
    assert np.abs(got - ref).max() < MAX_ABS, np.abs(got - ref).max()
    assert np_ref.rel_rms(got, ref) < REL_RMS, np_ref.rel_rms(got, ref)


def _check_tokens(got, ref_tokens, ref_logits, prompt_len):
    """Tokens must match until the first step where the oracle itself had a near-tie."""
    n = min(len(got), len(ref_tokens))
    for i in range(prompt_len, n):
        if got[i] != ref_tokens[i]:
            row = np.sort(ref_logits[i - prompt_len])[::-1]
            assert row[0] - row[1] < TIE_GAP, f"token {i}: {got[i]} != {ref_tokens[i]}, gap {row[0] - row[1]}"
            return
    assert len(got) == len(ref_tokens)


def _int4_oracle_weights(model, cfg, w, quant_head):
    """The oracle runs f64 math on exactly the nibbles and fp16 scales the GPU model holds."""
    w2 = dict(w)
    names = ["attn.c_attn.weight", "attn.c_proj.weight", "mlp.c_fc.weight", "mlp.c_proj.weight"]
    for i in range(cfg.n_layer):
        for which, nm in enumerate(names):
            p, s, K, N = model.get_int4(i, which)
            w2[f"h.{i}.{nm}"] = oracle.dequant_weight_int4(p, s, K, N, model.group_size())
    if quant_head:
        p, s, K, N = model.get_int4(-1, 0)
        w2["lm_head"] = oracle.dequant_weight_int4(p, s, K, N, model.group_size())
    return w2


def test_f32_model_forward_and_generate(reg):
    cfg = _mini()
    w = synth.gpt2_weights(cfg, base_seed=31, std=0.08, random_ln=True)
    m = Gpt2Model.from_weights(w, cfg, reg)
    om = oracle.Model(cfg.as_dict(), w)
    toks = synth.token_ids(1, (24,), cfg.vocab_size)
    _check_logits(m.forward(toks).to_host(), om.forward(toks))
    prompt = toks[:6]
    ref, lg = om.generate(prompt, 10, want_logits=True)  # the uncached CPU loop of the reference
    _check_tokens(m.generate(prompt, 10), ref, lg, 6)
    _check_tokens(m.generate_cached(prompt, 10), ref, lg, 6)


@pytest.mark.parametrize("tc", [2, 1, 0])
def test_f32_model_tensor_core_and_fma_paths(reg, tc):
    """The f32 family beyond four rows: fp16 activations times the weight as fp16 hi + lo on the tensor
    cores (the default, `f32_tc` = 2), the weight rounded to fp16 (1), or the f32 FMA kernels (0), each
    against the f64 oracle.  768 wide,
    200 tokens: one full 128-row tile plus a tail, K tails of the 64-wide blocks in no Linear, vocabulary
    not a multiple of the 128-feature tile."""
    cfg = Gpt2Config(n_layer=2, n_embd=768, n_head=12, vocab_size=1031, n_positions=256)
    w = synth.gpt2_weights(cfg, base_seed=33, std=0.04, random_ln=True)
    om = oracle.Model(cfg.as_dict(), w)
    toks = synth.token_ids(5, (200,), cfg.vocab_size)
    ref = om.forward(toks, flags=oracle.KV_FP16)
    reg.set_tuning("f32_tc", tc)
    try:
        m = Gpt2Model.from_weights(w, cfg, reg)
        got = m.forward(toks).to_host()
        _check_logits(got, ref)
        if not tc:  # f32 products; the fp16 K/V cache and the fp16 probabilities of long rows remain
            assert np_ref.rel_rms(got, ref) < 2e-4
        # eight sequences decode together: more than four rows, so the Linears of every step take the same path
        prompts = synth.token_ids(6, (8, 12), cfg.vocab_size)
        out, lens = m.generate_batch(prompts, 8)
        for b in (0, 3, 7):
            r, lg = om.generate_cached(prompts[b], 8, flags=oracle.KV_FP16, want_logits=True)
            _check_tokens(out[b][: lens[b]], r, lg, 12)
    finally:
        reg.set_tuning("f32_tc", -1)
    assert reg.device_error() == 0


def test_f32_model_sigmoid_gelu_flag(reg):
    cfg = _mini(n_layer=1)
    w = synth.gpt2_weights(cfg, base_seed=32, std=0.08)
    toks = synth.token_ids(2, (9,), cfg.vocab_size)
    m = Gpt2Model.from_weights(w, cfg, reg, flags=b200nn.GELU_SIGMOID)
    _check_logits(m.forward(toks).to_host(), oracle.Model(cfg.as_dict(), w).forward(toks, flags=oracle.GELU_SIGMOID))


@pytest.mark.parametrize("quant_head", [False, True])
def test_int4_model_forward_and_generate(reg, quant_head):
    cfg = _mini(n_layer=3, d=192, vocab=523)
    w = synth.gpt2_weights(cfg, base_seed=41, std=0.05, random_ln=True)
    flags = b200nn.QUANT_LM_HEAD if quant_head else 0
    m = Int4Gpt2Model.from_weights(w, cfg, reg, flags=flags, group_size=128)
    assert m.quantized_memory_bytes() > 0
    om = oracle.Model(cfg.as_dict(), _int4_oracle_weights(m, cfg, w, quant_head))
    toks = synth.token_ids(3, (20,), cfg.vocab_size)
    _check_logits(m.forward(toks).to_host(), om.forward(toks, flags=oracle.KV_FP16))
    prompt = toks[:7]
    ref, lg = om.generate_cached(prompt, 12, flags=oracle.KV_FP16, want_logits=True)
    _check_tokens(m.generate(prompt, 12), ref, lg, 7)


def test_int4_quantisation_matches_oracle_rule(reg):
    cfg = _mini(n_layer=1)
    w = synth.gpt2_weights(cfg, base_seed=43, std=0.02)
    m = Int4Gpt2Model.from_weights(w, cfg, reg)
    p, s, K, N = m.get_int4(0, 2)
    po, so = oracle.quantize_weight_int4(w["h.0.mlp.c_fc.weight"], K, N, 128)
    assert np.array_equal(p, po) and np.array_equal(s, oracle.f16_round(so))


def test_forward_cached_batched_equals_forward(reg):
    cfg = _mini()
    w = synth.gpt2_weights(cfg, base_seed=51, std=0.08)
    m = Gpt2Model.from_weights(w, cfg, reg)
    toks = synth.token_ids(4, (3, 10), cfg.vocab_size)
    cache = KvCache(m, batch=3, capacity=16)
    assert cache.is_empty()
    # f32 FMA Linears (0): the two ways differ by accumulation order only; default: both carry the
    # rounding of fp16 activations, of different row sets
    for mode, tol in ((0, 1e-3), (-1, 4e-3)):
        reg.set_tuning("f32_tc", mode)
        try:
            cache.reset()
            first = m.forward_cached(toks[:, :6], 6, cache).to_host().reshape(3, 6, -1)
            assert cache.len() == 6
            rest = m.forward_cached(toks[:, 6:], 4, cache).to_host().reshape(3, 4, -1)
            assert cache.len() == 10
            for b in range(3):
                full = m.forward(toks[b]).to_host()
                assert np.abs(first[b] - full[:6]).max() < tol
                assert np.abs(rest[b] - full[6:]).max() < tol
        finally:
            reg.set_tuning("f32_tc", -1)
    with pytest.raises(b200nn.NnError):  # capacity 16 exceeded
        m.forward_cached(toks[:, :7], 7, cache)
    cache.reset()
    assert cache.len() == 0


def test_generate_batch_equals_single_and_session(reg, one_k_split):
    cfg = _mini(n_layer=2, d=128, vocab=401)
    w = synth.gpt2_weights(cfg, base_seed=61, std=0.08, random_ln=True)
    m = Int4Gpt2Model.from_weights(w, cfg, reg)
    prompts = synth.token_ids(5, (5, 8), cfg.vocab_size)
    out, lens = m.generate_batch(prompts, 9)
    assert out.shape == (5, 17) and np.all(lens == 17)
    om = oracle.Model(cfg.as_dict(), _int4_oracle_weights(m, cfg, w, False))
    for b in range(5):
        single = m.generate(prompts[b], 9, flags=0)
        ref, lg = om.generate_cached(prompts[b], 9, flags=oracle.KV_FP16, want_logits=True)
        _check_tokens(single, ref, lg, 8)
        _check_tokens(out[b], ref, lg, 8)
    # the session API is the same loop in pieces (one eager step, then CUDA-graph replays)
    s = DecodeSession(m, batch=5, capacity=17)
    s.prefill(prompts)
    s.step(3)
    s.step(5)
    assert s.position() == 16
    assert np.array_equal(s.tokens(), out[:, 8:])
    lg = s.logits()
    assert lg.shape == (5, cfg.vocab_size) and np.isfinite(lg).all()
    assert np.array_equal(lg.argmax(1).astype(np.uint32), out[:, -1])
    t, nbytes = (lambda s2: (s2.prefill(prompts), s2.profile_step())[1])(DecodeSession(m, batch=5, capacity=17))
    assert set(t) == set(b200nn.PROF_NAMES) and t["linear"] > 0 and nbytes > 0
    assert reg.device_error() == 0


def test_int4_prefill_attention_tensor_core_long_sequences(reg):
    """The tensor-core prefill attention (fp16 activations) over several 128-query and 128-key tiles:
    a 300-token forward and a cached forward in two uneven pieces (past = 150, not a tile multiple),
    each against the oracle; and the CUDA-core kernel as a second opinion."""
    cfg = _mini(n_layer=2, d=128, vocab=257, npos=320)
    w = synth.gpt2_weights(cfg, base_seed=65, std=0.08, random_ln=True)
    m = Int4Gpt2Model.from_weights(w, cfg, reg)
    om = oracle.Model(cfg.as_dict(), _int4_oracle_weights(m, cfg, w, False))
    toks = synth.token_ids(8, (2, 300), cfg.vocab_size)
    refs = [om.forward(toks[b], flags=oracle.KV_FP16) for b in range(2)]
    full = m.forward(toks[0]).to_host()
    _check_logits(full, refs[0])
    cache = KvCache(m, batch=2, capacity=304)
    first = m.forward_cached(toks[:, :150], 150, cache).to_host().reshape(2, 150, -1)
    rest = m.forward_cached(toks[:, 150:], 150, cache).to_host().reshape(2, 150, -1)
    for b in range(2):
        _check_logits(first[b], refs[b][:150])
        _check_logits(rest[b], refs[b][150:])
    reg.set_tuning("attn_tc", 0)
    try:
        simt = m.forward(toks[0]).to_host()
    finally:
        reg.set_tuning("attn_tc", 1)
    _check_logits(simt, refs[0])
    assert np.abs(simt - full).max() < 5e-3
    assert reg.device_error() == 0


def test_prefill_attention_tensor_core_seq_1024_12_heads(reg):
    """GPT-2 Small's attention shape at the longest context: 12 heads, 1024 tokens (8 query tiles x up to
    8 key tiles per block), two sequences in one cached forward, against the oracle."""
    cfg = Gpt2Config(n_layer=1, n_embd=768, n_head=12, vocab_size=211, n_positions=1024)
    w = synth.gpt2_weights(cfg, base_seed=66, std=0.05, random_ln=True)
    m = Int4Gpt2Model.from_weights(w, cfg, reg)
    om = oracle.Model(cfg.as_dict(), _int4_oracle_weights(m, cfg, w, False))
    toks = synth.token_ids(10, (2, 1024), cfg.vocab_size)
    cache = KvCache(m, batch=2, capacity=1024)
    got = m.forward_cached(toks, 1024, cache).to_host().reshape(2, 1024, -1)
    for b in range(2):
        _check_logits(got[b], om.forward(toks[b], flags=oracle.KV_FP16))
    assert reg.device_error() == 0


def test_decode_attention_streaming_kernel_many_sequences(reg):
    """Enough (sequence, head) pairs to take the TMA-fed decode-attention kernel: 1800 sequences x 2
    heads, contexts 38..42 (not multiples of the 32-row stage).  Checked against the oracle on a few
    sequences and against the plain-load kernel on all of them."""
    cfg = _mini(n_layer=2, d=128, vocab=257, npos=48)
    w = synth.gpt2_weights(cfg, base_seed=67, std=0.08, random_ln=True)
    m = Int4Gpt2Model.from_weights(w, cfg, reg)
    om = oracle.Model(cfg.as_dict(), _int4_oracle_weights(m, cfg, w, False))
    B, P, N = 1800, 37, 5
    prompts = synth.token_ids(9, (B, P), cfg.vocab_size)

    def run():
        s = DecodeSession(m, batch=B, capacity=P + N + 1)
        s.prefill(prompts)
        s.step(1)      # eager
        s.step(N - 2)  # captured and replayed
        return s.tokens(), s.logits()

    tok_s, lg_s = run()
    reg.set_tuning("attn_stream", 0)
    try:
        tok_p, lg_p = run()
    finally:
        reg.set_tuning("attn_stream", 1)
    assert reg.device_error() == 0
    assert np.abs(lg_s - lg_p).max() < 2e-3
    assert (tok_s != tok_p).mean() < 0.01  # near-ties only
    for b in (0, 1, 777, B - 1):
        ref, lg = om.generate_cached(prompts[b], N, flags=oracle.KV_FP16, want_logits=True)
        _check_tokens(np.concatenate([prompts[b], tok_s[b]]), ref, lg, P)
    # a second session right away: the kernel's work counters must be back at zero
    tok_again, _ = run()
    assert (tok_again != tok_s).mean() < 0.01  # equal up to near-ties flipped by the order of the split-K additions
    # the optional half-item hand-out at the end of the grid (two records merged through scratch)
    reg.set_tuning("attn_split_items", 700)
    try:
        tok_h, lg_h = run()
    finally:
        reg.set_tuning("attn_split_items", 0)
    assert np.abs(lg_h - lg_s).max() < 2e-3
    assert (tok_h != tok_s).mean() < 0.01
    assert reg.device_error() == 0
    # the 16-warp shape of the block (16-row stages; by default only from 2.5 pairs per warp of its grid)
    reg.set_tuning("attn_stream_wide_min10", 1)
    reg.set_tuning("attn_stream_min10", 5)
    try:
        tok_w, lg_w = run()
    finally:
        reg.set_tuning("attn_stream_wide_min10", 25)
        reg.set_tuning("attn_stream_min10", 20)
    assert np.abs(lg_w - lg_s).max() < 2e-3
    assert (tok_w != tok_s).mean() < 0.01
    assert reg.device_error() == 0


@pytest.mark.parametrize("B,P", [(300, 37), (230, 270)])
def test_decode_attention_medium_batches_both_kernels(reg, B, P):
    """600 / 460 (sequence, head) pairs, contexts 38.. and 271..: the split-context kernel (the default at
    this size) against the oracle on a few sequences, and the TMA-fed kernel forced onto the same work
    (fewer items than warps: some warps of its grid get nothing) against the split kernel on all."""
    cfg = _mini(n_layer=2, d=128, vocab=257, npos=288)
    w = synth.gpt2_weights(cfg, base_seed=68, std=0.08, random_ln=True)
    m = Int4Gpt2Model.from_weights(w, cfg, reg)
    om = oracle.Model(cfg.as_dict(), _int4_oracle_weights(m, cfg, w, False))
    N = 5
    prompts = synth.token_ids(11, (B, P), cfg.vocab_size)

    def run():
        s = DecodeSession(m, batch=B, capacity=P + N + 1)
        s.prefill(prompts)
        s.step(1)
        s.step(N - 2)
        return s.tokens(), s.logits()

    tok_b, lg_b = run()
    reg.set_tuning("attn_stream_min10", 1)
    try:
        tok_p, lg_p = run()
    finally:
        reg.set_tuning("attn_stream_min10", 20)
    assert reg.device_error() == 0
    assert (tok_b != tok_p).mean() < 0.01
    same = (tok_b == tok_p).all(axis=1)  # a near-tie flipped by the order of the split-K additions changes a history
    # the two kernels add in different orders; where that moves an fp16 activation of order one by one unit
    # in the last place (1e-3), the logits move by a few 1e-3: a fifth of the path's tolerance is allowed
    assert np.abs(lg_b[same] - lg_p[same]).max() < MAX_ABS / 5
    reg.set_tuning("attn_stream_min10", 1)
    reg.set_tuning("attn_stream_wide_min10", 1)  # its 16-warp shape: 16-row stages, ragged last stage
    try:
        tok_w, lg_w = run()
    finally:
        reg.set_tuning("attn_stream_min10", 20)
        reg.set_tuning("attn_stream_wide_min10", 25)
    assert reg.device_error() == 0
    assert (tok_b != tok_w).mean() < 0.01
    same = (tok_b == tok_w).all(axis=1)
    assert np.abs(lg_b[same] - lg_w[same]).max() < MAX_ABS / 5
    for b in (0, B // 2, B - 1):
        ref, lg = om.generate_cached(prompts[b], N, flags=oracle.KV_FP16, want_logits=True)
        _check_tokens(np.concatenate([prompts[b], tok_b[b]]), ref, lg, P)
    tok_again, _ = run()  # the work counters are back at zero
    assert (tok_again != tok_b).mean() < 0.01  # equal up to near-ties flipped by the order of the split-K additions


def test_eos_stops_before_append(reg):
    # a vocabulary large enough to contain id 50256, with the head biased so that it wins
    cfg = Gpt2Config(n_layer=1, n_embd=64, n_head=1, vocab_size=50257, n_positions=32)
    w = synth.gpt2_weights(cfg, base_seed=71, std=0.02)
    w["wte"][50256] = 0.0
    m = Gpt2Model.from_weights(w, cfg, reg)
    prompt = np.array([5, 6, 7], dtype=np.uint32)
    free = m.generate(prompt, 6, flags=0)
    assert free.size == 9
    # force EOS at the second generated token: make that token's embedding row the EOS row's
    # strongest match by planting EOS = argmax target of step 2 via a crafted wte copy
    lg = oracle.Model(cfg.as_dict(), w).generate_cached(prompt, 2, want_logits=True)[1]
    target = int(np.argmax(lg[1]))
    w2 = dict(w)
    w2["wte"] = w["wte"].copy()
    w2["wte"][50256] = w["wte"][target] * 1.5  # same direction, larger: beats `target` at that step
    m2 = Gpt2Model.from_weights(w2, cfg, reg)
    ref = oracle.Model(cfg.as_dict(), w2).generate_cached(prompt, 6, flags=oracle.STOP_ON_EOS)[0]
    got = m2.generate(prompt, 6)  # default flags stop on EOS
    assert np.array_equal(got, ref)
    assert 50256 not in got.tolist()


def test_model_errors(reg):
    cfg = _mini(n_layer=1)
    w = synth.gpt2_weights(cfg, base_seed=81)
    m = Gpt2Model.from_weights(w, cfg, reg)
    with pytest.raises(b200nn.NnError) as e:
        m.forward(np.array([cfg.vocab_size], dtype=np.uint32))  # id out of range
    assert e.value.code == b200nn.ERR_DIM
    with pytest.raises(b200nn.NnError):
        m.generate(np.arange(60, dtype=np.uint32) % 300, 10)  # beyond n_positions
    bad = Gpt2Config(n_layer=1, n_embd=96, n_head=2, vocab_size=100, n_positions=16)  # head_dim 48
    with pytest.raises(b200nn.NnError) as e:
        Gpt2Model.from_weights(synth.gpt2_weights(bad, base_seed=82), bad, reg)
    assert e.value.code == b200nn.ERR_UNSUPPORTED
    w.pop("ln_f.bias")
    with pytest.raises(KeyError):
        Gpt2Model.from_weights(w, cfg, reg)


def _save_checkpoint(path, w, drop=(), replace=None):
    """An F32 checkpoint with Hugging Face key names (8-byte header length, JSON header, data)."""
    import json
    import struct
    header, blobs, off = {}, [], 0
    for k, v in w.items():
        name = "wte.weight" if k == "wte" else "wpe.weight" if k == "wpe" else k
        if name in drop:
            continue
        a = np.asarray((replace or {}).get(name, v))
        dt = {np.dtype(np.float32): "F32", np.dtype(np.float16): "F16"}[a.dtype]
        b = a.tobytes()
        header[name] = {"dtype": dt, "shape": list(a.shape), "data_offsets": [off, off + len(b)]}
        blobs.append(b)
        off += len(b)
    h = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h)) + h + b"".join(blobs))


def test_models_from_safetensors_checkpoint(reg, tmp_path):
    """load_gpt2_weights + from_weights inside the library: the same logits as the model built
    from the same arrays in memory; configuration given or read off the file; the loader's errors."""
    cfg = _mini(n_layer=2, d=128, vocab=307, npos=40)
    w = {k: np.asarray(v, np.float32) for k, v in synth.gpt2_weights(cfg, base_seed=95, std=0.08, random_ln=True).items()}
    d = cfg.n_embd
    shaped = dict(w)
    for i in range(cfg.n_layer):  # the checkpoint stores Conv1D weights as [in,out] matrices
        for nm, (k, n) in {"attn.c_attn.weight": (d, 3 * d), "attn.c_proj.weight": (d, d), "mlp.c_fc.weight": (d, 4 * d),
                           "mlp.c_proj.weight": (4 * d, d)}.items():
            shaped[f"h.{i}.{nm}"] = w[f"h.{i}.{nm}"].reshape(k, n)
    shaped["wte"] = w["wte"].reshape(cfg.vocab_size, d)
    shaped["wpe"] = w["wpe"].reshape(cfg.n_positions, d)
    p = tmp_path / "model.safetensors"
    _save_checkpoint(p, shaped)
    toks = synth.token_ids(12, (20,), cfg.vocab_size)
    for cls in (Gpt2Model, Int4Gpt2Model):
        ref = cls.from_weights(w, cfg, reg).forward(toks).to_host()
        a = cls.from_safetensors(p, reg, config=cfg)
        b = cls.from_safetensors(p, reg)  # configuration read off the tensor shapes
        assert b.config.as_dict() == pytest.approx(cfg.as_dict())
        # the residual GEMMs add their K splits in arrival order, so the last bits move between runs
        same = lambda x, y: np.abs(x - y).max() < 2e-3
        assert same(a.forward(toks).to_host(), ref)
        assert same(b.forward(toks).to_host(), ref)
        # the generic loader (model_generic.rs) + from_generic_weights: GPT-2's weight map hands the dense
        # weights over transposed to Linear layout; same logits as from_weights, as the reference's own
        # test_gpt2_generic_loader_regression asks (gpt2.rs:1690-1745)
        g = b200nn.load_safetensors_mapped(str(p), b200nn.gpt2_weight_map(cfg.n_layer))
        assert g.require("h.0.mlp.c_fc.weight").shape == [4 * d, d]
        assert same(cls.from_generic_weights(g, cfg, reg).forward(toks).to_host(), ref)
        with pytest.raises(b200nn.NnError) as e:  # a missing key: ShapeMismatch { expected: key, .. }
            cls.from_generic_weights(b200nn.load_safetensors_mapped(str(p), b200nn.gpt2_weight_map(1)), cfg, reg)
        assert e.value.code == b200nn.ERR_SHAPE and "h.1." in str(e.value)
    assert Int4Gpt2Model.from_safetensors(p, reg).quantized_memory_bytes() > 0
    # errors of the reference's loader (ModelError, model.rs:30-62)
    with pytest.raises(b200nn.NnError) as e:
        Gpt2Model.from_safetensors(tmp_path / "absent.safetensors", reg)
    assert e.value.code == b200nn.ERR_IO
    _save_checkpoint(p, shaped, drop=("h.1.mlp.c_proj.bias",))
    with pytest.raises(b200nn.NnError) as e:
        Gpt2Model.from_safetensors(p, reg)
    assert e.value.code == b200nn.ERR_MISSING and "h.1.mlp.c_proj.bias" in str(e.value)
    _save_checkpoint(p, shaped, replace={"ln_f.bias": shaped["ln_f.bias"].astype(np.float16)})
    with pytest.raises(b200nn.NnError) as e:
        Gpt2Model.from_safetensors(p, reg)
    assert e.value.code == b200nn.ERR_UNSUPPORTED and "F16" in str(e.value)
    _save_checkpoint(p, shaped, replace={"h.0.attn.c_attn.weight": shaped["h.0.attn.c_attn.weight"].T.copy()})
    with pytest.raises(b200nn.NnError) as e:
        Gpt2Model.from_safetensors(p, reg)
    assert e.value.code == b200nn.ERR_SHAPE


def test_gpt2_small_shapes_subset(reg):
    """GPT-2 Small dimensions (d 768, 12 heads, vocab 50257) with 2 layers: int4 + quantised head,
    2 sequences x 6 decode steps against the oracle."""
    cfg = Gpt2Config(n_layer=2, n_embd=768, n_head=12, vocab_size=50257, n_positions=64)
    w = synth.gpt2_weights(cfg, base_seed=91, std=0.02)
    m = Int4Gpt2Model.from_weights(w, cfg, reg, flags=b200nn.QUANT_LM_HEAD)
    om = oracle.Model(cfg.as_dict(), _int4_oracle_weights(m, cfg, w, True))
    prompts = synth.token_ids(6, (2, 16), cfg.vocab_size)
    out, _ = m.generate_batch(prompts, 6)
    for b in range(2):
        ref, lg = om.generate_cached(prompts[b], 6, flags=oracle.KV_FP16, want_logits=True)
        _check_tokens(out[b], ref, lg, 16)
    s = DecodeSession(m, batch=2, capacity=32)
    s.prefill(prompts)
    got = s.logits()
    for b in range(2):
        ref = om.forward(prompts[b], last_only=True, flags=oracle.KV_FP16)[0]
        _check_logits(got[b], ref)


@pytest.mark.parametrize("int4", [True, False])
def test_prefill_of_16384_rows_takes_the_persistent_gemm(reg, int4):
    """128 sequences x 128 prompt tokens, 640 wide: every Linear of the prefill pass has at least two
    256-row tiles per SM, so all four epilogues (q + K/V cache, residual twice, GELU) run in the
    persistent fp16 GEMM (int4 weights dequantised once per Linear on the way).  A few sequences are
    checked against the oracle, which runs them one at a time."""
    cfg = Gpt2Config(n_layer=2, n_embd=640, n_head=10, vocab_size=523, n_positions=160)
    w = synth.gpt2_weights(cfg, base_seed=77, std=0.04, random_ln=True)
    if int4:
        m = Int4Gpt2Model.from_weights(w, cfg, reg)
        om = oracle.Model(cfg.as_dict(), _int4_oracle_weights(m, cfg, w, False))
    else:
        m = Gpt2Model.from_weights(w, cfg, reg)
        om = oracle.Model(cfg.as_dict(), w)
    prompts = synth.token_ids(9, (128, 128), cfg.vocab_size)
    n0 = reg.launch_count()
    out, lens = m.generate_batch(prompts, 6)
    with_persistent = reg.launch_count() - n0
    for b in (0, 61, 127):
        ref, lg = om.generate_cached(prompts[b], 6, flags=oracle.KV_FP16, want_logits=True)
        _check_tokens(out[b][: lens[b]], ref, lg, 128)
    # the same through the one-tile-per-block kernels: same tokens, and (int4) four launches fewer per layer
    reg.set_tuning("tc_persistent", 0)
    try:
        n0 = reg.launch_count()
        out1, _ = m.generate_batch(prompts, 6)
        without = reg.launch_count() - n0
    finally:
        reg.set_tuning("tc_persistent", 1)
    assert with_persistent - without == (4 * cfg.n_layer if int4 else 0)
    same = (out == out1).all(axis=1).mean()
    assert same > 0.9, same  # different accumulation order may flip a near-tie in a few sequences
    assert reg.device_error() == 0


@pytest.mark.parametrize("preset,batch,prompt_len,new", [("small", 32, 24, 16), ("xl", 256, 16, 8)])
def test_full_size_int4_models_against_oracle(reg, preset, batch, prompt_len, new):
    """The benchmark's two model configurations at full size (GPT-2 Small and XL, every Linear and the LM
    head int4 g128, fp16 KV cache, 50257-token vocabulary) with their batch sizes, so that every kernel
    runs at the benchmark's shapes; the first and the last sequence of the batch are checked against the
    oracle token by token (it runs them one at a time), with shorter prompts than the benchmark's to
    keep the CPU side at seconds."""
    cfg = getattr(Gpt2Config, preset)()
    w = synth.gpt2_weights(cfg)
    m = Int4Gpt2Model.from_weights(w, cfg, reg, flags=b200nn.QUANT_LM_HEAD, group_size=128)
    om = oracle.Model(cfg.as_dict(), _int4_oracle_weights(m, cfg, w, True))
    del w
    prompts = synth.token_ids(synth.BASE_SEED + 7, (batch, prompt_len), cfg.vocab_size)
    out, lens = m.generate_batch(prompts, new)
    assert out.shape == (batch, prompt_len + new)
    for b in (0, batch - 1):
        ref, lg = om.generate_cached(prompts[b], new, flags=oracle.KV_FP16, want_logits=True)
        _check_tokens(out[b][: lens[b]], ref, lg, prompt_len)
    # logits of the last prompt position of one sequence through the public forward
    got = m.forward(prompts[0]).to_host()[-1]
    ref = om.forward(prompts[0], flags=oracle.KV_FP16)[-1]
    assert np.abs(got - ref).max() < MAX_ABS and np_ref.rel_rms(got, ref) < REL_RMS
    assert reg.device_error() == 0
    if preset != "xl":
        return
    # the benchmark's own decode window: 256 sequences with 128-token prompts, stepped to a context of 161;
    # the logits of that step (rows 0 and 255) against the oracle, where the greedy histories agree
    P, steps = 128, 33
    prompts = synth.token_ids(synth.BASE_SEED + 7, (batch, P), cfg.vocab_size)
    s = DecodeSession(m, batch=batch, capacity=P + steps + 2)
    s.prefill(prompts)
    s.step(1)
    s.step(steps - 1)
    assert s.position() == P + steps
    toks, lgs = s.tokens(), s.logits()
    compared = 0
    for b in (0, batch - 1):
        ref, lg = om.generate_cached(prompts[b], steps + 1, flags=oracle.KV_FP16, want_logits=True)
        _check_tokens(np.concatenate([prompts[b], toks[b]]), ref, lg, P)
        if np.array_equal(toks[b], ref[P:]):
            assert np.abs(lgs[b] - lg[-1]).max() < MAX_ABS and np_ref.rel_rms(lgs[b], lg[-1]) < REL_RMS
            compared += 1
    assert compared >= 1  # a near-tie may end one history early, not both
    assert reg.device_error() == 0


def test_forward_diagnostic_reports_the_reference_values(reg, capsys):
    """forward_diagnostic (gpt2.rs:595-667): the same logits as forward, and the reported values are the
    oracle's hidden states at the places the reference prints them."""
    cfg = _mini(n_layer=3)
    w = synth.gpt2_weights(cfg, base_seed=83, std=0.08, random_ln=True)
    m = Gpt2Model.from_weights(w, cfg, reg)
    toks = synth.token_ids(4, (11,), cfg.vocab_size)
    logits, rep = m.forward_diagnostic(toks)
    got = logits.to_host()
    ref = oracle.Model(cfg.as_dict(), w).forward(toks, flags=oracle.KV_FP16)
    _check_logits(got, ref)
    err = capsys.readouterr().err
    assert "[diag] Embedding pos0 first4:" in err and "[diag] Layer 2 pos10 first4:" in err and "Top-5 tokens at pos10" in err
    emb0 = w["wte"][toks[0]][:4] + w["wpe"][0][:4]
    assert np.allclose(rep["embedding_first"], emb0, atol=1e-6)
    emb_last = w["wte"][toks[-1]][:4] + w["wpe"][10][:4]
    assert np.allclose(rep["embedding_last"], emb_last, atol=1e-6)
    assert rep["block0_nonfinite"] == 0 and rep["final_block_nonfinite"] == 0
    order = np.argsort(-ref[-1], kind="stable")[:5]
    assert [t for t, _ in rep["top"]] == order.tolist() or np.abs(np.sort(ref[-1])[::-1][:5] - [v for _, v in rep["top"]]).max() < 2e-2
    assert np.allclose([v for _, v in rep["top"]], np.sort(got[-1])[::-1][:5], atol=1e-6)
    # hidden state after block 0, last position, against the oracle's block on the embedded rows
    x = (w["wte"][toks] + w["wpe"][: len(toks)]).astype(np.float32)
    h0, _, _ = oracle.Model(cfg.as_dict(), w).block_forward(0, x, flags=oracle.KV_FP16)
    assert np.abs(np.asarray(rep["block0_last"]) - h0[-1][:4]).max() < 5e-3


def test_two_contexts_in_one_process_one_host_thread_each(reg):
    """One context per GPU, one host thread per context (the threading model of the batch-sharded path):
    two contexts are created in this process (on two GPUs when there are two, else both on GPU 0), each
    thread builds its own int4 model and generates its half of the batch, then runs a four-row Int4Linear
    through the CUDA-core GEMV at a shape (K 4096, 149 feature tiles: no K split) whose block needs more than
    48 KB of dynamic shared memory, which is a per-device function attribute."""
    import threading

    import torch
    ndev = torch.cuda.device_count()
    devices = [0, 1 if ndev > 1 else 0]
    cfg = _mini(n_layer=2, d=128, vocab=257, npos=64)
    w = synth.gpt2_weights(cfg, base_seed=88, std=0.08, random_ln=True)
    prompts = synth.token_ids(6, (12, 9), cfg.vocab_size)
    K, N = 4096, 19072
    rng = np.random.default_rng(5)
    packed = rng.integers(0, 2 ** 32, (K // 8, N), dtype=np.uint32)  # eight random nibbles per word
    scales = rng.uniform(0.005, 0.02, (K // 128, N)).astype(np.float16).astype(np.float32)
    x = rng.standard_normal((4, K)).astype(np.float32)
    results, errors = {}, []

    def work(i):
        try:
            r = b200nn.KernelRegistry(devices[i])
            m = Int4Gpt2Model.from_weights(w, cfg, r)
            out, lens = m.generate_batch(prompts[i * 6:(i + 1) * 6], 6)
            r.set_gemv_max_rows(4)
            y = b200nn.Int4Linear(packed, scales, None, K, N, 128, r).forward(b200nn.GpuTensor.from_host(x, (4, K), r)).to_host()
            results[i] = (out, y, r.device_error())
            r.close()
        except Exception as e:  # surfaced below: a thread must not swallow a failure
            errors.append((i, repr(e)))

    th = [threading.Thread(target=work, args=(i,)) for i in range(2)]
    for t in th:
        t.start()
    for t in th:
        t.join()
    assert not errors, errors
    m0 = Int4Gpt2Model.from_weights(w, cfg, reg)
    ref, _ = m0.generate_batch(prompts, 6)
    yref = oracle.int4_linear(x, packed, scales, None, 4, N, K, 128)
    for i in range(2):
        out, y, err = results[i]
        assert err == 0
        assert (out == ref[i * 6:(i + 1) * 6]).mean() > 0.97
        assert np_ref.rel_rms(y, yref) < 1e-5


@pytest.mark.parametrize("quant_head", [False, True])
@pytest.mark.parametrize("B", [1, 2, 7, 40])
def test_greedy_pick_in_the_lm_head_epilogue_equals_the_separate_kernel(reg, one_k_split, quant_head, B):
    """Decode sessions take the greedy token inside the LM head's epilogue (a maximum and index per 32
    features, reduced by a second small kernel).  Same tokens, bit for bit, as argmax_kernel over the
    stored logits, under both tie rules; with every vocabulary row equal all logits of a row are equal
    (tensor-core path: every column goes through the same operations), so the first-index rule must give
    token 0 and the last-index rule the last token."""
    cfg = _mini(n_layer=1, d=128, vocab=523)
    w = synth.gpt2_weights(cfg, base_seed=97, std=0.08, random_ln=True)
    w["wte"][400] = w["wte"][17]
    w["wte"][522] = w["wte"][17]
    prompts = synth.token_ids(B, (B, 5), cfg.vocab_size)
    head = b200nn.QUANT_LM_HEAD if quant_head else 0
    for tie in (0, b200nn.ARGMAX_LAST):
        m = Int4Gpt2Model.from_weights(w, cfg, reg, flags=head | tie)
        fused, _ = m.generate_batch(prompts, 6)
        s = DecodeSession(m, batch=B, capacity=16)  # the same with the logits kept
        s.prefill(prompts)
        s.step(5)
        assert np.array_equal(s.tokens(), fused[:, 5:])
        assert np.array_equal(np.argmax(s.logits(), axis=1) if not tie else
                              s.logits().shape[1] - 1 - np.argmax(s.logits()[:, ::-1], axis=1), s.tokens()[:, -1])
        reg.set_tuning("fused_argmax", 0)
        try:
            plain, _ = m.generate_batch(prompts, 6)
        finally:
            reg.set_tuning("fused_argmax", 1)
        assert np.array_equal(fused, plain)
    if B > 2:
        flat = dict(w)
        flat["wte"] = np.repeat(w["wte"][:1], cfg.vocab_size, axis=0)
        for tie, want in ((0, 0), (b200nn.ARGMAX_LAST, cfg.vocab_size - 1)):
            m = Int4Gpt2Model.from_weights(flat, cfg, reg, flags=head | tie)
            out, _ = m.generate_batch(prompts, 3)
            assert (out[:, 5:] == want).all()
    with pytest.raises(b200nn.NnError):  # a session that keeps no logits cannot hand them out
        s = DecodeSession(m, batch=B, capacity=16, flags=b200nn.TOKENS_ONLY)
        s.prefill(prompts)
        s.logits()
    assert reg.device_error() == 0


@pytest.mark.parametrize("d,B,offset", [(192, 40, 0.0), (256, 33, 0.05), (320, 130, 0.0)])
def test_block_layernorms_folded_into_the_gemms(reg, d, B, offset):
    """Tuning key ln_fold = 1 (off by default: measured slower): decode steps of more than gemv_max_rows
    sequences run no LayerNorm kernel inside the blocks; the residual GEMMs hand fp16(x * g) and the row
    sums on, and the q/k/v and MLP GEMMs normalise after the product.  Same logits as the oracle and as
    the step with LayerNorm kernels, with random scale and shift vectors, a width whose last feature tile
    is ragged (192, 320), two token tiles (130 rows) and a residual stream whose mean is not small against
    its spread (offset).  Tolerance against the oracle: 1.5x the path's relative RMS, because x * g is
    rounded to fp16 before the mean is taken out instead of after."""
    cfg = _mini(n_layer=3, d=d, vocab=389)
    w = synth.gpt2_weights(cfg, base_seed=211, std=0.08, random_ln=True)
    w["wpe"] = w["wpe"] + np.float32(offset)
    m = Int4Gpt2Model.from_weights(w, cfg, reg, flags=b200nn.QUANT_LM_HEAD)
    om = oracle.Model(cfg.as_dict(), _int4_oracle_weights(m, cfg, w, True))
    P = 6
    prompts = synth.token_ids(d + B, (B, P), cfg.vocab_size)

    def first_steps(fold):
        reg.set_tuning("ln_fold", fold)
        try:
            s = DecodeSession(m, batch=B, capacity=P + 8)
            before = reg.launch_count()
            s.prefill(prompts)
            s.step(1)  # the tokens the prefill picked go through one decode step: same history on both paths
            lg1 = s.logits()
            n1 = reg.launch_count()
            s.step(3)
            return lg1, s.tokens(), s.logits(), n1 - before
        finally:
            reg.set_tuning("ln_fold", 0)

    lg_f, tok_f, lg3_f, launches_f = first_steps(1)
    lg_k, tok_k, lg3_k, launches_k = first_steps(0)
    assert launches_k - launches_f == 2 * cfg.n_layer  # the block LayerNorms of the one eager decode step
    assert (tok_f[:, :2] == tok_k[:, :2]).mean() > 0.97
    # two GPU paths, each near the oracle: twice the tolerance between them
    assert np.abs(lg_f - lg_k).max() < 2 * MAX_ABS and np_ref.rel_rms(lg_f, lg_k) < 2 * REL_RMS
    same = (tok_f == tok_k).all(axis=1)
    assert same.mean() > 0.9
    assert np.abs(lg3_f[same] - lg3_k[same]).max() < 2 * MAX_ABS and np_ref.rel_rms(lg3_f[same], lg3_k[same]) < 2 * REL_RMS
    for b in (0, B - 1):
        ref, lg = om.generate_cached(prompts[b], 2, flags=oracle.KV_FP16, want_logits=True)
        _check_tokens(np.concatenate([prompts[b], tok_f[b][:2]]), ref, lg, P)
        if np.array_equal(tok_f[b][:2], ref[P:]):
            assert np.abs(lg_f[b] - lg[-1]).max() < MAX_ABS and np_ref.rel_rms(lg_f[b], lg[-1]) < 1.5 * REL_RMS
            print(f"fold vs oracle {np_ref.rel_rms(lg_f[b], lg[-1]):.2e}, kernels vs oracle {np_ref.rel_rms(lg_k[b], lg[-1]):.2e}")
    assert reg.device_error() == 0
