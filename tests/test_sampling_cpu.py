"""SimpleRng and top_k_sample (host code of the library: runs without a GPU) against the oracle's
restatement of gpt2.rs:1000-1058 and against a third, pure-Python statement of the same arithmetic."""
import numpy as np
import pytest

import b200nn
from oracle import oracle

MASK = (1 << 64) - 1


def py_rng(seed):
    """xorshift64 as gpt2.rs:1012-1022 writes it: x ^= x<<13; x ^= x>>7; x ^= x<<17; (x>>40)/2^24."""
    x = seed if seed else 0xDEADBEEFCAFE1234
    while True:
        x ^= (x << 13) & MASK
        x ^= x >> 7
        x ^= (x << 17) & MASK
        yield np.float32(x >> 40) / np.float32(1 << 24)


def py_top_k(logits, k, temperature, r):
    """top_k_sample (gpt2.rs:1029-1058) in numpy float32, with the draw r given."""
    temp = np.float32(max(temperature, 1e-8))
    scaled = (np.asarray(logits, np.float32) / temp).astype(np.float32)
    order = sorted(range(scaled.size), key=lambda i: (-scaled[i], i))[: min(k, scaled.size)]  # stable descending
    e = np.exp((scaled[order] - scaled[order[0]]).astype(np.float32)).astype(np.float32)
    s = np.float32(0)
    for v in e:
        s = np.float32(s + v)
    cum = np.float32(0)
    for i, v in zip(order, e):
        cum = np.float32(cum + np.float32(v / s))
        if r < cum:
            return i
    return order[-1]


@pytest.mark.parametrize("seed", [0, 1, 42, 20260101, (1 << 63) + 12345])
def test_simple_rng_three_ways(seed):
    lib, orc, py = b200nn.SimpleRng(seed), oracle.SimpleRng(seed), py_rng(seed)
    for _ in range(200):
        a, b, c = lib.next_f32(), orc.next_f32(), float(next(py))
        assert a == b == c and 0.0 <= a < 1.0


def test_top_k_sample_matches_oracle_and_python():
    rng = np.random.default_rng(3)
    for case in range(60):
        n = int(rng.integers(1, 400))
        logits = rng.standard_normal(n).astype(np.float32) * np.float32(rng.choice([0.1, 1.0, 8.0]))
        if case % 3 == 0:  # ties: the stable sort keeps the lower index first
            logits = np.round(logits * 2) / 2
        k = int(rng.integers(1, 80))
        temp = float(rng.choice([1.0, 0.7, 1.5, 1e-3, 0.0]))  # 0 is clamped to 1e-8
        seed = int(rng.integers(1, 2**62))
        lib_r, orc_r, py_r = b200nn.SimpleRng(seed), oracle.SimpleRng(seed), py_rng(seed)
        for _ in range(5):
            a = b200nn.top_k_sample(logits, k, temp, lib_r)
            b, margin = oracle.top_k_sample(logits, k, temp, orc_r)
            assert a == b, (case, n, k, temp)
            r = next(py_r)
            if margin > 1e-6:  # expf of libm vs numpy may differ in the last bit right at a boundary
                assert py_top_k(logits, k, temp, r) == a
        assert lib_r.state.value == orc_r.state.value  # one draw per sample


def test_top_k_sample_edge_cases():
    r = b200nn.SimpleRng(9)
    assert b200nn.top_k_sample([3.0], 5, 1.0, r) == 0  # k larger than the vocabulary
    assert b200nn.top_k_sample([0.0, 5.0, 1.0], 1, 1.0, r) == 1  # k = 1 is greedy
    assert b200nn.top_k_sample([1.0, 7.0, 7.0, 2.0], 1, 0.5, r) == 1  # tie: first index wins the sort
    with pytest.raises(b200nn.NnError):
        b200nn.top_k_sample([1.0, 2.0], 0, 1.0, r)
    # tiny temperature: all mass on the maximum
    picks = {b200nn.top_k_sample([0.0, 0.2, 0.1], 3, 1e-6, r) for _ in range(50)}
    assert picks == {1}


def test_softmax_max_prob_oracle():
    assert oracle.softmax_max_prob(np.zeros(4, np.float32)) == pytest.approx(0.25)
    x = np.array([10.0, 0.0, -3.0], np.float32)
    assert oracle.softmax_max_prob(x) == pytest.approx(float(np.exp(10.0) / np.exp(x.astype(np.float64)).sum()), rel=1e-6)


def test_synthetic_weights_from_simple_rng_are_reproducible_from_the_reference_generator():
    """synth's "simple_rng" source: per-tensor SimpleRng streams, normals by Box-Muller on pairs of
    uniforms -- restated here in pure Python from the reference's xorshift64 (gpt2.rs:1000-1023), so a Rust
    caller with nothing but SimpleRng gets the same bits."""
    import math

    from b200nn import Gpt2Config, synth

    cfg = Gpt2Config(n_layer=1, n_embd=8, n_head=1, vocab_size=11, n_positions=4)
    w = synth.gpt2_weights(cfg, base_seed=77, std=0.02, source="simple_rng")
    w2 = synth.gpt2_weights(cfg, base_seed=77, std=0.02, source="simple_rng")
    assert all(np.array_equal(w[k], w2[k]) for k in w)

    def py_normals(seed, n, std):
        x = seed or 0xDEADBEEFCAFE1234
        out = []

        def nxt():
            nonlocal x
            x ^= (x << 13) & 0xFFFFFFFFFFFFFFFF
            x ^= x >> 7
            x ^= (x << 17) & 0xFFFFFFFFFFFFFFFF
            return float(np.float32((x >> 40) / float(1 << 24)))

        while len(out) < n:
            u1, u2 = nxt(), nxt()
            r = math.sqrt(-2.0 * math.log(1.0 - u1))
            out.append(np.float32(r * math.cos(2 * math.pi * u2) * float(np.float32(std))))
            out.append(np.float32(r * math.sin(2 * math.pi * u2) * float(np.float32(std))))
        return np.asarray(out[:n], dtype=np.float32)

    assert np.allclose(w["wte"].ravel(), py_normals(77 + 1, 11 * 8, 0.02), rtol=0, atol=1e-9)
    assert np.allclose(w["h.0.attn.c_attn.weight"].ravel(), py_normals(77 + 1000 + 3, 8 * 24, 0.02), rtol=0, atol=1e-9)
    big = synth._normal(5, (200000,), 1.0, "simple_rng")
    assert abs(float(big.mean())) < 0.01 and abs(float(big.std()) - 1.0) < 0.01
    # the default source is unchanged
    assert np.array_equal(synth.gpt2_weights(cfg, base_seed=77)["wte"],
                          (np.random.Generator(np.random.PCG64(78)).standard_normal((11, 8), dtype=np.float32) * np.float32(0.02)))


def test_argmax_and_softmax_max_prob_helpers():
    """gpt2.rs:983-997: the last maximum wins a tie (Rust max_by), an empty slice gives 0; the confidence of
    early exit is 1 / sum exp(x - max) in f32."""
    assert b200nn.argmax([1.0, 5.0, 2.0, 5.0, 0.0]) == 3
    assert b200nn.argmax([7.0]) == 0 and b200nn.argmax([]) == 0
    assert b200nn.argmax([-1.0, -1.0, -1.0]) == 2
    x = np.array([0.5, 2.0, -1.0, 2.0], dtype=np.float32)
    want = 1.0 / np.exp(x.astype(np.float64) - 2.0).sum()
    assert abs(b200nn.softmax_max_prob(x) - want) < 1e-6
    assert abs(b200nn.softmax_max_prob([3.0]) - 1.0) < 1e-7
