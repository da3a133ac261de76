"""Seeded synthetic GPT-2 weights and token ids (no checkpoint files are needed).

Every tensor is drawn from its own stream so that any two processes that agree on (config, base seed)
hold bit-identical weights: N(0, std) for embeddings, dense weights and biases, gamma = 1 and beta = 0
for LayerNorm unless ``random_ln``.  Dense weights use the checkpoint's Conv1D layout [in, out].

Two sources.  ``"pcg64"`` (the default): ``numpy.random.Generator(PCG64(seed))``.  ``"simple_rng"``:
the reference's own ``SimpleRng`` xorshift64 (gpt2.rs:1000-1023) seeded per tensor, normals by
Box-Muller on pairs of its uniforms (``b200nn_simple_rng_fill_normal``), so that a Rust caller that has
nothing but ``SimpleRng`` regenerates the same tensors.  The per-tensor seed is the same in both:
``base + 1`` wte, ``+ 2`` wpe, ``+ 3 / + 4`` ln_f, and for layer i with ``s = base + 1000 (i + 1)``:
``s+1 / s+2`` ln_1, ``s+3 / s+4`` c_attn weight / bias, ``s+5 / s+6`` attn c_proj, ``s+7 / s+8`` ln_2,
``s+9 / s+10`` mlp c_fc, ``s+11 / s+12`` mlp c_proj.
"""
from __future__ import annotations

import numpy as np

BASE_SEED = 20260101


def _normal(seed, shape, std, source="pcg64"):
    if source == "simple_rng":
        import ctypes as C

        from . import load_library
        lib = load_library()
        out = np.empty(int(np.prod(shape)), dtype=np.float32)
        state = C.c_uint64(lib.b200nn_simple_rng_new(seed))
        rc = lib.b200nn_simple_rng_fill_normal(C.byref(state), out.size, std, out.ctypes.data_as(C.POINTER(C.c_float)))
        assert rc == 0
        return out.reshape(shape)
    return (np.random.Generator(np.random.PCG64(seed)).standard_normal(shape, dtype=np.float32) * np.float32(std))


def gpt2_weights(cfg, base_seed: int = BASE_SEED, std: float = 0.02, random_ln: bool = False, source: str = "pcg64") -> dict:
    if source not in ("pcg64", "simple_rng"):
        raise ValueError("source must be 'pcg64' or 'simple_rng'")
    draw = _normal
    _normal_of = lambda seed, shape, s: draw(seed, shape, s, source)
    return _build(cfg, base_seed, std, random_ln, _normal_of)


def _build(cfg, base_seed, std, random_ln, _normal) -> dict:
    d, V, P = cfg.n_embd, cfg.vocab_size, cfg.n_positions
    w = {"wte": _normal(base_seed + 1, (V, d), std), "wpe": _normal(base_seed + 2, (P, d), std)}

    def ln(seed):
        if random_ln:
            return (1.0 + _normal(seed, (d,), 0.1)).astype(np.float32), _normal(seed + 1, (d,), 0.1)
        return np.ones(d, dtype=np.float32), np.zeros(d, dtype=np.float32)

    w["ln_f.weight"], w["ln_f.bias"] = ln(base_seed + 3)
    for i in range(cfg.n_layer):
        s = base_seed + 1000 * (i + 1)
        p = f"h.{i}."
        w[p + "ln_1.weight"], w[p + "ln_1.bias"] = ln(s + 1)
        w[p + "attn.c_attn.weight"] = _normal(s + 3, (d, 3 * d), std)
        w[p + "attn.c_attn.bias"] = _normal(s + 4, (3 * d,), std)
        w[p + "attn.c_proj.weight"] = _normal(s + 5, (d, d), std)
        w[p + "attn.c_proj.bias"] = _normal(s + 6, (d,), std)
        w[p + "ln_2.weight"], w[p + "ln_2.bias"] = ln(s + 7)
        w[p + "mlp.c_fc.weight"] = _normal(s + 9, (d, 4 * d), std)
        w[p + "mlp.c_fc.bias"] = _normal(s + 10, (4 * d,), std)
        w[p + "mlp.c_proj.weight"] = _normal(s + 11, (4 * d, d), std)
        w[p + "mlp.c_proj.bias"] = _normal(s + 12, (d,), std)
    return w


def token_ids(seed: int, shape, vocab: int) -> np.ndarray:
    """Uniform ids in [0, vocab)."""
    return np.random.Generator(np.random.PCG64(seed)).integers(0, vocab, size=shape, dtype=np.int64).astype(np.uint32)


def int4_linear_case(seed: int, m: int, k: int, n: int, group: int = 128):
    """Isolated int4 Linear inputs: signed nibbles uniform in [-8,7] packed in the reference layout
    [K/8,N] (stored +8), fp16-representable scales uniform in [0.005,0.02], activations N(0,1)."""
    g = np.random.Generator(np.random.PCG64(seed))
    q = g.integers(-8, 8, size=(k, n), dtype=np.int64)
    u = (q + 8).astype(np.uint32).reshape(k // 8, 8, n)
    packed = np.zeros((k // 8, n), dtype=np.uint32)
    for i in range(8):
        packed |= u[:, i, :] << np.uint32(4 * i)
    n_groups = (k + group - 1) // group
    scales = g.uniform(0.005, 0.02, size=(n_groups, n)).astype(np.float16).astype(np.float32)
    x = g.standard_normal((m, k), dtype=np.float32)
    return packed, scales, x, q
