"""Generates tests/golden/tiny_gpt2_golden.npz with the CPU oracle (run from the repository root:
``python tests/golden/make_golden.py``).  The reference is Rust and cannot run offline, so the
vectors are the oracle's own outputs, pinned so that later edits to the oracle cannot drift
unnoticed; the reference's known-answer tests live in reference_kats.json."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path[:0] = [ROOT, os.path.join(ROOT, "async-gpu_b200")]
from oracle import oracle  # noqa: E402
from b200nn import synth  # noqa: E402
from b200nn.gpt2 import Gpt2Config  # noqa: E402

TINY = dict(n_layer=2, n_embd=128, n_head=2, vocab_size=211, n_positions=32, layer_norm_epsilon=1e-5)
SEED = 21
w = synth.gpt2_weights(Gpt2Config(**TINY), base_seed=SEED, std=0.08, random_ln=True)
m = oracle.Model(TINY, w)
tokens = synth.token_ids(77, (10,), TINY["vocab_size"])
logits = m.forward(tokens)
generated, _ = m.generate_cached(tokens[:5], 8)
p, s = oracle.quantize_weight_int4(w["h.0.mlp.c_fc.weight"], 128, 512, 128)
# data-dependent decoding: one sampled run and one early-exit run (threshold = the median probe confidence)
sampled, _, _ = m.generate_cached_sampling(tokens[:5], 10, 20, 0.8, oracle.SimpleRng(2026))
rng = oracle.SimpleRng(7)
rng_draws = np.array([rng.next_f32() for _ in range(8)], dtype=np.float32)
conf = m.forward_early_exit(tokens, 2.0)[2]
for factor in (1.0, 0.9, 0.8, 0.7, 0.6, 0.5, 1.2, 1.5):  # the first threshold that gives steps of both depths
    threshold = np.float32(np.median(conf) * factor)
    ee_tokens, ee_layers, _, gap = m.generate_cached_early_exit(tokens[:5], 10, float(threshold))
    if len(set(ee_layers[1:].tolist())) == 2 and gap > 1e-4:
        break
np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "tiny_gpt2_golden.npz"),
                    seed=SEED, tokens=tokens, logits=logits, generated=generated, fc_packed=p, fc_scales=s,
                    sampled=sampled, rng_draws=rng_draws, probe_conf=conf, ee_threshold=threshold,
                    ee_tokens=ee_tokens, ee_layers=ee_layers)
print("written", logits.shape, generated, sampled, ee_layers)
