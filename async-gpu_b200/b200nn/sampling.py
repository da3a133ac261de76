"""``SimpleRng`` and ``top_k_sample`` of ``gpu_host::nn::models::gpt2`` (gpt2.rs:1000-1058), host code of
the library (no GPU needed)."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import NnError, _f32, load_library


class SimpleRng:
    """xorshift64; ``state`` is the u64 the library advances."""

    def __init__(self, seed: int):
        self.state = C.c_uint64(load_library().b200nn_simple_rng_new(seed))

    def next_f32(self) -> float:
        return float(load_library().b200nn_simple_rng_next_f32(C.byref(self.state)))


def top_k_sample(logits, k: int, temperature: float, rng: SimpleRng) -> int:
    a, ap = _f32(np.ravel(logits))
    tok = C.c_uint32()
    rc = load_library().b200nn_top_k_sample(ap, a.size, k, temperature, C.byref(rng.state), C.byref(tok))
    if rc != 0:
        raise NnError(rc, "top_k_sample: empty logits or k == 0")
    return int(tok.value)
