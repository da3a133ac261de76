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


def argmax(data) -> int:
    """``argmax`` (gpt2.rs:991-997): Rust's ``max_by`` keeps the LAST maximum on ties; an empty slice gives 0.
    (On the device the same rule is the flag ``ARGMAX_LAST``; the CPU reference of the test harness keeps
    the first.)"""
    a = np.ravel(np.asarray(data, dtype=np.float32))
    if a.size == 0:
        return 0
    return int(a.size - 1 - np.argmax(a[::-1]))


def softmax_max_prob(logits) -> float:
    """``softmax_max_prob`` (gpt2.rs:983-988): the probability of the most likely token, in f32 as there."""
    a = np.ravel(np.asarray(logits, dtype=np.float32))
    return float(np.float32(1.0) / np.sum(np.exp(a - a.max(), dtype=np.float32), dtype=np.float32))
