"""ctypes binding of the CPU oracle (``liboracle.so``, built from ``gpt2_oracle.c``).

TEST INFRASTRUCTURE ONLY: imported by the test-suite, the smoke check and the
benchmark's CPU-baseline leg.  The product library never uses it.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")

GELU_SIGMOID = 1 << 0
KV_FP16 = 1 << 1
ARGMAX_LAST = 1 << 2
STOP_ON_EOS = 1 << 3


def build(force: bool = False) -> str:
    """Compile liboracle.so with the Makefile beside this file (gcc only)."""
    src = os.path.join(_HERE, "gpt2_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-s", "-B"], check=True, capture_output=True)
    return _LIB_PATH


class OrcConfig(C.Structure):
    _fields_ = [
        ("n_layer", C.c_int32),
        ("n_embd", C.c_int32),
        ("n_head", C.c_int32),
        ("vocab_size", C.c_int32),
        ("n_positions", C.c_int32),
        ("layer_norm_epsilon", C.c_float),
    ]


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        L = C.CDLL(_LIB_PATH)
        f32p, u32p, i8p = C.POINTER(C.c_float), C.POINTER(C.c_uint32), C.POINTER(C.c_int8)
        sz = C.c_size_t
        L.orc_f16_round_array.argtypes = [f32p, sz, f32p]
        L.orc_num_threads.restype = C.c_int
        L.orc_set_num_threads.argtypes = [C.c_int]
        L.orc_quantize_int8_per_tensor.argtypes = [f32p, sz, i8p, f32p]
        L.orc_pack_int8_to_u32.argtypes = [i8p, sz, u32p]
        L.orc_quantize_int4_per_group.argtypes = [f32p, sz, sz, u32p, f32p]
        L.orc_quantize_weight_int4.argtypes = [f32p, sz, sz, sz, u32p, f32p]
        L.orc_quantize_weight_int4.restype = C.c_int
        L.orc_unpack_int4.argtypes = [C.c_uint32, C.c_int]
        L.orc_unpack_int4.restype = C.c_int
        L.orc_dequant_weight_int4.argtypes = [u32p, f32p, sz, sz, sz, f32p]
        for fn in (L.orc_int4_linear_f32, L.orc_int4_linear_f64):
            fn.argtypes = [f32p, u32p, f32p, f32p, sz, sz, sz, sz, f32p]
        L.orc_matmul_f64.argtypes = [f32p, f32p, sz, sz, sz, f32p]
        L.orc_layer_norm_f64.argtypes = [f32p, f32p, f32p, sz, sz, C.c_float, f32p]
        L.orc_softmax_f64.argtypes = [f32p, sz, sz, f32p]
        L.orc_attention_f64.argtypes = [f32p, f32p, f32p, sz, sz, f32p]
        L.orc_gelu_tanh.argtypes = [C.c_double]
        L.orc_gelu_tanh.restype = C.c_double
        L.orc_gelu_sigmoid.argtypes = [C.c_double]
        L.orc_gelu_sigmoid.restype = C.c_double
        L.orc_model_create.argtypes = [C.POINTER(OrcConfig), f32p, f32p, f32p, f32p]
        L.orc_model_create.restype = C.c_void_p
        L.orc_model_set_layer.argtypes = [C.c_void_p, C.c_int] + [f32p] * 12
        L.orc_model_set_lm_head.argtypes = [C.c_void_p, f32p]
        L.orc_model_destroy.argtypes = [C.c_void_p]
        L.orc_forward.argtypes = [C.c_void_p, u32p, C.c_int32, C.c_int32, C.c_uint32, f32p]
        L.orc_forward.restype = C.c_int
        for fn in (L.orc_generate, L.orc_generate_cached):
            fn.argtypes = [C.c_void_p, u32p, C.c_int32, C.c_int32, C.c_uint32, u32p, f32p]
            fn.restype = C.c_int
        L.orc_time_decode.argtypes = [C.c_void_p, u32p, C.c_int32, C.c_int32, C.c_uint32,
                                      C.POINTER(C.c_double), u32p]
        L.orc_time_decode.restype = C.c_int
        L.orc_mha_f64.argtypes = [f32p, sz, f32p, f32p, sz, sz, sz, sz, sz, f32p]
        L.orc_block_forward.argtypes = [C.c_void_p, C.c_int, f32p, sz, sz, f32p, f32p, sz, C.c_uint32, f32p]
        u64p, i32p = C.POINTER(C.c_uint64), C.POINTER(C.c_int32)
        L.orc_rng_new.argtypes = [C.c_uint64]
        L.orc_rng_new.restype = C.c_uint64
        L.orc_rng_next_f32.argtypes = [u64p]
        L.orc_rng_next_f32.restype = C.c_float
        L.orc_top_k_sample.argtypes = [f32p, sz, sz, C.c_float, u64p, f32p]
        L.orc_top_k_sample.restype = C.c_uint32
        L.orc_softmax_max_prob.argtypes = [f32p, sz]
        L.orc_softmax_max_prob.restype = C.c_float
        L.orc_generate_cached_sampling.argtypes = [C.c_void_p, u32p, C.c_int32, C.c_int32, C.c_int32, C.c_float, u64p,
                                                   C.c_uint32, u32p, f32p, f32p]
        L.orc_generate_cached_sampling.restype = C.c_int
        L.orc_forward_early_exit.argtypes = [C.c_void_p, u32p, C.c_int32, C.c_float, C.c_uint32, f32p, i32p, f32p]
        L.orc_forward_early_exit.restype = C.c_int
        L.orc_generate_cached_early_exit.argtypes = [C.c_void_p, u32p, C.c_int32, C.c_int32, C.c_float, C.c_uint32, u32p,
                                                     i32p, i32p, f32p, f32p]
        L.orc_generate_cached_early_exit.restype = C.c_int
        _lib = L
    return _lib


def _f32(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a, a.ctypes.data_as(C.POINTER(C.c_float))


def _u32(a):
    a = np.ascontiguousarray(a, dtype=np.uint32)
    return a, a.ctypes.data_as(C.POINTER(C.c_uint32))


def f16_round(x):
    x, xp = _f32(x)
    out = np.empty_like(x)
    lib().orc_f16_round_array(xp, x.size, out.ctypes.data_as(C.POINTER(C.c_float)))
    return out


def num_threads() -> int:
    return int(lib().orc_num_threads())


def quantize_int8_per_tensor(data):
    data, dp = _f32(data)
    q = np.empty(data.size, dtype=np.int8)
    s = C.c_float()
    lib().orc_quantize_int8_per_tensor(dp, data.size, q.ctypes.data_as(C.POINTER(C.c_int8)), C.byref(s))
    return q, float(s.value)


def pack_int8_to_u32(values):
    v = np.ascontiguousarray(values, dtype=np.int8)
    out = np.zeros((v.size + 3) // 4, dtype=np.uint32)
    lib().orc_pack_int8_to_u32(v.ctypes.data_as(C.POINTER(C.c_int8)), v.size,
                               out.ctypes.data_as(C.POINTER(C.c_uint32)))
    return out


def quantize_int4_per_group(data, group):
    data, dp = _f32(data)
    packed = np.zeros(data.size // 8, dtype=np.uint32)
    scales = np.zeros((data.size + group - 1) // group, dtype=np.float32)
    lib().orc_quantize_int4_per_group(dp, data.size, group, packed.ctypes.data_as(C.POINTER(C.c_uint32)),
                                      scales.ctypes.data_as(C.POINTER(C.c_float)))
    return packed, scales


def quantize_weight_int4(weight_t, k, n, group):
    """weight_t: [K,N] row-major f32 -> (packed [K/8,N] u32, scales [ceil(K/g),N] f32)."""
    w, wp = _f32(weight_t)
    assert w.size == k * n
    packed = np.zeros((k // 8, n), dtype=np.uint32)
    scales = np.zeros(((k + group - 1) // group, n), dtype=np.float32)
    rc = lib().orc_quantize_weight_int4(wp, k, n, group, packed.ctypes.data_as(C.POINTER(C.c_uint32)),
                                        scales.ctypes.data_as(C.POINTER(C.c_float)))
    if rc != 0:
        raise ValueError("K must be divisible by 8")
    return packed, scales


def unpack_int4(word, index):
    return int(lib().orc_unpack_int4(int(word), int(index)))


def dequant_weight_int4(packed, scales, k, n, group):
    p, pp = _u32(packed)
    s, sp = _f32(scales)
    out = np.empty((k, n), dtype=np.float32)
    lib().orc_dequant_weight_int4(pp, sp, k, n, group, out.ctypes.data_as(C.POINTER(C.c_float)))
    return out


def int4_linear(a, packed, scales, bias, m, n, k, group, f64=True):
    a, ap = _f32(a)
    p, pp = _u32(packed)
    s, sp = _f32(scales)
    if bias is not None:
        b, bp = _f32(bias)
    else:
        bp = None
    out = np.empty((m, n), dtype=np.float32)
    fn = lib().orc_int4_linear_f64 if f64 else lib().orc_int4_linear_f32
    fn(ap, pp, sp, bp, m, n, k, group, out.ctypes.data_as(C.POINTER(C.c_float)))
    return out


def matmul(a, b, m, k, n):
    a, ap = _f32(a)
    b, bp = _f32(b)
    out = np.empty((m, n), dtype=np.float32)
    lib().orc_matmul_f64(ap, bp, m, k, n, out.ctypes.data_as(C.POINTER(C.c_float)))
    return out


def layer_norm(x, gamma, beta, eps=1e-5):
    x, xp = _f32(x)
    g, gp = _f32(gamma)
    b, bp = _f32(beta)
    d = g.size
    out = np.empty_like(x)
    lib().orc_layer_norm_f64(xp, gp, bp, x.size // d, d, eps, out.ctypes.data_as(C.POINTER(C.c_float)))
    return out


def softmax(x, rows, cols):
    x, xp = _f32(x)
    out = np.empty_like(x)
    lib().orc_softmax_f64(xp, rows, cols, out.ctypes.data_as(C.POINTER(C.c_float)))
    return out


def attention(q, k, v, seq, d):
    q, qp = _f32(q)
    k, kp = _f32(k)
    v, vp = _f32(v)
    out = np.empty((seq, d), dtype=np.float32)
    lib().orc_attention_f64(qp, kp, vp, seq, d, out.ctypes.data_as(C.POINTER(C.c_float)))
    return out


def gelu_tanh(x):
    return np.array([lib().orc_gelu_tanh(float(v)) for v in np.ravel(x)], dtype=np.float64).reshape(np.shape(x))


def gelu_sigmoid(x):
    return np.array([lib().orc_gelu_sigmoid(float(v)) for v in np.ravel(x)], dtype=np.float64).reshape(np.shape(x))


def mha(q, kc, vc, H, dh, nq, past, cap):
    """q [nq,H*dh]; kc,vc [H,cap,dh] (new positions already appended) -> [nq,H*dh]."""
    q, qp = _f32(q)
    kc, kp = _f32(kc)
    vc, vp = _f32(vc)
    out = np.empty((nq, H * dh), dtype=np.float32)
    lib().orc_mha_f64(qp, H * dh, kp, vp, H, dh, nq, past, cap, out.ctypes.data_as(C.POINTER(C.c_float)))
    return out


class Model:
    """Oracle GPT-2 over f32 weights in checkpoint (Conv1D, [in,out]) layout.

    ``weights`` is a dict: wte [V,d], wpe [P,d], ln_f.weight/bias, and per layer
    ``h.{i}.ln_1.weight|bias``, ``h.{i}.attn.c_attn.weight [d,3d]|bias``,
    ``h.{i}.attn.c_proj.weight [d,d]|bias``, ``h.{i}.ln_2.weight|bias``,
    ``h.{i}.mlp.c_fc.weight [d,4d]|bias``, ``h.{i}.mlp.c_proj.weight [4d,d]|bias``;
    optional ``lm_head [d,V]`` replaces the tied head.
    """

    def __init__(self, cfg: dict, weights: dict):
        L = lib()
        self.cfg = OrcConfig(cfg["n_layer"], cfg["n_embd"], cfg["n_head"], cfg["vocab_size"],
                             cfg["n_positions"], cfg.get("layer_norm_epsilon", 1e-5))
        self._keep = {}

        def P(name):
            arr, ptr = _f32(weights[name])
            self._keep[name] = arr
            return ptr

        self._h = L.orc_model_create(C.byref(self.cfg), P("wte"), P("wpe"), P("ln_f.weight"), P("ln_f.bias"))
        for i in range(cfg["n_layer"]):
            p = f"h.{i}."
            L.orc_model_set_layer(self._h, i, P(p + "ln_1.weight"), P(p + "ln_1.bias"),
                                  P(p + "attn.c_attn.weight"), P(p + "attn.c_attn.bias"),
                                  P(p + "attn.c_proj.weight"), P(p + "attn.c_proj.bias"),
                                  P(p + "ln_2.weight"), P(p + "ln_2.bias"),
                                  P(p + "mlp.c_fc.weight"), P(p + "mlp.c_fc.bias"),
                                  P(p + "mlp.c_proj.weight"), P(p + "mlp.c_proj.bias"))
        if "lm_head" in weights:
            L.orc_model_set_lm_head(self._h, P("lm_head"))
        self.vocab = cfg["vocab_size"]

    def __del__(self):
        try:
            lib().orc_model_destroy(self._h)
        except Exception:
            pass

    def forward(self, tokens, last_only=False, flags=0):
        t, tp = _u32(tokens)
        rows = 1 if last_only else t.size
        out = np.empty((rows, self.vocab), dtype=np.float32)
        rc = lib().orc_forward(self._h, tp, t.size, int(last_only), flags, out.ctypes.data_as(C.POINTER(C.c_float)))
        if rc != 0:
            raise RuntimeError(f"orc_forward rc={rc}")
        return out

    def block_forward(self, layer, x, past=0, kc=None, vc=None, flags=0):
        """One block alone: x [nq,d] at positions past..; kc / vc [H,past,dh] are the cached rows.
        Returns (out [nq,d], k [H,past+nq,dh], v [H,past+nq,dh])."""
        x, xp = _f32(x)
        nq, d = x.shape
        H = self.cfg.n_head
        dh = d // H
        cap = past + nq
        k = np.zeros((H, cap, dh), dtype=np.float32)
        v = np.zeros((H, cap, dh), dtype=np.float32)
        if past:
            k[:, :past] = np.asarray(kc, dtype=np.float32).reshape(H, past, dh)
            v[:, :past] = np.asarray(vc, dtype=np.float32).reshape(H, past, dh)
        out = np.empty((nq, d), dtype=np.float32)
        f32p = C.POINTER(C.c_float)
        lib().orc_block_forward(self._h, layer, xp, nq, past, k.ctypes.data_as(f32p), v.ctypes.data_as(f32p), cap, flags,
                                out.ctypes.data_as(f32p))
        return out, k, v

    def _gen(self, fn, prompt, max_new, flags, want_logits):
        p, pp = _u32(prompt)
        out = np.zeros(p.size + max_new, dtype=np.uint32)
        lg = np.zeros((max_new, self.vocab), dtype=np.float32) if want_logits else None
        n = fn(self._h, pp, p.size, max_new, flags, out.ctypes.data_as(C.POINTER(C.c_uint32)),
               lg.ctypes.data_as(C.POINTER(C.c_float)) if want_logits else None)
        if n < 0:
            raise RuntimeError(f"oracle generate rc={n}")
        return (out[:n], lg[: n - p.size + (1 if n - p.size < max_new else 0)] if want_logits else None)

    def generate(self, prompt, max_new, flags=0, want_logits=False):
        """Uncached greedy loop (re-runs the whole sequence each step)."""
        return self._gen(lib().orc_generate, prompt, max_new, flags, want_logits)

    def generate_cached(self, prompt, max_new, flags=0, want_logits=False):
        return self._gen(lib().orc_generate_cached, prompt, max_new, flags, want_logits)

    def time_decode(self, prompt, steps, flags=0):
        p, pp = _u32(prompt)
        sec = C.c_double()
        toks = np.zeros(steps, dtype=np.uint32)
        rc = lib().orc_time_decode(self._h, pp, p.size, steps, flags, C.byref(sec),
                                   toks.ctypes.data_as(C.POINTER(C.c_uint32)))
        if rc != 0:
            raise RuntimeError(f"orc_time_decode rc={rc}")
        return float(sec.value), toks

    def generate_cached_sampling(self, prompt, max_new, top_k, temperature, rng: "SimpleRng", flags=0):
        """generate_cached_sampling (gpt2.rs:933-977) -> (tokens, step logits, margin of every draw)."""
        p, pp = _u32(prompt)
        out = np.zeros(p.size + max_new, dtype=np.uint32)
        lg = np.zeros((max_new, self.vocab), dtype=np.float32)
        mg = np.ones(max_new, dtype=np.float32)
        n = lib().orc_generate_cached_sampling(self._h, pp, p.size, max_new, top_k, temperature, C.byref(rng.state), flags,
                                               out.ctypes.data_as(C.POINTER(C.c_uint32)),
                                               lg.ctypes.data_as(C.POINTER(C.c_float)),
                                               mg.ctypes.data_as(C.POINTER(C.c_float)))
        if n < 0:
            raise RuntimeError(f"orc_generate_cached_sampling rc={n}")
        return out[:n], lg, mg

    def forward_early_exit(self, tokens, threshold, flags=0):
        """forward_early_exit (gpt2.rs:797-830) -> (logits [seq,vocab], layers used, probe confidences)."""
        t, tp = _u32(tokens)
        out = np.empty((t.size, self.vocab), dtype=np.float32)
        used = C.c_int32()
        conf = np.full(max(self.cfg.n_layer - 1, 1), np.nan, dtype=np.float32)
        rc = lib().orc_forward_early_exit(self._h, tp, t.size, threshold, flags, out.ctypes.data_as(C.POINTER(C.c_float)),
                                          C.byref(used), conf.ctypes.data_as(C.POINTER(C.c_float)))
        if rc != 0:
            raise RuntimeError(f"orc_forward_early_exit rc={rc}")
        return out, int(used.value), conf

    def generate_cached_early_exit(self, prompt, max_new, threshold, flags=0):
        """generate_cached_early_exit (gpt2.rs:837-924) -> (tokens, layers per step, step logits, smallest
        |confidence - threshold| met)."""
        p, pp = _u32(prompt)
        out = np.zeros(p.size + max_new, dtype=np.uint32)
        layers = np.zeros(1 + max_new, dtype=np.int32)
        steps, gap = C.c_int32(), C.c_float()
        lg = np.zeros((max(max_new, 1), self.vocab), dtype=np.float32)
        n = lib().orc_generate_cached_early_exit(self._h, pp, p.size, max_new, threshold, flags,
                                                 out.ctypes.data_as(C.POINTER(C.c_uint32)),
                                                 layers.ctypes.data_as(C.POINTER(C.c_int32)), C.byref(steps),
                                                 lg.ctypes.data_as(C.POINTER(C.c_float)), C.byref(gap))
        if n < 0:
            raise RuntimeError(f"orc_generate_cached_early_exit rc={n}")
        return out[:n], layers[: steps.value], lg, float(gap.value)


class SimpleRng:
    """SimpleRng (gpt2.rs:1000-1023)."""

    def __init__(self, seed: int):
        self.state = C.c_uint64(lib().orc_rng_new(seed))

    def next_f32(self) -> float:
        return float(lib().orc_rng_next_f32(C.byref(self.state)))


def top_k_sample(logits, k, temperature, rng: SimpleRng):
    """top_k_sample (gpt2.rs:1029-1058) -> (token, margin of the draw)."""
    a, ap = _f32(logits)
    mg = C.c_float()
    t = lib().orc_top_k_sample(ap, a.size, k, temperature, C.byref(rng.state), C.byref(mg))
    return int(t), float(mg.value)


def softmax_max_prob(logits):
    a, ap = _f32(logits)
    return float(lib().orc_softmax_max_prob(ap, a.size))
