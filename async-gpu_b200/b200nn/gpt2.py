"""GPT-2 models, named as in ``gpu_host::nn::models::gpt2`` (models/gpt2.rs)."""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass

import numpy as np

from . import (ERR_SHAPE, GpuTensor, KernelRegistry, NnError, PROF_NAMES, _BlockW, _Cfg, _Diag, _LayerW, _Weights, _f32,
               _f32p, _u32, _u32p)


@dataclass
class Gpt2Config:
    """``Gpt2Config`` (gpt2.rs:20-93)."""
    n_layer: int = 12
    n_embd: int = 768
    n_head: int = 12
    vocab_size: int = 50257
    n_positions: int = 1024
    layer_norm_epsilon: float = 1e-5

    @classmethod
    def small(cls):
        return cls(12, 768, 12)

    @classmethod
    def medium(cls):
        return cls(24, 1024, 16)

    @classmethod
    def large(cls):
        return cls(36, 1280, 20)

    @classmethod
    def xl(cls):
        return cls(48, 1600, 25)

    def head_dim(self):
        return self.n_embd // self.n_head

    def ffn_dim(self):
        return 4 * self.n_embd

    def as_dict(self):
        return dict(n_layer=self.n_layer, n_embd=self.n_embd, n_head=self.n_head, vocab_size=self.vocab_size,
                    n_positions=self.n_positions, layer_norm_epsilon=self.layer_norm_epsilon)

    def _c(self):
        return _Cfg(self.n_layer, self.n_embd, self.n_head, self.vocab_size, self.n_positions, self.layer_norm_epsilon)


_LAYER_KEYS = [("ln_1_weight", "ln_1.weight", 1), ("ln_1_bias", "ln_1.bias", 1),
               ("c_attn_weight", "attn.c_attn.weight", 3), ("c_attn_bias", "attn.c_attn.bias", 3),
               ("c_proj_weight", "attn.c_proj.weight", 1), ("c_proj_bias", "attn.c_proj.bias", 1),
               ("ln_2_weight", "ln_2.weight", 1), ("ln_2_bias", "ln_2.bias", 1),
               ("mlp_fc_weight", "mlp.c_fc.weight", 4), ("mlp_fc_bias", "mlp.c_fc.bias", 4),
               ("mlp_proj_weight", "mlp.c_proj.weight", 4), ("mlp_proj_bias", "mlp.c_proj.bias", 1)]


def _pack_weights(cfg: Gpt2Config, weights: dict):
    """``Gpt2Weights`` (model.rs:112-154) from a dict keyed as the checkpoint is: ``wte``, ``wpe``,
    ``ln_f.weight|bias`` and ``h.{i}.<name>`` with dense weights in Conv1D layout [in,out]."""
    keep = []
    d = cfg.n_embd

    def P(name, numel):
        a, p = _f32(weights[name])
        if a.size != numel:
            raise NnError(ERR_SHAPE, f"{name}: expected {numel} elements, got {a.size}")
        keep.append(a)
        return p

    layers = (_LayerW * cfg.n_layer)()
    for i in range(cfg.n_layer):
        for field, key, mult in _LAYER_KEYS:
            numel = mult * d * (d if field.endswith("_weight") and not field.startswith("ln_") else 1)
            setattr(layers[i], field, P(f"h.{i}.{key}", numel))
    w = _Weights(P("wte", cfg.vocab_size * d), P("wpe", cfg.n_positions * d), P("ln_f.weight", d), P("ln_f.bias", d),
                 layers)
    keep.append(layers)
    return w, keep


class KvCache:
    """Device KV cache (``KvCache``, gpt2.rs:1064-1117) with a batch axis."""

    def __init__(self, model: "Gpt2Model", batch: int = 1, capacity: int | None = None):
        self.model = model
        self.h = C.c_void_p()
        cap = capacity or model.config.n_positions
        model.reg.check(model.reg.lib.b200nn_kvcache_create(model.h, batch, cap, C.byref(self.h)))

    def len(self):
        return int(self.model.reg.lib.b200nn_kvcache_len(self.h))

    def is_empty(self):
        return self.len() == 0

    def reset(self):
        self.model.reg.check(self.model.reg.lib.b200nn_kvcache_reset(self.h))

    def __del__(self):
        try:
            if self.h and self.model.h and self.model.reg.h:
                self.model.reg.lib.b200nn_kvcache_destroy(self.h)
        except Exception:
            pass


class Gpt2Model:
    """``Gpt2Model::from_weights`` (gpt2.rs:337-404) and its forward / generate family."""
    _int4 = False

    def __init__(self, weights: dict, config: Gpt2Config, reg: KernelRegistry, flags: int = 0, group_size: int = 128):
        self.reg, self.config, self.flags = reg, config, flags
        cw, keep = _pack_weights(config, weights)
        cc = config._c()
        self.h = C.c_void_p()
        if self._int4:
            rc = reg.lib.b200nn_int4_gpt2_create(reg.h, C.byref(cc), C.byref(cw), group_size, flags, C.byref(self.h))
        else:
            rc = reg.lib.b200nn_gpt2_create(reg.h, C.byref(cc), C.byref(cw), flags, C.byref(self.h))
        del keep
        reg.check(rc)
        self._group_size = group_size

    @classmethod
    def from_weights(cls, weights, config, reg, **kw):
        return cls(weights, config, reg, **kw)

    @classmethod
    def from_generic_weights(cls, weights, config, reg, **kw):
        """``Gpt2Model::from_generic_weights`` / ``Int4Gpt2Model::from_generic_weights`` (gpt2.rs:410-476,
        1436-1500): ``weights`` is the generic loader's ``LoadedWeights`` under GPT-2's key names, the four
        dense weights of every block already transposed to Linear layout [out,in] (``gpt2_weight_map``).
        A key that is missing is the reference's ``ShapeMismatch { expected: key, .. }``."""
        from . import WEIGHTS_OUT_IN

        def need(key):
            t = weights.get(key)
            if t is None:
                raise NnError(ERR_SHAPE, f"ShapeMismatch: expected {key}, got MissingTensor")
            return t.data

        w = {"wte": need("wte.weight"), "wpe": need("wpe.weight"), "ln_f.weight": need("ln_f.weight"),
             "ln_f.bias": need("ln_f.bias")}
        for i in range(config.n_layer):
            for _, key, _ in _LAYER_KEYS:
                w[f"h.{i}.{key}"] = need(f"h.{i}.{key}")
        kw["flags"] = kw.get("flags", 0) | WEIGHTS_OUT_IN
        return cls(w, config, reg, **kw)

    @classmethod
    def from_safetensors(cls, path, reg: KernelRegistry, config: Gpt2Config | None = None, flags: int = 0,
                         group_size: int = 128):
        """``load_gpt2_weights`` (model.rs:308-386) + ``from_weights`` in the library: an F32 checkpoint
        with Hugging Face key names.  ``config=None`` reads the shape off the file."""
        self = cls.__new__(cls)
        self.reg, self.flags, self._group_size = reg, flags, group_size
        self.h = C.c_void_p()
        cc = config._c() if config is not None else None
        rc = reg.lib.b200nn_gpt2_load_safetensors(reg.h, os.fsencode(path), C.byref(cc) if cc is not None else None,
                                                  group_size if cls._int4 else 0, flags, C.byref(self.h))
        reg.check(rc)
        got = _Cfg()
        reg.check(reg.lib.b200nn_gpt2_get_config(self.h, C.byref(got)))
        self.config = Gpt2Config(n_layer=got.n_layer, n_embd=got.n_embd, n_head=got.n_head, vocab_size=got.vocab_size,
                                 n_positions=got.n_positions, layer_norm_epsilon=got.layer_norm_epsilon)
        return self

    def forward(self, token_ids, seq_len=None) -> GpuTensor:
        t, tp = _u32(token_ids)
        n = t.size if seq_len is None else seq_len
        h = C.c_void_p()
        self.reg.check(self.reg.lib.b200nn_gpt2_forward(self.h, tp, n, C.byref(h)))
        return GpuTensor(self.reg, h)

    def forward_auto_fused(self, token_ids, seq_len=None) -> GpuTensor:
        """``forward_auto_fused`` (gpt2.rs:500-522): here every forward already runs the fused epilogues."""
        return self.forward(token_ids, seq_len)

    def forward_features(self, token_ids) -> GpuTensor:
        """``forward_features`` (gpt2.rs:570-581): [seq, n_embd] after the final LayerNorm."""
        t, tp = _u32(token_ids)
        h = C.c_void_p()
        self.reg.check(self.reg.lib.b200nn_gpt2_forward_features(self.h, tp, t.size, C.byref(h)))
        return GpuTensor(self.reg, h)

    def embedding_table(self):
        """``embedding_table`` (gpt2.rs:584-586) -> (wte [vocab,d], wpe [positions,d]) on the device."""
        a, b = C.c_void_p(), C.c_void_p()
        self.reg.check(self.reg.lib.b200nn_gpt2_embedding_table(self.h, C.byref(a), C.byref(b)))
        return GpuTensor(self.reg, a), GpuTensor(self.reg, b)

    def forward_profiled(self, token_ids):
        """``forward_profiled`` (gpt2.rs:529-568) -> (logits, [(component, milliseconds), ...])."""
        t, tp = _u32(token_ids)
        n_max = self.config.n_layer + 3
        times = (C.c_float * n_max)()
        h, n = C.c_void_p(), C.c_int32()
        self.reg.check(self.reg.lib.b200nn_gpt2_forward_profiled(self.h, tp, t.size, C.byref(h), times, n_max, C.byref(n)))
        names = ["embedding"] + [f"block_{i}" for i in range(self.config.n_layer)] + ["ln_f", "lm_head"]
        return GpuTensor(self.reg, h), list(zip(names, [float(times[i]) for i in range(n.value)]))

    def forward_diagnostic(self, token_ids, file=None):
        """``forward_diagnostic`` (gpt2.rs:595-667): forward that prints the reference's ``[diag]`` lines
        (to ``file``, default stderr) and returns (logits, the reported values as a dict)."""
        import sys
        t, tp = _u32(token_ids)
        h, dg = C.c_void_p(), _Diag()
        self.reg.check(self.reg.lib.b200nn_gpt2_forward_diagnostic(self.h, tp, t.size, C.byref(h), C.byref(dg)))
        last, out = t.size - 1, file or sys.stderr
        f4 = lambda a: "[" + ", ".join(f"{float(v):.6f}" for v in a) + "]"
        print(f"[diag] Embedding pos0 first4: {f4(dg.embedding_first)}", file=out)
        print(f"[diag] Embedding pos{last} first4: {f4(dg.embedding_last)}", file=out)
        for i, vals, bad in ((0, dg.block0_last, dg.block0_nonfinite),
                             (self.config.n_layer - 1, dg.final_block_last, dg.final_block_nonfinite)):
            print(f"[diag] Layer {i} pos{last} first4: {f4(vals)}", file=out)
            if bad:
                print(f"[diag] WARNING: Layer {i} has {bad} NaN/Inf values!", file=out)
        print(f"[diag] Final LN pos{last} first4: {f4(dg.ln_f_last)}", file=out)
        print(f"[diag] Top-5 tokens at pos{last}:", file=out)
        top = [(int(dg.top_tokens[i]), float(dg.top_scores[i])) for i in range(dg.n_top)]
        for tok, score in top:
            print(f"  token {tok}: {score:.4f}", file=out)
        report = {"embedding_first": list(dg.embedding_first), "embedding_last": list(dg.embedding_last),
                  "block0_last": list(dg.block0_last), "final_block_last": list(dg.final_block_last),
                  "block0_nonfinite": dg.block0_nonfinite, "final_block_nonfinite": dg.final_block_nonfinite,
                  "ln_f_last": list(dg.ln_f_last), "top": top}
        return GpuTensor(self.reg, h), report

    def forward_cached(self, token_ids, new_len, cache: KvCache) -> GpuTensor:
        t, tp = _u32(token_ids)
        h = C.c_void_p()
        self.reg.check(self.reg.lib.b200nn_gpt2_forward_cached(self.h, tp, new_len, cache.h, C.byref(h)))
        return GpuTensor(self.reg, h)

    def _gen(self, fn, prompt, max_new, flags):
        p, pp = _u32(prompt)
        out = np.zeros(p.size + max_new, dtype=np.uint32)
        n = C.c_size_t()
        self.reg.check(fn(self.h, pp, p.size, max_new, self.flags | flags, out.ctypes.data_as(_u32p), C.byref(n)))
        return out[: n.value]

    def generate(self, prompt_tokens, max_new_tokens, flags: int = 8):
        """Greedy; by default stops before appending token 50256 as the reference does."""
        return self._gen(self.reg.lib.b200nn_gpt2_generate, prompt_tokens, max_new_tokens, flags)

    def generate_cached(self, prompt_tokens, max_new_tokens, flags: int = 8):
        return self._gen(self.reg.lib.b200nn_gpt2_generate_cached, prompt_tokens, max_new_tokens, flags)

    def generate_cached_sampling(self, prompt_tokens, max_new_tokens, top_k, temperature, rng: "SimpleRng"):
        """``generate_cached_sampling`` (gpt2.rs:933-977); ``rng`` advances one draw per token."""
        p, pp = _u32(prompt_tokens)
        out = np.zeros(p.size + max_new_tokens, dtype=np.uint32)
        n = C.c_size_t()
        self.reg.check(self.reg.lib.b200nn_gpt2_generate_cached_sampling(
            self.h, pp, p.size, max_new_tokens, top_k, temperature, C.byref(rng.state), out.ctypes.data_as(_u32p),
            C.byref(n)))
        return out[: n.value]

    def forward_early_exit(self, token_ids, threshold):
        """``forward_early_exit`` (gpt2.rs:797-830) -> (logits tensor [seq,vocab], layers used)."""
        t, tp = _u32(token_ids)
        h, used = C.c_void_p(), C.c_int32()
        self.reg.check(self.reg.lib.b200nn_gpt2_forward_early_exit(self.h, tp, t.size, threshold, C.byref(h),
                                                                   C.byref(used)))
        return GpuTensor(self.reg, h), int(used.value)

    def generate_cached_early_exit(self, prompt_tokens, max_new_tokens, threshold):
        """``generate_cached_early_exit`` (gpt2.rs:837-924) -> (tokens, layers used per step, prefill first)."""
        p, pp = _u32(prompt_tokens)
        out = np.zeros(p.size + max_new_tokens, dtype=np.uint32)
        layers = np.zeros(1 + max_new_tokens, dtype=np.int32)
        n, steps = C.c_size_t(), C.c_size_t()
        self.reg.check(self.reg.lib.b200nn_gpt2_generate_cached_early_exit(
            self.h, pp, p.size, max_new_tokens, threshold, out.ctypes.data_as(_u32p), C.byref(n),
            layers.ctypes.data_as(C.POINTER(C.c_int32)), C.byref(steps)))
        return out[: n.value], layers[: steps.value]

    def generate_batch(self, prompts, max_new_tokens, flags: int = 0):
        """prompts [batch, prompt_len] -> (tokens [batch, prompt_len+max_new], lengths [batch])."""
        p = np.ascontiguousarray(prompts, dtype=np.uint32)
        batch, plen = p.shape
        out = np.zeros((batch, plen + max_new_tokens), dtype=np.uint32)
        lens = (C.c_size_t * batch)()
        self.reg.check(self.reg.lib.b200nn_gpt2_generate_batch(
            self.h, p.ctypes.data_as(_u32p), batch, plen, max_new_tokens, self.flags | flags,
            out.ctypes.data_as(_u32p), lens))
        return out, np.array(list(lens), dtype=np.int64)

    def quantized_memory_bytes(self):
        return int(self.reg.lib.b200nn_gpt2_quantized_memory_bytes(self.h))

    def get_int4(self, layer: int, which: int):
        """(packed [K/8,N], scales [ceil(K/g),N] fp16-rounded, K, N) the model holds for one Linear."""
        k, n = C.c_size_t(), C.c_size_t()
        self.reg.check(self.reg.lib.b200nn_gpt2_get_int4(self.h, layer, which, None, None, C.byref(k), C.byref(n)))
        K, N, g = k.value, n.value, self._group_size
        packed = np.zeros((K // 8, N), dtype=np.uint32)
        scales = np.zeros(((K + g - 1) // g, N), dtype=np.float32)
        self.reg.check(self.reg.lib.b200nn_gpt2_get_int4(self.h, layer, which, packed.ctypes.data_as(_u32p),
                                                         scales.ctypes.data_as(_f32p), None, None))
        return packed, scales, K, N

    def __del__(self):
        try:
            if self.h and self.reg.h:
                self.reg.lib.b200nn_gpt2_destroy(self.h)
                self.h = None
        except Exception:
            pass


class Int4Gpt2Model(Gpt2Model):
    """``Int4Gpt2Model::from_weights(weights, config, group_size, &registry)`` (gpt2.rs:1356-1436)."""
    _int4 = True
    DEFAULT_GROUP_SIZE = 128

    def group_size(self):
        return self._group_size


class DecodeSession:
    """The batched greedy loop in pieces with all state on the device: prefill, then steps."""

    def __init__(self, model: Gpt2Model, batch: int, capacity: int, flags: int = 0):
        self.model, self.reg, self.batch, self.capacity = model, model.reg, batch, capacity
        self.h = C.c_void_p()
        self.reg.check(self.reg.lib.b200nn_session_create(model.h, batch, capacity, model.flags | flags, C.byref(self.h)))

    def prefill(self, prompts):
        p = np.ascontiguousarray(prompts, dtype=np.uint32)
        assert p.shape[0] == self.batch
        self.reg.check(self.reg.lib.b200nn_session_prefill(self.h, p.ctypes.data_as(_u32p), p.shape[1]))

    def step(self, n_steps: int = 1):
        self.reg.check(self.reg.lib.b200nn_session_step(self.h, n_steps))

    def rewind(self, position: int):
        """Timing aid: moves the position counter back; the cache keeps its contents."""
        self.reg.check(self.reg.lib.b200nn_session_rewind(self.h, position))

    def position(self):
        return int(self.reg.lib.b200nn_session_position(self.h))

    def tokens(self):
        out = np.zeros((self.batch, self.capacity), dtype=np.uint32)
        n = C.c_size_t()
        self.reg.check(self.reg.lib.b200nn_session_tokens(self.h, out.ctypes.data_as(_u32p), self.capacity, C.byref(n)))
        return out[:, : n.value]

    def logits(self):
        out = np.empty((self.batch, self.model.config.vocab_size), dtype=np.float32)
        self.reg.check(self.reg.lib.b200nn_session_logits(self.h, out.ctypes.data_as(_f32p)))
        return out

    def profile_step(self):
        t = (C.c_float * len(PROF_NAMES))()
        b = C.c_uint64()
        self.reg.check(self.reg.lib.b200nn_session_profile_step(self.h, t, C.byref(b)))
        return {n: float(t[i]) for i, n in enumerate(PROF_NAMES)}, int(b.value)

    def time_family(self, family: str, reps: int = 3):
        """(milliseconds, launches) of one kernel family run alone `reps` times; prefill again afterwards."""
        ms = C.c_float()
        n = C.c_uint64()
        self.reg.check(self.reg.lib.b200nn_session_time_family(self.h, PROF_NAMES.index(family), reps, C.byref(ms),
                                                               C.byref(n)))
        return float(ms.value), int(n.value)

    def __del__(self):
        try:
            if self.h and self.model.h and self.reg.h:
                self.reg.lib.b200nn_session_destroy(self.h)
        except Exception:
            pass


class TransformerBlock:
    """``TransformerBlock::new(ln_1_weight, ln_1_bias, attn_qkv_weight, attn_qkv_bias, attn_out_weight,
    attn_out_bias, ln_2_weight, ln_2_bias, ffn_up_weight, ffn_up_bias, ffn_down_weight, ffn_down_bias, &config,
    &registry)`` (gpt2.rs:98-170): one pre-LN block; dense weights in Linear layout [out,in]."""
    _create = "b200nn_block_create"

    def __init__(self, ln_1_weight, ln_1_bias, attn_qkv_weight, attn_qkv_bias, attn_out_weight, attn_out_bias,
                 ln_2_weight, ln_2_bias, ffn_up_weight, ffn_up_bias, ffn_down_weight, ffn_down_bias,
                 config: Gpt2Config, reg: KernelRegistry, flags: int = 0, **extra):
        d = config.n_embd
        sizes = [d, d, 3 * d * d, 3 * d, d * d, d, d, d, 4 * d * d, 4 * d, 4 * d * d, d]
        arrs = [np.ascontiguousarray(a, dtype=np.float32) for a in (
            ln_1_weight, ln_1_bias, attn_qkv_weight, attn_qkv_bias, attn_out_weight, attn_out_bias, ln_2_weight,
            ln_2_bias, ffn_up_weight, ffn_up_bias, ffn_down_weight, ffn_down_bias)]
        for a, n in zip(arrs, sizes):
            if a.size != n:
                raise NnError(ERR_SHAPE, f"TransformerBlock: expected {n} elements, got {a.size}")
        self.reg, self.config, self._keep = reg, config, arrs
        w = _BlockW(*[a.ctypes.data_as(_f32p) for a in arrs])
        cfg = config._c()
        self.h = C.c_void_p()
        reg.check(self._call_create(reg, cfg, w, flags, extra))

    def _call_create(self, reg, cfg, w, flags, extra):
        return reg.lib.b200nn_block_create(reg.h, C.byref(cfg), C.byref(w), flags, C.byref(self.h))

    def forward(self, x: GpuTensor) -> GpuTensor:
        """input [seq_len, n_embd] -> output [seq_len, n_embd] (gpt2.rs:172-204)."""
        h = C.c_void_p()
        self.reg.check(self.reg.lib.b200nn_block_forward(self.h, x.h, C.byref(h)))
        return GpuTensor(self.reg, h)

    forward_auto_fused = forward  # the fused epilogues are always on (gpt2.rs:206-243)

    def forward_auto_fused(self, x: GpuTensor) -> GpuTensor:
        """``TransformerBlock::forward_auto_fused`` (gpt2.rs:206-247): the fused epilogues are always on here."""
        return self.forward(x)

    def forward_cached(self, x: GpuTensor, cached_k, cached_v, kv_len: int):
        """``forward_cached(input, cached_k, cached_v, kv_len) -> (output, new_k, new_v)`` (gpt2.rs:249-288);
        cached_k / cached_v: [n_head][kv_len*64]; new_k / new_v: [n_head, new_len*64]."""
        H, new_len = self.config.n_head, x.shape()[0]
        ck = cv = None
        if kv_len:
            ka, ck = _f32(np.asarray(cached_k, dtype=np.float32))
            va, cv = _f32(np.asarray(cached_v, dtype=np.float32))
            if ka.size != H * kv_len * 64 or va.size != H * kv_len * 64:
                raise NnError(ERR_SHAPE, "forward_cached: cached K/V must hold n_head x kv_len x 64 values")
        nk = np.empty((H, new_len * 64), dtype=np.float32)
        nv = np.empty_like(nk)
        h = C.c_void_p()
        self.reg.check(self.reg.lib.b200nn_block_forward_cached(self.h, x.h, ck, cv, kv_len, C.byref(h),
                                                                nk.ctypes.data_as(_f32p), nv.ctypes.data_as(_f32p)))
        return GpuTensor(self.reg, h), nk, nv

    def __del__(self):
        try:
            if self.h and self.reg.h:
                self.reg.lib.b200nn_block_destroy(self.h)
        except Exception:
            pass


class Int4TransformerBlock(TransformerBlock):
    """``Int4TransformerBlock::new(..., &config, group_size, &registry)`` (gpt2.rs:1219-1296): the same twelve
    slices, every dense weight quantised to int4 with ``group_size`` (attention through
    ``Int4MultiHeadAttention``, gpt2.rs:1127-1214)."""

    def __init__(self, *args, group_size: int = 128, **kw):
        super().__init__(*args, group_size=group_size, **kw)

    def _call_create(self, reg, cfg, w, flags, extra):
        return reg.lib.b200nn_int4_block_create(reg.h, C.byref(cfg), C.byref(w), extra.get("group_size", 128), flags,
                                                C.byref(self.h))
