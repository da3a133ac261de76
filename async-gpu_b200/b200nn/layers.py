"""Layers, named as in ``gpu_host::nn::layers`` (layers/mod.rs:36-39: ``Module::forward``)."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import (ACT_NONE, ERR_SHAPE, GpuTensor, KernelRegistry, NnError, _f32, _f32p, _out, _u32, _u32p)
from . import ops


class _Module:
    _destroy = None

    def __del__(self):
        try:
            if getattr(self, "h", None) and self.reg.h and self._destroy:
                getattr(self.reg.lib, self._destroy)(self.h)
        except Exception:
            pass


class Linear(_Module):
    """``Linear::new(weight [out,in], bias, in, out, &registry)`` (layers/linear.rs:58-88)."""
    _destroy = "b200nn_linear_destroy"

    def __init__(self, weight, bias, in_features, out_features, reg: KernelRegistry):
        w, wp = _f32(weight)
        if w.size != in_features * out_features:
            raise NnError(ERR_SHAPE, f"weight: expected {out_features}x{in_features}, got {w.size} elements")
        bp = None
        if bias is not None:
            b, bp = _f32(bias)
            if b.size != out_features:
                raise NnError(ERR_SHAPE, f"bias: expected {out_features}, got {b.size}")
        self.reg = reg
        self.h = C.c_void_p()
        reg.check(reg.lib.b200nn_linear_create(reg.h, wp, bp, in_features, out_features, C.byref(self.h)))

    @classmethod
    def with_codegen(cls, weight, bias, in_features, out_features, reg: KernelRegistry, codegen=None):
        """``Linear::with_codegen`` (layers/linear.rs:94-125).  The reference hands over its run-time kernel
        generator for ``forward_auto_fused``; the epilogues are compiled into the library here, so the
        argument is accepted and not used."""
        return cls(weight, bias, in_features, out_features, reg)

    def forward(self, x: GpuTensor) -> GpuTensor:
        h = C.c_void_p()
        return _out(self.reg, self.reg.lib.b200nn_linear_forward(self.h, x.h, C.byref(h)), h)

    def forward_fused(self, x: GpuTensor, activation: int = ACT_NONE) -> GpuTensor:
        h = C.c_void_p()
        return _out(self.reg, self.reg.lib.b200nn_linear_forward_fused(self.h, x.h, activation, C.byref(h)), h)

    forward_auto_fused = forward_fused


class Int4Linear(_Module):
    """``Int4Linear::new(packed [K/8,N], scales [ceil(K/g),N], bias, in, out, group, &registry)``
    (layers/int4_linear.rs:40-68)."""
    _destroy = "b200nn_int4_linear_destroy"

    def __init__(self, packed, scales, bias, in_features, out_features, group_size, reg: KernelRegistry):
        p, pp = _u32(packed)
        s, sp = _f32(scales)
        n_groups = (in_features + group_size - 1) // group_size if group_size else 0
        if in_features % 8 or p.size != (in_features // 8) * out_features or s.size != n_groups * out_features:
            raise NnError(ERR_SHAPE, "packed must be [K/8,N] and scales [ceil(K/group),N] with K%8==0")
        bp = None
        if bias is not None:
            b, bp = _f32(bias)
            if b.size != out_features:
                raise NnError(ERR_SHAPE, f"bias: expected {out_features}, got {b.size}")
        self.reg = reg
        self.in_features, self.out_features = in_features, out_features
        self.h = C.c_void_p()
        reg.check(reg.lib.b200nn_int4_linear_create(reg.h, pp, sp, bp, in_features, out_features, group_size,
                                                    C.byref(self.h)))

    def forward(self, x: GpuTensor) -> GpuTensor:
        h = C.c_void_p()
        return _out(self.reg, self.reg.lib.b200nn_int4_linear_forward(self.h, x.h, C.byref(h)), h)

    def forward_dev(self, x_ptr: int, m: int, y_ptr: int):
        """Device pointers in and out, enqueued on the registry's stream, no synchronisation."""
        self.reg.check(self.reg.lib.b200nn_int4_linear_forward_dev(self.h, x_ptr, m, y_ptr))

    def forward_host(self, x: np.ndarray) -> np.ndarray:
        a, ap = _f32(x)
        m = a.size // self.in_features
        out = np.empty((m, self.out_features), dtype=np.float32)
        self.reg.check(self.reg.lib.b200nn_int4_linear_forward_host(self.h, ap, m, out.ctypes.data_as(_f32p)))
        return out

    def memory_bytes(self) -> int:
        return int(self.reg.lib.b200nn_int4_linear_memory_bytes(self.h))


class LayerNorm(_Module):
    """``LayerNorm::new(gamma, beta, eps, &registry)`` (layers/norm.rs:24-38)."""
    _destroy = "b200nn_layernorm_destroy"

    def __init__(self, gamma, beta, eps, reg: KernelRegistry):
        g, gp = _f32(gamma)
        b, bp = _f32(beta)
        if g.size != b.size or g.size == 0:
            raise NnError(ERR_SHAPE, "gamma and beta must have the same non-zero length")
        self.reg = reg
        self.h = C.c_void_p()
        reg.check(reg.lib.b200nn_layernorm_create(reg.h, gp, bp, g.size, eps, C.byref(self.h)))
        self._g, self._b, self._gt, self._bt = g.copy(), b.copy(), None, None

    def gamma(self) -> GpuTensor:
        """``LayerNorm::gamma`` (layers/norm.rs:41-43): the scale vector as a device tensor."""
        if self._gt is None:
            self._gt = GpuTensor.from_host(self._g, (self._g.size,), self.reg)
        return self._gt

    def beta(self) -> GpuTensor:
        """``LayerNorm::beta`` (layers/norm.rs:46-48): the shift vector as a device tensor."""
        if self._bt is None:
            self._bt = GpuTensor.from_host(self._b, (self._b.size,), self.reg)
        return self._bt

    def forward(self, x: GpuTensor) -> GpuTensor:
        h = C.c_void_p()
        return _out(self.reg, self.reg.lib.b200nn_layernorm_forward(self.h, x.h, C.byref(h)), h)


class Embedding(_Module):
    """``Embedding::new(wte, wpe, vocab, max_seq, d, &registry)`` (layers/embedding.rs:25-40)."""
    _destroy = "b200nn_embedding_destroy"

    def __init__(self, wte, wpe, vocab_size, max_seq_len, d_model, reg: KernelRegistry):
        w, wp = _f32(wte)
        p, pp = _f32(wpe)
        if w.size != vocab_size * d_model or p.size != max_seq_len * d_model:
            raise NnError(ERR_SHAPE, "wte must be [vocab,d] and wpe [max_seq,d]")
        self.reg = reg
        self.h = C.c_void_p()
        reg.check(reg.lib.b200nn_embedding_create(reg.h, wp, pp, vocab_size, max_seq_len, d_model, C.byref(self.h)))

    def forward_tokens(self, token_ids, seq_len=None) -> GpuTensor:
        return self.forward_tokens_with_offset(token_ids, seq_len, 0)

    def forward_tokens_with_offset(self, token_ids, seq_len=None, pos_offset=0) -> GpuTensor:
        t, tp = _u32(token_ids)
        n = t.size if seq_len is None else seq_len
        h = C.c_void_p()
        return _out(self.reg, self.reg.lib.b200nn_embedding_forward_tokens(self.h, tp, n, pos_offset, C.byref(h)), h)


class MultiHeadAttention(_Module):
    """``MultiHeadAttention::new(qkv_w [3d,d], qkv_b, out_w [d,d], out_b, d, heads, &registry)``
    (layers/attention.rs:30-52)."""
    _destroy = "b200nn_attention_destroy"

    def __init__(self, qkv_weight, qkv_bias, out_weight, out_bias, n_embd, n_heads, reg: KernelRegistry):
        qw, qwp = _f32(qkv_weight)
        qb, qbp = _f32(qkv_bias)
        ow, owp = _f32(out_weight)
        ob, obp = _f32(out_bias)
        if qw.size != 3 * n_embd * n_embd or qb.size != 3 * n_embd or ow.size != n_embd * n_embd or ob.size != n_embd:
            raise NnError(ERR_SHAPE, "attention weights do not match n_embd")
        self.reg = reg
        self.n_heads, self.d_head = n_heads, n_embd // n_heads
        self.h = C.c_void_p()
        reg.check(reg.lib.b200nn_attention_create(reg.h, qwp, qbp, owp, obp, n_embd, n_heads, C.byref(self.h)))

    def forward_causal(self, x: GpuTensor) -> GpuTensor:
        h = C.c_void_p()
        return _out(self.reg, self.reg.lib.b200nn_attention_forward_causal(self.h, x.h, C.byref(h)), h)

    def forward_cached(self, x: GpuTensor, cached_k, cached_v, kv_len):
        """cached_k/v: [n_heads][kv_len*d_head]; returns (output, new_k [H,new*dh], new_v)."""
        new_len = x.shape()[0]
        ck = cv = None
        if kv_len:
            ka, ck = _f32(np.asarray(cached_k, dtype=np.float32))
            va, cv = _f32(np.asarray(cached_v, dtype=np.float32))
        nk = np.empty((self.n_heads, new_len * self.d_head), dtype=np.float32)
        nv = np.empty_like(nk)
        h = C.c_void_p()
        self.reg.check(self.reg.lib.b200nn_attention_forward_cached(
            self.h, x.h, ck, cv, kv_len, C.byref(h), nk.ctypes.data_as(_f32p), nv.ctypes.data_as(_f32p)))
        return GpuTensor(self.reg, h), nk, nv


class Int4MultiHeadAttention(MultiHeadAttention):
    """``Int4MultiHeadAttention::new(qkv_w [3d,d], qkv_b, out_w [d,d], out_b, d, heads, group_size, &registry)``
    (models/gpt2.rs:1127-1214): both projections quantised to int4 at construction."""

    def __init__(self, qkv_weight, qkv_bias, out_weight, out_bias, n_embd, n_heads, group_size, reg: KernelRegistry):
        qw, qwp = _f32(qkv_weight)
        qb, qbp = _f32(qkv_bias)
        ow, owp = _f32(out_weight)
        ob, obp = _f32(out_bias)
        if qw.size != 3 * n_embd * n_embd or qb.size != 3 * n_embd or ow.size != n_embd * n_embd or ob.size != n_embd:
            raise NnError(ERR_SHAPE, "attention weights do not match n_embd")
        self.reg = reg
        self.n_heads, self.d_head = n_heads, n_embd // n_heads
        self.h = C.c_void_p()
        reg.check(reg.lib.b200nn_int4_attention_create(reg.h, qwp, qbp, owp, obp, n_embd, n_heads, group_size, C.byref(self.h)))


class GELU:
    """``GELU::new(&registry)`` (layers/activation.rs:15-33)."""

    def __init__(self, reg: KernelRegistry, sigmoid_form: bool = False):
        self.reg, self.sigmoid_form = reg, sigmoid_form

    def forward(self, x: GpuTensor) -> GpuTensor:
        return ops.gelu(x, self.reg, self.sigmoid_form)


class SiLU:
    """``SiLU::new(&registry)`` (layers/activation.rs:36-54): x * sigmoid(x)."""

    def __init__(self, reg: KernelRegistry):
        self.reg = reg

    def forward(self, x: GpuTensor) -> GpuTensor:
        return ops.silu(x, self.reg)


class Sigmoid:
    """``Sigmoid::new(&registry)`` (layers/activation.rs:57-75)."""

    def __init__(self, reg: KernelRegistry):
        self.reg = reg

    def forward(self, x: GpuTensor) -> GpuTensor:
        return ops.sigmoid(x, self.reg)


class ReLU:
    """``ReLU::new(&registry)`` (layers/activation.rs:78-96)."""

    def __init__(self, reg: KernelRegistry):
        self.reg = reg

    def forward(self, x: GpuTensor) -> GpuTensor:
        return ops.relu(x, self.reg)
