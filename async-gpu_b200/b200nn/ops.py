"""Stateless ops, named as in ``gpu_host::nn::ops`` (ops/mod.rs:19-37)."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import (ACT_GELU_SIGMOID, ACT_GELU_TANH, ACT_RELU, ACT_SIGMOID, ACT_SILU, ERR_SHAPE, GpuTensor, KernelRegistry, NnError, _f32,
               _f32p, _out, _u32p, load_library)


# ---- quantize (ops/quantize.rs) ----
def quantize_weight_int4(weight_t, k, n, group_size):
    """[K,N] f32 -> (packed [K/8,N] u32, scales [ceil(K/g),N] f32); raises ShapeMismatch if K%8 != 0."""
    lib = load_library()
    w, wp = _f32(weight_t)
    if w.size != k * n:
        raise NnError(ERR_SHAPE, "weight_t must be [K, N]")
    packed = np.zeros((k // 8, n), dtype=np.uint32)
    scales = np.zeros(((k + group_size - 1) // group_size, n), dtype=np.float32)
    rc = lib.b200nn_quantize_weight_int4(wp, k, n, group_size, packed.ctypes.data_as(_u32p), scales.ctypes.data_as(_f32p))
    if rc != 0:
        raise NnError(rc, "K must be divisible by 8")
    return packed, scales


def quantize_int4_per_group(data, group_size):
    lib = load_library()
    d, dp = _f32(data)
    packed = np.zeros(d.size // 8, dtype=np.uint32)
    scales = np.zeros((d.size + group_size - 1) // group_size, dtype=np.float32)
    rc = lib.b200nn_quantize_int4_per_group(dp, d.size, group_size, packed.ctypes.data_as(_u32p), scales.ctypes.data_as(_f32p))
    if rc != 0:
        raise NnError(rc, "length must be divisible by 8")
    return packed, scales


def unpack_int4(word, index):
    return int(load_library().b200nn_unpack_int4(int(word), int(index)))


def pack_int8_to_u32(values):
    v = np.ascontiguousarray(values, dtype=np.int8)
    out = np.zeros((v.size + 3) // 4, dtype=np.uint32)
    load_library().b200nn_pack_int8_to_u32(v.ctypes.data_as(C.POINTER(C.c_int8)), v.size, out.ctypes.data_as(_u32p))
    return out


def quantize_int8_per_tensor(data):
    d, dp = _f32(data)
    q = np.zeros(d.size, dtype=np.int8)
    s = C.c_float()
    load_library().b200nn_quantize_int8_per_tensor(dp, d.size, q.ctypes.data_as(C.POINTER(C.c_int8)), C.byref(s))
    return q, float(s.value)


# ---- device ops ----
def layer_norm(x: GpuTensor, gamma: GpuTensor, beta: GpuTensor, eps: float, reg: KernelRegistry):
    h = C.c_void_p()
    return _out(reg, reg.lib.b200nn_layer_norm(reg.h, x.h, gamma.h, beta.h, eps, C.byref(h)), h)


def layer_norm_residual_dual(a, b, gamma, beta, eps, reg):
    hs, hn = C.c_void_p(), C.c_void_p()
    reg.check(reg.lib.b200nn_layer_norm_residual_dual(reg.h, a.h, b.h, gamma.h, beta.h, eps, C.byref(hs), C.byref(hn)))
    return GpuTensor(reg, hs), GpuTensor(reg, hn)


def _act(x, act, reg):
    h = C.c_void_p()
    return _out(reg, reg.lib.b200nn_activation(reg.h, x.h, act, C.byref(h)), h)


def gelu(x, reg, sigmoid_form=False):
    """tanh GELU by default; ``sigmoid_form`` selects x*sigmoid(1.702x) (the reference's v2 kernel)."""
    return _act(x, ACT_GELU_SIGMOID if sigmoid_form else ACT_GELU_TANH, reg)


def relu(x, reg):
    return _act(x, ACT_RELU, reg)


def silu(x, reg):
    """``ops::silu`` (ops/activation.rs:21-26): x * sigmoid(x)."""
    return _act(x, ACT_SILU, reg)


def sigmoid(x, reg):
    """``ops::sigmoid`` (ops/activation.rs:28-33)."""
    return _act(x, ACT_SIGMOID, reg)


def matmul(a: GpuTensor, b: GpuTensor, reg: KernelRegistry):
    """``ops::matmul`` (ops/gemm.rs:20-212): [M,K] x [K,N] -> [M,N] on device tensors."""
    h = C.c_void_p()
    return _out(reg, reg.lib.b200nn_matmul(reg.h, a.h, b.h, C.byref(h)), h)


# ``matmul_v2`` / ``matmul_v4`` / ``matmul_v4_1`` (ops/gemm.rs:220-346, 353-560, 568-800) are the reference's other
# kernels for the same contract, [M,K] x [K,N] -> [M,N] row-major; one implementation serves them here.
matmul_v2 = matmul_v4 = matmul_v4_1 = matmul

FUSED_GELU, FUSED_RELU = "gelu", "relu"  # ``FusedActivation`` (ops/gemm.rs:803-808)


def matmul_fused(a: GpuTensor, b: GpuTensor, bias: GpuTensor, activation, reg: KernelRegistry):
    """``ops::matmul_fused`` (ops/gemm.rs:814-977): activation(a [M,K] x b [K,N] + bias [N]); its GELU is the
    sigmoid form x * sigmoid(1.702 x).  Device tensors in, a new tensor out; the product, the bias and the
    activation run as three launches here (a Linear that keeps its weight fuses them: ``Linear.forward_fused``)."""
    if a.ndim() != 2 or b.ndim() != 2:
        raise NnError(ERR_SHAPE, f"ShapeMismatch: expected 2D tensors, actual a.ndim={a.ndim()}, b.ndim={b.ndim()}")
    if a.shape()[1] != b.shape()[0]:
        raise NnError(ERR_SHAPE, f"ShapeMismatch: expected a.shape[1]={a.shape()[1]} == b.shape[0], actual b.shape[0]={b.shape()[0]}")
    n = b.shape()[1]
    if bias.ndim() != 1 or bias.shape()[0] != n:
        raise NnError(ERR_SHAPE, f"ShapeMismatch: expected bias.shape=[{n}], actual bias.shape={list(bias.shape())}")
    if activation not in (FUSED_GELU, FUSED_RELU):
        raise NnError(ERR_SHAPE, "activation must be FUSED_GELU or FUSED_RELU")
    y = matmul(a, b, reg)
    bias_add(y, bias, reg)
    return gelu(y, reg, sigmoid_form=True) if activation == FUSED_GELU else relu(y, reg)


def layer_norm_residual(x, residual, gamma, beta, eps, reg):
    """``ops::layer_norm_residual`` (ops/norm.rs:88-246): LayerNorm(x + residual); the sum itself is not kept."""
    return layer_norm_residual_dual(x, residual, gamma, beta, eps, reg)[1]


def elementwise_add_out(a, b, reg):
    """``ops::elementwise_add_out`` (ops/reshape.rs:219-290): a + b into a new tensor."""
    if a.numel() != b.numel():
        raise NnError(ERR_SHAPE, f"ShapeMismatch: expected same numel, a has {a.numel()}, b has {b.numel()}")
    out = a.clone_tensor()
    elementwise_add(out, b, reg)
    return out


def embedding_lookup(wte: GpuTensor, wpe: GpuTensor, token_ids, seq_len, reg):
    """``ops::embedding_lookup`` (ops/reshape.rs:301-335): out[p] = wte[tok[p]] + wpe[p] for the first
    ``seq_len`` ids.  The tables are device tensors; the layer form that keeps them is ``Embedding``."""
    from .layers import Embedding
    v, d = wte.shape()
    e = Embedding(wte.to_host(), wpe.to_host(), v, wpe.shape()[0], d, reg)
    return e.forward_tokens(np.asarray(token_ids, dtype=np.uint32)[:seq_len])


def bias_add(data, bias, reg):
    reg.check(reg.lib.b200nn_bias_add(reg.h, data.h, bias.h))


def elementwise_add(a, b, reg):
    reg.check(reg.lib.b200nn_elementwise_add(reg.h, a.h, b.h))


def split_qkv(qkv, seq_len, n_heads, d_head, reg):
    q, k, v = C.c_void_p(), C.c_void_p(), C.c_void_p()
    reg.check(reg.lib.b200nn_split_qkv(reg.h, qkv.h, seq_len, n_heads, d_head, C.byref(q), C.byref(k), C.byref(v)))
    return GpuTensor(reg, q), GpuTensor(reg, k), GpuTensor(reg, v)


def concat_heads(heads, seq_len, n_heads, d_head, reg):
    h = C.c_void_p()
    return _out(reg, reg.lib.b200nn_concat_heads(reg.h, heads.h, seq_len, n_heads, d_head, C.byref(h)), h)


def multi_head_flash_attention(q, k, v, seq_len, n_heads, d_head, causal, reg):
    h = C.c_void_p()
    return _out(reg, reg.lib.b200nn_multi_head_flash_attention(reg.h, q.h, k.h, v.h, seq_len, n_heads, d_head,
                                                               int(causal), C.byref(h)), h)


# ``multi_head_flash_attention_v3`` / ``_nvrtc`` (ops/attention.rs:210-374): the same contract through the
# reference's run-time compiled kernels (their last argument is the device; the registry stands for it here).
multi_head_flash_attention_v3 = multi_head_flash_attention_nvrtc = multi_head_flash_attention


def scaled_dot_product_attention(q, k, v, causal, reg):
    """``ops::scaled_dot_product_attention`` (ops/attention.rs:17-103): one head, q, k, v [seq_len, d_head]."""
    if len(q.shape()) != 2 or len(k.shape()) != 2 or len(v.shape()) != 2:
        raise NnError(ERR_SHAPE, "ShapeMismatch: expected 2D tensors [seq_len, d_head]")
    return scaled_dot_product_attention_kv(q, k, v, causal, k.shape()[0] - q.shape()[0], reg)


def scaled_dot_product_attention_kv(q, k, v, causal, q_offset, reg):
    h = C.c_void_p()
    return _out(reg, reg.lib.b200nn_attention_kv(reg.h, q.h, k.h, v.h, int(causal), q_offset, C.byref(h)), h)


def int4_matmul(a: GpuTensor, b_host, k, n, group_size, reg):
    b, bp = _f32(b_host)
    h = C.c_void_p()
    return _out(reg, reg.lib.b200nn_int4_matmul(reg.h, a.h, bp, k, n, group_size, C.byref(h)), h)


def prefill_attention_f16(q_ptr, k_cache_ptr, v_cache_ptr, batch, n_heads, capacity, seq_len, past, out_ptr, reg):
    """Causal attention of ``seq_len`` new rows per sequence on caller-owned fp16 device buffers (device
    pointers as ints): q / out ``[batch*seq_len, n_heads*64]``, caches ``[batch][n_heads][capacity][64]``."""
    reg.check(reg.lib.b200nn_prefill_attention_f16(reg.h, q_ptr, k_cache_ptr, v_cache_ptr, batch, n_heads, capacity,
                                                   seq_len, past, out_ptr))


def decode_attention_f16(q_ptr, k_cache_ptr, v_cache_ptr, batch, n_heads, capacity, ctx_len, out_ptr, reg):
    """One query row per sequence against the first ``ctx_len`` cached positions, fp16 device buffers."""
    reg.check(reg.lib.b200nn_decode_attention_f16(reg.h, q_ptr, k_cache_ptr, v_cache_ptr, batch, n_heads, capacity,
                                                  ctx_len, out_ptr))
