"""Host-side mirror of async-gpu's ``gpu_host::nn`` API over ``libb200nn.so`` (ctypes).

Names follow the reference (``KernelRegistry``, ``GpuTensor``, ``Linear``, ``Int4Linear``,
``LayerNorm``, ``Embedding``, ``MultiHeadAttention``, ``Gpt2Config``, ``Gpt2Model``,
``Int4Gpt2Model``, ``KvCache``, ``ops.*``); a Rust ``-sys`` crate binds the same C symbols.
There is no CPU fallback: if the CUDA library is missing or no B200 is present, construction
raises ``NnError``.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(os.path.dirname(_HERE), "libb200nn.so")

OK, ERR_SHAPE, ERR_DIM, ERR_UNSUPPORTED, ERR_CUDA, ERR_DEVICE, ERR_ARG, ERR_IO, ERR_MISSING = range(9)
ACT_NONE, ACT_GELU_TANH, ACT_GELU_SIGMOID, ACT_RELU, ACT_SILU, ACT_SIGMOID = range(6)
GELU_SIGMOID, QUANT_LM_HEAD, ARGMAX_LAST, STOP_ON_EOS, TOKENS_ONLY, WEIGHTS_OUT_IN = 1, 2, 4, 8, 16, 32
PROF_NAMES = ("embed", "layernorm", "linear", "attention", "lm_head", "argmax")

_KINDS = {ERR_SHAPE: "ShapeMismatch", ERR_DIM: "DimOutOfRange", ERR_UNSUPPORTED: "KernelNotFound",
          ERR_CUDA: "Cuda", ERR_DEVICE: "DeviceTimeout", ERR_ARG: "InvalidArgument", ERR_IO: "Io",
          ERR_MISSING: "MissingTensor"}


class NnError(RuntimeError):
    """Mirrors ``NnError`` (nn/error.rs:7-29); ``kind`` names the variant."""

    def __init__(self, code, message=""):
        self.code = code
        self.kind = _KINDS.get(code, f"code {code}")
        super().__init__(f"{self.kind}: {message}")


class _Cfg(C.Structure):
    _fields_ = [("n_layer", C.c_int32), ("n_embd", C.c_int32), ("n_head", C.c_int32), ("vocab_size", C.c_int32),
                ("n_positions", C.c_int32), ("layer_norm_epsilon", C.c_float)]


_f32p, _u32p = C.POINTER(C.c_float), C.POINTER(C.c_uint32)


class _LayerW(C.Structure):
    _fields_ = [(n, _f32p) for n in (
        "ln_1_weight", "ln_1_bias", "c_attn_weight", "c_attn_bias", "c_proj_weight", "c_proj_bias",
        "ln_2_weight", "ln_2_bias", "mlp_fc_weight", "mlp_fc_bias", "mlp_proj_weight", "mlp_proj_bias")]


class _BlockW(C.Structure):
    _fields_ = [(n, _f32p) for n in (
        "ln_1_weight", "ln_1_bias", "attn_qkv_weight", "attn_qkv_bias", "attn_out_weight", "attn_out_bias",
        "ln_2_weight", "ln_2_bias", "ffn_up_weight", "ffn_up_bias", "ffn_down_weight", "ffn_down_bias")]


class _Diag(C.Structure):
    _fields_ = [("embedding_first", C.c_float * 4), ("embedding_last", C.c_float * 4), ("block0_last", C.c_float * 4),
                ("final_block_last", C.c_float * 4), ("block0_nonfinite", C.c_int32), ("final_block_nonfinite", C.c_int32),
                ("ln_f_last", C.c_float * 4), ("top_tokens", C.c_uint32 * 5), ("top_scores", C.c_float * 5),
                ("n_top", C.c_int32)]


class _Weights(C.Structure):
    _fields_ = [("wte", _f32p), ("wpe", _f32p), ("ln_f_weight", _f32p), ("ln_f_bias", _f32p),
                ("layers", C.POINTER(_LayerW))]


_lib = None


def load_library() -> C.CDLL:
    """Loads the CUDA library; raises if it has not been built (no fallback exists)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise NnError(ERR_UNSUPPORTED, f"{LIB_PATH} is missing: build it with async-gpu_b200/build.py")
        L = C.CDLL(LIB_PATH)
        vp, sz, i32, u32 = C.c_void_p, C.c_size_t, C.c_int32, C.c_uint32
        szp, vpp = C.POINTER(C.c_size_t), C.POINTER(C.c_void_p)
        sig = {
            "b200nn_version": (C.c_char_p, []),
            "b200nn_ctx_create": (i32, [i32, vpp]), "b200nn_ctx_destroy": (None, [vp]),
            "b200nn_ctx_synchronize": (i32, [vp]), "b200nn_ctx_stream": (vp, [vp]),
            "b200nn_ctx_trim": (i32, [vp]),
            "b200nn_last_error_message": (C.c_char_p, [vp]), "b200nn_last_cuda_error": (i32, [vp]),
            "b200nn_ctx_device_error": (i32, [vp, _u32p]), "b200nn_ctx_launch_count": (C.c_uint64, [vp]),
            "b200nn_ctx_set_gemv_max_rows": (i32, [vp, i32]),
            "b200nn_ctx_set_tuning": (i32, [vp, C.c_char_p, i32]),
            "b200nn_ctx_read_trace": (i32, [vp, C.POINTER(C.c_longlong)]),
            "b200nn_ctx_read_persist_trace": (i32, [vp, C.POINTER(C.c_uint64), sz]),
            "b200nn_tensor_from_host": (i32, [vp, _f32p, szp, i32, vpp]),
            "b200nn_tensor_from_device": (i32, [vp, vp, szp, i32, vpp]),
            "b200nn_tensor_zeros": (i32, [vp, szp, i32, vpp]), "b200nn_tensor_to_host": (i32, [vp, _f32p, sz]),
            "b200nn_tensor_ndim": (i32, [vp]), "b200nn_tensor_numel": (sz, [vp]),
            "b200nn_tensor_shape": (i32, [vp, szp, i32]), "b200nn_tensor_reshape": (i32, [vp, szp, i32, vpp]),
            "b200nn_tensor_clone": (i32, [vp, vpp]), "b200nn_tensor_data": (vp, [vp]),
            "b200nn_tensor_transpose": (i32, [vp, sz, sz, vpp]),
            "b200nn_tensor_concat": (i32, [vpp, sz, sz, vpp]),
            "b200nn_tensor_split": (i32, [vp, sz, szp, sz, vpp]),
            "b200nn_tensor_destroy": (None, [vp]),
            "b200nn_quantize_weight_int4": (i32, [_f32p, sz, sz, sz, _u32p, _f32p]),
            "b200nn_quantize_int4_per_group": (i32, [_f32p, sz, sz, _u32p, _f32p]),
            "b200nn_unpack_int4": (i32, [u32, i32]),
            "b200nn_pack_int8_to_u32": (i32, [C.POINTER(C.c_int8), sz, _u32p]),
            "b200nn_quantize_int8_per_tensor": (i32, [_f32p, sz, C.POINTER(C.c_int8), _f32p]),
            "b200nn_layer_norm": (i32, [vp, vp, vp, vp, C.c_float, vpp]),
            "b200nn_layer_norm_residual_dual": (i32, [vp, vp, vp, vp, vp, C.c_float, vpp, vpp]),
            "b200nn_activation": (i32, [vp, vp, i32, vpp]), "b200nn_bias_add": (i32, [vp, vp, vp]),
            "b200nn_elementwise_add": (i32, [vp, vp, vp]),
            "b200nn_split_qkv": (i32, [vp, vp, sz, sz, sz, vpp, vpp, vpp]),
            "b200nn_concat_heads": (i32, [vp, vp, sz, sz, sz, vpp]),
            "b200nn_multi_head_flash_attention": (i32, [vp, vp, vp, vp, sz, sz, sz, i32, vpp]),
            "b200nn_attention_kv": (i32, [vp, vp, vp, vp, i32, sz, vpp]),
            "b200nn_int4_matmul": (i32, [vp, vp, _f32p, sz, sz, sz, vpp]),
            "b200nn_matmul": (i32, [vp, vp, vp, vpp]),
            "b200nn_linear_create": (i32, [vp, _f32p, _f32p, sz, sz, vpp]),
            "b200nn_linear_forward": (i32, [vp, vp, vpp]), "b200nn_linear_forward_fused": (i32, [vp, vp, i32, vpp]),
            "b200nn_linear_destroy": (None, [vp]),
            "b200nn_int4_linear_create": (i32, [vp, _u32p, _f32p, _f32p, sz, sz, sz, vpp]),
            "b200nn_int4_linear_forward": (i32, [vp, vp, vpp]),
            "b200nn_int4_linear_forward_dev": (i32, [vp, vp, sz, vp]),
            "b200nn_int4_linear_forward_host": (i32, [vp, _f32p, sz, _f32p]),
            "b200nn_int4_linear_memory_bytes": (sz, [vp]), "b200nn_int4_linear_destroy": (None, [vp]),
            "b200nn_layernorm_create": (i32, [vp, _f32p, _f32p, sz, C.c_float, vpp]),
            "b200nn_layernorm_forward": (i32, [vp, vp, vpp]), "b200nn_layernorm_destroy": (None, [vp]),
            "b200nn_embedding_create": (i32, [vp, _f32p, _f32p, sz, sz, sz, vpp]),
            "b200nn_embedding_forward_tokens": (i32, [vp, _u32p, sz, sz, vpp]),
            "b200nn_embedding_destroy": (None, [vp]),
            "b200nn_attention_create": (i32, [vp, _f32p, _f32p, _f32p, _f32p, sz, sz, vpp]),
            "b200nn_int4_attention_create": (i32, [vp, _f32p, _f32p, _f32p, _f32p, sz, sz, sz, vpp]),
            "b200nn_attention_forward_causal": (i32, [vp, vp, vpp]),
            "b200nn_attention_forward_cached": (i32, [vp, vp, _f32p, _f32p, sz, vpp, _f32p, _f32p]),
            "b200nn_attention_destroy": (None, [vp]),
            "b200nn_gpt2_config_preset": (i32, [C.c_char_p, C.POINTER(_Cfg)]),
            "b200nn_gpt2_create": (i32, [vp, C.POINTER(_Cfg), C.POINTER(_Weights), u32, vpp]),
            "b200nn_int4_gpt2_create": (i32, [vp, C.POINTER(_Cfg), C.POINTER(_Weights), sz, u32, vpp]),
            "b200nn_gpt2_destroy": (None, [vp]), "b200nn_gpt2_get_config": (i32, [vp, C.POINTER(_Cfg)]),
            "b200nn_gpt2_quantized_memory_bytes": (sz, [vp]),
            "b200nn_gpt2_get_int4": (i32, [vp, i32, i32, _u32p, _f32p, szp, szp]),
            "b200nn_gpt2_forward": (i32, [vp, _u32p, sz, vpp]),
            "b200nn_block_create": (i32, [vp, C.POINTER(_Cfg), C.POINTER(_BlockW), u32, vpp]),
            "b200nn_int4_block_create": (i32, [vp, C.POINTER(_Cfg), C.POINTER(_BlockW), sz, u32, vpp]),
            "b200nn_block_forward": (i32, [vp, vp, vpp]),
            "b200nn_block_forward_cached": (i32, [vp, vp, _f32p, _f32p, sz, vpp, _f32p, _f32p]),
            "b200nn_block_destroy": (None, [vp]),
            "b200nn_kvcache_create": (i32, [vp, sz, sz, vpp]), "b200nn_kvcache_len": (sz, [vp]),
            "b200nn_kvcache_reset": (i32, [vp]), "b200nn_kvcache_destroy": (None, [vp]),
            "b200nn_gpt2_forward_cached": (i32, [vp, _u32p, sz, vp, vpp]),
            "b200nn_gpt2_generate": (i32, [vp, _u32p, sz, sz, u32, _u32p, szp]),
            "b200nn_gpt2_generate_cached": (i32, [vp, _u32p, sz, sz, u32, _u32p, szp]),
            "b200nn_gpt2_generate_batch": (i32, [vp, _u32p, sz, sz, sz, u32, _u32p, szp]),
            "b200nn_session_create": (i32, [vp, sz, sz, u32, vpp]),
            "b200nn_session_prefill": (i32, [vp, _u32p, sz]), "b200nn_session_step": (i32, [vp, sz]),
            "b200nn_session_rewind": (i32, [vp, sz]), "b200nn_session_position": (sz, [vp]),
            "b200nn_session_tokens": (i32, [vp, _u32p, sz, szp]), "b200nn_session_logits": (i32, [vp, _f32p]),
            "b200nn_session_profile_step": (i32, [vp, _f32p, C.POINTER(C.c_uint64)]),
            "b200nn_session_time_family": (i32, [vp, i32, i32, _f32p, C.POINTER(C.c_uint64)]),
            "b200nn_gpt2_forward_features": (i32, [vp, _u32p, sz, vpp]),
            "b200nn_gpt2_embedding_table": (i32, [vp, vpp, vpp]),
            "b200nn_gpt2_forward_profiled": (i32, [vp, _u32p, sz, vpp, _f32p, i32, C.POINTER(i32)]),
            "b200nn_simple_rng_new": (C.c_uint64, [C.c_uint64]),
            "b200nn_simple_rng_next_f32": (C.c_float, [C.POINTER(C.c_uint64)]),
            "b200nn_simple_rng_fill_uniform": (i32, [C.POINTER(C.c_uint64), sz, _f32p]),
            "b200nn_simple_rng_fill_normal": (i32, [C.POINTER(C.c_uint64), sz, C.c_float, _f32p]),
            "b200nn_top_k_sample": (i32, [_f32p, sz, sz, C.c_float, C.POINTER(C.c_uint64), _u32p]),
            "b200nn_gpt2_generate_cached_sampling": (i32, [vp, _u32p, sz, sz, sz, C.c_float, C.POINTER(C.c_uint64), _u32p,
                                                           szp]),
            "b200nn_gpt2_forward_early_exit": (i32, [vp, _u32p, sz, C.c_float, vpp, C.POINTER(i32)]),
            "b200nn_gpt2_generate_cached_early_exit": (i32, [vp, _u32p, sz, sz, C.c_float, _u32p, szp, C.POINTER(i32),
                                                             szp]),
            "b200nn_safetensors_open": (i32, [C.c_char_p, vpp]), "b200nn_safetensors_close": (None, [vp]),
            "b200nn_safetensors_count": (i32, [vp]),
            "b200nn_safetensors_info": (i32, [vp, i32, C.POINTER(C.c_char_p), C.POINTER(C.c_char_p), szp, i32,
                                              C.POINTER(i32), szp]),
            "b200nn_safetensors_find": (i32, [vp, C.c_char_p]),
            "b200nn_safetensors_read": (i32, [vp, i32, vp, sz]),
            "b200nn_safetensors_last_error": (C.c_char_p, []),
            "b200nn_gpt2_load_safetensors": (i32, [vp, C.c_char_p, C.POINTER(_Cfg), sz, u32, vpp]),
            "b200nn_bpe_load": (i32, [C.c_char_p, u32, vpp]),
            "b200nn_bpe_create": (i32, [C.c_char_p, szp, _u32p, sz, u32, vpp]),
            "b200nn_bpe_destroy": (None, [vp]), "b200nn_bpe_vocab_size": (sz, [vp]),
            "b200nn_bpe_encode": (i32, [vp, C.c_char_p, sz, _u32p, sz, szp]),
            "b200nn_bpe_encode_piece": (i32, [vp, C.c_char_p, sz, _u32p, sz, szp]),
            "b200nn_bpe_decode": (i32, [vp, _u32p, sz, C.c_char_p, sz, szp]),
            "b200nn_bpe_last_error": (C.c_char_p, []),
            "b200nn_gpt2_forward_diagnostic": (i32, [vp, _u32p, sz, vpp, C.POINTER(_Diag)]),
            "b200nn_prefill_attention_f16": (i32, [vp, vp, vp, vp, i32, i32, i32, i32, i32, vp]),
            "b200nn_decode_attention_f16": (i32, [vp, vp, vp, vp, i32, i32, i32, i32, vp]),
            "b200nn_decode_attention_noalloc": (i32, [i32, vp, vp, vp, vp, i32, i32, i32, i32, vp]),
            "b200nn_noalloc_last_error": (C.c_char_p, []),
            "b200nn_session_destroy": (None, [vp]),
        }
        for name, (res, args) in sig.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        L._declared = sorted(sig)
        _lib = L
    return _lib


def _f32(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a, a.ctypes.data_as(_f32p)


def _u32(a):
    a = np.ascontiguousarray(a, dtype=np.uint32)
    return a, a.ctypes.data_as(_u32p)


def _shape(shape):
    arr = (C.c_size_t * len(shape))(*[int(s) for s in shape])
    return arr, len(shape)


class KernelRegistry:
    """``KernelRegistry::init_default()`` (nn/registry.rs:131-135): one context per GPU."""

    def __init__(self, device: int = 0):
        self.lib = load_library()
        h = C.c_void_p()
        rc = self.lib.b200nn_ctx_create(device, C.byref(h))
        if rc != OK:
            raise NnError(rc, "no usable B200 (sm_100) CUDA device; this library has no CPU path")
        self.h = h
        self.device = device

    @classmethod
    def init_default(cls):
        return cls(0)

    def check(self, rc):
        if rc != OK:
            raise NnError(rc, (self.lib.b200nn_last_error_message(self.h) or b"").decode())

    def synchronize(self):
        self.check(self.lib.b200nn_ctx_synchronize(self.h))

    def trim(self):
        """Returns the device blocks the context keeps for reuse to the driver."""
        self.check(self.lib.b200nn_ctx_trim(self.h))

    @property
    def stream(self) -> int:
        return int(self.lib.b200nn_ctx_stream(self.h) or 0)

    def launch_count(self) -> int:
        return int(self.lib.b200nn_ctx_launch_count(self.h))

    def set_gemv_max_rows(self, rows: int):
        self.check(self.lib.b200nn_ctx_set_gemv_max_rows(self.h, rows))

    def set_tuning(self, key: str, value: int):
        self.check(self.lib.b200nn_ctx_set_tuning(self.h, key.encode(), value))

    def read_persist_trace(self, blocks: int = 148) -> np.ndarray:
        """[block, 32, 2] nanosecond stamps of the persistent decode kernel's last launch (measurement aid)."""
        out = np.zeros((blocks, 32, 2), dtype=np.uint64)
        self.check(self.lib.b200nn_ctx_read_persist_trace(self.h, out.ctypes.data_as(C.POINTER(C.c_uint64)), out.size))
        return out

    def device_error(self) -> int:
        w = C.c_uint32()
        self.lib.b200nn_ctx_device_error(self.h, C.byref(w))
        return int(w.value)

    def close(self):
        if self.h:
            self.lib.b200nn_ctx_destroy(self.h)
            self.h = None


class GpuTensor:
    """f32 N-dim device tensor (nn/tensor.rs:45-60)."""

    def __init__(self, reg: KernelRegistry, handle):
        self.reg, self.h = reg, handle

    @classmethod
    def from_host(cls, data, shape, reg: KernelRegistry):
        a, p = _f32(data)
        sh, nd = _shape(shape)
        if a.size != int(np.prod(shape)):
            raise NnError(ERR_SHAPE, f"expected {int(np.prod(shape))} elements, got {a.size}")
        h = C.c_void_p()
        reg.check(reg.lib.b200nn_tensor_from_host(reg.h, p, sh, nd, C.byref(h)))
        return cls(reg, h)

    @classmethod
    def from_data(cls, device_ptr: int, shape, reg: KernelRegistry):
        """``GpuTensor::from_data`` (tensor.rs:67-77): a tensor over f32 data already on the registry's device
        (``device_ptr`` = its address).  The values are copied; the caller keeps its buffer."""
        sh, nd = _shape(shape)
        h = C.c_void_p()
        reg.check(reg.lib.b200nn_tensor_from_device(reg.h, C.c_void_p(int(device_ptr)), sh, nd, C.byref(h)))
        return cls(reg, h)

    @classmethod
    def zeros(cls, shape, reg: KernelRegistry):
        sh, nd = _shape(shape)
        h = C.c_void_p()
        reg.check(reg.lib.b200nn_tensor_zeros(reg.h, sh, nd, C.byref(h)))
        return cls(reg, h)

    def shape(self):
        nd = self.reg.lib.b200nn_tensor_ndim(self.h)
        arr = (C.c_size_t * nd)()
        self.reg.check(self.reg.lib.b200nn_tensor_shape(self.h, arr, nd))
        return tuple(int(x) for x in arr)

    def numel(self):
        return int(self.reg.lib.b200nn_tensor_numel(self.h))

    def to_host(self) -> np.ndarray:
        out = np.empty(self.numel(), dtype=np.float32)
        self.reg.check(self.reg.lib.b200nn_tensor_to_host(self.h, out.ctypes.data_as(_f32p), out.size))
        return out.reshape(self.shape())

    def reshape(self, shape):
        sh, nd = _shape(shape)
        h = C.c_void_p()
        self.reg.check(self.reg.lib.b200nn_tensor_reshape(self.h, sh, nd, C.byref(h)))
        return GpuTensor(self.reg, h)

    def ndim(self):
        return len(self.shape())

    def strides(self):
        """Row-major strides in elements (tensor.rs:140; every tensor here is contiguous)."""
        st, acc = [], 1
        for n in reversed(self.shape()):
            st.append(acc)
            acc *= n
        return tuple(reversed(st))

    def is_contiguous(self):
        return True

    def size_bytes(self):
        return self.numel() * 4

    def transpose(self, dim0: int, dim1: int):
        """``GpuTensor::transpose`` (tensor.rs:227-268), on the device."""
        h = C.c_void_p()
        return _out(self.reg, self.reg.lib.b200nn_tensor_transpose(self.h, dim0, dim1, C.byref(h)), h)

    @staticmethod
    def concat(tensors, dim: int):
        """``GpuTensor::concat`` (tensor.rs:287-349), on the device."""
        if not tensors:
            raise NnError(ERR_SHAPE, "ShapeMismatch: expected at least one tensor, got empty list")
        reg = tensors[0].reg
        arr = (C.c_void_p * len(tensors))(*[t.h for t in tensors])
        h = C.c_void_p()
        return _out(reg, reg.lib.b200nn_tensor_concat(arr, len(tensors), dim, C.byref(h)), h)

    def split(self, dim: int, sizes):
        """``GpuTensor::split`` (tensor.rs:351-393), on the device."""
        sizes = [int(x) for x in sizes]
        arr = (C.c_size_t * max(1, len(sizes)))(*sizes)
        outs = (C.c_void_p * max(1, len(sizes)))()
        self.reg.check(self.reg.lib.b200nn_tensor_split(self.h, dim, arr, len(sizes), outs))
        return [GpuTensor(self.reg, C.c_void_p(outs[i])) for i in range(len(sizes))]

    def clone_tensor(self):
        h = C.c_void_p()
        self.reg.check(self.reg.lib.b200nn_tensor_clone(self.h, C.byref(h)))
        return GpuTensor(self.reg, h)

    def data_ptr(self) -> int:
        return int(self.reg.lib.b200nn_tensor_data(self.h) or 0)

    def __del__(self):
        try:
            if self.h and self.reg.h:
                self.reg.lib.b200nn_tensor_destroy(self.h)
        except Exception:
            pass


def _out(reg, rc, h):
    reg.check(rc)
    return GpuTensor(reg, h)


from . import ops  # noqa: E402
from .layers import (Embedding, Int4Linear, LayerNorm, Linear, MultiHeadAttention, Int4MultiHeadAttention,  # noqa: E402
                     GELU, SiLU, Sigmoid, ReLU)
from .gpt2 import (Gpt2Config, Gpt2Model, Int4Gpt2Model, KvCache, DecodeSession, TransformerBlock,  # noqa: E402
                   Int4TransformerBlock)
from .sampling import SimpleRng, top_k_sample, argmax, softmax_max_prob  # noqa: E402
from .tokenizer import Gpt2Tokenizer, TokenizerError, GPT2_VOCAB_SIZE, ENDOFTEXT_TOKEN_ID  # noqa: E402
from .checkpoint import (SafeTensorsFile, TensorInfo, list_tensors, load_all_tensors, load_gpt2_weights,  # noqa: E402
                         load_int4_tensors, TensorData, WeightMapping, LoadedWeights, map_weight, map_weight_t,
                         load_safetensors_raw, load_safetensors_mapped, load_safetensors, gpt2_weight_map)
