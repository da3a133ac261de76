"""Checkpoint reading, named as in ``gpu_host::model`` (crates/core/gpu-host/src/model.rs): the
safetensors container is parsed by the library (host code, no GPU needed)."""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass

import numpy as np

from . import ERR_UNSUPPORTED, NnError, load_library

_NP = {"F64": np.float64, "F32": np.float32, "F16": np.float16, "I64": np.int64, "I32": np.int32, "I16": np.int16,
       "I8": np.int8, "U64": np.uint64, "U32": np.uint32, "U16": np.uint16, "U8": np.uint8, "BOOL": np.bool_}


@dataclass
class TensorInfo:
    """``TensorInfo`` (model.rs:186-198)."""
    name: str
    shape: tuple
    dtype: str
    num_elements: int
    size_bytes: int


class SafeTensorsFile:
    """An open checkpoint: header parsed and validated, tensors read on demand."""

    def __init__(self, path):
        self.lib = load_library()
        self.h = C.c_void_p()
        rc = self.lib.b200nn_safetensors_open(os.fsencode(path), C.byref(self.h))
        if rc != 0:
            raise NnError(rc, (self.lib.b200nn_safetensors_last_error() or b"").decode())

    def _check(self, rc):
        if rc != 0:
            raise NnError(rc, (self.lib.b200nn_safetensors_last_error() or b"").decode())

    def __len__(self):
        return int(self.lib.b200nn_safetensors_count(self.h))

    def info(self, index: int) -> TensorInfo:
        name, dtype = C.c_char_p(), C.c_char_p()
        shape = (C.c_size_t * 8)()
        ndim, nbytes = C.c_int32(), C.c_size_t()
        self._check(self.lib.b200nn_safetensors_info(self.h, index, C.byref(name), C.byref(dtype), shape, 8,
                                                     C.byref(ndim), C.byref(nbytes)))
        shp = tuple(int(shape[i]) for i in range(ndim.value))
        return TensorInfo(name.value.decode(), shp, dtype.value.decode(), int(np.prod(shp, dtype=np.int64)) if shp else 1,
                          int(nbytes.value))

    def find(self, name: str) -> int:
        return int(self.lib.b200nn_safetensors_find(self.h, name.encode()))

    def read(self, index: int) -> np.ndarray:
        ti = self.info(index)
        if ti.dtype not in _NP:
            raise NnError(ERR_UNSUPPORTED, f"{ti.name}: dtype {ti.dtype} has no numpy equivalent")
        out = np.empty(ti.shape, dtype=_NP[ti.dtype])
        self._check(self.lib.b200nn_safetensors_read(self.h, index, out.ctypes.data_as(C.c_void_p), out.nbytes))
        return out

    def close(self):
        if self.h:
            self.lib.b200nn_safetensors_close(self.h)
            self.h = C.c_void_p()

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def list_tensors(path):
    """``list_tensors`` (model.rs:201-221): metadata of every tensor, sorted by name."""
    with SafeTensorsFile(path) as f:
        return [f.info(i) for i in range(len(f))]


def load_all_tensors(path):
    """``load_all_tensors`` (model.rs:388-397): name -> f32 array; a tensor of another dtype is an error."""
    out = {}
    with SafeTensorsFile(path) as f:
        for i in range(len(f)):
            ti = f.info(i)
            if ti.dtype != "F32":
                raise NnError(ERR_UNSUPPORTED, f"tensor {ti.name}: expected dtype F32, got {ti.dtype}")
            out[ti.name] = f.read(i)
    return out


def load_int4_tensors(path):
    """Reads a checkpoint in the layout ``scripts/quantize_gpt2_int4.py`` writes (the reference has no
    reader for it): every quantised matrix is a pair ``<key>.int4_packed`` (U32 ``[in/8, out]``, eight
    nibbles per word, nibble i at bits 4i, stored value q + 8) and ``<key>.int4_scales`` (F32
    ``[ceil(in/group), out]``); everything else is F32.  Returns ``(int4, dense)``: ``int4[key]`` =
    ``(packed, scales, in_features, out_features, group_size)`` exactly as ``Int4Linear`` takes them
    (int4_linear.rs:40-48), ``dense[key]`` = f32 array.  The group size is read off the shapes (the
    script's 128 whenever 128-wide groups tile the matrix, else in_features / scale rows)."""
    int4, dense, packed, scales = {}, {}, {}, {}
    with SafeTensorsFile(path) as f:
        for i in range(len(f)):
            ti = f.info(i)
            if ti.name.endswith(".int4_packed"):
                if ti.dtype != "U32" or len(ti.shape) != 2:
                    raise NnError(ERR_UNSUPPORTED, f"tensor {ti.name}: expected a 2-D U32 tensor, got {ti.dtype} {ti.shape}")
                packed[ti.name[: -len(".int4_packed")]] = f.read(i)
            elif ti.name.endswith(".int4_scales"):
                if ti.dtype != "F32" or len(ti.shape) != 2:
                    raise NnError(ERR_UNSUPPORTED, f"tensor {ti.name}: expected a 2-D F32 tensor, got {ti.dtype} {ti.shape}")
                scales[ti.name[: -len(".int4_scales")]] = f.read(i)
            elif ti.dtype == "F32":
                dense[ti.name] = f.read(i)
            else:
                raise NnError(ERR_UNSUPPORTED, f"tensor {ti.name}: expected dtype F32, got {ti.dtype}")
    for key in sorted(set(packed) | set(scales)):
        if key not in packed or key not in scales:
            raise NnError(ERR_UNSUPPORTED, f"{key}: int4_packed and int4_scales must come as a pair")
        p, s = packed[key], scales[key]
        k, n = p.shape[0] * 8, p.shape[1]
        if s.shape[1] != n or s.shape[0] < 1:
            raise NnError(ERR_UNSUPPORTED, f"{key}: scales {s.shape} do not match packed {p.shape}")
        g = s.shape[0]
        # the writer's groups are 128 wide with a ragged last one: that reading comes first; only a file
        # it does not fit (another group size) falls back to in_features / rows
        if -(-k // 128) == g:
            group = min(128, k)
        else:
            group = k if g == 1 else -(-k // g)
        if group % 8 or -(-k // group) != g:
            raise NnError(ERR_UNSUPPORTED, f"{key}: {g} scale rows do not tile in_features = {k}")
        int4[key] = (np.ascontiguousarray(p), np.ascontiguousarray(s), k, n, group)
    return int4, dense


def load_gpt2_weights(path):
    """``load_gpt2_weights`` (model.rs:308-386) as the dict ``Gpt2Model.from_weights`` takes: keys
    ``wte``, ``wpe``, ``ln_f.weight|bias``, ``h.{i}.<name>``; dense weights stay [in,out]."""
    t = load_all_tensors(path)
    out = {}
    for k, v in t.items():
        out["wte" if k == "wte.weight" else "wpe" if k == "wpe.weight" else k] = v
    return out
