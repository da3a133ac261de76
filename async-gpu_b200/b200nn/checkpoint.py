"""Checkpoint reading, named as in ``gpu_host::model`` (crates/core/gpu-host/src/model.rs): the
safetensors container is parsed by the library (host code, no GPU needed)."""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass

import numpy as np

from . import ERR_MISSING, ERR_SHAPE, ERR_UNSUPPORTED, NnError, load_library

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


# ---------------------------------------------------------------------------------------------
# The generic loader (gpu-host/src/model_generic.rs): weights by logical name, with the transforms a
# weight map asks for.  Host code over the same safetensors reader.
# ---------------------------------------------------------------------------------------------
class TensorData:
    """``TensorData`` (model_generic.rs:24-58): f32 data + shape."""

    def __init__(self, data, shape):
        self.data = np.ascontiguousarray(data, dtype=np.float32).reshape(-1)
        self.shape = [int(s) for s in shape]
        if int(np.prod(self.shape, dtype=np.int64)) != self.data.size:
            raise NnError(ERR_SHAPE, f"TensorData: shape {self.shape} does not hold {self.data.size} elements")

    def numel(self):
        return int(self.data.size)

    def transpose_2d(self):
        """[rows, cols] -> [cols, rows]; anything but a 2-D tensor is the reference's MissingTensor error."""
        if len(self.shape) != 2:
            raise NnError(ERR_MISSING, f"transpose_2d requires 2D, got {self.shape}")
        r, c = self.shape
        return TensorData(self.data.reshape(r, c).T.copy(), [c, r])


TRANSFORM_NONE, TRANSFORM_TRANSPOSE_2D = "None", "Transpose2D"  # ``Transform`` (model_generic.rs:61-67)


class WeightMapping:
    """``WeightMapping`` (model_generic.rs:70-78): safetensors key -> logical name, with a transform."""

    def __init__(self, safetensors_key, name, transform=TRANSFORM_NONE):
        self.safetensors_key, self.name, self.transform = safetensors_key, name, transform


def map_weight(st_key, name):
    """``map_weight`` (model_generic.rs:190-196)."""
    return WeightMapping(st_key, name, TRANSFORM_NONE)


def map_weight_t(st_key, name):
    """``map_weight_t`` (model_generic.rs:199-205): with the Conv1D -> Linear transpose."""
    return WeightMapping(st_key, name, TRANSFORM_TRANSPOSE_2D)


class LoadedWeights:
    """``LoadedWeights`` (model_generic.rs:84-120): tensors by logical name."""

    def __init__(self, weights):
        self._w = dict(weights)

    def get(self, name):
        return self._w.get(name)

    def require(self, name):
        t = self._w.get(name)
        if t is None:
            raise NnError(ERR_MISSING, name)
        return t

    def __len__(self):
        return len(self._w)

    def is_empty(self):
        return not self._w

    def total_params(self):
        return sum(t.numel() for t in self._w.values())

    def items(self):
        return self._w.items()


def load_safetensors_raw(path):
    """``load_safetensors_raw`` (model_generic.rs:126-150): key -> TensorData; a tensor that is not F32 is
    ``UnexpectedDtype``."""
    return {k: TensorData(v, v.shape) for k, v in load_all_tensors(path).items()}


def load_safetensors_mapped(path, weight_map):
    """``load_safetensors_mapped`` (model_generic.rs:156-177): a missing key is ``MissingTensor``."""
    raw = load_safetensors_raw(path)
    out = {}
    for m in weight_map:
        t = raw.get(m.safetensors_key)
        if t is None:
            raise NnError(ERR_MISSING, m.safetensors_key)
        out[m.name] = t.transpose_2d() if m.transform == TRANSFORM_TRANSPOSE_2D else TensorData(t.data.copy(), t.shape)
    return LoadedWeights(out)


def load_safetensors(path):
    """``load_safetensors`` (model_generic.rs:183-187): every tensor under its own key, no transform."""
    return LoadedWeights(load_safetensors_raw(path))


def gpt2_weight_map(num_layers):
    """``gpt2_weight_map`` (model_generic.rs:210-277): GPT-2's keys under their own names, the four Conv1D
    weights of every block transposed to Linear layout [out,in]."""
    m = [map_weight(k, k) for k in ("wte.weight", "wpe.weight", "ln_f.weight", "ln_f.bias")]
    for i in range(num_layers):
        p = f"h.{i}"
        for k in ("ln_1.weight", "ln_1.bias", "ln_2.weight", "ln_2.bias"):
            m.append(map_weight(f"{p}.{k}", f"{p}.{k}"))
        for k in ("attn.c_attn", "attn.c_proj", "mlp.c_fc", "mlp.c_proj"):
            m.append(map_weight_t(f"{p}.{k}.weight", f"{p}.{k}.weight"))
            m.append(map_weight(f"{p}.{k}.bias", f"{p}.{k}.bias"))
    return m
