"""The safetensors reader of the library (host code: runs without a GPU), against files written by
hand from the format's public description and, where the `safetensors` Python package is present,
against files written by that package (the format's own implementation)."""
import json
import struct

import numpy as np
import pytest

import b200nn
from b200nn import checkpoint

_DT = {np.dtype(np.float32): "F32", np.dtype(np.uint32): "U32", np.dtype(np.float16): "F16", np.dtype(np.int64): "I64",
       np.dtype(np.uint8): "U8"}


def write_safetensors(path, tensors, metadata=None, pad_header_to=None):
    """8-byte little-endian header length, JSON header, raw little-endian data."""
    header, blobs, off = {}, [], 0
    if metadata is not None:
        header["__metadata__"] = metadata
    for name, a in tensors.items():
        a = np.asarray(a)
        b = a.tobytes()  # C order; a 0-d array keeps its empty shape
        header[name] = {"dtype": _DT[a.dtype], "shape": list(a.shape), "data_offsets": [off, off + len(b)]}
        blobs.append(b)
        off += len(b)
    h = json.dumps(header).encode()
    if pad_header_to:
        h += b" " * (pad_header_to - len(h))
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h)) + h + b"".join(blobs))


def _sample():
    rng = np.random.default_rng(5)
    return {
        "wte.weight": rng.standard_normal((7, 4)).astype(np.float32),
        "h.0.attn.c_attn.weight.int4_packed": rng.integers(0, 2**32, (3, 5), dtype=np.uint32),
        "scalar": np.array(3.5, dtype=np.float32),
        "empty": np.zeros((0, 4), dtype=np.float32),
        'odd "name"\\ é': np.arange(6, dtype=np.int64).reshape(2, 3),
        "bytes": np.arange(10, dtype=np.uint8),
        "half": np.array([1.5, -2.0], dtype=np.float16),
    }


def test_list_and_read_hand_written_file(tmp_path):
    p = tmp_path / "a.safetensors"
    t = _sample()
    write_safetensors(p, t, metadata={"format": "pt", "note": "x"}, pad_header_to=1000)
    infos = checkpoint.list_tensors(p)
    assert [i.name for i in infos] == sorted(t)  # list_tensors sorts by name
    with checkpoint.SafeTensorsFile(p) as f:
        assert len(f) == len(t)
        for i, ti in enumerate(infos):
            a = t[ti.name]
            assert ti.shape == a.shape and ti.dtype == _DT[a.dtype]
            assert ti.num_elements == a.size and ti.size_bytes == a.nbytes
            got = f.read(i)
            assert got.dtype == a.dtype and np.array_equal(got, a)
            assert f.find(ti.name) == i
        assert f.find("nope") == -1


def test_load_all_tensors_is_f32_only(tmp_path):
    p = tmp_path / "b.safetensors"
    good = {"x": np.ones((2, 2), np.float32), "y": np.arange(3, dtype=np.float32)}
    write_safetensors(p, good)
    got = checkpoint.load_all_tensors(p)
    assert set(got) == {"x", "y"} and np.array_equal(got["y"], good["y"])
    write_safetensors(p, dict(good, z=np.zeros(2, np.float16)))
    with pytest.raises(b200nn.NnError) as e:
        checkpoint.load_all_tensors(p)
    assert e.value.code == b200nn.ERR_UNSUPPORTED and "F16" in str(e.value)


def test_reads_files_written_by_the_safetensors_package(tmp_path):
    st = pytest.importorskip("safetensors.numpy")
    p = tmp_path / "c.safetensors"
    t = {k: v for k, v in _sample().items() if v.size}  # the package rejects nothing here; keep it simple
    st.save_file(t, str(p), metadata={"made_by": "safetensors"})
    with checkpoint.SafeTensorsFile(p) as f:
        assert sorted(f.info(i).name for i in range(len(f))) == sorted(t)
        for i in range(len(f)):
            ti = f.info(i)
            assert np.array_equal(f.read(i), t[ti.name]) and ti.shape == t[ti.name].shape
    back = st.load_file(str(p))
    assert all(np.array_equal(back[k], t[k]) for k in t)


@pytest.mark.parametrize("case", ["missing", "short", "hdr_len", "not_json", "range", "size", "dtype", "dup", "no_offsets",
                                  "overflow", "overlap", "gap", "uncovered"])
def test_malformed_files_are_rejected(tmp_path, case):
    p = tmp_path / "bad.safetensors"
    data = np.arange(4, dtype=np.float32).tobytes()

    def put(header: bytes, body: bytes = data):
        p.write_bytes(struct.pack("<Q", len(header)) + header + body)

    if case == "missing":
        pass
    elif case == "short":
        p.write_bytes(b"\x01\x02")
    elif case == "hdr_len":
        p.write_bytes(struct.pack("<Q", 10**6) + b"{}")
    elif case == "not_json":
        put(b"[1,2,3]")
    elif case == "range":
        put(json.dumps({"a": {"dtype": "F32", "shape": [8], "data_offsets": [0, 32]}}).encode())
    elif case == "size":
        put(json.dumps({"a": {"dtype": "F32", "shape": [3], "data_offsets": [0, 16]}}).encode())
    elif case == "dtype":
        put(json.dumps({"a": {"dtype": "Q4", "shape": [4], "data_offsets": [0, 16]}}).encode())
    elif case == "dup":
        put(b'{"a":{"dtype":"F32","shape":[2],"data_offsets":[0,8]},"a":{"dtype":"F32","shape":[2],"data_offsets":[8,16]}}')
    elif case == "no_offsets":
        put(json.dumps({"a": {"dtype": "F32", "shape": [4]}}).encode())
    elif case == "overflow":  # 2^32 x 2^32 x 4 bytes wraps to 0 in 64 bits: must not pass as an empty tensor
        put(json.dumps({"a": {"dtype": "F32", "shape": [2**32, 2**32], "data_offsets": [0, 0]},
                        "b": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode())
    elif case == "overlap":
        put(json.dumps({"a": {"dtype": "F32", "shape": [3], "data_offsets": [0, 12]},
                        "b": {"dtype": "F32", "shape": [2], "data_offsets": [8, 16]}}).encode())
    elif case == "gap":
        put(json.dumps({"a": {"dtype": "F32", "shape": [1], "data_offsets": [0, 4]},
                        "b": {"dtype": "F32", "shape": [2], "data_offsets": [8, 16]}}).encode())
    elif case == "uncovered":  # the last 8 bytes of the data section belong to no tensor
        put(json.dumps({"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}}).encode())
    with pytest.raises(b200nn.NnError) as e:
        checkpoint.SafeTensorsFile(p)
    assert e.value.code == b200nn.ERR_IO and str(e.value)


def test_load_gpt2_weights_key_names(tmp_path):
    """The dict has the checkpoint's Hugging Face names, with wte / wpe as from_weights expects them."""
    from b200nn import Gpt2Config, synth
    cfg = Gpt2Config(n_layer=2, n_embd=64, n_head=1, vocab_size=50, n_positions=16)
    w = synth.gpt2_weights(cfg, base_seed=3)
    p = tmp_path / "m.safetensors"
    write_safetensors(p, {("wte.weight" if k == "wte" else "wpe.weight" if k == "wpe" else k): v for k, v in w.items()})
    got = checkpoint.load_gpt2_weights(p)
    assert set(got) == set(w)
    assert all(np.array_equal(got[k], np.asarray(w[k], np.float32).reshape(got[k].shape)) for k in w)
    assert got["h.1.mlp.c_fc.weight"].shape == (64, 256)  # Conv1D layout [in,out] kept


def test_load_int4_tensors_layout_of_the_reference_script(tmp_path):
    """The int4 checkpoint layout of scripts/quantize_gpt2_int4.py:21-62, 85-99: `<key>.int4_packed` U32
    [in/8,out] + `<key>.int4_scales` F32 [ceil(in/128),out]; other tensors F32.  The quantiser here is the
    oracle's (quantize.rs:102-153), which packs the same way (nibble i of a word at bits 4i, value + 8)."""
    from oracle import oracle
    rng = np.random.default_rng(11)
    tensors, want = {}, {}
    # 1080 rows: nine 128-wide groups (the last ragged), although 1080 / 9 = 120 would tile as well
    for key, (k, n) in {"h.0.mlp.c_fc.weight": (256, 40), "h.0.attn.c_proj.weight": (200, 24), "small": (64, 8),
                        "ragged9": (1080, 8)}.items():
        w = (rng.standard_normal((k, n)) * 0.05).astype(np.float32)
        p, s = oracle.quantize_weight_int4(w, k, n, 128)
        tensors[key + ".int4_packed"], tensors[key + ".int4_scales"] = p.reshape(k // 8, n), s.reshape(-1, n)
        want[key] = (p.reshape(k // 8, n), s.reshape(-1, n), k, n)
    tensors["ln_f.bias"] = rng.standard_normal(16).astype(np.float32)
    path = tmp_path / "model_int4.safetensors"
    write_safetensors(path, tensors)
    int4, dense = checkpoint.load_int4_tensors(path)
    assert set(dense) == {"ln_f.bias"} and np.array_equal(dense["ln_f.bias"], tensors["ln_f.bias"])
    assert set(int4) == set(want)
    for key, (p, s, k, n) in want.items():
        gp, gs, gk, gn, group = int4[key]
        assert (gk, gn) == (k, n) and np.array_equal(gp, p) and np.array_equal(gs, s)
        assert group == (128 if k > 128 else k)  # 200 rows: two groups, the second ragged
        # the pair is what the oracle's int4 Linear takes
        x = rng.standard_normal((2, k)).astype(np.float32)
        ref = x.astype(np.float64) @ oracle.dequant_weight_int4(gp, gs, k, n, group).reshape(k, n).astype(np.float64)
        assert np.allclose(oracle.int4_linear(x, gp, gs, None, 2, n, k, group, f64=True), ref, atol=1e-9)
    # a lone half of a pair, or a pair of the wrong dtype, is an error
    bad = dict(tensors)
    del bad["small.int4_scales"]
    write_safetensors(path, bad)
    with pytest.raises(b200nn.NnError):
        checkpoint.load_int4_tensors(path)
    bad = dict(tensors)
    bad["small.int4_packed"] = bad["small.int4_packed"].astype(np.int64)
    write_safetensors(path, bad)
    with pytest.raises(b200nn.NnError):
        checkpoint.load_int4_tensors(path)


def _tiny_gpt2_checkpoint(n_layer=2, d=8, vocab=11, npos=6, seed=3):
    """A checkpoint with Hugging Face GPT-2 key names: dense weights in Conv1D layout [in,out]."""
    rng = np.random.default_rng(seed)
    t = {"wte.weight": rng.standard_normal((vocab, d)), "wpe.weight": rng.standard_normal((npos, d)),
         "ln_f.weight": rng.standard_normal(d), "ln_f.bias": rng.standard_normal(d)}
    for i in range(n_layer):
        p = f"h.{i}"
        for k in ("ln_1", "ln_2"):
            t[f"{p}.{k}.weight"], t[f"{p}.{k}.bias"] = rng.standard_normal(d), rng.standard_normal(d)
        for k, (a, b) in {"attn.c_attn": (d, 3 * d), "attn.c_proj": (d, d), "mlp.c_fc": (d, 4 * d), "mlp.c_proj": (4 * d, d)}.items():
            t[f"{p}.{k}.weight"], t[f"{p}.{k}.bias"] = rng.standard_normal((a, b)), rng.standard_normal(b)
    return {k: np.asarray(v, np.float32) for k, v in t.items()}


def test_generic_loader_maps_names_and_transposes(tmp_path):
    """model_generic.rs: raw loading (F32 only), a weight map with renames and Conv1D -> Linear transposes,
    GPT-2's own map, the LoadedWeights accessors and their errors."""
    t = _tiny_gpt2_checkpoint()
    path = str(tmp_path / "model.safetensors")
    write_safetensors(path, t)
    raw = checkpoint.load_safetensors_raw(path)
    assert set(raw) == set(t) and raw["h.1.mlp.c_fc.weight"].shape == [8, 32]
    assert np.array_equal(raw["wte.weight"].data.reshape(11, 8), t["wte.weight"])
    lw = checkpoint.load_safetensors(path)
    assert len(lw) == len(t) and not lw.is_empty() and lw.total_params() == sum(v.size for v in t.values())
    m = [checkpoint.map_weight("wte.weight", "embedding.tokens"), checkpoint.map_weight_t("h.0.attn.c_attn.weight", "block.0.qkv")]
    mapped = checkpoint.load_safetensors_mapped(path, m)
    assert len(mapped) == 2 and mapped.get("wte.weight") is None
    qkv = mapped.require("block.0.qkv")
    assert qkv.shape == [24, 8] and np.array_equal(qkv.data.reshape(24, 8), t["h.0.attn.c_attn.weight"].T)
    with pytest.raises(b200nn.NnError) as e:
        mapped.require("block.1.qkv")
    assert e.value.code == b200nn.ERR_MISSING
    with pytest.raises(b200nn.NnError) as e:
        checkpoint.load_safetensors_mapped(path, [checkpoint.map_weight("no.such.key", "x")])
    assert e.value.code == b200nn.ERR_MISSING
    with pytest.raises(b200nn.NnError):  # transpose_2d of a vector is the reference's error, too
        checkpoint.load_safetensors_mapped(path, [checkpoint.map_weight_t("ln_f.bias", "x")])
    gm = checkpoint.gpt2_weight_map(2)
    assert len(gm) == 4 + 2 * 12 and sum(x.transform == checkpoint.TRANSFORM_TRANSPOSE_2D for x in gm) == 8
    g = checkpoint.load_safetensors_mapped(path, gm)
    assert g.require("h.1.mlp.c_proj.weight").shape == [8, 32]  # [out,in]
    assert g.require("h.1.mlp.c_proj.bias").shape == [8] and g.require("ln_f.weight").shape == [8]
    # a tensor of another dtype is refused by the raw loader
    t2 = dict(t)
    t2["extra"] = np.arange(4, dtype=np.uint32)
    write_safetensors(path, t2)
    with pytest.raises(b200nn.NnError):
        checkpoint.load_safetensors_raw(path)
