"""CPU tests of the C-ABI library: it loads, exports every declared symbol, its host-side logic
(the quantiser) matches the oracle, and without a GPU it fails loudly instead of falling back."""
import ctypes as C
import os
import re

import numpy as np
import pytest

import b200nn
from b200nn import ops
from oracle import oracle

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "b200nn.h")).read()
    return sorted(set(re.findall(r"B200NN_API[^;]*?\b(b200nn_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = b200nn.load_library()
    names = _declared_symbols()
    assert len(names) > 70
    for n in names:
        assert hasattr(lib, n), f"libb200nn.so does not export {n}"
    # and the Python mirror binds each of them with a signature
    assert set(names) == set(lib._declared)


def test_rust_sys_crate_declares_exactly_the_header(): 
    """crates/b200nn-sys/src/lib.rs (the binding the reference's Rust host links against; it cannot be
    compiled where there is no cargo) must declare every exported function once, with the header's
    parameter count, and the #[repr(C)] structs must have the header's fields in the header's order."""
    text = open(os.path.join(ROOT, "include", "b200nn.h")).read()
    header = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    h_fns = {}
    for m in re.finditer(r"B200NN_API\s+[^;#]*?\b(b200nn_\w+)\s*\(([^;]*?)\)\s*;", header, flags=re.S):
        args = " ".join(m.group(2).split())
        h_fns[m.group(1)] = 0 if args == "void" else args.count(",") + 1
    rs = open(os.path.join(ROOT, "crates", "b200nn-sys", "src", "lib.rs")).read()
    r_fns = {}
    for m in re.finditer(r"pub fn (b200nn_\w+)\s*\((.*?)\)\s*(?:->\s*[^;]+)?;", rs, flags=re.S):
        args = m.group(2).strip().rstrip(",")
        assert m.group(1) not in r_fns, f"{m.group(1)} declared twice"
        r_fns[m.group(1)] = 0 if not args else args.count(":")
    assert set(r_fns) == set(h_fns) == set(_declared_symbols())
    assert r_fns == h_fns
    # struct fields: C `const float *a, *b;` lists against Rust `pub a: *const f32,`
    for name in ("b200nn_gpt2_config", "b200nn_gpt2_layer_weights", "b200nn_gpt2_weights", "b200nn_block_weights",
                 "b200nn_gpt2_diagnostic"):
        c_body = re.search(r"typedef struct \{([^}]*)\}\s*" + name + r"\s*;", header).group(1)
        c_fields = []
        for stmt in c_body.split(";"):
            stmt = stmt.strip()
            if stmt:
                c_fields += [re.sub(r"\[\d+\]|[^\w]", "", part.split()[-1]) for part in stmt.split(",")]
        r_body = re.search(r"pub struct " + name + r"\s*\{([^}]*)\}", rs).group(1)
        r_fields = re.findall(r"pub (\w+):", r_body)
        assert r_fields == c_fields, name
    for const in re.findall(r"\b(B200NN_[A-Z0-9_]+)\s*=", header):
        assert re.search(r"pub const " + const + r":", rs), f"{const} missing from the crate"


def test_version_string():
    assert b"sm_100a" in b200nn.load_library().b200nn_version()


def _has_gpu():
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


@pytest.mark.skipif(_has_gpu(), reason="checks the no-GPU behaviour")
def test_no_gpu_means_error_not_fallback():
    with pytest.raises(b200nn.NnError) as e:
        b200nn.KernelRegistry.init_default()
    assert e.value.code == b200nn.ERR_CUDA


@pytest.mark.parametrize("k,n,group", [(8, 4, 128), (64, 24, 32), (768, 96, 128), (1600, 33, 128)])
def test_host_quantizer_matches_oracle(k, n, group):
    rng = np.random.default_rng(k + n)
    w = (rng.standard_normal((k, n)) * 0.02).astype(np.float32)
    w[:, -1] = 0.0
    p, s = ops.quantize_weight_int4(w, k, n, group)
    po, so = oracle.quantize_weight_int4(w, k, n, group)
    assert np.array_equal(p, po) and np.array_equal(s, so)


def test_host_quantizer_rejects_bad_k():
    with pytest.raises(b200nn.NnError) as e:
        ops.quantize_weight_int4(np.zeros((12, 4), np.float32), 12, 4, 128)
    assert e.value.code == b200nn.ERR_SHAPE


def test_host_pack_helpers_match_reference_kats():
    assert ops.pack_int8_to_u32([1, 2, 3, 4, 5, 6, 7, 8]).tolist() == [0x04030201, 0x08070605]
    assert ops.pack_int8_to_u32([1, 2, 3]).tolist() == [0x00030201]
    q, s = ops.quantize_int8_per_tensor([0.0, 1.0, -1.0, 0.5])
    assert abs(s - 1 / 127) < 1e-6 and q[:3].tolist() == [0, 127, -127]
    data = np.array([0.0, 1.0, -1.0, 0.5, 0.25, -0.5, 0.75, -0.75], dtype=np.float32)
    p, sc = ops.quantize_int4_per_group(data, 128)
    po, so = oracle.quantize_int4_per_group(data, 128)
    assert np.array_equal(p, po) and np.array_equal(sc, so)
    word = sum(((v + 8) & 0xF) << (4 * i) for i, v in enumerate(range(-4, 4)))
    assert [ops.unpack_int4(word, i) for i in range(8)] == list(range(-4, 4))


def test_config_presets():
    lib = b200nn.load_library()
    for name, (l, d, h) in dict(small=(12, 768, 12), medium=(24, 1024, 16), large=(36, 1280, 20),
                                xl=(48, 1600, 25)).items():
        c = b200nn._Cfg()
        assert lib.b200nn_gpt2_config_preset(name.encode(), C.byref(c)) == 0
        assert (c.n_layer, c.n_embd, c.n_head, c.vocab_size, c.n_positions) == (l, d, h, 50257, 1024)
        py = getattr(b200nn.Gpt2Config, name)()
        assert (py.n_layer, py.n_embd, py.n_head) == (l, d, h) and py.head_dim() == 64 and py.ffn_dim() == 4 * d
    assert lib.b200nn_gpt2_config_preset(b"huge", C.byref(b200nn._Cfg())) == b200nn.ERR_UNSUPPORTED


def test_null_handles_are_rejected():
    lib = b200nn.load_library()
    assert lib.b200nn_ctx_synchronize(None) == b200nn.ERR_ARG
    assert lib.b200nn_session_step(None, 1) == b200nn.ERR_ARG
    assert lib.b200nn_tensor_numel(None) == 0
    assert lib.b200nn_kvcache_len(None) == 0


def test_mirror_carries_the_reference_names_of_the_path():
    """The host-side mirror keeps the reference's public names for the GPT-2 inference path, so that a test
    written against ``gpu_host::nn`` reads the same here (nn/ops/*.rs, nn/layers/*.rs, nn/tensor.rs,
    nn/models/gpt2.rs, by file)."""
    want = {
        ops: ["matmul", "matmul_v2", "matmul_v4", "matmul_v4_1", "matmul_fused", "int4_matmul",           # ops/gemm.rs
              "layer_norm", "layer_norm_residual", "layer_norm_residual_dual",                             # ops/norm.rs
              "scaled_dot_product_attention", "scaled_dot_product_attention_kv", "split_qkv", "concat_heads",
              "multi_head_flash_attention", "multi_head_flash_attention_v3", "multi_head_flash_attention_nvrtc",
              "gelu", "silu", "sigmoid", "relu",                                                           # ops/activation.rs
              "bias_add", "elementwise_add", "elementwise_add_out", "embedding_lookup",                    # ops/reshape.rs
              "quantize_int4_per_group", "quantize_weight_int4", "unpack_int4"],                           # ops/quantize.rs
        b200nn.GpuTensor: ["from_data", "from_host", "to_host", "zeros", "numel", "ndim", "shape", "strides",
                           "is_contiguous", "size_bytes", "reshape", "transpose", "clone_tensor", "concat", "split"],
        b200nn.Linear: ["with_codegen", "forward", "forward_fused", "forward_auto_fused"],
        b200nn.Int4Linear: ["forward", "memory_bytes"],
        b200nn.LayerNorm: ["forward", "gamma", "beta"],
        b200nn.Embedding: ["forward_tokens", "forward_tokens_with_offset"],
        b200nn.MultiHeadAttention: ["forward_causal", "forward_cached"],
        b200nn.Int4MultiHeadAttention: ["forward_causal"],
        b200nn.Gpt2Config: ["small", "medium", "large", "xl", "head_dim", "ffn_dim"],
        b200nn.Gpt2Model: ["from_weights", "from_generic_weights", "forward", "forward_auto_fused", "forward_profiled",
                           "forward_features", "embedding_table", "forward_diagnostic", "generate", "forward_cached",
                           "generate_cached", "forward_early_exit", "generate_cached_early_exit",
                           "generate_cached_sampling"],
        b200nn.Int4Gpt2Model: ["from_weights", "from_generic_weights", "group_size", "forward", "generate",
                               "quantized_memory_bytes"],
        b200nn.TransformerBlock: ["forward", "forward_auto_fused", "forward_cached"],
        b200nn.Int4TransformerBlock: ["forward"],
        b200nn.KernelRegistry: ["init_default"],
        b200nn.SimpleRng: ["next_f32"],
        b200nn: ["GELU", "SiLU", "Sigmoid", "ReLU", "KvCache", "top_k_sample", "NnError"],
    }
    missing = [f"{getattr(o, '__name__', o)}.{n}" for o, names in want.items() for n in names if not hasattr(o, n)]
    assert not missing, missing


def test_safe_rust_crate_names_only_what_the_sys_crate_declares():
    """crates/b200nn (the safe layer with the reference's names; not compiled where there is no cargo): every
    `sys::` item it uses is declared by crates/b200nn-sys, its brackets balance, and it carries the same types
    as the C++ host layer it follows (include/b200nn.hpp)."""
    safe = open(os.path.join(ROOT, "crates", "b200nn", "src", "lib.rs")).read()
    sysrs = open(os.path.join(ROOT, "crates", "b200nn-sys", "src", "lib.rs")).read()
    used = sorted(set(re.findall(r"\bsys::(\w+)", safe)))
    assert len(used) > 60
    missing = [n for n in used if not re.search(r"\b(fn|const|struct)\s+%s\b" % n, sysrs) and not re.search(r"^\s+%s,$" % n, sysrs, flags=re.M)]
    assert not missing, missing
    for o, c in ("{}", "()", "[]"):
        assert safe.count(o) == safe.count(c)
    hpp = open(os.path.join(ROOT, "include", "b200nn.hpp")).read()
    for name in ["KernelRegistry", "GpuTensor", "Linear", "Int4Linear", "LayerNorm", "Embedding", "MultiHeadAttention",
                 "Gpt2Config", "Gpt2Weights", "TransformerLayerWeights", "Gpt2Model", "Int4Gpt2Model", "KvCache", "SimpleRng",
                 "NnError", "Activation", "FusedActivation", "TransformerBlock", "BlockWeights", "DecodeSession"]:
        assert re.search(r"\b(struct|enum)\s+%s\b" % name, safe), name
        assert re.search(r"\b(class|struct|enum class|using)\s+%s\b" % name, hpp), name
