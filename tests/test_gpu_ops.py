"""GPU parity tests of the single ops and layers, through the C ABI, against the CPU oracle.

Tolerances: f32 CUDA-core kernels are compared at 1e-5 relative RMS (f32 accumulation against the
oracle's f64); kernels that feed fp16 operands to the tensor cores at 5e-4 relative RMS, inside
the path's budget of 1e-3 relative RMS / 2e-2 max-abs on logits."""
import json
import os

import numpy as np
import pytest

import b200nn
import np_ref
from b200nn import GpuTensor, ops, synth
from oracle import oracle

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
KATS = json.load(open(os.path.join(HERE, "golden", "reference_kats.json")))


def _formula(expr, n, **env):
    return np.array([eval(expr, {}, dict(i=i, **env)) for i in range(n)], dtype=np.float32)


# ---- isolated int4 Linear: the shapes of the benchmark's second configuration -------------------
@pytest.mark.parametrize("k,n", [(768, 3072), (3072, 768), (768, 2304), (768, 50257)])
@pytest.mark.parametrize("m", [1, 8, 64])
def test_int4_linear_shapes(reg, m, k, n):
    packed, scales, x, _ = synth.int4_linear_case(100 + m, m, k, n, 128)
    lin = b200nn.Int4Linear(packed, scales, None, k, n, 128, reg)
    y = lin.forward(GpuTensor.from_host(x, (m, k), reg)).to_host()
    ref = oracle.int4_linear(x, packed, scales, None, m, n, k, 128, f64=True)
    assert y.shape == (m, n)
    rr = np_ref.rel_rms(y, ref)
    tc = m > 2  # rows above the GEMV threshold take the fp16 tensor-core path
    assert rr < (5e-4 if tc else 1e-5), rr
    assert np.abs(y - ref).max() < (2e-2 if tc else 1e-3)
    assert lin.memory_bytes() == packed.size * 4 + scales.size * 4


@pytest.mark.parametrize("m,k,n,group", [(1, 1600, 1600, 128), (2, 6400, 1600, 128), (3, 1600, 4800, 128),
                                         (4, 128, 130, 64), (7, 192, 257, 64), (5, 64, 1, 64)])
def test_int4_linear_ragged(reg, m, k, n, group):
    # K=1600 has a ragged last group of 64; N not a multiple of the 128-row tile; bias present
    packed, scales, x, _ = synth.int4_linear_case(7 * m + k, m, k, n, group)
    bias = np.linspace(-0.5, 0.5, n).astype(np.float32)
    reg.set_gemv_max_rows(8)  # exercise the CUDA-core path for every row count here
    try:
        y = b200nn.Int4Linear(packed, scales, bias, k, n, group, reg).forward(GpuTensor.from_host(x, (m, k), reg)).to_host()
    finally:
        reg.set_gemv_max_rows(-1)
    ref = oracle.int4_linear(x, packed, scales, bias, m, n, k, group, f64=True)
    assert np_ref.rel_rms(y, ref) < 1e-5


@pytest.mark.parametrize("k,n,group", [(8, 4, 128), (24, 5, 16), (40, 3, 128)])
def test_int4_linear_odd_shapes_take_generic_kernel(reg, k, n, group):
    # shapes the tiled layout cannot hold (K % 64 != 0) still work, as in the reference
    rng = np.random.default_rng(k)
    w = (rng.standard_normal((k, n)) * 0.1).astype(np.float32)
    packed, scales = ops.quantize_weight_int4(w, k, n, group)
    x = rng.standard_normal((3, k)).astype(np.float32)
    y = b200nn.Int4Linear(packed, scales, None, k, n, group, reg).forward(GpuTensor.from_host(x, (3, k), reg)).to_host()
    sc16 = oracle.f16_round(scales)  # the library keeps group scales in fp16
    ref = oracle.int4_linear(x, packed, sc16, None, 3, n, k, group, f64=True)
    assert np.abs(y - ref).max() < 1e-5


def test_int4_linear_host_entry_and_errors(reg):
    packed, scales, x, _ = synth.int4_linear_case(5, 2, 768, 768, 128)
    lin = b200nn.Int4Linear(packed, scales, None, 768, 768, 128, reg)
    y = lin.forward_host(x)
    ref = oracle.int4_linear(x, packed, scales, None, 2, 768, 768, 128)
    assert np_ref.rel_rms(y, ref) < 1e-5
    with pytest.raises(b200nn.NnError) as e:  # int4_linear.rs:74-79 shape check
        lin.forward(GpuTensor.zeros((2, 700), reg))
    assert e.value.code == b200nn.ERR_SHAPE
    with pytest.raises(b200nn.NnError):
        b200nn.Int4Linear(packed, scales, None, 770, 768, 128, reg)


def test_int4_matmul_op(reg):
    rng = np.random.default_rng(1)
    b = (rng.standard_normal((256, 96)) * 0.05).astype(np.float32)
    a = rng.standard_normal((2, 256)).astype(np.float32)
    y = ops.int4_matmul(GpuTensor.from_host(a, (2, 256), reg), b, 256, 96, 128, reg).to_host()
    p, s = oracle.quantize_weight_int4(b, 256, 96, 128)
    ref = oracle.int4_linear(a, p, oracle.f16_round(s), None, 2, 96, 256, 128)
    assert np_ref.rel_rms(y, ref) < 1e-5


# ---- f32 Linear: the reference's own arithmetic-pattern tests (layers/linear.rs:388-464) ---------
# Tuning key f32_tc selects how more than four rows are multiplied: 2 (default) fp16 activations times
# the weight as fp16 hi + lo on the tensor cores, 1 the weight rounded to fp16 only, 0 the f32 FMA kernels.
@pytest.mark.parametrize("idx", [0, 1])
def test_linear_reference_patterns(reg, idx):
    c = KATS["patterns"][idx]
    b, k, n = c["batch"], c["in"], c["out"]
    w = _formula(c["weight_formula"], n * k)
    bias = _formula(c["bias_formula"], n)
    x = _formula(c["input_formula"], b * k)
    lin = b200nn.Linear(w, bias, k, n, reg)
    ref = oracle.matmul(x, np.ascontiguousarray(w.reshape(n, k).T), b, k, n) + bias
    for mode in (2, 1, 0):
        reg.set_tuning("f32_tc", mode)
        try:
            y = lin.forward(GpuTensor.from_host(x, (b, k), reg)).to_host()
        finally:
            reg.set_tuning("f32_tc", -1)
        assert y.shape == (b, n)
        # fp16 activations on the tensor-core paths: inside the reference's own tolerance
        assert np.abs(y - ref).max() < min(c["tol"], 1e-4 if (b <= 4 or mode == 0) else 2e-3)


@pytest.mark.parametrize("m", [1, 3, 70])
def test_linear_fused_activation(reg, m):
    rng = np.random.default_rng(m)
    w = (rng.standard_normal((200, 96)) * 0.1).astype(np.float32)  # [out,in]
    bias = rng.standard_normal(200).astype(np.float32)
    x = rng.standard_normal((m, 96)).astype(np.float32)
    lin = b200nn.Linear(w, bias, 96, 200, reg)
    pre = x.astype(np.float64) @ w.astype(np.float64).T + bias
    for mode in (2, 1, 0):
        reg.set_tuning("f32_tc", mode)
        try:
            tol = 2e-3 if (mode and m > 4) else 1e-4
            y = lin.forward_fused(GpuTensor.from_host(x, (m, 96), reg), b200nn.ACT_GELU_TANH).to_host()
            assert np.abs(y - np_ref.gelu_tanh(pre)).max() < tol
            y = lin.forward_fused(GpuTensor.from_host(x, (m, 96), reg), b200nn.ACT_RELU).to_host()
            assert np.abs(y - np.maximum(pre, 0)).max() < tol
        finally:
            reg.set_tuning("f32_tc", -1)
    with pytest.raises(b200nn.NnError):
        lin.forward(GpuTensor.zeros((m, 95), reg))


@pytest.mark.parametrize("mode", [2, 1])
@pytest.mark.parametrize("m,k,n", [(5, 768, 768), (33, 768, 2304), (128, 1600, 6400), (300, 6400, 1600),
                                   (1000, 768, 3072), (64, 1600, 50257), (7, 72, 130), (260, 200, 1), (9, 8, 129)])
def test_linear_tensor_core_shapes(reg, m, k, n, mode):
    """f32 Linear of more than four rows (linear.rs:283-313) on the tensor cores, f32 accumulation.
    Checked twice: against the f64 product of the f32 operands at the fp16 tolerance, and against the
    f64 product of exactly the operands the kernel multiplies (fp16-rounded activations; the weight as
    fp16 hi + lo, or rounded to fp16) at f32 accumulation accuracy, which pins tiling, swizzle, K tail
    (K % 64 != 0), ragged N and row tails."""
    rng = np.random.default_rng(m * 7 + n)
    w = (rng.standard_normal((n, k)) * 0.05).astype(np.float32)
    bias = rng.standard_normal(n).astype(np.float32)
    x = rng.standard_normal((m, k)).astype(np.float32)
    reg.set_tuning("f32_tc", mode)
    try:
        launches = reg.launch_count()
        y = b200nn.Linear(w, bias, k, n, reg).forward(GpuTensor.from_host(x, (m, k), reg)).to_host()
        assert reg.launch_count() - launches == 2  # activation conversion + the GEMM
    finally:
        reg.set_tuning("f32_tc", -1)
    ref = x.astype(np.float64) @ w.astype(np.float64).T + bias
    assert np_ref.rel_rms(y, ref) < (3.5e-4 if mode == 2 else 5e-4)
    hi = w.astype(np.float16)
    w_used = hi.astype(np.float64)
    if mode == 2:
        w_used = w_used + (w - hi.astype(np.float32)).astype(np.float16).astype(np.float64)
        assert np.abs(w_used - w).max() < 1e-7  # hi + lo carries the f32 weight to about 22 bits
    ref16 = x.astype(np.float16).astype(np.float64) @ w_used.T + bias
    assert np_ref.rel_rms(y, ref16) < 5e-6
    assert np.abs(y - ref16).max() < 1e-4 * max(1.0, float(np.abs(ref16).max()))
    assert reg.device_error() == 0


def test_linear_tensor_core_fallbacks(reg):
    """K not a multiple of 8 (no 16-byte row stride for the tensor map) and weights beyond fp16's range
    keep the f32 FMA kernels."""
    rng = np.random.default_rng(5)
    for k, scale in [(100, 0.05), (96, 1e6)]:
        w = (rng.standard_normal((40, k)) * scale).astype(np.float32)
        x = rng.standard_normal((9, k)).astype(np.float32)
        y = b200nn.Linear(w, None, k, 40, reg).forward(GpuTensor.from_host(x, (9, k), reg)).to_host()
        ref = x.astype(np.float64) @ w.astype(np.float64).T
        assert np_ref.rel_rms(y, ref) < 1e-5


# ---- LayerNorm, activations, element-wise -------------------------------------------------------
def test_layernorm_reference_pattern(reg):
    c = KATS["patterns"][2]
    b, d = c["batch"], c["d"]
    g = _formula(c["gamma_formula"], d)
    be = _formula(c["beta_formula"], d)
    x = _formula(c["input_formula"], b * d, batch=b, d=d)
    y = b200nn.LayerNorm(g, be, c["eps"], reg).forward(GpuTensor.from_host(x, (b, d), reg)).to_host()
    assert np.abs(y - oracle.layer_norm(x, g, be, c["eps"]).reshape(b, d)).max() < 1e-5


@pytest.mark.parametrize("rows,d", [(1, 768), (33, 1600), (5, 64), (3, 5000), (1024, 768), (1531, 1600), (2050, 64),
                                    (1100, 2048), (1025, 1284)])
def test_layernorm_and_residual_dual(reg, rows, d):
    # from 1024 rows on (and d a multiple of 4 up to 2048) the plain form takes the warp-per-row kernel
    rng = np.random.default_rng(d)
    x = (rng.standard_normal((rows, d)) * 3 + 50).astype(np.float32)  # large mean: needs the two-pass variance
    r = rng.standard_normal((rows, d)).astype(np.float32)
    g = rng.standard_normal(d).astype(np.float32)
    b = rng.standard_normal(d).astype(np.float32)
    tg, tb = GpuTensor.from_host(g, (d,), reg), GpuTensor.from_host(b, (d,), reg)
    y = ops.layer_norm(GpuTensor.from_host(x, (rows, d), reg), tg, tb, 1e-5, reg).to_host()
    assert np.abs(y - oracle.layer_norm(x, g, b).reshape(rows, d)).max() < 2e-4
    s, nrm = ops.layer_norm_residual_dual(GpuTensor.from_host(x, (rows, d), reg), GpuTensor.from_host(r, (rows, d), reg),
                                          tg, tb, 1e-5, reg)
    assert np.array_equal(s.to_host(), x + r)
    assert np.abs(nrm.to_host() - oracle.layer_norm(x + r, g, b).reshape(rows, d)).max() < 2e-4


def test_gelu_forms(reg):
    x = np.linspace(-5, 5, 1001).astype(np.float32)  # range of tests_transformer.rs:128-207
    t = GpuTensor.from_host(x, (1001,), reg)
    assert np.abs(ops.gelu(t, reg).to_host() - oracle.gelu_tanh(x)).max() < 1e-5
    assert np.abs(ops.gelu(t, reg, sigmoid_form=True).to_host() - oracle.gelu_sigmoid(x)).max() < 1e-5
    assert np.abs(b200nn.GELU(reg).forward(t).to_host() - np_ref.gelu_tanh(x)).max() < 1e-5


def test_bias_add_elementwise_add_reshape(reg):
    rng = np.random.default_rng(2)
    a = rng.standard_normal((6, 10)).astype(np.float32)
    b = rng.standard_normal((6, 10)).astype(np.float32)
    bias = rng.standard_normal(10).astype(np.float32)
    ta = GpuTensor.from_host(a, (6, 10), reg)
    ops.bias_add(ta, GpuTensor.from_host(bias, (10,), reg), reg)
    ops.elementwise_add(ta, GpuTensor.from_host(b, (6, 10), reg), reg)
    assert np.allclose(ta.to_host(), a + bias + b, atol=1e-6)
    v = ta.reshape((3, 20))
    assert v.shape() == (3, 20) and np.array_equal(v.to_host().ravel(), ta.to_host().ravel())
    with pytest.raises(b200nn.NnError):
        ta.reshape((7, 7))
    z = GpuTensor.zeros((4, 4), reg)
    assert not z.to_host().any() and z.clone_tensor().numel() == 16


def test_embedding_with_offset(reg):
    rng = np.random.default_rng(3)
    wte = rng.standard_normal((50, 64)).astype(np.float32)
    wpe = rng.standard_normal((16, 64)).astype(np.float32)
    e = b200nn.Embedding(wte, wpe, 50, 16, 64, reg)
    ids = np.array([3, 49, 0, 7], dtype=np.uint32)
    assert np.array_equal(e.forward_tokens(ids).to_host(), wte[ids] + wpe[:4])   # tests_transformer.rs:739-836
    assert np.array_equal(e.forward_tokens_with_offset(ids, 4, 9).to_host(), wte[ids] + wpe[9:13])
    with pytest.raises(b200nn.NnError):
        e.forward_tokens(np.array([50], dtype=np.uint32))
    with pytest.raises(b200nn.NnError):
        e.forward_tokens_with_offset(ids, 4, 13)


def test_split_qkv_concat_heads_roundtrip(reg):
    rng = np.random.default_rng(4)
    seq, H, dh = 7, 3, 64
    qkv = rng.standard_normal((seq, 3 * H * dh)).astype(np.float32)
    q, k, v = ops.split_qkv(GpuTensor.from_host(qkv, qkv.shape, reg), seq, H, dh, reg)
    d = H * dh
    for t, off in ((q, 0), (k, d), (v, 2 * d)):
        ref = qkv[:, off:off + d].reshape(seq, H, dh).transpose(1, 0, 2)
        assert np.array_equal(t.to_host(), ref)
    back = ops.concat_heads(q, seq, H, dh, reg).to_host()
    assert np.array_equal(back, qkv[:, :d])


def test_int4_linear_from_int4_checkpoint_pair(reg, tmp_path):
    """`<key>.int4_packed` / `<key>.int4_scales` of the reference script's int4 checkpoint
    (scripts/quantize_gpt2_int4.py:85-99) go straight into Int4Linear (int4_linear.rs:40-48)."""
    from test_checkpoint_cpu import write_safetensors
    rng = np.random.default_rng(21)
    k, n = 768, 200
    w = (rng.standard_normal((k, n)) * 0.05).astype(np.float32)
    p, s = oracle.quantize_weight_int4(w, k, n, 128)
    path = tmp_path / "model_int4.safetensors"
    write_safetensors(path, {"h.0.mlp.c_fc.weight.int4_packed": p.reshape(k // 8, n),
                             "h.0.mlp.c_fc.weight.int4_scales": s.reshape(-1, n),
                             "h.0.mlp.c_fc.bias": np.linspace(-1, 1, n).astype(np.float32)})
    int4, dense = b200nn.load_int4_tensors(path)
    gp, gs, gk, gn, group = int4["h.0.mlp.c_fc.weight"]
    lin = b200nn.Int4Linear(gp, gs, dense["h.0.mlp.c_fc.bias"], gk, gn, group, reg)
    for m in (1, 40):
        x = rng.standard_normal((m, k)).astype(np.float32)
        y = lin.forward(GpuTensor.from_host(x, (m, k), reg)).to_host()
        ref = oracle.int4_linear(x, gp, oracle.f16_round(gs), dense["h.0.mlp.c_fc.bias"], m, n, k, group, f64=True)
        assert np_ref.rel_rms(y, ref) < (1e-5 if m == 1 else 5e-4)


@pytest.mark.parametrize("mode", [2, 1])
@pytest.mark.parametrize("m,k,n", [(9000, 256, 1100), (9000, 200, 1100), (16384, 768, 768)])
def test_linear_tensor_core_many_tiles_take_the_persistent_kernel(reg, m, k, n, mode):
    """From two 256-row tiles per SM on, one persistent block per SM walks the tiles with two accumulators
    (the epilogue of one tile overlaps the K loop of the next).  Ragged N, a row tail, a K tail; compared
    with the one-tile-per-block kernel (tuning key tc_persistent = 0: same operands, same order of the K
    blocks) and with the f64 product of the operands the kernel multiplies."""
    rng = np.random.default_rng(m + k + n)
    w = (rng.standard_normal((n, k)) * 0.05).astype(np.float32)
    bias = rng.standard_normal(n).astype(np.float32)
    x = rng.standard_normal((m, k)).astype(np.float32)
    lin = b200nn.Linear(w, bias, k, n, reg)
    t = GpuTensor.from_host(x, (m, k), reg)
    reg.set_tuning("f32_tc", mode)
    try:
        y = lin.forward_fused(t, b200nn.ACT_GELU_TANH).to_host()
        reg.set_tuning("tc_persistent", 0)
        y1 = lin.forward_fused(t, b200nn.ACT_GELU_TANH).to_host()
    finally:
        reg.set_tuning("tc_persistent", 1)
        reg.set_tuning("f32_tc", -1)
    assert np.array_equal(y, y1)
    hi = w.astype(np.float16)
    w_used = hi.astype(np.float64)
    if mode == 2:
        w_used = w_used + (w - hi.astype(np.float32)).astype(np.float16).astype(np.float64)
    ref16 = np_ref.gelu_tanh(x.astype(np.float16).astype(np.float64) @ w_used.T + bias)
    assert np_ref.rel_rms(y, ref16) < 5e-6
    assert reg.device_error() == 0


def test_tensor_transpose_concat_split(reg):
    """GpuTensor::transpose / concat / split (tensor.rs:227-393) on the device, against numpy, with the
    reference's errors (DimOutOfRange, ShapeMismatch)."""
    rng = np.random.default_rng(21)
    a = rng.standard_normal((3, 4, 5, 2)).astype(np.float32)
    t = GpuTensor.from_host(a, a.shape, reg)
    assert t.ndim() == 4 and t.strides() == (40, 10, 2, 1) and t.is_contiguous() and t.size_bytes() == a.size * 4
    for d0, d1 in [(0, 1), (1, 3), (0, 3), (2, 2), (3, 1)]:
        got = t.transpose(d0, d1)
        ref = np.swapaxes(a, d0, d1)
        assert got.shape() == ref.shape and np.array_equal(got.to_host(), ref)
    m = rng.standard_normal((257, 130)).astype(np.float32)  # a 2-D case larger than a block
    assert np.array_equal(GpuTensor.from_host(m, m.shape, reg).transpose(0, 1).to_host(), m.T)
    with pytest.raises(b200nn.NnError) as e:
        t.transpose(0, 4)
    assert e.value.code == b200nn.ERR_DIM
    parts = [rng.standard_normal(s).astype(np.float32) for s in [(3, 2, 5), (3, 4, 5), (3, 1, 5)]]
    tp = [GpuTensor.from_host(p, p.shape, reg) for p in parts]
    for dim, ps in [(1, parts), (0, [parts[0], parts[0]]), (2, [parts[1], parts[1], parts[1]])]:
        got = GpuTensor.concat([GpuTensor.from_host(p, p.shape, reg) for p in ps], dim)
        ref = np.concatenate(ps, axis=dim)
        assert got.shape() == ref.shape and np.array_equal(got.to_host(), ref)
    with pytest.raises(b200nn.NnError) as e:
        GpuTensor.concat([tp[0], tp[1]], 0)  # sizes differ in a dimension that is not the concatenated one
    assert e.value.code == b200nn.ERR_SHAPE
    with pytest.raises(b200nn.NnError) as e:
        GpuTensor.concat([tp[0]], 3)
    assert e.value.code == b200nn.ERR_DIM
    with pytest.raises(b200nn.NnError):
        GpuTensor.concat([], 0)
    big = np.concatenate(parts, axis=1)
    tb = GpuTensor.from_host(big, big.shape, reg)
    chunks = tb.split(1, [2, 4, 1])
    assert [c.shape() for c in chunks] == [(3, 2, 5), (3, 4, 5), (3, 1, 5)]
    for c, p in zip(chunks, parts):
        assert np.array_equal(c.to_host(), p)
    last = tb.split(2, [1, 4])
    assert np.array_equal(last[0].to_host(), big[:, :, :1]) and np.array_equal(last[1].to_host(), big[:, :, 1:])
    with pytest.raises(b200nn.NnError) as e:
        tb.split(1, [2, 4])  # sizes must add up to the dimension
    assert e.value.code == b200nn.ERR_SHAPE
    with pytest.raises(b200nn.NnError) as e:
        tb.split(5, [7])
    assert e.value.code == b200nn.ERR_DIM


def test_ops_matmul_activations_and_small_wrappers(reg):
    """ops::matmul (gemm.rs:20-212), the Activation kinds Silu and Sigmoid (linear.rs:24-33, activation.rs:21-33),
    scaled_dot_product_attention, layer_norm_residual, elementwise_add_out, embedding_lookup: against numpy."""
    rng = np.random.default_rng(33)
    for m, k, n in [(1, 64, 5), (3, 130, 257), (7, 768, 96), (200, 96, 33)]:
        a = rng.standard_normal((m, k)).astype(np.float32)
        b = rng.standard_normal((k, n)).astype(np.float32)
        y = ops.matmul(GpuTensor.from_host(a, a.shape, reg), GpuTensor.from_host(b, b.shape, reg), reg).to_host()
        ref = a.astype(np.float64) @ b.astype(np.float64)
        assert y.shape == (m, n) and np_ref.rel_rms(y, ref) < 1e-5
    with pytest.raises(b200nn.NnError) as e:
        ops.matmul(GpuTensor.from_host(a, a.shape, reg), GpuTensor.from_host(a, a.shape, reg), reg)
    assert e.value.code == b200nn.ERR_SHAPE
    x = np.linspace(-6, 6, 999).astype(np.float32)
    t = GpuTensor.from_host(x, x.shape, reg)
    sig = 1.0 / (1.0 + np.exp(-x.astype(np.float64)))
    assert np.abs(ops.sigmoid(t, reg).to_host() - sig).max() < 1e-6
    assert np.abs(ops.silu(t, reg).to_host() - x * sig).max() < 1e-5
    # Linear::forward_fused with the two kinds (more than four rows: tensor-core path; one row: GEMV)
    w = (rng.standard_normal((40, 64)) * 0.1).astype(np.float32)
    bias = rng.standard_normal(40).astype(np.float32)
    lin = b200nn.Linear(w, bias, 64, 40, reg)
    for rows in (1, 9):
        xi = rng.standard_normal((rows, 64)).astype(np.float32)
        pre = xi.astype(np.float64) @ w.T.astype(np.float64) + bias
        got = lin.forward_fused(GpuTensor.from_host(xi, xi.shape, reg), b200nn.ACT_SILU).to_host()
        assert np.abs(got - pre / (1 + np.exp(-pre))).max() < (1e-5 if rows == 1 else 5e-3)
        got = lin.forward_fused(GpuTensor.from_host(xi, xi.shape, reg), b200nn.ACT_SIGMOID).to_host()
        assert np.abs(got - 1 / (1 + np.exp(-pre))).max() < (1e-5 if rows == 1 else 2e-3)
    # one head, full causal attention == the kv form with no offset
    q, k, v = [rng.standard_normal((33, 64)).astype(np.float32) for _ in range(3)]
    tq, tk, tv = [GpuTensor.from_host(z, z.shape, reg) for z in (q, k, v)]
    full = ops.scaled_dot_product_attention(tq, tk, tv, True, reg).to_host()
    ref = oracle.mha(q, oracle.f16_round(k)[None], oracle.f16_round(v)[None], 1, 64, 33, 0, 33)
    assert np.abs(full - ref).max() < 1e-4
    # LayerNorm(x + r), the sum not kept; a + b into a new tensor
    xr, rr = rng.standard_normal((5, 96)).astype(np.float32), rng.standard_normal((5, 96)).astype(np.float32)
    g, be = rng.standard_normal(96).astype(np.float32), rng.standard_normal(96).astype(np.float32)
    tg, tb = GpuTensor.from_host(g, g.shape, reg), GpuTensor.from_host(be, be.shape, reg)
    ta, tr = GpuTensor.from_host(xr, xr.shape, reg), GpuTensor.from_host(rr, rr.shape, reg)
    nrm = ops.layer_norm_residual(ta, tr, tg, tb, 1e-5, reg).to_host()
    assert np.abs(nrm - oracle.layer_norm(xr + rr, g, be).reshape(5, 96)).max() < 2e-4
    s = ops.elementwise_add_out(ta, tr, reg)
    assert np.array_equal(s.to_host(), xr + rr) and np.array_equal(ta.to_host(), xr)
    wte, wpe = rng.standard_normal((11, 8)).astype(np.float32), rng.standard_normal((6, 8)).astype(np.float32)
    ids = np.array([3, 0, 10, 7], dtype=np.uint32)
    out = ops.embedding_lookup(GpuTensor.from_host(wte, wte.shape, reg), GpuTensor.from_host(wpe, wpe.shape, reg), ids, 4, reg)
    assert np.array_equal(out.to_host(), wte[ids] + wpe[:4])


@pytest.mark.gpu
def test_matmul_fused_layernorm_accessors_and_with_codegen(reg):
    """ops::matmul_fused (gemm.rs:814-977: bias then the sigmoid-form GELU or ReLU, with its shape errors),
    LayerNorm::gamma / beta (norm.rs:41-48) and Linear::with_codegen (linear.rs:94-125)."""
    rng = np.random.default_rng(91)
    a = rng.standard_normal((6, 70)).astype(np.float32)
    b = (rng.standard_normal((70, 45)) * 0.2).astype(np.float32)
    bias = rng.standard_normal(45).astype(np.float32)
    ta, tb, tbias = [GpuTensor.from_host(z, z.shape, reg) for z in (a, b, bias)]
    pre = a.astype(np.float64) @ b.astype(np.float64) + bias
    got = ops.matmul_fused(ta, tb, tbias, ops.FUSED_GELU, reg).to_host()
    assert got.shape == (6, 45) and np.abs(got - pre / (1 + np.exp(-1.702 * pre))).max() < 3e-5
    got = ops.matmul_fused(ta, tb, tbias, ops.FUSED_RELU, reg).to_host()
    assert np.abs(got - np.maximum(pre, 0)).max() < 3e-5
    assert np.array_equal(ta.to_host(), a) and np.array_equal(tb.to_host(), b)  # inputs untouched
    for bad in [(ta.reshape((6, 70, 1)), tb, tbias), (ta, ta, tbias), (ta, tb, GpuTensor.from_host(a[0], (70,), reg)),
                (ta, tb, tbias.reshape((1, 45)))]:
        with pytest.raises(b200nn.NnError) as e:
            ops.matmul_fused(*bad, ops.FUSED_RELU, reg)
        assert e.value.code == b200nn.ERR_SHAPE and "ShapeMismatch" in str(e.value)
    g, be = rng.standard_normal(96).astype(np.float32), rng.standard_normal(96).astype(np.float32)
    ln = b200nn.LayerNorm(g, be, 1e-5, reg)
    assert np.array_equal(ln.gamma().to_host(), g) and np.array_equal(ln.beta().to_host(), be)
    assert ln.gamma().shape() == (96,) and ln.gamma() is ln.gamma()
    w = (rng.standard_normal((45, 70)) * 0.2).astype(np.float32)
    lin = b200nn.Linear.with_codegen(w, bias, 70, 45, reg, codegen=None)
    y = lin.forward(ta).to_host()
    assert np.abs(y - (a.astype(np.float64) @ w.T.astype(np.float64) + bias)).max() < 5e-3
    # the zero-parameter activation layers (layers/activation.rs:36-96)
    x = np.linspace(-6, 6, 501).astype(np.float32)
    t = GpuTensor.from_host(x, x.shape, reg)
    sig = 1.0 / (1.0 + np.exp(-x.astype(np.float64)))
    assert np.abs(b200nn.SiLU(reg).forward(t).to_host() - x * sig).max() < 1e-5
    assert np.abs(b200nn.Sigmoid(reg).forward(t).to_host() - sig).max() < 1e-6
    assert np.array_equal(b200nn.ReLU(reg).forward(t).to_host(), np.maximum(x, 0))
    assert np.array_equal(t.to_host(), x)
    # GpuTensor::from_data (tensor.rs:67-77): over device data of another owner; a copy, so later writes
    # to the source do not show
    import torch
    src = torch.arange(24, dtype=torch.float32, device="cuda").reshape(2, 3, 4) * 0.5
    torch.cuda.synchronize()
    d = GpuTensor.from_data(src.data_ptr(), (2, 3, 4), reg)
    assert d.shape() == (2, 3, 4) and np.array_equal(d.to_host(), src.cpu().numpy())
    src += 1.0
    torch.cuda.synchronize()
    assert np.array_equal(d.to_host(), src.cpu().numpy() - 1.0)
    own = GpuTensor.from_data(t.data_ptr(), (501,), reg)
    assert np.array_equal(own.to_host(), x)
    with pytest.raises(b200nn.NnError):
        GpuTensor.from_data(0, (4,), reg)
