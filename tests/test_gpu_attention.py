"""GPU parity tests of the attention kernels against the f64 oracle.

K and V are held in fp16 inside the library, so the oracle is given K and V rounded to fp16
(the same inputs the kernels see); what remains is f32 accumulation error: tolerance 1e-4 absolute
on outputs of order one (the reference's own attention tests use 1e-3 / 1e-4,
crates/test/gpu-test-harness/src/tests_transformer.rs:443-581, 1963-2121)."""
import numpy as np
import pytest

import b200nn
from b200nn import GpuTensor, ops
from oracle import oracle

pytestmark = pytest.mark.gpu


def _qkv(seed, H, n, scale=1.0):
    rng = np.random.default_rng(seed)
    return [(rng.standard_normal((H, n, 64)) * scale).astype(np.float32) for _ in range(3)]


def _oracle_mha(q, k, v, past):
    H, nq, _ = q.shape
    cap = k.shape[1]
    qrow = np.ascontiguousarray(q.transpose(1, 0, 2).reshape(nq, H * 64))
    out = oracle.mha(qrow, oracle.f16_round(k), oracle.f16_round(v), H, 64, nq, past, cap)
    return out.reshape(nq, H, 64).transpose(1, 0, 2)


@pytest.mark.parametrize("H,n", [(12, 128), (12, 256), (3, 1), (2, 65), (25, 100), (1, 1024)])
def test_causal_flash_attention(reg, H, n):
    q, k, v = _qkv(n + H, H, n)
    out = ops.multi_head_flash_attention(GpuTensor.from_host(q, q.shape, reg), GpuTensor.from_host(k, k.shape, reg),
                                         GpuTensor.from_host(v, v.shape, reg), n, H, 64, True, reg).to_host()
    ref = _oracle_mha(q, k, v, 0)
    assert out.shape == (H, n, 64)
    assert np.abs(out - ref).max() < 1e-4
    # row 0 of causal attention is V[0] (tests_transformer.rs:2176-2191)
    assert np.abs(out[:, 0] - oracle.f16_round(v[:, 0])).max() < 1e-6


@pytest.mark.parametrize("kv_len,q_len", [(1024, 1), (1, 1), (17, 1), (300, 1), (200, 8), (64, 64)])
def test_attention_kv_with_offset(reg, kv_len, q_len):
    # new queries at the end of a longer K/V history: causal with q_offset = kv_len - q_len
    q, _, _ = _qkv(kv_len, 1, q_len)
    _, k, v = _qkv(kv_len + 1, 1, kv_len)
    off = kv_len - q_len
    out = ops.scaled_dot_product_attention_kv(GpuTensor.from_host(q[0], (q_len, 64), reg),
                                              GpuTensor.from_host(k[0], (kv_len, 64), reg),
                                              GpuTensor.from_host(v[0], (kv_len, 64), reg), True, off, reg).to_host()
    ref = _oracle_mha(q, k, v, off)[0]
    assert out.shape == (q_len, 64)
    assert np.abs(out - ref).max() < 1e-4


def test_cached_equals_last_rows_of_full(reg):
    # flash_attention_kv must reproduce the last row of the full causal result (tolerance 1e-4,
    # tests_transformer.rs:1963-2121)
    q, k, v = _qkv(9, 1, 96)
    full = ops.multi_head_flash_attention(GpuTensor.from_host(q, q.shape, reg), GpuTensor.from_host(k, k.shape, reg),
                                          GpuTensor.from_host(v, v.shape, reg), 96, 1, 64, True, reg).to_host()
    last = ops.scaled_dot_product_attention_kv(GpuTensor.from_host(q[0, 95:], (1, 64), reg),
                                               GpuTensor.from_host(k[0], (96, 64), reg),
                                               GpuTensor.from_host(v[0], (96, 64), reg), True, 95, reg).to_host()
    assert np.abs(full[0, 95] - last[0]).max() < 1e-4


def test_large_scores_do_not_overflow(reg):
    q, k, v = _qkv(5, 2, 80, scale=6.0)  # scores of several hundred before the softmax
    out = ops.multi_head_flash_attention(GpuTensor.from_host(q, q.shape, reg), GpuTensor.from_host(k, k.shape, reg),
                                         GpuTensor.from_host(v, v.shape, reg), 80, 2, 64, True, reg).to_host()
    assert np.isfinite(out).all()
    assert np.abs(out - _oracle_mha(q, k, v, 0)).max() < 2e-3


def test_attention_rejects_bad_shapes(reg):
    t = GpuTensor.zeros((2, 8, 32), reg)
    with pytest.raises(b200nn.NnError):
        ops.multi_head_flash_attention(t, t, t, 8, 2, 32, True, reg)  # d_head != 64
    a, b = GpuTensor.zeros((4, 64), reg), GpuTensor.zeros((3, 64), reg)
    with pytest.raises(b200nn.NnError):
        ops.scaled_dot_product_attention_kv(a, b, b, True, 0, reg)  # more queries than keys


@pytest.mark.parametrize("seq", [1, 9, 70])
def test_multi_head_attention_layer(reg, seq):
    rng = np.random.default_rng(seq)
    d, H = 128, 2
    qkv_w = (rng.standard_normal((3 * d, d)) * 0.08).astype(np.float32)
    qkv_b = (rng.standard_normal(3 * d) * 0.1).astype(np.float32)
    out_w = (rng.standard_normal((d, d)) * 0.08).astype(np.float32)
    out_b = (rng.standard_normal(d) * 0.1).astype(np.float32)
    x = rng.standard_normal((seq, d)).astype(np.float32)
    layer = b200nn.MultiHeadAttention(qkv_w, qkv_b, out_w, out_b, d, H, reg)
    y = layer.forward_causal(GpuTensor.from_host(x, (seq, d), reg)).to_host()

    qkv = x.astype(np.float64) @ qkv_w.astype(np.float64).T + qkv_b
    k = qkv[:, d:2 * d].reshape(seq, H, 64).transpose(1, 0, 2).astype(np.float32)
    v = qkv[:, 2 * d:].reshape(seq, H, 64).transpose(1, 0, 2).astype(np.float32)
    att = oracle.mha(qkv[:, :d].astype(np.float32), oracle.f16_round(k), oracle.f16_round(v), H, 64, seq, 0, seq)
    ref = att.astype(np.float64) @ out_w.astype(np.float64).T + out_b
    assert np.abs(y - ref).max() < 2e-3  # fp16 rounding of K,V may flip on f32-vs-f64 differences

    if seq > 2:  # forward_cached: feed the last row on top of the history of the first seq-1 rows
        past = seq - 1
        ck = oracle.f16_round(k[:, :past]).reshape(H, past * 64)
        cv = oracle.f16_round(v[:, :past]).reshape(H, past * 64)
        yc, nk, nv = layer.forward_cached(GpuTensor.from_host(x[past:], (1, d), reg), ck, cv, past)
        assert np.abs(yc.to_host()[0] - y[past]).max() < 2e-3
        assert np.abs(nk.reshape(H, 64) - k[:, past]).max() < 2e-3
        assert np.abs(nv.reshape(H, 64) - v[:, past]).max() < 2e-3


@pytest.mark.parametrize("B,H,S,past,cap", [(2, 3, 128, 0, 128), (1, 12, 1024, 0, 1024), (2, 2, 200, 77, 300),
                                            (1, 1, 1, 0, 5), (3, 5, 257, 128, 640), (1, 2, 130, 511, 641)])
def test_prefill_attention_fp16_buffers_tensor_cores(reg, B, H, S, past, cap):
    """The tensor-core prefill kernel on caller-owned fp16 buffers (what the models call): several key
    tiles, a query count and a history that are no multiples of the 128-row tiles, more capacity than
    rows, several sequences and heads.  Cache rows past the last written one hold NaN: they must not
    reach the result (the copies zero-fill past the written extent).  Oracle on the same fp16 values;
    tolerance: the output's fp16 rounding plus f32 accumulation."""
    import torch
    dev = torch.device("cuda", reg.device)
    rng = np.random.default_rng(B * 1000 + S + past)
    n = past + S
    q = oracle.f16_round(rng.standard_normal((B, S, H * 64)).astype(np.float32))
    k = oracle.f16_round(rng.standard_normal((B, H, n, 64)).astype(np.float32))
    v = oracle.f16_round(rng.standard_normal((B, H, n, 64)).astype(np.float32))
    kc = np.full((B, H, cap, 64), np.nan, np.float16)
    vc = np.full((B, H, cap, 64), np.nan, np.float16)
    kc[:, :, :n] = k
    vc[:, :, :n] = v
    q_d = torch.from_numpy(q.astype(np.float16).reshape(B * S, H * 64)).to(dev)
    k_d, v_d = torch.from_numpy(kc).to(dev), torch.from_numpy(vc).to(dev)
    out_d = torch.zeros((B * S, H * 64), device=dev, dtype=torch.float16)
    torch.cuda.synchronize()
    ops.prefill_attention_f16(q_d.data_ptr(), k_d.data_ptr(), v_d.data_ptr(), B, H, cap, S, past, out_d.data_ptr(), reg)
    reg.synchronize()
    out = out_d.cpu().numpy().astype(np.float32).reshape(B, S, H * 64)
    for b in range(B):
        ref = oracle.mha(q[b], k[b], v[b], H, 64, S, past, n)
        assert np.isfinite(out[b]).all()
        assert np.abs(out[b] - ref).max() < 2e-3, (b, np.abs(out[b] - ref).max())
    assert reg.device_error() == 0


@pytest.mark.parametrize("seq", [1, 2, 7, 150])
def test_int4_multi_head_attention_layer(reg, seq):
    """Int4MultiHeadAttention (gpt2.rs:1127-1214): both projections quantised at construction (group 128 along
    the input dimension of the transposed weight); reference = the f64 path on the dequantised weights the
    quantisation rule gives, K and V rounded to fp16 as the layer's cache holds them.  1 and 2 rows take the
    GEMV, 7 and 150 the tensor-core GEMMs and attention with fp16 activations."""
    rng = np.random.default_rng(seq + 40)
    d, H, g = 128, 2, 128
    qkv_w = (rng.standard_normal((3 * d, d)) * 0.08).astype(np.float32)
    qkv_b = (rng.standard_normal(3 * d) * 0.1).astype(np.float32)
    out_w = (rng.standard_normal((d, d)) * 0.08).astype(np.float32)
    out_b = (rng.standard_normal(d) * 0.1).astype(np.float32)
    x = rng.standard_normal((seq, d)).astype(np.float32)
    layer = b200nn.Int4MultiHeadAttention(qkv_w, qkv_b, out_w, out_b, d, H, g, reg)
    y = layer.forward_causal(GpuTensor.from_host(x, (seq, d), reg)).to_host()

    def deq(w_out_in):  # the weight the layer multiplies with: quantise [in,out], fp16 scales, dequantise
        k, n = w_out_in.shape[1], w_out_in.shape[0]
        p, s = oracle.quantize_weight_int4(np.ascontiguousarray(w_out_in.T), k, n, g)
        return oracle.dequant_weight_int4(p, oracle.f16_round(s), k, n, g).astype(np.float64)  # [in,out]

    qkv = x.astype(np.float64) @ deq(qkv_w) + qkv_b
    k = qkv[:, d:2 * d].reshape(seq, H, 64).transpose(1, 0, 2).astype(np.float32)
    v = qkv[:, 2 * d:].reshape(seq, H, 64).transpose(1, 0, 2).astype(np.float32)
    att = oracle.mha(qkv[:, :d].astype(np.float32), oracle.f16_round(k), oracle.f16_round(v), H, 64, seq, 0, seq)
    ref = att.astype(np.float64) @ deq(out_w) + out_b
    tol = 2e-3 if seq <= 2 else 6e-3  # fp16 activations on the tensor-core path
    assert np.abs(y - ref).max() < tol, np.abs(y - ref).max()
    if seq > 2:
        past = seq - 1
        ck = oracle.f16_round(k[:, :past]).reshape(H, past * 64)
        cv = oracle.f16_round(v[:, :past]).reshape(H, past * 64)
        yc, nk, nv = layer.forward_cached(GpuTensor.from_host(x[past:], (1, d), reg), ck, cv, past)
        assert np.abs(yc.to_host()[0] - y[past]).max() < tol
        assert np.abs(nk.reshape(H, 64) - k[:, past]).max() < 2e-3
    assert reg.device_error() == 0
