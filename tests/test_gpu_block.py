"""GPU parity tests of the single transformer block handles (`TransformerBlock`, `Int4TransformerBlock`:
gpt2.rs:98-289, 1219-1339) against the oracle's block on the same seeded weights: the full causal forward
and the cached forward with K/V handed in and out as host vectors, as the reference's per-block cache does."""
import numpy as np
import pytest

import np_ref
from b200nn import Gpt2Config, GpuTensor, Int4TransformerBlock, TransformerBlock, synth
from oracle import oracle

pytestmark = pytest.mark.gpu

_NAMES = ["ln_1.weight", "ln_1.bias", "attn.c_attn.weight", "attn.c_attn.bias", "attn.c_proj.weight", "attn.c_proj.bias",
          "ln_2.weight", "ln_2.bias", "mlp.c_fc.weight", "mlp.c_fc.bias", "mlp.c_proj.weight", "mlp.c_proj.bias"]


def _slices(w):
    """The twelve slices of layer 0 as TransformerBlock::new takes them: dense weights [out,in]."""
    out = []
    for nm in _NAMES:
        a = w["h.0." + nm]
        out.append(np.ascontiguousarray(a.T) if a.ndim == 2 else a)
    return out


def _int4_oracle(w, cfg, group):
    """Oracle weights of the int4 block: every dense matrix quantised with the reference rule, the scales
    rounded to fp16, dequantised again (what the block multiplies)."""
    w2 = dict(w)
    d = cfg.n_embd
    for nm, (k, n) in {"attn.c_attn.weight": (d, 3 * d), "attn.c_proj.weight": (d, d), "mlp.c_fc.weight": (d, 4 * d),
                       "mlp.c_proj.weight": (4 * d, d)}.items():
        p, s = oracle.quantize_weight_int4(w["h.0." + nm], k, n, group)
        w2["h.0." + nm] = oracle.dequant_weight_int4(p, oracle.f16_round(s), k, n, group)
    return w2


@pytest.mark.parametrize("int4", [False, True])
@pytest.mark.parametrize("d,seq", [(128, 23), (192, 70)])
def test_block_forward_and_forward_cached(reg, int4, d, seq):
    cfg = Gpt2Config(n_layer=1, n_embd=d, n_head=d // 64, vocab_size=64, n_positions=128)
    w = synth.gpt2_weights(cfg, base_seed=91 + d, std=0.06, random_ln=True)
    if int4:
        blk = Int4TransformerBlock(*_slices(w), cfg, reg, group_size=128)
        om = oracle.Model(cfg.as_dict(), _int4_oracle(w, cfg, 128))
    else:
        blk = TransformerBlock(*_slices(w), cfg, reg)
        om = oracle.Model(cfg.as_dict(), w)
    rng = np.random.default_rng(d + seq)
    x = rng.standard_normal((seq, d)).astype(np.float32)
    # full causal forward
    got = blk.forward(GpuTensor.from_host(x, (seq, d), reg)).to_host()
    ref, k_ref, v_ref = om.block_forward(0, x, flags=oracle.KV_FP16)
    assert np_ref.rel_rms(got, ref) < 1e-3, np_ref.rel_rms(got, ref)
    # the same launches (the split-K sums of the two projections are added in no fixed order: last bits may differ)
    assert np_ref.rel_rms(blk.forward_auto_fused(GpuTensor.from_host(x, (seq, d), reg)).to_host(), got) < 1e-5
    # the same rows in two cached calls: positions [0, past) first, then the rest on top of the returned K/V
    H, past = cfg.n_head, seq - 4
    y0, k0, v0 = blk.forward_cached(GpuTensor.from_host(x[:past], (past, d), reg), None, None, 0)
    assert k0.shape == (H, past * 64)
    assert np.abs(k0.reshape(H, past, 64) - k_ref[:, :past]).max() < 2e-3
    y1, k1, v1 = blk.forward_cached(GpuTensor.from_host(x[past:], (seq - past, d), reg), k0, v0, past)
    both = np.concatenate([y0.to_host(), y1.to_host()])
    assert np_ref.rel_rms(both, ref) < 1e-3
    assert np.abs(v1.reshape(H, seq - past, 64) - v_ref[:, past:]).max() < 2e-3
    # one new row on top of everything before it (the decode shape)
    y2, _, _ = blk.forward_cached(GpuTensor.from_host(x[-1:], (1, d), reg), np.concatenate([k0.reshape(H, past, 64), k1.reshape(H, -1, 64)[:, :-1]], axis=1).reshape(H, -1),
                                  np.concatenate([v0.reshape(H, past, 64), v1.reshape(H, -1, 64)[:, :-1]], axis=1).reshape(H, -1), seq - 1)
    assert np_ref.rel_rms(y2.to_host()[0], ref[-1]) < 1e-3
    assert reg.device_error() == 0


def test_block_rejects_bad_arguments(reg):
    cfg = Gpt2Config(n_layer=1, n_embd=128, n_head=2, vocab_size=64, n_positions=32)
    w = synth.gpt2_weights(cfg, base_seed=5)
    blk = TransformerBlock(*_slices(w), cfg, reg)
    import b200nn
    with pytest.raises(b200nn.NnError) as e:
        blk.forward(GpuTensor.from_host(np.zeros((3, 64), np.float32), (3, 64), reg))
    assert e.value.code == b200nn.ERR_SHAPE
    with pytest.raises(b200nn.NnError):
        TransformerBlock(*_slices(w)[:-1], np.zeros(5, np.float32), cfg, reg)  # a slice of the wrong size
    bad = Gpt2Config(n_layer=1, n_embd=96, n_head=2, vocab_size=64, n_positions=32)  # head_dim 48
    with pytest.raises(b200nn.NnError):
        TransformerBlock(*[np.zeros(n, np.float32) for n in (96, 96, 3 * 96 * 96, 3 * 96, 96 * 96, 96, 96, 96, 4 * 96 * 96,
                                                                4 * 96, 4 * 96 * 96, 96)], bad, reg)
