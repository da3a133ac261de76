"""GPU tests of the persistent decode kernel (all transformer blocks of an int4 decode step in one
cooperative launch; opt-in through the tuning key "persist"): parity against the oracle and against the
one-kernel-per-operation path on the same seeded weights, and the bounded-wait failure path.

The failure test makes a wait run out on the host's terms: block 0 is told to leave out one arrival at
the grid counter (a flag that nothing sets), every other block's bounded wait gives up after a
millisecond, the kernel returns, the call that fetches results reports B200NN_ERR_DEVICE, and the
context keeps working.  Nothing faults, traps or spins without a limit."""
import numpy as np
import pytest

import b200nn
import np_ref
from b200nn import DecodeSession, Gpt2Config, Int4Gpt2Model, synth
from oracle import oracle
from test_gpu_model import MAX_ABS, REL_RMS, _check_tokens, _int4_oracle_weights

pytestmark = pytest.mark.gpu


def _run(reg, m, prompts, n_new, persist):
    reg.set_tuning("persist", persist)
    try:
        B, P = prompts.shape
        s = DecodeSession(m, batch=B, capacity=P + n_new + 2)
        s.prefill(prompts)
        s.step(1)
        s.step(n_new - 2)
        return s.tokens(), s.logits()
    finally:
        reg.set_tuning("persist", 0)


# rows 3 (the smallest batch that takes the kernel), 8 (most blocks have no GEMM units), 40 and 100 (64- and
# 128-row token tiles), 256 (the 256-row tile, four operand stages); widths 128 / 192 and GPT-2 XL's 1600
@pytest.mark.parametrize("d,layers,B,P", [(128, 2, 3, 9), (128, 2, 8, 9), (128, 2, 40, 17), (192, 3, 100, 70),
                                         (128, 2, 256, 33), (1600, 2, 32, 130), (1600, 2, 200, 40)])
def test_persistent_decode_matches_oracle_and_per_operation_path(reg, d, layers, B, P):
    cfg = Gpt2Config(n_layer=layers, n_embd=d, n_head=d // 64, vocab_size=257 if d < 512 else 1031, n_positions=256)
    w = synth.gpt2_weights(cfg, base_seed=300 + B, std=0.08 if d < 512 else 0.02, random_ln=True)
    m = Int4Gpt2Model.from_weights(w, cfg, reg)
    N = 6
    prompts = synth.token_ids(B, (B, P), cfg.vocab_size)
    launches0 = reg.launch_count()
    tok_p, lg_p = _run(reg, m, prompts, N, 1)
    launches_p = reg.launch_count() - launches0
    assert reg.device_error() == 0
    launches0 = reg.launch_count()
    tok_o, lg_o = _run(reg, m, prompts, N, 0)
    launches_o = reg.launch_count() - launches0
    assert launches_p < launches_o  # one launch per step for all blocks instead of seven per block
    same = (tok_p == tok_o).all(axis=1)  # a near-tie that flips a token changes everything after it
    assert (~same).sum() <= max(2, B // 32)  # the order of the split-K additions differs between the two paths (and from run to run)
    assert np.abs(lg_p - lg_o)[same].max() < 5e-3
    om = oracle.Model(cfg.as_dict(), _int4_oracle_weights(m, cfg, w, False))
    for b in sorted({0, B // 2, B - 1}):
        ref, lg = om.generate_cached(prompts[b], N, flags=oracle.KV_FP16, want_logits=True)
        _check_tokens(np.concatenate([prompts[b], tok_p[b]]), ref, lg, P)
        if np.array_equal(tok_p[b], ref[P:]):  # same history: the last step's logits are comparable
            assert np.abs(lg_p[b] - lg[-1]).max() < MAX_ABS and np_ref.rel_rms(lg_p[b], lg[-1]) < REL_RMS


def test_persistent_decode_wait_runs_out_and_context_survives(reg):
    cfg = Gpt2Config(n_layer=2, n_embd=128, n_head=2, vocab_size=257, n_positions=64)
    w = synth.gpt2_weights(cfg, base_seed=77, std=0.08, random_ln=True)
    m = Int4Gpt2Model.from_weights(w, cfg, reg)
    prompts = synth.token_ids(5, (16, 9), cfg.vocab_size)
    good_tok, good_lg = _run(reg, m, prompts, 4, 1)
    reg.set_tuning("persist", 1)
    reg.set_tuning("persist_wait_kcycles", 2000)  # about a millisecond of SM clocks
    reg.set_tuning("persist_fault_phase", 5)      # block 0 never arrives after the sixth phase
    try:
        s = DecodeSession(m, batch=16, capacity=16)
        s.prefill(prompts)
        s.step(1)
        with pytest.raises(b200nn.NnError) as e:
            s.logits()
        assert e.value.code == b200nn.ERR_DEVICE
        assert reg.device_error() == 0  # the word was cleared by the call that reported it
    finally:
        reg.set_tuning("persist_fault_phase", -1)
        reg.set_tuning("persist_wait_kcycles", 0)
        reg.set_tuning("persist", 0)
    # the context still works, on both paths, and gives the results from before
    tok, lg = _run(reg, m, prompts, 4, 1)
    assert np.array_equal(tok, good_tok) or np.abs(lg - good_lg).max() < 5e-3
    tok0, lg0 = _run(reg, m, prompts, 4, 0)
    assert (tok0 == good_tok).mean() > 0.95
    assert reg.device_error() == 0
