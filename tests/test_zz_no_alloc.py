"""GPU test of the allocation-free decode-attention entry point.

Some hosts of this library may not let it allocate device memory: they have given away their whole
memory budget up front, or they call from a place where cudaMalloc would stall the device.  For
them `b200nn_decode_attention_noalloc` runs the split-context decode-attention kernel with its
scratch in a fixed array inside the library image.  This test calls it through the C ABI on
caller-owned buffers, twice in a row (the calls share the scratch, so the second call proves that
nothing stale is left behind), and compares each result with the regular entry point
(`b200nn_attention_kv`, one head at a time) and with the CPU oracle's f64 attention at the attention
tests' tolerance of 1e-4.  That nothing is allocated is checked on the driver's own figure
(free device bytes from cudaMemGetInfo, which a cudaMalloc inside the library would lower), after
a first call has done the per-device set-up.

The file sorts last on purpose: if it fails, `pytest -x` has already run every other test.
"""
import ctypes as C

import numpy as np
import pytest

import b200nn
from b200nn import GpuTensor, ops
from oracle import oracle

pytestmark = pytest.mark.gpu


def _oracle_rows(q, k16, v16, ctx_len):
    """f64 attention of the CPU oracle over the first ctx_len cached positions, one sequence at a time."""
    B, H, cap = q.shape[0], k16.shape[1], k16.shape[2]
    out = np.zeros((B, H * 64), dtype=np.float32)
    for b in range(B):
        out[b] = oracle.mha(q[b:b + 1], k16[b].astype(np.float32), v16[b].astype(np.float32), H, 64, 1, ctx_len - 1, cap)[0]
    return out


def _reference_rows(reg, q, k16, v16, ctx_len):
    """The existing entry point, one (sequence, head) pair per call; K and V given as the f32 values
    the fp16 cache holds, so both paths see identical inputs."""
    B, H = q.shape[0], k16.shape[1]
    out = np.zeros((B, H * 64), dtype=np.float32)
    for b in range(B):
        for h in range(H):
            qt = GpuTensor.from_host(q[b, h * 64:(h + 1) * 64], (1, 64), reg)
            kt = GpuTensor.from_host(k16[b, h, :ctx_len].astype(np.float32), (ctx_len, 64), reg)
            vt = GpuTensor.from_host(v16[b, h, :ctx_len].astype(np.float32), (ctx_len, 64), reg)
            out[b, h * 64:(h + 1) * 64] = ops.scaled_dot_product_attention_kv(qt, kt, vt, True, ctx_len - 1, reg).to_host()[0]
    return out


@pytest.mark.parametrize("B,H,cap,ctx_lens", [(3, 4, 320, (300, 77)), (2, 12, 1024, (1024, 1))])
def test_no_alloc_entry_matches_regular_entry_twice(reg, B, H, cap, ctx_lens):
    import torch

    lib = b200nn.load_library()
    rng = np.random.default_rng(B * 100 + H)
    dev = torch.device("cuda", reg.device)
    for call, ctx_len in enumerate(ctx_lens):  # two calls in a row on the same scratch, different shapes of work
        q = rng.standard_normal((B, H * 64)).astype(np.float32)
        k16 = rng.standard_normal((B, H, cap, 64)).astype(np.float16)
        v16 = rng.standard_normal((B, H, cap, 64)).astype(np.float16)
        # caller-owned device buffers (the entry point itself allocates nothing)
        q_d = torch.from_numpy(q).to(dev)
        k_d = torch.from_numpy(k16).to(dev)
        v_d = torch.from_numpy(v16).to(dev)
        out_d = torch.full((B, H * 64), float("nan"), device=dev, dtype=torch.float32)
        args = (reg.device, None, q_d.data_ptr(), k_d.data_ptr(), v_d.data_ptr(), B, H, cap, ctx_len, out_d.data_ptr())
        if call == 0:  # the first call on a device looks the scratch's address up (module load, symbol lookup)
            assert lib.b200nn_decode_attention_noalloc(*args) == 0, lib.b200nn_noalloc_last_error()
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info(dev)[0]
        rc = lib.b200nn_decode_attention_noalloc(*args)
        assert rc == 0, lib.b200nn_noalloc_last_error()
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info(dev)[0] == free_before  # the driver's free bytes: no cudaMalloc anywhere
        got = out_d.cpu().numpy()
        ref = _reference_rows(reg, q, k16, v16, ctx_len)
        assert np.isfinite(got).all(), f"call {call}"
        assert np.abs(got - ref).max() < 1e-4, f"call {call}: {np.abs(got - ref).max()}"
        orc = _oracle_rows(q, k16, v16, ctx_len)
        assert np.abs(got - orc).max() < 1e-4, f"call {call} vs oracle: {np.abs(got - orc).max()}"


def test_no_alloc_entry_at_the_largest_accepted_size(reg):
    """batch x heads = 4096, the most the fixed scratch takes: the split count is then limited by the
    fixed record array (16384 / 4096 = 4 splits of a 300-row context), not by the kernel's own rule.
    Checked against the oracle on a sample of sequences and for two calls in a row giving the same bits."""
    import torch

    lib = b200nn.load_library()
    B, H, cap, ctx_len = 1024, 4, 304, 300
    rng = np.random.default_rng(7)
    dev = torch.device("cuda", reg.device)
    q = rng.standard_normal((B, H * 64)).astype(np.float32)
    k16 = rng.standard_normal((B, H, cap, 64)).astype(np.float16)
    v16 = rng.standard_normal((B, H, cap, 64)).astype(np.float16)
    q_d, k_d, v_d = (torch.from_numpy(a).to(dev) for a in (q, k16, v16))
    outs = []
    for _ in range(2):
        out_d = torch.full((B, H * 64), float("nan"), device=dev, dtype=torch.float32)
        rc = lib.b200nn_decode_attention_noalloc(reg.device, None, q_d.data_ptr(), k_d.data_ptr(), v_d.data_ptr(), B, H,
                                                 cap, ctx_len, out_d.data_ptr())
        assert rc == 0, lib.b200nn_noalloc_last_error()
        torch.cuda.synchronize()
        outs.append(out_d.cpu().numpy())
    assert np.isfinite(outs[0]).all()
    assert np.array_equal(outs[0], outs[1])
    sample = [0, 1, 511, 1023]
    orc = _oracle_rows(q[sample], k16[sample], v16[sample], ctx_len)
    assert np.abs(outs[0][sample] - orc).max() < 1e-4


def test_no_alloc_entry_rejects_oversized_and_bad_arguments(reg):
    import torch

    lib = b200nn.load_library()
    dev = torch.device("cuda", reg.device)
    buf = torch.zeros(64, device=dev)
    p = buf.data_ptr()
    # 4097 (sequence, head) pairs: beyond the fixed scratch
    assert lib.b200nn_decode_attention_noalloc(reg.device, None, p, p, p, 4097, 1, 8, 4, p) == b200nn.ERR_SHAPE
    assert b"4096" in lib.b200nn_noalloc_last_error()
    assert lib.b200nn_decode_attention_noalloc(reg.device, None, p, p, p, 1, 1, 8, 9, p) == b200nn.ERR_SHAPE  # ctx > capacity
    assert lib.b200nn_decode_attention_noalloc(reg.device, None, None, p, p, 1, 1, 8, 4, p) == b200nn.ERR_ARG
    assert lib.b200nn_decode_attention_noalloc(-1, None, p, p, p, 1, 1, 8, 4, p) == b200nn.ERR_ARG
    # a cache pointer that is not 16-byte aligned is refused on the host (the kernel reads rows 16 bytes at a time)
    assert lib.b200nn_decode_attention_noalloc(reg.device, None, p, p + 2, p, 1, 1, 8, 4, p) == b200nn.ERR_ARG
    assert b"aligned" in lib.b200nn_noalloc_last_error()
