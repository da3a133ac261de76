"""GPU parity tests of the tcgen05 int4 GEMM (rows above the GEMV threshold) against the f64 oracle.

The kernel rounds activations and dequantised weights to fp16 before the MMA (f32 accumulation in
TMEM): tolerance 5e-4 relative RMS per Linear, inside the path's 1e-3 budget on logits."""
import numpy as np
import pytest

import b200nn
import np_ref
from b200nn import GpuTensor, synth
from oracle import oracle

pytestmark = pytest.mark.gpu


def _run(reg, m, k, n, group=128, bias=True, seed=0):
    packed, scales, x, _ = synth.int4_linear_case(seed + m + k + n, m, k, n, group)
    b = np.linspace(-1, 1, n).astype(np.float32) if bias else None
    y = b200nn.Int4Linear(packed, scales, b, k, n, group, reg).forward(GpuTensor.from_host(x, (m, k), reg)).to_host()
    ref = oracle.int4_linear(x, packed, scales, b, m, n, k, group, f64=True)
    return y, ref


@pytest.mark.parametrize("m", [3, 16, 17, 32, 33, 64, 100, 128, 129, 256, 300, 700])
def test_row_counts_cover_every_tile_width(reg, m):
    y, ref = _run(reg, m, 768, 768)
    assert y.shape == ref.shape
    assert np_ref.rel_rms(y, ref) < 5e-4, np_ref.rel_rms(y, ref)
    assert reg.device_error() == 0


@pytest.mark.parametrize("k,n", [(64, 128), (64, 130), (1600, 1600), (1600, 4800), (6400, 1600), (1600, 6400),
                                 (3072, 768), (768, 50257), (128, 1)])
@pytest.mark.parametrize("m", [32, 256])
def test_model_shapes_with_split_k_and_ragged_edges(reg, m, k, n):
    y, ref = _run(reg, m, k, n)
    assert np_ref.rel_rms(y, ref) < 5e-4, np_ref.rel_rms(y, ref)
    assert np.abs(y - ref).max() < 2e-2 * max(1.0, float(np.abs(ref).max()))
    assert reg.device_error() == 0


def test_group_64_and_no_bias(reg):
    y, ref = _run(reg, 48, 1024, 384, group=64, bias=False)
    assert np_ref.rel_rms(y, ref) < 5e-4


def test_repeatable_bitwise(reg):
    # split-K partials are summed in split order by the last block: results do not depend on arrival order
    packed, scales, x, _ = synth.int4_linear_case(3, 32, 6400, 1600, 128)
    lin = b200nn.Int4Linear(packed, scales, None, 6400, 1600, 128, reg)
    t = GpuTensor.from_host(x, (32, 6400), reg)
    a = lin.forward(t).to_host()
    for _ in range(3):
        assert np.array_equal(a, lin.forward(t).to_host())


def test_gemv_and_tensor_core_paths_agree(reg):
    packed, scales, x, _ = synth.int4_linear_case(4, 8, 1600, 1600, 128)
    lin = b200nn.Int4Linear(packed, scales, None, 1600, 1600, 128, reg)
    t = GpuTensor.from_host(x, (8, 1600), reg)
    tc = lin.forward(t).to_host()
    reg.set_gemv_max_rows(8)
    try:
        cc = lin.forward(t).to_host()
    finally:
        reg.set_gemv_max_rows(-1)
    assert np_ref.rel_rms(tc, cc) < 5e-4
    assert np_ref.rel_rms(cc, oracle.int4_linear(x, packed, scales, None, 8, 1600, 1600, 128)) < 1e-5


@pytest.mark.parametrize("m,k,n,group", [(2100, 1600, 4800, 128), (5900, 3200, 1600, 128), (9000, 192, 1100, 64)])
def test_prefill_rows_dequantise_once_then_persistent_gemm(reg, m, k, n, group):
    """With at least two 256-row tiles per SM the weight is written out once as the fp16 matrix the int4
    GEMM builds tile by tile, and the persistent fp16 GEMM multiplies it (tuning key int4_via_f16): the same
    operand values, so the two ways agree to accumulation order, and both match the oracle."""
    packed, scales, x, _ = synth.int4_linear_case(m + n, m, k, n, group)
    bias = np.linspace(-1, 1, n).astype(np.float32)
    lin = b200nn.Int4Linear(packed, scales, bias, k, n, group, reg)
    t = GpuTensor.from_host(x, (m, k), reg)
    n0 = reg.launch_count()
    y = lin.forward(t).to_host()
    n_new = reg.launch_count() - n0
    reg.set_tuning("int4_via_f16", 0)
    try:
        n0 = reg.launch_count()
        y_int4 = lin.forward(t).to_host()
        assert reg.launch_count() - n0 == n_new - 1  # no dequantisation launch on the int4 GEMM's way
    finally:
        reg.set_tuning("int4_via_f16", 1)
    assert np_ref.rel_rms(y, y_int4) < 5e-6
    ref = oracle.int4_linear(x, packed, scales, bias, m, n, k, group, f64=True)
    assert np_ref.rel_rms(y, ref) < 5e-4
    assert np.abs(y - ref).max() < 2e-2 * max(1.0, float(np.abs(ref).max()))
    assert reg.device_error() == 0
