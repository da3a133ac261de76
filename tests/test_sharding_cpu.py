"""CPU tests of the multi-GPU host logic: the batch is block-partitioned over ranks, every rank
works on its own sequences with no data-path collective, and only timing / token gathering cross
ranks.  Run here with two gloo ranks; the per-rank "model" is the CPU oracle on a tiny GPT-2."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path[:0] = [ROOT, os.path.join(ROOT, "async-gpu_b200")]

import bench  # noqa: E402


@pytest.mark.parametrize("total,world", [(256, 1), (256, 2), (256, 8), (10, 4), (3, 8), (0, 2)])
def test_shard_bounds_partition(total, world):
    parts = [bench.shard_bounds(total, world, r) for r in range(world)]
    assert parts[0][0] == 0 and parts[-1][1] == total
    for (a0, a1), (b0, b1) in zip(parts, parts[1:]):
        assert a1 == b0 and a0 <= a1 and b0 <= b1
    sizes = [b - a for a, b in parts]
    assert max(sizes) - min(sizes) <= 1 and sizes == sorted(sizes, reverse=True)


TINY = dict(n_layer=1, n_embd=64, n_head=1, vocab_size=97, n_positions=24, layer_norm_epsilon=1e-5)


def _generate_slice(lo, hi):
    from b200nn import synth
    from b200nn.gpt2 import Gpt2Config
    from oracle import oracle
    w = synth.gpt2_weights(Gpt2Config(**TINY), base_seed=5, std=0.1)
    prompts = synth.token_ids(9, (5, 4), TINY["vocab_size"])
    m = oracle.Model(TINY, w)
    return np.stack([m.generate_cached(prompts[b], 6)[0] for b in range(lo, hi)]) if hi > lo else np.zeros((0, 10), np.uint32)


def _worker(rank, world, port, q):
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    lo, hi = bench.shard_bounds(5, world, rank)
    mine = _generate_slice(lo, hi)
    # what crosses ranks: a barrier, the max of the per-rank times, and the final token gather
    dist.barrier()
    t = torch.tensor([float(rank + 1)], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    gathered = [None] * world
    dist.all_gather_object(gathered, (lo, hi, mine))
    if rank == 0:
        q.put((float(t.item()), gathered))
    dist.destroy_process_group()


def test_two_rank_gloo_run_equals_single_process():
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    tmax, gathered = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert tmax == 2.0
    whole = _generate_slice(0, 5)
    parts = sorted(gathered, key=lambda g: g[0])
    assert [(g[0], g[1]) for g in parts] == [(0, 3), (3, 5)]
    assert np.array_equal(np.concatenate([g[2] for g in parts]), whole)
