#!/usr/bin/env python
"""Benchmark of the int4 GPT-2 decode path.

    python bench.py --gpus N --steps K --warmup W            # this library, one rank per GPU
    python bench.py --impl reference --steps K --warmup W    # the reference's CPU path (oracle port)

Workload (the reference benchmark's largest case, its fifth configuration): GPT-2 XL, every Linear int4 group-128 (LM head included), fp16
KV cache, 256 independent sequences sharded over the ranks (256/N each, no data-path collective),
prompt of 128 random token ids, greedy decode of 128 tokens.  A "step" is one greedy decode step of
every sequence of the batch (all layers, LM head, argmax, token fed back on the device) at context
128 + (step mod 128).  Weights and token ids are seeded synthetic data.

One JSON line is printed by rank 0: `value` = sequences x steps / max-over-ranks CUDA-event time with
all state resident in HBM (the K timed steps sit in the middle of the decode window, so their mean
context is the window's mean whatever K is; the timed region is repeated and the median reported);
`e2e` = the same metric through generate_batch (host prompt ids in, host tokens out, prefill included,
every rank's tokens gathered on rank 0 inside the timed region); `roofline` = the dominant kernel
family of a step timed alone (algorithmic bytes / time against the measured HBM peak); `prefill` =
this rank's prompts through all layers; `gemv` = one-row dequant-GEMV bandwidth; at N=1 also
`int4_linear` (the isolated int4 Linear at 1 / 8 / 64 rows on GPT-2 Small's four shapes, L2-cold and
L2-warm), `attention` (isolated causal attention, batch 8 x 12 heads x 256 / 512 / 1024, and decode
attention of 64 sequences over 1024 cached positions) and `cpu_baseline` = the oracle on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path[:0] = [os.path.join(ROOT, "async-gpu_b200"), ROOT]

WORKLOADS = {
    # name: (preset, total batch, prompt, max_new, model family)
    "gpt2-xl-int4-b256": ("xl", 256, 128, 128, "int4"),
    "gpt2-small-int4-b32": ("small", 32, 512, 256, "int4"),
    # the unquantised family (f32 weights; Linears of more than four rows on the tensor cores):
    # not the headline, kept for its prefill figure and profiler captures
    "gpt2-xl-f32-b16": ("xl", 16, 512, 32, "f32"),
}
METRIC = "int4 GPT-2 decode tokens/sec"
UNIT = "tokens/s"


def shard_bounds(total: int, world: int, rank: int):
    """Contiguous block partition of `total` sequences: the first total % world ranks get one more."""
    base, extra = divmod(total, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def traffic_ratio(kernel: str):
    """DRAM bytes / algorithmic bytes of a kernel's profiler capture, from profiles/dram_traffic.json
    (written by hand from the capture summarised beside it)."""
    p = os.path.join(ROOT, "profiles", "dram_traffic.json")
    try:
        e = json.load(open(p))[kernel]
        return float(e["dram_bytes"]) / float(e["algorithmic_bytes"]), e.get("source")
    except Exception:
        return None, None


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "measured"
    return 6650.0, 1400.0, "fallback"


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while the timed region runs."""

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index, self.rows, self._halt = index, [], threading.Event()

    def run(self):
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        while not self._halt.is_set():
            try:
                out = subprocess.run(["nvidia-smi", "-i", str(self.index), f"--query-gpu={q}",
                                      "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5).stdout
                f = [x.strip() for x in out.strip().split(",")]
                if len(f) >= 6:
                    self.rows.append(f)
            except Exception:
                pass
            self._halt.wait(0.2)

    def finish(self):
        self._halt.set()
        self.join(timeout=6)
        if not self.rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        sm = sorted(float(r[0]) for r in self.rows)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": float(self.rows[0][1]), "reasons": reasons,
                "samples": len(self.rows)}


def build_int4_oracle_weights(cfg, w, group=128):
    """int4-quantises every dense weight and the LM head with the ORACLE's quantiser, rounds the scales
    to fp16 and dequantises again: the f32 matrices the CPU reference path multiplies."""
    from oracle import oracle
    d = cfg.n_embd
    out = dict(w)
    for i in range(cfg.n_layer):
        for nm, (k, n) in {"attn.c_attn.weight": (d, 3 * d), "attn.c_proj.weight": (d, d),
                           "mlp.c_fc.weight": (d, 4 * d), "mlp.c_proj.weight": (4 * d, d)}.items():
            key = f"h.{i}.{nm}"
            p, s = oracle.quantize_weight_int4(w[key], k, n, group)
            out[key] = oracle.dequant_weight_int4(p, oracle.f16_round(s), k, n, group)
    wt = np.ascontiguousarray(w["wte"].T)
    p, s = oracle.quantize_weight_int4(wt, d, cfg.vocab_size, group)
    out["lm_head"] = oracle.dequant_weight_int4(p, oracle.f16_round(s), d, cfg.vocab_size, group)
    return out


def cpu_decode_sample(cfg, w, prompt, steps, warmup):
    """Times `steps` KV-cached greedy decode steps of ONE sequence on the host cores with the oracle."""
    from oracle import oracle
    om = oracle.Model(cfg.as_dict(), w)
    flags = oracle.KV_FP16
    if warmup:
        om.time_decode(prompt, warmup, flags)
    sec, _ = om.time_decode(prompt, steps, flags)
    return sec, oracle.num_threads()


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    # torchrun pins OMP_NUM_THREADS=1 for its workers; this arm is the host-cores baseline and runs
    # alone (the other ranks have exited), so it takes every core the process may run on.  Set before
    # the OpenMP runtime of the oracle library is loaded.
    os.environ["OMP_NUM_THREADS"] = str(len(os.sched_getaffinity(0)))
    from b200nn import synth  # seeded data generator only (numpy); no library code runs on this arm
    from b200nn.gpt2 import Gpt2Config
    preset, total, prompt_len, max_new, family = WORKLOADS[args.workload]
    cfg = getattr(Gpt2Config, preset)()
    w = synth.gpt2_weights(cfg)
    if family == "int4":
        w = build_int4_oracle_weights(cfg, w)
    prompt = synth.token_ids(synth.BASE_SEED + 7, (total, prompt_len), cfg.vocab_size)[0, : args.cpu_prompt]
    steps = min(args.steps, args.cpu_max_steps)
    sec, threads = cpu_decode_sample(cfg, w, prompt, steps, min(args.warmup, 2))
    value = steps / sec
    sample = (f"1 of {total} sequences, prompt {args.cpu_prompt} tokens, {steps} KV-cached greedy decode steps, "
              f"f64 accumulate, OpenMP over output columns")
    line = {
        "impl": "reference", "metric": METRIC.replace("int4", family), "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": min(args.warmup, 2), "ms_per_step": 1e3 * sec / steps, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": family + " weights, f64 accumulate", "data": "synthetic",
        "config": {"workload": args.workload, "note": "CPU restatement of the reference path (Rust reference "
                   "cannot be built offline); each step is one decode step of a 1-sequence sample"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)
    return 0


def gemv_bandwidth(reg, cfg, hbm_peak, iters=96, only=None):
    """Dequant-GEMV (one input row, CUDA cores) HBM bandwidth on the model's four Linear shapes: each
    launch reads a different copy of the weight (copies add up to more than the L2), launches are
    back to back on the library's stream between two CUDA events.  Bytes per launch are algorithmic:
    nibbles + fp16 scales + input row + output row."""
    import torch
    import b200nn
    from b200nn import synth
    d = cfg.n_embd
    stream = torch.cuda.ExternalStream(reg.stream)
    out = {}
    shapes = {"qkv": (d, 3 * d), "proj": (d, d), "fc": (d, 4 * d), "fcproj": (4 * d, d), "lm_head": (d, cfg.vocab_size)}
    for name, (k, n) in shapes.items():
        if only and name != only:
            continue
        packed, scales, _, _ = synth.int4_linear_case(11, 1, k, n, 128)
        copies = max(2, int(256e6 // (k * n / 2)))
        lins = [b200nn.Int4Linear(packed, scales, None, k, n, 128, reg) for _ in range(copies)]
        x = torch.randn(1, k, device="cuda")
        y = torch.empty(1, n, device="cuda")
        for l in lins:
            l.forward_dev(x.data_ptr(), 1, y.data_ptr())
        reg.synchronize()
        # the launches are captured into one CUDA graph so that the host's launch rate is not what
        # is being measured
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream, capture_error_mode="thread_local"):
            for i in range(iters):
                lins[i % copies].forward_dev(x.data_ptr(), 1, y.data_ptr())
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            g.replay()
            e0.record(stream)
            g.replay()
            e1.record(stream)
        torch.cuda.synchronize()
        del g
        us = e0.elapsed_time(e1) / iters * 1e3
        nbytes = k * n // 2 + ((k + 127) // 128) * n * 2 + k * 4 + n * 4
        out[name] = {"k": k, "n": n, "us_per_launch": round(us, 2), "GBps": round(nbytes / us / 1e3, 1),
                     "frac_of_hbm_peak": round(nbytes / us / 1e3 / hbm_peak, 4)}
        del lins
    return out


def _graph_time(reg, stream, launch, iters):
    """Microseconds per call of `launch(i)`, i = 0..iters-1, captured into one CUDA graph and replayed
    (the host's launch rate is not what is being measured); one untimed replay first."""
    import torch
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=stream, capture_error_mode="thread_local"):
        for i in range(iters):
            launch(i)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        g.replay()
        e0.record(stream)
        g.replay()
        e1.record(stream)
    torch.cuda.synchronize()
    del g
    return e0.elapsed_time(e1) / iters * 1e3


def int4_linear_isolated(reg, hbm_peak, tf_peak, iters=64):
    """The isolated int4 Linear of GPT-2 Small (K, N) in {(768,3072), (3072,768), (768,2304), (768,50257)}
    at M in {1, 8, 64} rows through Int4Linear.forward on device buffers (f32 in, f32 out: the reference's
    interface, int4_linear.rs:60-130).  Nibbles uniform in [-8,7], group 128, fp16-representable scales,
    activations N(0,1).  `cold`: every launch reads another copy of the weight (copies add up to > 256 MB,
    twice the L2); `warm`: the same weight every launch.  Bytes are algorithmic: nibbles + fp16 scales +
    f32 input rows + f32 output rows; flops 2*M*K*N."""
    import torch
    import b200nn
    from b200nn import synth
    stream = torch.cuda.ExternalStream(reg.stream)
    out = {}
    for (k, n) in ((768, 3072), (3072, 768), (768, 2304), (768, 50257)):
        packed, scales, _, _ = synth.int4_linear_case(21, 1, k, n, 128)
        copies = max(2, int(256e6 // (k * n / 2)) + 1)
        lins = [b200nn.Int4Linear(packed, scales, None, k, n, 128, reg) for _ in range(copies)]
        for m in (1, 8, 64):
            x = torch.randn(m, k, device="cuda")
            y = torch.empty(m, n, device="cuda")
            for l in lins:  # every copy once outside the capture: staging buffers and scratch get their size
                l.forward_dev(x.data_ptr(), m, y.data_ptr())
            reg.synchronize()
            nbytes = k * n // 2 + ((k + 127) // 128) * n * 2 + m * k * 4 + m * n * 4
            rec = {"bytes": nbytes}
            for mode in ("cold", "warm"):
                us = _graph_time(reg, stream, lambda i: lins[i % copies if mode == "cold" else 0].forward_dev(
                    x.data_ptr(), m, y.data_ptr()), iters)
                rec[mode] = {"us": round(us, 2), "GBps": round(nbytes / us / 1e3, 1),
                             "frac_of_hbm_peak": round(nbytes / us / 1e3 / hbm_peak, 4),
                             "tflops": round(2 * m * k * n / us / 1e6, 2)}
            out[f"M{m}_K{k}_N{n}"] = rec
        del lins
    return out


def attention_isolated(reg, hbm_peak, tf_peak, seqs=(256, 512, 1024), decode=True):
    """Isolated attention on fp16 device buffers in the library's cache layout.  Prefill: causal, batch 8,
    12 heads, head_dim 64, seq 256 / 512 / 1024, Q/K/V N(0,1); flops 4 * 0.5 * B * H * n^2 * 64 (the
    convention of tests_transformer.rs:2219-2224 times the batch); both a single launch between events
    and the graph-replayed rate are given (these are microseconds of tensor work).  Decode: one query
    per sequence, 64 sequences x 12 heads against 1024 cached positions; bytes B*H*1024*64*2*2 + q + out,
    rotating over copies of the cache that add up to more than the L2."""
    import torch
    from b200nn import ops
    stream = torch.cuda.ExternalStream(reg.stream)
    out = {"prefill": {}, "decode": {}}
    B, H = 8, 12
    for n in seqs:
        q = torch.randn(B * n, H * 64, device="cuda", dtype=torch.float16)
        kc = torch.randn(B, H, n, 64, device="cuda", dtype=torch.float16)
        vc = torch.randn(B, H, n, 64, device="cuda", dtype=torch.float16)
        o = torch.empty_like(q)
        call = lambda i: ops.prefill_attention_f16(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), B, H, n, n, 0, o.data_ptr(), reg)
        call(0)
        reg.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            e0.record(stream)
            call(0)
            e1.record(stream)
        torch.cuda.synchronize()
        single_us = e0.elapsed_time(e1) * 1e3
        us = _graph_time(reg, stream, call, 32)
        flops = 4 * 0.5 * B * H * n * n * 64
        out["prefill"][f"seq{n}"] = {"us_graph": round(us, 2), "us_single_launch": round(single_us, 2),
                                     "tflops": round(flops / us / 1e6, 2),
                                     "frac_of_bf16_peak": round(flops / us / 1e6 / tf_peak, 4)}
    if not decode:
        return out
    B, ctx = 64, 1024
    copies = 3  # 3 x 201 MB of K and V: more than the 126 MB L2 between two uses of a copy
    q = torch.randn(B, H * 64, device="cuda", dtype=torch.float16)
    kcs = [torch.randn(B, H, ctx, 64, device="cuda", dtype=torch.float16) for _ in range(copies)]
    vcs = [torch.randn(B, H, ctx, 64, device="cuda", dtype=torch.float16) for _ in range(copies)]
    o = torch.empty_like(q)
    call = lambda i: ops.decode_attention_f16(q.data_ptr(), kcs[i % copies].data_ptr(), vcs[i % copies].data_ptr(), B, H,
                                              ctx, ctx, o.data_ptr(), reg)
    call(0)
    reg.synchronize()
    us = _graph_time(reg, stream, call, 30)
    nbytes = B * H * ctx * 64 * 2 * 2 + 2 * B * H * 64 * 2
    out["decode"]["b64_kv1024"] = {"us": round(us, 2), "bytes": nbytes, "GBps": round(nbytes / us / 1e3, 1),
                                   "frac_of_hbm_peak": round(nbytes / us / 1e3 / hbm_peak, 4)}
    return out


def cpu_reference_form(steps=1):
    """The reference benchmark's first configuration the way the reference's CPU test runs it (tests_inference.rs:4393-4540): GPT-2
    Small, f32 weights, f64 accumulation, greedy decode WITHOUT a KV cache (every step recomputes the
    whole sequence), one thread.  Bounded sample: the 64-token prompt and `steps` generated tokens."""
    from oracle import oracle
    from b200nn import synth
    from b200nn.gpt2 import Gpt2Config
    cfg = Gpt2Config.small()
    w = synth.gpt2_weights(cfg)
    prompt = synth.token_ids(synth.BASE_SEED + 7, (1, 64), cfg.vocab_size)[0]
    om = oracle.Model(cfg.as_dict(), w)
    threads = oracle.num_threads()
    oracle.lib().orc_set_num_threads(1)
    try:
        t0 = time.perf_counter()
        om.generate(prompt, steps)
        sec = time.perf_counter() - t0
    finally:
        oracle.lib().orc_set_num_threads(threads)
    return {"value": steps / sec, "unit": UNIT, "cores": 1, "kind": "port",
            "sample": f"GPT-2 Small f32, prompt 64, {steps} greedy token(s) without KV cache, f64, single thread "
                      f"({sec:.1f} s)"}


def run_b200(args):
    import torch
    import torch.distributed as dist
    import b200nn
    from b200nn import DecodeSession, Gpt2Config, Gpt2Model, Int4Gpt2Model, synth

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        args.gpus = world
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    def barrier():
        if world > 1:
            dist.barrier()

    preset, total, prompt_len, max_new, family = WORKLOADS[args.workload]
    if args.batch:
        total = args.batch
    cfg = getattr(Gpt2Config, preset)()
    if args.layers:
        cfg.n_layer = args.layers  # reduced depth: for profiler captures only, never a benchmark number
    lo, hi = shard_bounds(total, world, rank)
    batch = hi - lo
    reg = b200nn.KernelRegistry(local)
    for kv in args.tune:
        key, val = kv.split("=")
        reg.set_tuning(key, int(val))
    w = synth.gpt2_weights(cfg)
    t0 = time.time()
    if family == "int4":
        model = Int4Gpt2Model.from_weights(w, cfg, reg, flags=b200nn.QUANT_LM_HEAD, group_size=128)
    else:
        model = Gpt2Model.from_weights(w, cfg, reg)
    build_s = time.time() - t0
    prompts_all = synth.token_ids(synth.BASE_SEED + 7, (total, prompt_len), cfg.vocab_size)
    prompts = np.ascontiguousarray(prompts_all[lo:hi])

    capacity = prompt_len + max_new + 8
    # greedy decoding needs tokens only: the step's logits stay in the LM head's epilogue
    sess = DecodeSession(model, batch, capacity, flags=b200nn.TOKENS_ONLY)
    sess.prefill(prompts)
    stream = torch.cuda.ExternalStream(reg.stream, device=torch.device("cuda", local))
    window = max_new  # context goes prompt_len .. prompt_len + window - 1, then wraps

    def run_steps(n):
        done = 0
        while done < n:
            room = prompt_len + window - sess.position()
            if room <= 0:
                sess.rewind(prompt_len)
                room = window
            k = min(room, n - done)
            sess.step(k)
            done += k

    run_steps(max(args.warmup, 3))
    # fill the rest of the decode window once, so that every context of it has its cached rows and the
    # timed region can start anywhere inside it
    if sess.position() < prompt_len + window:
        sess.step(prompt_len + window - sess.position())
    reg.synchronize()
    launches0 = reg.launch_count()
    # The K timed steps sit in the middle of the decode window [prompt_len, prompt_len + window): their
    # mean context is the window's mean whatever K is (K > window wraps around the whole window).  The
    # timed region runs `reps` times from the same start (the cache keeps its rows); the median counts.
    first_ctx = prompt_len + max(0, (window - args.steps) // 2)
    reps = max(1, args.reps)
    sampler = ClockSampler(local)
    sampler.start()
    rep_ms = []
    for _ in range(reps):
        sess.rewind(first_ctx)
        barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            e0.record(stream)
            run_steps(args.steps)
            e1.record(stream)
        torch.cuda.synchronize()
        barrier()
        t = torch.tensor([e0.elapsed_time(e1)], device="cuda", dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        rep_ms.append(float(t.item()))
    clocks = sampler.finish()
    ms = sorted(rep_ms)[len(rep_ms) // 2]
    launches = (reg.launch_count() - launches0) // reps
    value = total * args.steps / (ms / 1e3)
    last_ctx = first_ctx + args.steps - 1
    contexts = [first_ctx, last_ctx] if args.steps <= window else [prompt_len, prompt_len + window - 1]

    # per-kernel-family device time of single decode steps at mid-window context (CUDA events
    # around every launch on the library's stream), for the roofline of the dominant kernel
    sess.rewind(prompt_len)
    run_steps(window // 2)
    ctx_mid = sess.position() + 1
    _, lin_bytes = sess.profile_step()  # algorithmic bytes of the Linear kernels of one step
    sess.rewind(sess.position() - 1)
    # each family alone: its launches of one step, three passes back to back between two CUDA
    # events on the library's stream (the activations are scratch afterwards)
    fam, fam_launches, fam_reps = {}, {}, 3
    for name in ("attention", "linear", "layernorm", "lm_head"):
        ms_f, n_f = sess.time_family(name, fam_reps)
        fam[name] = ms_f / fam_reps
        fam_launches[name] = n_f // fam_reps
    hbm_peak, tf_peak, peak_kind = peaks()
    H, L, d = cfg.n_head, cfg.n_layer, cfg.n_embd
    act_b = 2 if batch > 2 else 4
    attn_bytes_launch = batch * H * ctx_mid * 64 * 2 * 2 + 2 * batch * d * act_b
    lin_flops = sum(2 * batch * k * n for k, n in ((d, 3 * d), (d, d), (d, 4 * d), (4 * d, d))) * L
    roofs = {
        "attention": {"kernel": "decode_attn_stream_kernel" if batch * H >= 2 * 148 * 8 else "decode_attn_kernel",
                      "bound": "hbm", "unit": "GB/s", "peak": hbm_peak,
                      "achieved": attn_bytes_launch * L / (fam["attention"] * 1e-3) / 1e9 if fam["attention"] else 0.0},
        "linear": {"kernel": family + " Linear kernels (4 per layer)", "bound": "hbm", "unit": "GB/s", "peak": hbm_peak,
                   "achieved": lin_bytes / (fam["linear"] * 1e-3) / 1e9 if fam["linear"] else 0.0,
                   "tensor_tflops": lin_flops / (fam["linear"] * 1e-3) / 1e12 if fam["linear"] else 0.0},
    }
    dominant = max(("attention", "linear"), key=lambda k2: fam[k2])
    roof = dict(roofs[dominant])
    roof["frac"] = roof["achieved"] / roof["peak"] if roof["peak"] else None
    roof["frac_of_nominal_8000_GBps"] = roof["achieved"] / 8000.0  # the data-sheet HBM3e figure, for context
    # DRAM bytes per launch: the ratio dram bytes / algorithmic bytes of the kernel's ncu capture on a
    # smaller case of the same workload (2 layers, context 130: 218.1 MB moved for 213.0 MB), applied
    # to this launch's algorithmic bytes -- the kernel streams, so its traffic grows with the rows read
    ratio, ratio_src = traffic_ratio(roofs[dominant]["kernel"])
    roof["traffic"] = ratio * attn_bytes_launch if dominant == "attention" and ratio else None
    roof["traffic_source"] = (ratio_src + ", scaled by the rows this launch reads") if roof["traffic"] else None
    roof["peak_source"] = peak_kind
    roof["launch_ms"] = fam[dominant] / max(1, fam_launches[dominant])
    roof["launches_per_step"] = fam_launches
    roof["step_family_ms"] = {k2: round(v, 4) for k2, v in fam.items()}
    roof["other"] = {k2: {"achieved": v["achieved"], "frac": v["achieved"] / v["peak"]} for k2, v in roofs.items()
                     if k2 != dominant}

    # end to end through the public batched generate call: host prompts in, host tokens out; with more
    # than one rank every rank's [sequences, prompt + new] token matrix is gathered on rank 0 inside the
    # timed region (the one cross-GPU step of the batch-sharded path)
    e2e_runs = []
    gathered_rows = None
    for _ in range(args.e2e_runs):
        barrier()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        out, lens = model.generate_batch(prompts, max_new)
        if world > 1:
            mine = torch.from_numpy(out.astype(np.int32)).cuda()
            sizes = [shard_bounds(total, world, r)[1] - shard_bounds(total, world, r)[0] for r in range(world)]
            pad = torch.zeros((max(sizes), mine.shape[1]), dtype=torch.int32, device="cuda")
            pad[: mine.shape[0]] = mine
            parts = [torch.empty_like(pad) for _ in range(world)] if rank == 0 else None
            dist.gather(pad, parts, dst=0)
            if rank == 0:
                allt = torch.cat([parts[r][: sizes[r]] for r in range(world)]).cpu().numpy()
                gathered_rows = int(allt.shape[0])
        else:
            gathered_rows = int(out.shape[0])
        t1 = time.perf_counter()
        dt = torch.tensor([t1 - t0], device="cuda", dtype=torch.float64)
        if world > 1:
            dist.all_reduce(dt, op=dist.ReduceOp.MAX)
        e2e_runs.append(float(dt.item()))
    e2e = None
    if e2e_runs:
        best = min(e2e_runs)
        e2e = {"value": total * max_new / best, "unit": UNIT, "h2d_bytes_per_step": batch * prompt_len * 4 / max_new,
               "d2h_bytes_per_step": batch * (prompt_len + max_new) * 4 / max_new, "seconds_per_generate": best,
               "sequences_on_rank0": gathered_rows,
               "note": "generate_batch: prefill + %d decode steps, host token ids in, host tokens out, all ranks' "
                       "tokens gathered on rank 0; bytes are per decode step per rank" % max_new}

    # the prefill of this rank's prompts on its own (second of two passes), device time on the library's stream
    p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        sess.prefill(prompts)
        p0.record(stream)
        sess.prefill(prompts)
        p1.record(stream)
    torch.cuda.synchronize()
    prefill_ms = p0.elapsed_time(p1)
    pre_flops = lin_flops * prompt_len + 4 * 0.5 * batch * H * prompt_len * prompt_len * 64 * L
    prefill = {"ms": prefill_ms, "tokens_per_s": batch * prompt_len / (prefill_ms * 1e-3),
               "tflops": pre_flops / (prefill_ms * 1e-3) / 1e12, "tokens": batch * prompt_len,
               "note": "this rank's prompts through all layers (Linear + causal attention flops; LM head on the last rows only)"}

    line = {
        "metric": METRIC.replace("int4", family), "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": ("int4 weights / fp16 operands / f32 accumulate" if family == "int4" else
                  "f32 weights as fp16 hi + lo / fp16 activations / f32 accumulate"), "data": "synthetic",
        "config": {"workload": args.workload, "total_sequences": total, "sequences_per_gpu": batch,
                   "prompt_len": prompt_len, "decode_window": [prompt_len, prompt_len + window - 1],
                   "timed_contexts": contexts, "timed_region_repeats": reps, "timed_region_ms": [round(x, 3) for x in rep_ms],
                   "l2": "inputs larger than L2 (weights + KV read per step: %.1f GB)" %
                         ((lin_bytes + attn_bytes_launch * L) / 1e9),
                   "model_build_s": round(build_s, 1)},
        "roofline": roof, "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks, "prefill": prefill,
    }
    if args.layers:
        line["config"]["layers_override"] = args.layers
        line["config"]["note"] = "reduced depth for a profiler capture: not a benchmark number"
    if args.tune:
        line["config"]["tuning_overrides"] = args.tune
    if rank == 0 and not args.no_gemv and family == "int4":
        line["gemv"] = gemv_bandwidth(reg, cfg, hbm_peak)
    if world == 1 and not args.no_isolated and family == "int4" and not args.layers:
        del sess
        reg.trim()
        line["int4_linear"] = int4_linear_isolated(reg, hbm_peak, tf_peak)
        line["attention"] = attention_isolated(reg, hbm_peak, tf_peak)
    if world == 1 and not args.no_cpu_baseline:
        wq = build_int4_oracle_weights(cfg, w) if family == "int4" else w
        steps = args.cpu_steps
        sec, threads = cpu_decode_sample(cfg, wq, prompts_all[0, : args.cpu_prompt], steps, 1)
        line["cpu_baseline"] = {"value": steps / sec, "unit": UNIT, "cores": threads, "kind": "port",
                                "sample": f"1 of {total} sequences, prompt {args.cpu_prompt}, {steps} KV-cached decode "
                                          f"steps with the oracle (f64 accumulate)"}
        if not args.no_cpu_reference_form:
            line["cpu_baseline"]["reference_form_gpt2_small"] = cpu_reference_form()
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="gpt2-xl-int4-b256", choices=sorted(WORKLOADS))
    ap.add_argument("--batch", type=int, default=0, help="override the total number of sequences")
    ap.add_argument("--layers", type=int, default=0, help="profiling aid: build only this many layers")
    ap.add_argument("--no-gemv", action="store_true", help="skip the dequant-GEMV bandwidth measurement")
    ap.add_argument("--e2e-runs", type=int, default=2)
    ap.add_argument("--reps", type=int, default=5, help="repeats of the timed region (the median is reported)")
    ap.add_argument("--no-isolated", action="store_true", help="skip the isolated int4 Linear / attention measurements")
    ap.add_argument("--isolated-only", action="store_true",
                    help="profiling aid: only the isolated attention measurements (no model is built); with "
                         "--attention-seq N only the causal prefill case of that length, with --gemv-shape NAME "
                         "only the one-row dequant-GEMV of that GPT-2 XL shape (qkv, proj, fc, fcproj, lm_head)")
    ap.add_argument("--attention-seq", type=int, default=0)
    ap.add_argument("--gemv-shape", default="")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-cpu-reference-form", action="store_true",
                    help="skip the single-thread, cache-less GPT-2 Small CPU run (the reference's own CPU test form)")
    ap.add_argument("--tune", action="append", default=[], metavar="KEY=VALUE",
                    help="measurement aid: b200nn_ctx_set_tuning override, e.g. --tune attn_stream=0 (repeatable)")
    ap.add_argument("--cpu-steps", type=int, default=8)
    ap.add_argument("--cpu-prompt", type=int, default=32)
    ap.add_argument("--cpu-max-steps", type=int, default=64)
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if args.isolated_only:
        sys.path.insert(0, os.path.join(ROOT, "async-gpu_b200"))
        import b200nn
        reg = b200nn.KernelRegistry(0)
        for kv in args.tune:
            key, val = kv.split("=")
            reg.set_tuning(key, int(val))
        hbm_peak, tf_peak, _ = peaks()
        if args.gemv_shape:
            from b200nn.gpt2 import Gpt2Config
            print(json.dumps({"gemv": gemv_bandwidth(reg, Gpt2Config.xl(), hbm_peak, only=args.gemv_shape),
                              "note": "isolated kernels only: not the benchmark line"}), flush=True)
            return 0
        seqs = (args.attention_seq,) if args.attention_seq else (256, 512, 1024)
        print(json.dumps({"attention": attention_isolated(reg, hbm_peak, tf_peak, seqs, decode=not args.attention_seq),
                          "note": "isolated kernels only: not the benchmark line"}), flush=True)
        return 0
    if args.gpus > 1 and "RANK" not in os.environ:
        # convenience: relaunch under torchrun when called plainly with --gpus N
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", "29511", os.path.abspath(__file__)] + sys.argv[1:]
        return subprocess.call(cmd)
    return run_b200(args)


if __name__ == "__main__":
    sys.exit(main())
