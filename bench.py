#!/usr/bin/env python
"""Benchmark of the attention hot path on B200.

Headline workload (one "step"): one decode step of the batched-decode configuration --
Llama-3-8B attention shape (32 query / 8 KV heads, head_dim 128), 64 concurrent sequences with
seeded context lengths ~U[512, 8192], paged fp16 KV in 16-token blocks, one new token per
sequence: KV append + split-KV attention + combine, for one attention layer.  The KV working set
(~1.1 GB per GPU) is far larger than L2, so no L2 flush is needed between steps.

  python bench.py --gpus N --steps K --warmup W            (N > 1: launched under torchrun)
  python bench.py --impl reference ...                     (CPU oracle on the host cores)

With N > 1 every rank owns its own 64 sequences (weak scaling, no collective on the data path);
the timed region is bracketed by a barrier + synchronize and the maximum over ranks is reported.
One JSON line is printed by rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

METRIC = "decode_attn_tok_per_s"
UNIT = "tok/s"


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "tflops": d["bf16_tflops"],
                "tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "src": "measured"}
    return {"hbm_gbs": 6650.0, "tflops": 1590.0, "tflops_sustained": 1400.0, "src": "fallback"}


class ClockSampler:
    """Samples nvidia-smi SM clocks and throttle reasons of one GPU while a region is timed."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc = index, None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for n, val in zip(names, f[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------------------------
# workloads
# ------------------------------------------------------------------------------------------------
def setup_decode(ctx, cfg, rank, device):
    """Paged pools filled (through the append kernel) with seeded N(0,1) K/V for `cfg.batch`
    sequences; returns everything a decode step needs."""
    import torch

    import hippo_leap_b200 as hl
    from hippo_leap_b200 import synth

    ctx_lens = synth.gen_ctx_lens(cfg, rank=rank)
    tables, num_blocks = synth.gen_block_tables(ctx_lens, cfg.block_tokens, cfg.seed + rank)
    shape = hl.AttnShape(cfg.n_head, cfg.n_head_kv, cfg.head_dim, cfg.head_dim, hl.HL_ROPE_SPLIT_HALF, cfg.rms_eps)
    ctx.set_rope(cfg.theta())
    kv = ctx.kv_create(1, cfg.n_head_kv, cfg.head_dim, cfg.block_tokens, num_blocks)
    ttab = torch.from_numpy(tables).to(device)
    gen = torch.Generator(device=device)
    gen.manual_seed(1000 + cfg.seed + rank)
    for i, c in enumerate(ctx_lens):
        k = torch.randn((int(c), cfg.n_head_kv, cfg.head_dim), generator=gen, device=device)
        v = torch.randn((int(c), cfg.n_head_kv, cfg.head_dim), generator=gen, device=device)
        nb = (int(c) + cfg.block_tokens - 1) // cfg.block_tokens
        ctx.kv_append_seq(kv, 0, shape, k, v, 0, ttab[i, :nb].contiguous())
    B = len(ctx_lens)
    q = torch.randn((B, cfg.n_head, cfg.head_dim), generator=gen, device=device)
    kn = torch.randn((B, cfg.n_head_kv, cfg.head_dim), generator=gen, device=device)
    vn = torch.randn((B, cfg.n_head_kv, cfg.head_dim), generator=gen, device=device)
    out = torch.empty_like(q)
    tctx = torch.from_numpy(ctx_lens).to(device)
    ctx.sync()
    return dict(shape=shape, kv=kv, ctx_lens=ctx_lens, tctx=tctx, ttab=ttab, q=q, kn=kn, vn=vn, out=out,
                max_ctx=int(ctx_lens.max()))


def cpu_decode_sample(cfg, n_seq, steps, n_threads):
    """The CPU oracle on the first n_seq sequences of the same seeded workload: `steps` decode steps.
    Returns seconds per step."""
    import oracle
    from hippo_leap_b200 import synth

    ctx_lens = synth.gen_ctx_lens(cfg, rank=0)[:n_seq]
    theta = cfg.theta()
    g = np.random.Generator(np.random.PCG64(77))
    caches = []
    for c in ctx_lens:
        sc = oracle.SeqCache(int(c), cfg.n_head_kv, cfg.head_dim)
        sc.k[:] = g.standard_normal(sc.k.shape, dtype=np.float32)
        sc.v[:] = g.standard_normal(sc.v.shape, dtype=np.float32)
        caches.append(sc)
    q = g.standard_normal((n_seq, 1, cfg.n_head, cfg.head_dim), dtype=np.float32)
    k = g.standard_normal((n_seq, 1, cfg.n_head_kv, cfg.head_dim), dtype=np.float32)
    v = g.standard_normal((n_seq, 1, cfg.n_head_kv, cfg.head_dim), dtype=np.float32)
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        for i, sc in enumerate(caches):
            sc.cur_len = int(ctx_lens[i]) - 1  # the step appends at ctx-1 and attends ctx keys
            oracle.attn_forward(q[i], k[i], v[i], sc, theta=theta, rope_mode=oracle.ROPE_SPLIT_HALF,
                                n_threads=n_threads)
        times.append(time.perf_counter() - t0)
    return times, ctx_lens


def run_reference(args, rank, world, result_out):
    """The reference arm: the CPU restatement of the reference's float32 ops (the reference itself is
    Nim and cannot be built here), all host threads, on a bounded sample of the same workload."""
    if rank != 0:
        return
    import oracle
    from hippo_leap_b200 import synth

    cfg = synth.CONFIGS[4]
    n_threads = os.cpu_count() or oracle.max_threads()  # torchrun pins OMP_NUM_THREADS=1; ask for all cores
    # Size the per-step sample so that the whole run stays within about two minutes.
    probe, _ = cpu_decode_sample(cfg, 4, 2, n_threads)
    per_seq = probe[1] / 4
    n_seq = int(max(1, min(16, 120.0 / ((args.warmup + args.steps) * per_seq))))
    times, ctx_lens = cpu_decode_sample(cfg, n_seq, args.warmup + args.steps, n_threads)
    t = sum(times[args.warmup:])
    value = n_seq * args.steps / t
    sample = (f"first {n_seq} of the 64 seeded sequences (ctx sum {int(ctx_lens.sum())}), one layer, "
              f"{args.steps} steps, {n_threads} threads")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * t / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(cfg, args.gpus),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": n_threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), file=result_out, flush=True)


def workload_config(cfg, n_gpus):
    return {"workload": "config 4: batched decode attention, Llama-3-8B shape, one layer",
            "n_head": cfg.n_head, "n_head_kv": cfg.n_head_kv, "head_dim": cfg.head_dim,
            "sequences_per_gpu": cfg.batch, "ctx_range": list(cfg.ctx_range), "kv": "paged fp16",
            "block_tokens": cfg.block_tokens, "sharding": f"batch x{n_gpus} (own sequences per GPU, no collective)",
            "l2": "KV working set ~1.1 GB per GPU >> 126 MB L2 (no flush needed)"}


def timed_loop(torch, fn, steps):
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1)  # ms


def extras_single_gpu(ctx, torch, device, peaks, quick, configs=(2, 3, 5)):
    """Prefill TFLOP/s on the prefill configurations (one layer each), device-resident inputs."""
    import hippo_leap_b200 as hl
    from hippo_leap_b200 import synth

    res = {}
    for ci in configs:
        cfg = synth.CONFIGS[ci]
        S = cfg.prefill
        gen = torch.Generator(device=device)
        gen.manual_seed(2000 + ci)
        qw = kw = None
        if cfg.qk_norm:
            qw = (torch.rand(cfg.head_dim, generator=gen, device=device) * 0.2 + 0.9)
            kw = (torch.rand(cfg.head_dim, generator=gen, device=device) * 0.2 + 0.9)
        shape = hl.AttnShape(cfg.n_head, cfg.n_head_kv, cfg.head_dim, cfg.head_dim, hl.HL_ROPE_SPLIT_HALF,
                             cfg.rms_eps, qw, kw)
        ctx.set_rope(cfg.theta())
        bt = 128
        nb = (S + bt - 1) // bt
        kv = ctx.kv_create(1, cfg.n_head_kv, cfg.head_dim, bt, nb)
        table = torch.randperm(nb, generator=gen, device=device).to(torch.int32)
        q = torch.randn((S, cfg.n_head, cfg.head_dim), generator=gen, device=device)
        k = torch.randn((S, cfg.n_head_kv, cfg.head_dim), generator=gen, device=device)
        v = torch.randn((S, cfg.n_head_kv, cfg.head_dim), generator=gen, device=device)
        if cfg.bf16_range:    # values a bf16 model would produce, still handed over as float32
            q, k, v = (x.bfloat16().float() for x in (q, k, v))
        if cfg.fp16_inputs:   # activations arrive as fp16
            q, k, v = (x.half() for x in (q, k, v))
        out = torch.empty((S, cfg.n_head, cfg.head_dim), dtype=torch.float16, device=device)
        ctx.kv_append_seq(kv, 0, shape, k, v, 0, table)
        n = 2 if quick else 5
        for _ in range(2):
            ctx.attn_prefill(kv, 0, shape, q, 0, table, out)
        ms = timed_loop(torch, lambda: ctx.attn_prefill(kv, 0, shape, q, 0, table, out), n) / n
        ms_app = timed_loop(torch, lambda: ctx.kv_append_seq(kv, 0, shape, k, v, 0, table), n) / n
        fl = synth.prefill_flops(cfg.n_head, cfg.head_dim, S)
        tf = fl / (ms * 1e-3) / 1e12
        res[f"config{ci}_prefill"] = {
            "workload": f"{cfg.name}: causal prefill of {S} tokens, one layer, "
                        f"{'fp16' if cfg.fp16_inputs else 'float32'} Q/K/V in, fp16 out", "ms_attn": ms, "ms_kv_append": ms_app,
            "tflops": tf, "frac_of_tensor_peak": tf / peaks["tflops"], "peak_tflops": peaks["tflops"],
            "peak_src": peaks["src"], "flops": fl}
        kv.destroy()
        del q, k, v, out
        torch.cuda.empty_cache()
    return res


def extra_linear(ctx, torch, device, peaks):
    """The dense fp16 projection next to the hot path: a Wo-shaped GEMM at config 3 size, and the decode projections
    of Llama-3.2-1B (M = 1) timed as chains of 16 launches over 16 different weight matrices (more than L2 holds)
    replayed from one CUDA graph, so that the figures are device time, not the launch rate of this script."""
    import hippo_leap_b200 as hl
    gen = torch.Generator(device=device)
    gen.manual_seed(7)
    res = {}
    M, N, K = 8192, 4096, 4096
    a = torch.randn((M, K), generator=gen, device=device).half()
    w = (torch.randn((N, K), generator=gen, device=device) / K ** 0.5).half()
    out = torch.empty((M, N), dtype=torch.float32, device=device)
    for _ in range(3):
        ctx.linear_f16(a, w, out)
    n = 20
    ms = timed_loop(torch, lambda: ctx.linear_f16(a, w, out), n) / n
    fl = 2.0 * M * N * K
    res[f"gemm_{M}x{N}x{K}"] = {"ms": ms, "tflops": fl / (ms * 1e-3) / 1e12,
                                "frac_of_tensor_peak": fl / (ms * 1e-3) / 1e12 / peaks["tflops"]}
    del a, w, out
    side = torch.cuda.Stream(device=device)
    ctx2 = hl.Context(device.index or 0, side)
    try:
        for name, (N, K, L) in {"qkv_3072x2048": (3072, 2048, 16), "wo_2048x2048": (2048, 2048, 16),
                                "gate_up_16384x2048": (16384, 2048, 16), "down_2048x8192": (2048, 8192, 16),
                                "vocab_128256x2048": (128256, 2048, 2)}.items():
            ws = (torch.randn((L, N, K), generator=gen, device=device) / K ** 0.5).half()
            for M in (1, 4, 16, 64):
                a = torch.randn((M, K), generator=gen, device=device).half()
                out = torch.empty((M, N), dtype=torch.float32, device=device)
                torch.cuda.synchronize()
                with torch.cuda.stream(side):
                    for l in range(L):
                        ctx2.linear_f16(a, ws[l], out)
                    side.synchronize()
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=side):
                        for l in range(L):
                            ctx2.linear_f16(a, ws[l], out)
                    for _ in range(3):
                        g.replay()
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    reps = 20
                    e0.record(side)
                    for _ in range(reps):
                        g.replay()
                    e1.record(side)
                    side.synchronize()
                us = e0.elapsed_time(e1) * 1e3 / (reps * L)
                by = N * K * 2
                res[f"gemv_{name}" + ("" if M == 1 else f"_x{M}rows")] = {
                    "us_per_launch": us, "weight_gbs": by / (us * 1e-6) / 1e9,
                    "frac_of_hbm_peak": by / (us * 1e-6) / 1e9 / peaks["hbm_gbs"]}
                del a, out, g
            del ws
            torch.cuda.empty_cache()
    finally:
        ctx2.close()
    return res


def extra_config2_pipeline(torch, device_index):
    """Config 2 end to end through the backend contract (the calls hippo_leap's generate loop makes):
    one 2048-token prefill, then 256 greedy decode steps, 16 attention layers, llama3-scaled theta,
    host token ids in, host logits / token id out, one synchronisation per call."""
    from hippo_leap_b200 import backend as B
    from hippo_leap_b200 import synth

    cfg = synth.CONFIGS[2]
    hp = B.HParams(nVocab=512, nLayer=cfg.layers, nHead=cfg.n_head, nHeadKv=cfg.n_head_kv, headDim=cfg.head_dim,
                   ropeFreqBase=cfg.rope_base, llama3Scaling=True)
    m = B.standin_model(hp, cfg.seed)
    cache = B.initKvCache(hp, cfg.prefill + cfg.decode_steps + 8, device_index)
    B.loadModelBackend(m, hp, device_index)
    try:
        prompt = np.random.Generator(np.random.PCG64([cfg.seed, 1])).integers(0, hp.nVocab, cfg.prefill).astype(np.int32)
        res = {}
        for rep in range(2):  # first pass warms up (allocations, cos/sin table), second is timed
            cache.curLen = 0
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            tok = B.argmaxLast(B.forwardPrefill(m, prompt, cache), hp.nVocab)
            t1 = time.perf_counter()
            gpu_ms = 0.0
            for _ in range(cfg.decode_steps):
                tok, ms = B.forwardDecodeTokenTimed(m, tok, cache)
                gpu_ms += ms
            t2 = time.perf_counter()
            res = {"workload": "config 2: Llama-3.2-1B attention shape, 16 layers, prefill 2048 + 256 greedy decode "
                               "steps through the backend contract (attention-only stand-in model)",
                   "prefill_ms": (t1 - t0) * 1e3, "prefill_tok_per_s": cfg.prefill / (t1 - t0),
                   "decode_ms_per_token": (t2 - t1) * 1e3 / cfg.decode_steps,
                   "decode_tok_per_s": cfg.decode_steps / (t2 - t1),
                   "decode_gpu_ms_per_token": gpu_ms / cfg.decode_steps,
                   "launches": B.launchCount()}
        return res
    finally:
        B.freeKvCache(cache)
        B.unloadModelBackend()


def extra_dense_model(torch, device_index, prefill=2048, decode_steps=64):
    """The whole dense Llama-3.2-1B layer stack (16 layers, n_emb 2048, n_ffn 8192, vocabulary 128256, 32 / 8 heads of
    64, fp16 weights, llama3-scaled theta) through the dense backend contract: one prefill, then greedy decode steps.
    Weights repeat a seeded pool of 4 Mi normals (the kernels do not care; it keeps host set-up short)."""
    from hippo_leap_b200 import dense as D
    import hippo_leap_b200 as hl

    L = 16
    hp = D.DenseHParams(nVocab=128256, nEmb=2048, nLayer=L, nFfn=8192, nHead=32, nHeadKv=8, headDim=64,
                        ropeFreqBase=500000.0, rmsEps=1e-5, ropeMode=hl.HL_ROPE_SPLIT_HALF, llama3Scaling=True)
    g = np.random.Generator(np.random.PCG64([5, 77]))
    pool = g.standard_normal(1 << 22, dtype=np.float32)

    def rep(src, shape):  # src (4 Mi values) repeated to fill shape
        n = int(np.prod(shape))
        out = np.empty(-(-n // src.size) * src.size, src.dtype)
        out.reshape(-1, src.size)[:] = src
        return out[:n].reshape(shape)

    def mat(*shape):  # scaled 1/sqrt(fan_in)
        return rep((pool / np.sqrt(shape[-1])).astype(np.float16), shape)

    def gain(*shape):
        return g.uniform(0.9, 1.1, shape).astype(np.float32)

    E, F, V, qd, kd = hp.nEmb, hp.nFfn, hp.nVocab, hp.nHead * hp.headDim, hp.nHeadKv * hp.headDim
    w = dict(tok_emb=rep(pool.astype(np.float16), (V, E)), attn_norm=gain(L, E), wq=mat(L, qd, E), wk=mat(L, kd, E),
             wv=mat(L, kd, E), wo=mat(L, E, qd), q_norm=None, k_norm=None, ffn_norm=gain(L, E), w_gate=mat(L, F, E),
             w_up=mat(L, F, E), w_down=mat(L, E, F), out_norm=gain(E), w_out=mat(V, E))
    m = D.DenseModel(hp, w)
    weight_bytes = sum(v.nbytes for k, v in w.items() if v is not None and k != "tok_emb")
    cache = D.initKvCache(hp, prefill + decode_steps + 8, device_index)
    D.loadModelBackend(m, hp, device_index)
    try:
        prompt = np.random.Generator(np.random.PCG64([5, 1])).integers(0, hp.nVocab, prefill).astype(np.int32)
        res = {}
        for rep in range(2):
            cache.curLen = 0
            t0 = time.perf_counter()
            tok = D.argmaxLast(D.forwardPrefill(m, prompt, cache), hp.nVocab)
            t1 = time.perf_counter()
            gpu_ms = 0.0
            for _ in range(decode_steps):
                tok, ms = D.forwardDecodeTokenTimed(m, tok, cache)
                gpu_ms += ms
            t2 = time.perf_counter()
            gemm_flops = 2.0 * prefill * L * (E * (qd + 2 * kd) + qd * E + 3 * E * F)
            res = {"workload": f"Llama-3.2-1B dense model, fp16 weights, prefill {prefill} + {decode_steps} greedy decode "
                               "steps through the dense backend contract",
                   "prefill_ms": (t1 - t0) * 1e3, "prefill_tok_per_s": prefill / (t1 - t0),
                   "prefill_projection_tflops": gemm_flops / (t1 - t0) / 1e12,
                   "decode_ms_per_token": (t2 - t1) * 1e3 / decode_steps, "decode_tok_per_s": decode_steps / (t2 - t1),
                   "decode_gpu_ms_per_token": gpu_ms / decode_steps,
                   "decode_weight_gbs": weight_bytes / (gpu_ms / decode_steps * 1e-3) / 1e9,
                   "weight_bytes": weight_bytes}
        # several sequences decoded together from one shared page pool: every weight is read once per step for all of them
        batched = {}
        pool = D.DecodeBatch(m, 64, 512 + 40)
        try:
            short = prompt[:512]
            for s in range(64):
                pool.prefill(s, short)
            for nb in (1, 4, 16, 64):
                ids = np.arange(nb, dtype=np.int32)
                toks = np.full(nb, 11, np.int32)
                for _ in range(2):
                    toks, _ = pool.decode(ids, toks)
                gpu_ms, steps = 0.0, 8
                t0 = time.perf_counter()
                for _ in range(steps):
                    toks, _, ms = pool.decode(ids, toks, timed=True)
                    gpu_ms += ms
                wall = time.perf_counter() - t0
                batched[f"{nb}_sequences"] = {"ms_per_step": wall * 1e3 / steps, "gpu_ms_per_step": gpu_ms / steps,
                                              "tok_per_s": nb * steps / wall}
        finally:
            pool.close()
        res["batched_decode_ctx512"] = batched
        return res
    finally:
        D.freeKvCache(cache)
        D.unloadModelBackend()


def extra_head_sharded_prefill(ctx, torch, dist, device, rank, world, peaks):
    """Config 5 with KV heads split across ranks and one all-gather of the head outputs (fp16)."""
    import hippo_leap_b200 as hl
    from hippo_leap_b200 import synth

    from hippo_leap_b200 import sharding

    cfg = synth.CONFIGS[5]
    S = cfg.prefill
    sh = sharding.head_shard(rank, world, cfg.n_head, cfg.n_head_kv)
    hkv_l, hq_l = sh.n_head_kv, sh.n_head
    gen = torch.Generator(device=device)
    gen.manual_seed(3000 + rank)
    shape = hl.AttnShape(hq_l, hkv_l, cfg.head_dim, cfg.head_dim, hl.HL_ROPE_SPLIT_HALF, cfg.rms_eps)
    ctx.set_rope(cfg.theta())
    bt = 128
    nb = (S + bt - 1) // bt
    kv = ctx.kv_create(1, hkv_l, cfg.head_dim, bt, nb)
    table = torch.arange(nb, device=device, dtype=torch.int32)
    q = torch.randn((S, hq_l, cfg.head_dim), generator=gen, device=device)
    k = torch.randn((S, hkv_l, cfg.head_dim), generator=gen, device=device)
    v = torch.randn((S, hkv_l, cfg.head_dim), generator=gen, device=device)
    if cfg.fp16_inputs:
        q, k, v = (x.half() for x in (q, k, v))
    ctx.kv_append_seq(kv, 0, shape, k, v, 0, table)
    results = {}
    fused = sharding.FusedHeadShardedPrefill(ctx, kv, shape, S, cfg.n_head, device)
    plain = sharding.HeadShardedPrefill(ctx, kv, shape, S, 1, device, world)
    for name, runner in (("fused_in_kernel", fused), ("nccl_allgather_after", plain)):
        for _ in range(2):
            runner.run(q, table)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        n = 5
        results[name] = sharding.max_over_ranks(timed_loop(torch, lambda: runner.run(q, table), n) / n, device)
    # cross-check: both ways must produce the same gathered tensor
    a_ = fused.run(q, table)
    b_ = plain.run(q, table)
    torch.cuda.synchronize()
    same = bool(torch.equal(a_, b_[0]))

    ms = results["fused_in_kernel"]
    fl = synth.prefill_flops(cfg.n_head, cfg.head_dim, S)
    tf = fl / (ms * 1e-3) / 1e12
    kv.destroy()
    return {"workload": f"{cfg.name}: 32768-token causal prefill, KV heads {hkv_l}/GPU, fp16 head outputs stored to "
                        "every GPU by the attention kernel itself (peer stores over NVLink, no collective kernel)",
            "ms_nccl_allgather_after": results["nccl_allgather_after"], "ms_fused_in_kernel": results["fused_in_kernel"],
            "fused_equals_allgather": same,
            "ms": ms, "tflops_aggregate": tf, "frac_of_tensor_peak_per_gpu": tf / world / peaks["tflops"],
            "scaling": "strong"}


def _protect_stdout():
    """Libraries (NCCL's version banner, for one) write to stdout; the contract is ONE JSON line
    there.  Point fd 1 at stderr for the run and keep the real stdout for the result line."""
    sys.stdout.flush()
    real = os.dup(1)
    os.dup2(2, 1)
    return os.fdopen(real, "w")


def main():
    result_out = _protect_stdout()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-extras", action="store_true", help="skip the prefill side measurements")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--decode-chunk", type=int, default=0)
    ap.add_argument("--prefill-kernel", type=int, default=0, help="0 auto, 1 warp-MMA, 2 tcgen05, 3 tcgen05 on SM pairs")
    ap.add_argument("--linear-only", action="store_true", help="measure only the dense fp16 projection kernels")
    ap.add_argument("--dense-only", action="store_true", help="measure only the dense Llama-3.2-1B model")
    ap.add_argument("--pipeline-only", action="store_true", help="measure only the config 2 backend pipeline")
    ap.add_argument("--head-sharded-only", action="store_true",
                    help="measure only the head-sharded config 5 prefill + all-gather at N GPUs")
    ap.add_argument("--prefill-only", type=int, default=0, metavar="CFG",
                    help="measure only the prefill kernel of configuration 2, 3 or 5 (small profiling target)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, rank, world, result_out)
        return

    import torch
    import torch.distributed as dist

    import hippo_leap_b200 as hl
    from hippo_leap_b200 import synth

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a B200: there is no CPU fallback (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    peaks = load_peaks()
    cfg = synth.CONFIGS[4]
    ctx = hl.Context(local_rank, torch.cuda.current_stream())
    ctx.set_tuning(args.decode_chunk, args.prefill_kernel)
    if args.linear_only:
        print(json.dumps(extra_linear(ctx, torch, device, peaks)), file=result_out, flush=True)
        ctx.close()
        return
    if args.dense_only:
        print(json.dumps(extra_dense_model(torch, local_rank)), file=result_out, flush=True)
        ctx.close()
        return
    if args.pipeline_only:
        print(json.dumps(extra_config2_pipeline(torch, local_rank)), file=result_out, flush=True)
        ctx.close()
        return
    if args.head_sharded_only:
        res = extra_head_sharded_prefill(ctx, torch, dist, device, rank, world, peaks)
        if rank == 0:
            print(json.dumps(res), file=result_out, flush=True)
        ctx.close()
        if world > 1:
            dist.destroy_process_group()
        return
    if args.prefill_only:
        res = extras_single_gpu(ctx, torch, device, peaks, quick=True, configs=(args.prefill_only,))
        print(json.dumps(res), file=result_out, flush=True)
        ctx.close()
        return
    w = setup_decode(ctx, cfg, rank, device)
    B = len(w["ctx_lens"])

    def step():
        ctx.kv_append_batch(w["kv"], 0, w["shape"], w["kn"], w["vn"], w["tctx"], w["ttab"])
        ctx.attn_decode(w["kv"], 0, w["shape"], w["q"], w["tctx"], w["max_ctx"], w["ttab"], w["out"])

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    l0 = ctx.launch_count()
    ms_local = timed_loop(torch, step, args.steps)
    launches = ctx.launch_count() - l0
    t = torch.tensor([ms_local], device=device, dtype=torch.float64)
    if world > 1:
        dist.barrier()
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total = float(t.item())
    value = world * B * args.steps / (ms_total * 1e-3)

    # roofline of the dominant kernel pair (split-KV decode + combine), timed alone
    for _ in range(3):
        ctx.attn_decode(w["kv"], 0, w["shape"], w["q"], w["tctx"], w["max_ctx"], w["ttab"], w["out"])
    ms_attn = timed_loop(torch, lambda: ctx.attn_decode(w["kv"], 0, w["shape"], w["q"], w["tctx"], w["max_ctx"],
                                                        w["ttab"], w["out"]), args.steps) / args.steps
    alg_bytes = synth.decode_bytes(w["ctx_lens"], cfg.n_head, cfg.n_head_kv, cfg.head_dim)
    achieved = alg_bytes / (ms_attn * 1e-3) / 1e9
    roofline = {"bound": "hbm", "kernel": "attn_decode_kernel<128,...> + attn_combine_kernel<128>",
                "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                "peak_src": peaks["src"], "traffic": None, "algorithmic_bytes_per_launch": alg_bytes,
                "ms_per_launch": ms_attn}

    # end to end through the host-buffer C ABI call: pinned host inputs, host result, every step
    q_h, k_h, v_h = (x.cpu().pin_memory() for x in (w["q"], w["kn"], w["vn"]))
    out_h = torch.empty_like(q_h).pin_memory()

    def step_host():
        ctx.decode_step_host(w["kv"], 0, w["shape"], q_h, k_h, v_h, w["tctx"], w["max_ctx"], w["ttab"], out_h)

    for _ in range(3):
        step_host()
    if world > 1:
        dist.barrier()
    ms_e2e = timed_loop(torch, step_host, args.steps)
    t2 = torch.tensor([ms_e2e], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t2, op=dist.ReduceOp.MAX)
    e2e_value = world * B * args.steps / (float(t2.item()) * 1e-3)
    h2d = q_h.numel() * 4 + k_h.numel() * 4 + v_h.numel() * 4
    d2h = out_h.numel() * 4
    clocks = sampler.stop()  # sampled across the three timed loops above (device, kernel-only, end-to-end)
    code, detail = ctx.device_status()
    if code != 0:
        raise SystemExit(f"device status {code} (detail {detail}) after the timed region")

    extra = {}
    if not args.no_extras:
        if world == 1:
            extra.update(extras_single_gpu(ctx, torch, device, peaks, quick=False))
            extra["config2_backend_pipeline"] = extra_config2_pipeline(torch, local_rank)
            extra["linear_f16"] = extra_linear(ctx, torch, device, peaks)
            extra["dense_llama32_1b"] = extra_dense_model(torch, local_rank)
        if cfg.n_head_kv % world == 0:
            extra["config5_head_sharded_prefill"] = extra_head_sharded_prefill(ctx, torch, dist, device, rank, world,
                                                                               peaks)

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu:
        n_threads = os.cpu_count() or 1
        n_seq = 16
        times, cl = cpu_decode_sample(cfg, n_seq, 3, n_threads)
        tt = sum(times[1:]) / 2
        cpu_baseline = {"value": n_seq / tt, "unit": UNIT, "cores": n_threads, "kind": "port",
                        "sample": f"first {n_seq} of the 64 seeded sequences (ctx sum {int(cl.sum())}), one layer, "
                                  f"2 timed steps after 1 warm-up, {tt:.2f} s per step"}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_total / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16 KV, f32 accumulate", "data": "synthetic",
            "config": workload_config(cfg, world),
            "hbm_gbs": achieved, "roofline": roofline, "cpu_baseline": cpu_baseline,
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": float(t2.item()) / args.steps},
            "gpu_launches": int(launches), "clocks": clocks, "extra": extra,
        }
        print(json.dumps(line), file=result_out, flush=True)
    w["kv"].destroy()
    ctx.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
