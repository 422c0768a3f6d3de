#!/usr/bin/env python
"""Benchmark of the attention hot path on B200.

Headline workload (one "step"): one decode step of the batched-decode configuration --
Llama-3-8B attention shape (32 query / 8 KV heads, head_dim 128), 64 concurrent sequences with
seeded context lengths ~U[512, 8192], paged fp16 KV in 16-token blocks, one new token per
sequence: KV append + split-KV attention + combine, for one attention layer.  The KV working set
(~1.1 GB per GPU) is far larger than L2, so no L2 flush is needed between steps.

  python bench.py --gpus N --steps K --warmup W            (N > 1: launched under torchrun)
  python bench.py --impl reference ...                     (CPU oracle on the host cores)

With N > 1 the workload is N instances of the 64-sequence set, dealt to the ranks greedy longest-first as one set of
64 * N sequences: every rank streams the KV bytes of the one-GPU workload (weak scaling, no collective on the data path); every timed region is bracketed
by a barrier + synchronize, the maximum over ranks is taken, and the median of several such regions is reported.
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

NCU_DECODE_TRAFFIC_RATIO = 1005.96 / 997.376  # ncu DRAM traffic / algorithmic bytes of the decode + combine launch
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
        sm, mx, pw, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
                pw.append(float(f[2]))
            except ValueError:
                continue
            for n, val in zip(names, f[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w": statistics.median(pw) if pw else None, "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------------------------
# workloads
# ------------------------------------------------------------------------------------------------
def setup_decode(ctx, cfg, rank, world, device):
    """This rank's share of the set of `cfg.batch * world` sequences -- `world` instances of the seeded 64-sequence
    workload dealt greedy longest-first on context length: every rank gets one sequence of each length, i.e. the KV
    bytes of the one-GPU workload; paged pools filled (through the append kernel) with this rank's own seeded N(0,1)
    K/V in its own page order; returns everything a decode step needs."""
    import torch

    import hippo_leap_b200 as hl
    from hippo_leap_b200 import synth

    all_ctx, owners = synth.gen_sharded_ctx_lens(cfg, world)
    ctx_lens = all_ctx[owners[rank]]
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
                max_ctx=int(ctx_lens.max()), total_sequences=int(len(all_ctx)))


def cpu_decode_sample(cfg, n_seq, steps, n_threads):
    """The CPU oracle on the first n_seq sequences of the same seeded workload: `steps` decode steps.
    Returns seconds per step."""
    import oracle
    from hippo_leap_b200 import synth  # workload shapes and seeds only: nothing here loads the CUDA library

    ctx_lens = synth.gen_ctx_lens(cfg, rank=0)[:n_seq]
    theta = oracle.theta_table(cfg.head_dim, cfg.rope_base)
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
    try:    # this arm is the CPU oracle alone: the CUDA library must not even be mapped into the process
        cuda_lib_mapped = any("libhl_b200" in ln for ln in open("/proc/self/maps"))
    except OSError:
        cuda_lib_mapped = None
    config = workload_config(cfg, args.gpus)
    config["sequences_timed_per_step"] = n_seq   # the CPU arm times a bounded sample of the 64 sequences per step
    config["sample"] = sample
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * t / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config,
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": n_threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "cuda_library_mapped": cuda_lib_mapped,
    }
    print(json.dumps(line), file=result_out, flush=True)


def workload_config(cfg, n_gpus):
    return {"workload": "config 4: batched decode attention, Llama-3-8B shape, one layer",
            "n_head": cfg.n_head, "n_head_kv": cfg.n_head_kv, "head_dim": cfg.head_dim,
            "sequences_per_gpu": cfg.batch, "ctx_range": list(cfg.ctx_range), "kv": "paged fp16",
            "block_tokens": cfg.block_tokens,
            "sharding": f"{n_gpus} instance(s) of the seeded 64-sequence set = {cfg.batch * n_gpus} sequences, dealt to {n_gpus} "
                        "GPU(s) greedy longest-first (every GPU carries the KV bytes of the one-GPU workload), no collective",
            "l2": "KV working set ~1.1 GB per GPU >> 126 MB L2 (no flush needed)"}


def timed_loop(torch, fn, steps):
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1)  # ms


# DRAM bytes per launch of the prefill kernels from ncu captures (dram__bytes_read.sum + dram__bytes_write.sum; the
# summaries under profiles/ give the commands).  None: not captured for that configuration.
PREFILL_NCU_TRAFFIC = {3: 170.6e6 + 42.7e6, 5: 3770.3e6 + 514.8e6}


def median_ms(torch, fn, n, min_sample_ms=2.0):
    """Median over n samples of the device time per call (CUDA events on the current stream).  A sample is a run of
    back-to-back calls long enough (>= min_sample_ms) that the host's launch latency hides behind the kernels: timed
    one by one with a synchronise in between, a 50 us kernel reads 20 us too long."""
    est = timed_loop(torch, fn, 1)
    k = max(1, int(np.ceil(min_sample_ms / max(est, 1e-3))))
    return statistics.median(timed_loop(torch, fn, k) / k for _ in range(n))


def cpu_prefill_rows(cfg, theta, q, k, v, qw, kw, n_rows, n_threads):
    """The CPU oracle on a seeded sample of (token, head) rows of one prefill: returns (seconds for the rows,
    seconds to norm / rotate / append all K and V, rows, their outputs).  Positions are uniform over the prompt, so
    the mean row attends about half the prompt and the measured rate extrapolates to the whole causal problem."""
    import oracle

    S = q.shape[0]
    g = np.random.Generator(np.random.PCG64([cfg.seed, 4242]))
    rows = np.stack([g.integers(0, S, n_rows), g.integers(0, cfg.n_head, n_rows)], axis=1).astype(np.int32)
    cache = oracle.SeqCache(S, cfg.n_head_kv, cfg.head_dim)
    t0 = time.perf_counter()
    oracle.attn_forward(q, k, v, cache, theta=theta, rope_mode=oracle.ROPE_SPLIT_HALF, q_norm_w=qw, k_norm_w=kw,
                        eps=cfg.rms_eps, rows=rows[:1], n_threads=n_threads)
    t_append = time.perf_counter() - t0
    cache.cur_len = 0
    t0 = time.perf_counter()
    out = oracle.attn_forward(q, k, v, cache, theta=theta, rope_mode=oracle.ROPE_SPLIT_HALF, q_norm_w=qw, k_norm_w=kw,
                              eps=cfg.rms_eps, rows=rows, n_threads=n_threads)
    return max(time.perf_counter() - t0 - t_append, 1e-9), t_append, rows, out


def extras_single_gpu(ctx, torch, device, peaks, quick, configs=(2, 3, 5), cpu=True):
    """Prefill TFLOP/s on the prefill configurations (one layer each): device-resident inputs (the kernel's
    roofline), end to end through hl_b200_prefill_host (pinned float32 host Q/K/V in, host output back, every call),
    and the CPU oracle on a row sample of the same problem beside it."""
    import hippo_leap_b200 as hl
    from hippo_leap_b200 import synth

    res = {}
    n_threads = os.cpu_count() or 1
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
        q32 = torch.randn((S, cfg.n_head, cfg.head_dim), generator=gen, device=device)
        k32 = torch.randn((S, cfg.n_head_kv, cfg.head_dim), generator=gen, device=device)
        v32 = torch.randn((S, cfg.n_head_kv, cfg.head_dim), generator=gen, device=device)
        if cfg.bf16_range:    # values a bf16 model would produce, still handed over as float32
            q32, k32, v32 = (x.bfloat16().float() for x in (q32, k32, v32))
        if cfg.fp16_inputs:   # activations arrive as fp16
            q, k, v = (x.half() for x in (q32, k32, v32))
            q32, k32, v32 = (x.float() for x in (q, k, v))   # the same values widened, for the host-buffer and CPU legs
        else:
            q, k, v = q32, k32, v32
        out = torch.empty((S, cfg.n_head, cfg.head_dim), dtype=torch.float16, device=device)
        ctx.kv_append_seq(kv, 0, shape, k, v, 0, table)
        n = 3 if quick else 7
        for _ in range(3):
            ctx.attn_prefill(kv, 0, shape, q, 0, table, out)
        # Two regimes.  "burst": a few calls after an idle second, SM clocks at their maximum (a kernel timed alone; compare
        # with the burst GEMM peak).  "sustained": ~0.5 s of back-to-back calls, where the 1 kW power cap has pulled the
        # clocks down (a kernel inside a long step; compare with the sustained GEMM peak).  Short prompts never reach it.
        run = lambda: ctx.attn_prefill(kv, 0, shape, q, 0, table, out)  # noqa: E731
        torch.cuda.synchronize()
        time.sleep(1.0)
        run()
        ms = median_ms(torch, run, 3)
        sampler = ClockSampler(device.index or 0)
        sampler.start()
        k_sus = 8 if quick else max(8, int(500.0 / ms))  # (the quick form is the small profiling target: few launches)
        timed_loop(torch, run, k_sus // 2)                      # bring the power governor to its steady state
        ms_sus = timed_loop(torch, run, k_sus // 2) / (k_sus // 2)
        clocks = sampler.stop()
        ms_app = median_ms(torch, lambda: ctx.kv_append_seq(kv, 0, shape, k, v, 0, table), n)
        fl = synth.prefill_flops(cfg.n_head, cfg.head_dim, S)
        tf = fl / (ms * 1e-3) / 1e12
        entry = {
            "workload": f"{cfg.name}: causal prefill of {S} tokens, one layer, "
                        f"{'fp16' if cfg.fp16_inputs else 'float32'} Q/K/V in, fp16 out", "ms_attn": ms, "ms_kv_append": ms_app,
            "tflops": tf, "frac_of_tensor_peak": tf / peaks["tflops"], "peak_tflops": peaks["tflops"],
            "regime": "burst (first calls after an idle second, clocks at maximum) against the burst GEMM peak",
            "sustained": {"ms_attn": ms_sus, "tflops": fl / (ms_sus * 1e-3) / 1e12,
                          "frac_of_sustained_tensor_peak": fl / (ms_sus * 1e-3) / 1e12 / peaks["tflops_sustained"],
                          "peak_tflops_sustained": peaks["tflops_sustained"], "calls": k_sus // 2, "clocks": clocks,
                          "regime": "0.5 s of back-to-back calls (power-capped clocks) against the sustained GEMM peak"},
            "peak_src": peaks["src"], "flops": fl,
            "roofline": {"bound": "tensor", "achieved": tf, "peak": peaks["tflops"], "unit": "TFLOP/s",
                         "frac": tf / peaks["tflops"], "traffic": PREFILL_NCU_TRAFFIC.get(ci)}}
        del q, k, v, out
        # end to end: page-locked float32 host buffers in and out through the host-buffer entry point, every call
        if not quick:
            q_h, k_h, v_h = (x.cpu().pin_memory() for x in (q32, k32, v32))
            out_h = torch.empty_like(q_h).pin_memory()
            for _ in range(2):
                ctx.prefill_host(kv, 0, shape, q_h, k_h, v_h, 0, table, out_h)
            walls = []
            for _ in range(5):
                t0 = time.perf_counter()
                ctx.prefill_host(kv, 0, shape, q_h, k_h, v_h, 0, table, out_h)   # synchronises before it returns
                walls.append(time.perf_counter() - t0)
            w = statistics.median(walls)
            entry["e2e"] = {"value": fl / w / 1e12, "unit": "TFLOP/s", "ms": w * 1e3, "tok_per_s": S / w,
                            "h2d_bytes_per_step": (q_h.numel() + k_h.numel() + v_h.numel()) * 4,
                            "d2h_bytes_per_step": out_h.numel() * 4,
                            "call": "hl_b200_prefill_host (float32 host Q/K/V in, KV append + attention, float32 host out)"}
            if cpu:
                n_rows = {2: 4096, 3: 1024, 5: 256}.get(ci, 256)
                qn, kn, vn = (x.numpy() for x in (q_h, k_h, v_h))
                wn = (None if qw is None else qw.cpu().numpy(), None if kw is None else kw.cpu().numpy())
                t_rows, t_append, rows, want = cpu_prefill_rows(cfg, cfg.theta(), qn, kn, vn, wn[0], wn[1], n_rows,
                                                                n_threads)
                pairs = float((rows[:, 0].astype(np.int64) + 1).sum())
                row_flops = 4.0 * cfg.head_dim * pairs
                full_s = t_append + fl / (row_flops / t_rows)
                entry["cpu_baseline"] = {
                    "value": row_flops / t_rows / 1e12, "unit": "TFLOP/s", "cores": n_threads, "kind": "port",
                    "rows_per_s": n_rows / t_rows,
                    "sample": f"{n_rows} seeded (token, head) rows of the same {S}-token problem (positions uniform over the "
                              f"prompt, {int(pairs)} query-key pairs) in {t_rows:.2f} s on {n_threads} threads, after "
                              f"{t_append:.2f} s of norm / RoPE / append of all K, V",
                    "extrapolated_full_problem_s": full_s,
                    "extrapolation": "measured flop rate of the sampled rows applied to the whole causal problem "
                                     "(an estimate: the full CPU run was not made)"}
                # the rows double as a parity check of the benchmarked call
                got = out_h[torch.from_numpy(rows[:, 0]).long(), torch.from_numpy(rows[:, 1]).long()].numpy()
                entry["max_abs_vs_oracle_rows"] = float(np.abs(got - want).max())
            del q_h, k_h, v_h, out_h
        res[f"config{ci}_prefill"] = entry
        kv.destroy()
        del q32, k32, v32
        torch.cuda.empty_cache()
    return res


def extra_config1_full(ctx, torch, device):
    """Configuration 1 in full, driven like the reference's integration test (tests/integration_inference.nim:34-46):
    a 128-token causal prefill, then 32 decode steps, one attention layer (32 / 4 heads of 64, theta 1e4), float32
    ~N(0,1) from seed 0 -- on the GPU through the host-buffer entry points (host in, host out, one synchronisation per
    call) and on the CPU oracle, single-threaded (the reference's tensor ops are) and with all host threads."""
    import hippo_leap_b200 as hl
    import oracle
    from hippo_leap_b200 import synth

    cfg = synth.CONFIGS[1]
    S, T = cfg.prefill, cfg.decode_steps
    q, k, v = synth.gen_qkv(cfg, S + T)
    theta = oracle.theta_table(cfg.head_dim, cfg.rope_base)
    ctx.set_rope(theta)
    shape = hl.AttnShape(cfg.n_head, cfg.n_head_kv, cfg.head_dim, cfg.head_dim, hl.HL_ROPE_SPLIT_HALF, cfg.rms_eps)
    bt = 16
    nb = (S + T + bt - 1) // bt
    kv = ctx.kv_create(1, cfg.n_head_kv, cfg.head_dim, bt, nb)
    table = torch.arange(nb, dtype=torch.int32, device=device)
    tq, tk, tv = (torch.from_numpy(x).pin_memory() for x in (q, k, v))
    out = torch.empty_like(tq).pin_memory()
    ctx_len_steps = [torch.tensor([S + t + 1], dtype=torch.int32, device=device) for t in range(T)]

    def gpu_run():
        ctx.prefill_host(kv, 0, shape, tq[:S], tk[:S], tv[:S], 0, table, out[:S])
        for t in range(T):
            p = S + t
            ctx.decode_step_host(kv, 0, shape, tq[p:p + 1], tk[p:p + 1], tv[p:p + 1], ctx_len_steps[t], p + 1,
                                 table.view(1, -1), out[p:p + 1])

    for _ in range(2):
        gpu_run()
    walls = []
    for _ in range(5):
        t0 = time.perf_counter()
        gpu_run()
        walls.append(time.perf_counter() - t0)
    gpu_s = statistics.median(walls)

    def cpu_run(n_threads):
        cache = oracle.SeqCache(S + T, cfg.n_head_kv, cfg.head_dim)
        t0 = time.perf_counter()
        outs = [oracle.attn_forward(q[:S], k[:S], v[:S], cache, theta=theta, rope_mode=oracle.ROPE_SPLIT_HALF,
                                    n_threads=n_threads)]
        for t in range(S, S + T):
            outs.append(oracle.attn_forward(q[t:t + 1], k[t:t + 1], v[t:t + 1], cache, theta=theta,
                                            rope_mode=oracle.ROPE_SPLIT_HALF, n_threads=n_threads))
        return time.perf_counter() - t0, np.concatenate(outs)

    cpu1_s, want = cpu_run(1)
    n_threads = os.cpu_count() or 1
    cpun_s, _ = cpu_run(n_threads)
    kv.destroy()
    return {"workload": "config 1 in full: TinyLlama-1.1B single-layer attention, 128-token causal prefill + 32 decode steps, "
                        "float32 host buffers in and out of every call",
            "gpu_ms": gpu_s * 1e3, "gpu_tok_per_s": (S + T) / gpu_s, "gpu_calls": 1 + T,
            "cpu_baseline": {"value": (S + T) / cpu1_s, "unit": "tok/s", "cores": 1, "kind": "port",
                             "sample": f"the whole configuration, {cpu1_s * 1e3:.1f} ms", "ms": cpu1_s * 1e3,
                             "all_threads": {"cores": n_threads, "ms": cpun_s * 1e3, "tok_per_s": (S + T) / cpun_s}},
            "max_abs_vs_oracle": float(np.abs(out.numpy() - want).max())}


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


def extra_head_sharded_decode(ctx, torch, dist, device, rank, world, peaks):
    """Configuration 4 with KV heads split across ranks: every rank holds its Hkv/N heads of ALL 64 sequences' pages,
    runs the decode step on its n_head/N query heads, and the head-major rows are gathered -- once with one NCCL
    all-gather after the kernels, once by the kernels' own stores to every peer (symmetric memory).  Strong scaling:
    the 64 sequences are fixed, each rank streams 1/N of the KV bytes."""
    import hippo_leap_b200 as hl
    from hippo_leap_b200 import sharding, synth

    cfg = synth.CONFIGS[4]
    sh = sharding.head_shard(rank, world, cfg.n_head, cfg.n_head_kv)
    ctx_lens = synth.gen_ctx_lens(cfg)                       # the same 64 sequences and page tables on every rank
    tables, num_blocks = synth.gen_block_tables(ctx_lens, cfg.block_tokens, cfg.seed)
    shape = hl.AttnShape(sh.n_head, sh.n_head_kv, cfg.head_dim, cfg.head_dim, hl.HL_ROPE_SPLIT_HALF, cfg.rms_eps)
    ctx.set_rope(cfg.theta())
    kv = ctx.kv_create(1, sh.n_head_kv, cfg.head_dim, cfg.block_tokens, num_blocks)
    ttab = torch.from_numpy(tables).to(device)
    tctx = torch.from_numpy(ctx_lens).to(device)
    B = len(ctx_lens)
    gen = torch.Generator(device=device)
    gen.manual_seed(4000)                                     # the SAME full-width tensors on every rank, sliced by head
    check_seqs = [int(i) for i in np.argsort(ctx_lens)[:2]]  # the two shortest: checked against the CPU oracle below
    kept = {}
    for i, c in enumerate(ctx_lens):
        k_all = torch.randn((int(c), cfg.n_head_kv, cfg.head_dim), generator=gen, device=device)
        v_all = torch.randn((int(c), cfg.n_head_kv, cfg.head_dim), generator=gen, device=device)
        if rank == 0 and i in check_seqs:
            kept[i] = (k_all.cpu().numpy(), v_all.cpu().numpy())
        nb = (int(c) + cfg.block_tokens - 1) // cfg.block_tokens
        ctx.kv_append_seq(kv, 0, shape, k_all[:, sh.kv_lo:sh.kv_hi], v_all[:, sh.kv_lo:sh.kv_hi], 0,
                          ttab[i, :nb].contiguous())
    q_full = torch.randn((B, cfg.n_head, cfg.head_dim), generator=gen, device=device)
    kn_full = torch.randn((B, cfg.n_head_kv, cfg.head_dim), generator=gen, device=device)
    vn_full = torch.randn((B, cfg.n_head_kv, cfg.head_dim), generator=gen, device=device)
    q, kn, vn = q_full[:, sh.q_lo:sh.q_hi], kn_full[:, sh.kv_lo:sh.kv_hi], vn_full[:, sh.kv_lo:sh.kv_hi]
    max_ctx = int(ctx_lens.max())
    plain = sharding.HeadShardedDecode(ctx, kv, shape, B, device, world)
    fused = sharding.FusedHeadShardedDecode(ctx, kv, shape, B, cfg.n_head, device)
    results = {}
    n = 50
    for name, runner in (("fused_in_kernel", fused), ("nccl_allgather_after", plain)):
        for _ in range(5):
            runner.run(q, kn, vn, tctx, max_ctx, ttab)
        vals = []
        for _ in range(5):
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            vals.append(sharding.max_over_ranks(timed_loop(torch, lambda: runner.run(q, kn, vn, tctx, max_ctx, ttab), n) / n,
                                                device))
        results[name] = statistics.median(vals)
    a_ = fused.run(q, kn, vn, tctx, max_ctx, ttab).clone()
    b_ = plain.run(q, kn, vn, tctx, max_ctx, ttab).clone()
    torch.cuda.synchronize()
    same = bool(torch.equal(a_, b_))
    # the GATHERED tensor against the CPU oracle's unsharded step, all heads of the two shortest sequences (rank 0)
    max_abs = None
    if rank == 0:
        import oracle
        theta = cfg.theta()
        max_abs = 0.0
        for i, (kk, vv) in kept.items():
            kk, vv = kk.copy(), vv.copy()
            kk[-1], vv[-1] = kn_full[i].cpu().numpy(), vn_full[i].cpu().numpy()   # the step's own new token
            sc = oracle.SeqCache(kk.shape[0], cfg.n_head_kv, cfg.head_dim)
            if kk.shape[0] > 1:
                oracle.attn_forward(np.zeros((kk.shape[0] - 1, cfg.n_head, cfg.head_dim), np.float32), kk[:-1], vv[:-1], sc,
                                    theta=theta, rope_mode=oracle.ROPE_SPLIT_HALF, rows=[[0, 0]])
            want = oracle.attn_forward(q_full[i:i + 1].cpu().numpy(), kk[-1:], vv[-1:], sc, theta=theta,
                                       rope_mode=oracle.ROPE_SPLIT_HALF)[0]
            max_abs = max(max_abs, float(np.abs(a_[:, i].cpu().numpy() - want).max()))
    ms = min(results.values())
    alg = synth.decode_bytes(ctx_lens, cfg.n_head, cfg.n_head_kv, cfg.head_dim)
    kv.destroy()
    return {"workload": f"config 4, KV heads {sh.n_head_kv}/GPU: 64 sequences, one decode step (append + split-KV attention + "
                        "gather of head outputs to every GPU), float32 rows",
            "ms_nccl_allgather_after": results["nccl_allgather_after"], "ms_fused_in_kernel": results["fused_in_kernel"],
            "fused_equals_allgather": same, "max_abs_vs_oracle_two_sequences": max_abs, "ms": ms,
            "tok_per_s": B / (ms * 1e-3),
            "aggregate_kv_gbs": alg / (ms * 1e-3) / 1e9, "frac_of_hbm_peak_per_gpu": alg / world / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
            "gathered_bytes_per_gpu": int(B * cfg.n_head * cfg.head_dim * 4), "scaling": "strong"}


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
                    help="measure only the head-sharded config 5 prefill and config 4 decode (+ gather) at N GPUs")
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
    from hippo_leap_b200 import sharding, synth

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
        res = {"config5_head_sharded_prefill": extra_head_sharded_prefill(ctx, torch, dist, device, rank, world, peaks),
               "config4_head_sharded_decode": extra_head_sharded_decode(ctx, torch, dist, device, rank, world, peaks)}
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
    w = setup_decode(ctx, cfg, rank, world, device)
    B = len(w["ctx_lens"])            # this rank's sequences
    B_total = w["total_sequences"]    # all ranks': cfg.batch * world
    REPEATS = 5                       # every figure below is the median of this many K-step regions

    def region(fn, steps):
        """One timed region: barrier + synchronize on both sides, K steps, CUDA events, max over ranks."""
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        ms = timed_loop(torch, fn, steps)   # ends with a synchronize
        if world > 1:
            dist.barrier()
        return sharding.max_over_ranks(ms, device)

    def step():
        ctx.kv_append_batch(w["kv"], 0, w["shape"], w["kn"], w["vn"], w["tctx"], w["ttab"])
        ctx.attn_decode(w["kv"], 0, w["shape"], w["q"], w["tctx"], w["max_ctx"], w["ttab"], w["out"])

    for _ in range(args.warmup):
        step()
    sampler = ClockSampler(local_rank)
    sampler.start()
    l0 = ctx.launch_count()
    region_ms = [region(step, args.steps) for _ in range(REPEATS)]
    launches = (ctx.launch_count() - l0) // REPEATS
    ms_total = statistics.median(region_ms)
    value = B_total * args.steps / (ms_total * 1e-3)

    # roofline of the dominant kernel pair (split-KV decode + combine), timed alone on every rank; the line reports
    # the SLOWEST rank's launch (the one that bounds the step) and lists all ranks
    def attn_only():
        ctx.attn_decode(w["kv"], 0, w["shape"], w["q"], w["tctx"], w["max_ctx"], w["ttab"], w["out"])

    for _ in range(3):
        attn_only()
    ms_attn = statistics.median(timed_loop(torch, attn_only, args.steps) / args.steps for _ in range(REPEATS))
    alg_bytes = synth.decode_bytes(w["ctx_lens"], cfg.n_head, cfg.n_head_kv, cfg.head_dim)
    mine = torch.tensor([alg_bytes, ms_attn, float(B)], device=device, dtype=torch.float64)
    per = [mine.clone() for _ in range(world)]
    if world > 1:
        dist.all_gather(per, mine)
    per_rank = [{"rank": r, "sequences": int(x[2].item()), "algorithmic_bytes_per_launch": float(x[0].item()),
                 "ms_per_launch": float(x[1].item()), "gbs": float(x[0].item() / (x[1].item() * 1e-3) / 1e9)}
                for r, x in enumerate(per)]
    slow = max(per_rank, key=lambda e: e["ms_per_launch"])
    achieved = slow["gbs"]
    # ncu (the decode summary under profiles/): 1006.0 MB of DRAM traffic per launch for the 997.4 MB one-GPU workload,
    # i.e. 1.0086 x the algorithmic bytes; a rank's share of a larger set scales with its algorithmic bytes
    roofline = {"bound": "hbm", "kernel": "attn_decode_kernel<128,4,3> + attn_combine_kernel<128>",
                "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                "peak_src": peaks["src"], "traffic": NCU_DECODE_TRAFFIC_RATIO * slow["algorithmic_bytes_per_launch"],
                "traffic_src": "ncu dram__bytes_read.sum + dram__bytes_write.sum of the one-GPU workload, scaled by "
                               "algorithmic bytes",
                "algorithmic_bytes_per_launch": slow["algorithmic_bytes_per_launch"],
                "ms_per_launch": slow["ms_per_launch"], "rank": slow["rank"], "per_rank": per_rank}

    # end to end through the host-buffer C ABI call: pinned host inputs, host result, every step
    q_h, k_h, v_h = (x.cpu().pin_memory() for x in (w["q"], w["kn"], w["vn"]))
    out_h = torch.empty_like(q_h).pin_memory()

    # the C call itself, arguments marshalled once (a serving loop refills the same pinned buffers every step)
    step_host = ctx.decode_step_host_call(w["kv"], 0, w["shape"], q_h, k_h, v_h, w["tctx"], w["max_ctx"], w["ttab"], out_h)

    for _ in range(3):
        step_host()
    e2e_ms = [region(step_host, args.steps) for _ in range(REPEATS)]
    ms_e2e = statistics.median(e2e_ms)
    e2e_value = B_total * args.steps / (ms_e2e * 1e-3)
    io = torch.tensor([q_h.numel() * 4 + k_h.numel() * 4 + v_h.numel() * 4, out_h.numel() * 4], device=device,
                      dtype=torch.float64)
    if world > 1:
        dist.all_reduce(io)               # whole-job bytes per step: the sum over ranks
    h2d, d2h = int(io[0].item()), int(io[1].item())
    clocks = sampler.stop()  # sampled across the timed loops above (device, kernel-only, end-to-end)
    code, detail = ctx.device_status()
    if code != 0:
        raise SystemExit(f"device status {code} (detail {detail}) after the timed region")

    extra = {}
    if not args.no_extras:
        if world == 1:
            extra.update(extras_single_gpu(ctx, torch, device, peaks, quick=False, cpu=not args.no_cpu))
            extra["config1_full"] = extra_config1_full(ctx, torch, device)
            extra["config2_backend_pipeline"] = extra_config2_pipeline(torch, local_rank)
            extra["linear_f16"] = extra_linear(ctx, torch, device, peaks)
            extra["dense_llama32_1b"] = extra_dense_model(torch, local_rank)
        if cfg.n_head_kv % world == 0:
            # side measurements after the headline: a failure here (it would be the same on every rank: a missing
            # symmetric-memory feature, an allocation) is recorded and must not cost the line above
            for name, fn in (("config5_head_sharded_prefill", extra_head_sharded_prefill),
                             ("config4_head_sharded_decode", extra_head_sharded_decode)):
                try:
                    extra[name] = fn(ctx, torch, dist, device, rank, world, peaks)
                except Exception as e:  # noqa: BLE001
                    extra[name] = {"error": f"{type(e).__name__}: {e}"[:300]}

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
            "warmup": args.warmup, "ms_per_step": ms_total / args.steps, "repeats": REPEATS,
            "ms_per_step_each_repeat": [m / args.steps for m in region_ms], "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16 KV, f32 accumulate", "data": "synthetic",
            "config": workload_config(cfg, world),
            "hbm_gbs": achieved,
            # tok/s counts sequences, the work is KV bytes: the whole job's algorithmic bytes per second
            "kv_gbs_aggregate": sum(e["algorithmic_bytes_per_launch"] for e in per_rank) / (ms_total / args.steps * 1e-3) / 1e9,
            "roofline": roofline, "cpu_baseline": cpu_baseline,
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": ms_e2e / args.steps, "ms_per_step_each_repeat": [m / args.steps for m in e2e_ms],
                    "call": "hl_b200_decode_step_host (pinned float32 host q / k / v in, host out, every step)"},
            "gpu_launches": int(launches), "clocks": clocks, "extra": extra,
        }
        print(json.dumps(line), file=result_out, flush=True)
    w["kv"].destroy()
    ctx.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
