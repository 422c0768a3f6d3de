"""`hippo_leap bench` for the B200 attention backend: same runs / warm-up / table / statistics as the
reference's structured benchmark command (src/hippo_leap/cmd_bench.nim:93-136), on the attention-only
stand-in model or (``--model dense``) a dense llama / qwen3 layer stack with seeded fp16 weights (there is no
GGUF model or tokenizer on this path, so the prompt is seeded token ids).

    python -m hippo_leap_b200.cmd_bench --config 2 --prompt-tokens 2048 --tokens 128 --runs 5 --warmup 3
    python -m hippo_leap_b200.cmd_bench --model dense --config 2 --layers 4 --emb 2048 --ffn 8192 --vocab 32000
"""
from __future__ import annotations

import argparse
import math

import numpy as np

from . import backend as B
from . import synth

USAGE_DEFAULTS = dict(tokens=128, context=2048, runs=5, warmup=3)


def stats_line(label: str, data) -> str:
    """mean +- population standard deviation, min, max -- cmd_bench.nim:118-133."""
    if not data:
        return ""
    mean = sum(data) / len(data)
    std = math.sqrt(sum((v - mean) ** 2 for v in data) / len(data))
    return f"{label}: {mean:.2f} ± {std:.2f} tok/s  (min {min(data):.1f}, max {max(data):.1f})"


def run_table(generate, a, context) -> None:
    """Warm-up runs, the per-run table and the two statistics lines (cmd_bench.nim:93-136)."""
    for w in range(a.warmup):
        print(f"Warmup {w + 1}/{a.warmup}...")
        generate()
    print()
    print(" Run  Tokens  Time(ms)   tok/s   GPU(ms)  gpu tok/s")
    toks, gpu_toks = [], []
    for r in range(a.runs):
        res = generate()
        tps = res.completionTokens / (res.elapsedMs / 1e3) if res.elapsedMs > 0 else 0.0
        dec = res.completionTokens - 1
        gtps = dec / (res.gpuMs / 1e3) if res.gpuMs > 0 and dec > 0 else 0.0
        toks.append(tps)
        gpu_toks.append(gtps)
        print(f"{r + 1:>4}  {res.completionTokens:>6}  {res.elapsedMs:>9.1f}  {tps:>6.1f}  {res.gpuMs:>8.1f}  {gtps:>9.1f}")
    print()
    print(stats_line("Wall", toks))
    print(stats_line("GPU ", gpu_toks))


def main_dense(a) -> int:
    from . import dense as D

    cfg = synth.CONFIGS[a.config]
    hp = D.DenseHParams(nVocab=a.vocab, nEmb=a.emb, nLayer=a.layers or cfg.layers, nFfn=a.ffn, nHead=cfg.n_head,
                        nHeadKv=cfg.n_head_kv, headDim=cfg.head_dim, ropeFreqBase=cfg.rope_base, rmsEps=cfg.rms_eps,
                        llama3Scaling=cfg.llama3_scaling)
    context = max(a.context, a.prompt_tokens + a.tokens)
    print("Loading model...")
    m = D.random_dense_model(hp, cfg.seed, cfg.qk_norm)
    cache = D.initKvCache(hp, context, a.device)
    D.loadModelBackend(m, hp, a.device)
    try:
        prompt = np.random.Generator(np.random.PCG64([cfg.seed, 1])).integers(0, hp.nVocab, a.prompt_tokens).tolist()
        print(f"Model: dense layer stack, seeded fp16 weights, {cfg.name} attention shape, {hp.nLayer} layers, "
              f"n_emb {hp.nEmb}, n_ffn {hp.nFfn}, vocabulary {hp.nVocab}")
        print(f"Prompt: {a.prompt_tokens} seeded token ids")
        print(f"Max tokens: {a.tokens}")
        print(f"Context: {context}")
        print(f"Runs: {a.runs} ({a.warmup} warmup)")
        print()
        run_table(lambda: B.generate(m, cache, prompt, a.tokens, context, procs=D), a, context)
    finally:
        D.freeKvCache(cache)
        D.unloadModelBackend()
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="hippo_leap bench (b200 attention backend)")
    ap.add_argument("--config", type=int, default=2, choices=[1, 2, 3], help="attention shape of benchmark config 1-3")
    ap.add_argument("--layers", type=int, default=0, help="override the layer count of the config")
    ap.add_argument("--prompt-tokens", "-p", type=int, default=128)
    ap.add_argument("--tokens", "-n", type=int, default=USAGE_DEFAULTS["tokens"])
    ap.add_argument("--context", type=int, default=USAGE_DEFAULTS["context"])
    ap.add_argument("--runs", "-r", type=int, default=USAGE_DEFAULTS["runs"])
    ap.add_argument("--warmup", type=int, default=USAGE_DEFAULTS["warmup"])
    ap.add_argument("--device", type=int, default=0)
    ap.add_argument("--model", default="standin", choices=["standin", "dense"])
    ap.add_argument("--emb", type=int, default=2048, help="dense model: embedding width")
    ap.add_argument("--ffn", type=int, default=8192, help="dense model: FFN width")
    ap.add_argument("--vocab", type=int, default=32000, help="dense model: vocabulary size")
    a = ap.parse_args(argv)
    if a.model == "dense":
        return main_dense(a)

    cfg = synth.CONFIGS[a.config]
    hp = B.HParams(nVocab=512, nLayer=a.layers or cfg.layers, nHead=cfg.n_head, nHeadKv=cfg.n_head_kv,
                   headDim=cfg.head_dim, ropeFreqBase=cfg.rope_base, rmsEps=cfg.rms_eps,
                   llama3Scaling=cfg.llama3_scaling)
    context = max(a.context, a.prompt_tokens + a.tokens)
    print("Loading model...")
    m = B.standin_model(hp, cfg.seed, cfg.qk_norm)
    cache = B.initKvCache(hp, context, a.device)
    B.loadModelBackend(m, hp, a.device)
    try:
        prompt = np.random.Generator(np.random.PCG64([cfg.seed, 1])).integers(0, hp.nVocab, a.prompt_tokens).tolist()
        print(f"Model: attention-only stand-in, {cfg.name} shape, {hp.nLayer} layers")
        print(f"Prompt: {a.prompt_tokens} seeded token ids")
        print(f"Max tokens: {a.tokens}")
        print(f"Context: {context}")
        print(f"Runs: {a.runs} ({a.warmup} warmup)")
        print()
        run_table(lambda: B.generate(m, cache, prompt, a.tokens, context), a, context)
    finally:
        B.freeKvCache(cache)
        B.unloadModelBackend()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
