"""`bench.py --config c`: a hybrid Gated-DeltaNet + attention decoder under agent-style traffic, one GPU.

Sessions share long prefixes, every turn resends the conversation so far plus a new suffix (`testing/agent_traffic.py`),
the scheduler's prefix cache and its turn-boundary snapshots of the per-sequence state turn most of every later prompt
into a cache hit. The figure is output tokens per second of the closed loop, with requests served, TTFT / ITL percentiles
and the share of prompt tokens that came out of the cache.

This is the 27B-class hybrid of `models/hybrid.py` on ONE GPU without the draft model: config (c) of the benchmark names
tensor parallelism over eight GPUs and a one-layer draft, neither of which this decoder family has here, so the line says
`"same_config": false`. Reference: docs/vllm-rsi-example.md:233-239 (the metric set of its agent benchmark).
"""
from __future__ import annotations

import argparse
import json
import os
import time


def main(args) -> int:
    import torch

    from ..cli import make_runtime
    from ..engine import Engine
    from ..serve.scheduler import Scheduler
    from . import agent_traffic as T

    sessions = int(os.environ.get("KERN_B200_AGENT_SESSIONS", "16"))
    turns = int(os.environ.get("KERN_B200_AGENT_TURNS", "3"))
    prefix, suffix, output = (8192, 32768), (256, 2048), (64, 1024)
    worst = prefix[1] + turns * (suffix[1] + output[1]) + 64
    chunk = 2048
    ns = argparse.Namespace(manifest=None, model="hybrid-27b", cpu=False, kernels=None, gpu=0, capacity=None, weights=None,
                            layers=None if args.layers == 36 else args.layers, max_tokens=chunk + 64,
                            max_seqs=3 * min(sessions, 64),      # state slots: the live sequences and their turn-boundary snapshots
                            max_context=worst, tokenizer=None)
    rt = make_runtime(ns)
    sched = Scheduler(Engine(rt), chunk=chunk, max_seqs=min(sessions, 64))
    vocab = next(int(b["domain"]["max"]) + 1 for b in rt.doc["buffers"].values() if b.get("fill") == "token")
    # warm-up: graphs, tensor maps, allocator
    T.replay(sched, T.generate(seed=99, sessions=2, turns=1, prefix=(3000, 3000), suffix=(64, 64), output=(8, 8), vocab=vocab), deadline_s=300)
    torch.cuda.synchronize()
    work = T.generate(seed=args.seed, sessions=sessions, turns=turns, prefix=prefix, suffix=suffix, output=output, vocab=vocab)
    launches0 = rt.launches_total
    t0 = time.monotonic()
    res = T.replay(sched, work, concurrent=min(sessions, 64), deadline_s=1500)
    torch.cuda.synchronize()
    rt.check_error()
    wall = time.monotonic() - t0
    line = {
        "metric": "output tok/s of a closed loop of agent sessions; requests served; p50 TTFT & ITL", "value": round(res["output_tokens"] / wall, 1),
        "unit": "tok/s", "n_gpus": 1, "higher_is_better": True, "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic (uniform-random token ids, random-init bf16 weights)",
        "config": {"model": "hybrid GDN + attention decoder, 27B class (64 layers, 3 GDN : 1 GQA, hidden 5120)", "same_config": False,
                   "why": "config (c) names TP=8 and a one-layer draft model; this decoder family runs on one GPU without a draft here",
                   "sessions": sessions, "turns": turns, "prefix_tokens": list(prefix), "suffix_tokens": list(suffix),
                   "output_tokens": list(output), "families": 4, "chunk": chunk},
        "requests_served": res["requests_served"], "unfinished": res["unfinished"], "wall_s": round(wall, 2),
        "prompt_tokens": res["prompt_tokens"], "prefix_cache_share": round(res["prefix_cache_share"], 3),
        "ttft_ms_p50": res["ttft_ms_p50"] and round(res["ttft_ms_p50"], 1), "ttft_ms_p90": res["ttft_ms_p90"] and round(res["ttft_ms_p90"], 1),
        "itl_ms_p50": res["itl_ms_p50"] and round(res["itl_ms_p50"], 2), "itl_ms_p90": res["itl_ms_p90"] and round(res["itl_ms_p90"], 2),
        "gpu_launches": int(rt.launches_total - launches0),
    }
    print(json.dumps(line), flush=True)
    return 0
