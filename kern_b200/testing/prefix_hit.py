"""Time to first token of a long prompt, cold and again after its pages are in the prefix cache.

    python -m kern_b200.testing.prefix_hit --model dense-8b --tokens 13983

Prints one JSON line: cold and repeat time to first token (wall clock around the scheduler steps, device synchronised),
tokens taken from the cache, and the chunk size used. Reference counterpart: docs/serve.md:213-216 (a 13 983-token prompt,
888 ms cold, 27 ms after the hit).
"""
from __future__ import annotations

import argparse
import json
import time

import numpy as np


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="dense-8b")
    ap.add_argument("--tokens", type=int, default=13983)
    ap.add_argument("--chunk", type=int, default=2048)
    ap.add_argument("--cpu", action="store_true")
    a = ap.parse_args(argv)
    import torch

    from ..cli import make_runtime
    from ..engine import Engine
    from ..serve.scheduler import Request, Scheduler

    ns = argparse.Namespace(manifest=None, model=a.model, cpu=a.cpu, kernels=None, gpu=0, capacity=2 * a.tokens + 4096, weights=None,
                            layers=None, max_tokens=max(a.chunk, 2048), max_seqs=None, max_context=a.tokens + 64, tokenizer=None)
    rt = make_runtime(ns)
    sched = Scheduler(Engine(rt), chunk=a.chunk)
    rng = np.random.default_rng(0)
    vocab = next(int(b["domain"]["max"]) + 1 for b in rt.doc["buffers"].values() if b.get("fill") == "token")
    prompt = rng.integers(1, vocab, a.tokens).tolist()
    sync = (lambda: None) if a.cpu else torch.cuda.synchronize

    def ttft(req):
        sync()
        t0 = time.perf_counter()
        sched.submit(req)
        while req.first_token_at is None and req.finished is None:
            sched.step()
        sync()
        dt = time.perf_counter() - t0
        sched.run_until_idle(1000)
        return dt

    warm = Request(id="w", prompt=rng.integers(1, vocab, min(a.tokens, 3 * a.chunk)).tolist(), max_tokens=2)
    ttft(warm)                                   # graphs, tensor maps, allocator
    # a turn boundary one page before the end: where a model with per-sequence state snapshots it
    page = rt.page_unit
    hist = max(page, (a.tokens - 2) // page * page)
    cold = Request(id="a", prompt=prompt, max_tokens=2, history_tokens=hist)
    t_cold = ttft(cold)
    again = Request(id="b", prompt=prompt, max_tokens=2, history_tokens=hist)
    t_hit = ttft(again)
    print(json.dumps({"model": a.model, "prompt_tokens": a.tokens, "chunk": a.chunk, "ttft_cold_ms": round(t_cold * 1e3, 1),
                      "ttft_repeat_ms": round(t_hit * 1e3, 1), "cached_tokens": again.cached,
                      "same_first_token": cold.out[:1] == again.out[:1]}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
