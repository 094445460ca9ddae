"""Agent-style sessions (shared prefixes, growing conversations) replayed in a closed loop against the scheduler:
requests served, output tokens per second, TTFT / ITL percentiles and how much of every prompt came out of the prefix cache.

    python examples/python/agent_replay.py --cpu                                  # the toy decoder in host memory
    python examples/python/agent_replay.py --model dense-8b --sessions 16 --prefix 2000 8000

Reference counterpart: crates/kern-run/examples/agentx_replay.rs.
"""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--cpu", action="store_true")
    ap.add_argument("--model", default=None)
    ap.add_argument("--sessions", type=int, default=6)
    ap.add_argument("--turns", type=int, default=3)
    ap.add_argument("--prefix", type=int, nargs=2, default=None)
    ap.add_argument("--suffix", type=int, nargs=2, default=None)
    ap.add_argument("--output", type=int, nargs=2, default=None)
    ap.add_argument("--chunk", type=int, default=None)
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args()
    from kern_b200.cli import make_runtime
    from kern_b200.engine import Engine
    from kern_b200.serve.scheduler import Scheduler
    from kern_b200.testing import agent_traffic as T

    small = a.cpu and a.model is None
    prefix = tuple(a.prefix or ((16, 28) if small else (2000, 8000)))
    suffix = tuple(a.suffix or ((2, 4) if small else (64, 512)))
    output = tuple(a.output or ((2, 4) if small else (16, 128)))
    worst = prefix[1] + a.turns * (suffix[1] + output[1]) + 8
    ns = argparse.Namespace(manifest=None, model=a.model or "toy", cpu=a.cpu, kernels=None, gpu=0,
                            capacity=(worst + 64) * a.sessions if a.cpu else None, weights=None, layers=None,
                            max_tokens=None if small else max(a.chunk or 2048, 256) + 64, max_seqs=None if small else 3 * a.sessions,
                            max_context=None if small else worst + 64, tokenizer=None)
    rt = make_runtime(ns)
    vocab = next(int(b["domain"]["max"]) + 1 for b in rt.doc["buffers"].values() if b.get("fill") == "token")
    sched = Scheduler(Engine(rt), chunk=a.chunk or (32 if small else 2048), max_seqs=None if small else a.sessions)
    work = T.generate(seed=a.seed, sessions=a.sessions, turns=a.turns, prefix=prefix, suffix=suffix, output=output, vocab=vocab, families=2)
    res = T.replay(sched, work, concurrent=min(a.sessions, 4 if small else a.sessions), deadline_s=600)
    res = {k: (round(v, 3) if isinstance(v, float) else v) for k, v in res.items()}
    print(json.dumps({"example": "agent_replay", "model": a.model or "toy", **res, "ok": res["unfinished"] == 0}))
    return 0 if res["unfinished"] == 0 else 1


if __name__ == "__main__":
    raise SystemExit(main())
