"""Headline benchmark: output tokens/s of the serving engine at fixed concurrency, dense GQA 8B-class
decoder (36 layers, hidden 4096, 32 Q / 8 KV heads of 128, SwiGLU 12288, vocab 151936, bf16 random
init), 256 concurrent requests with prompts of 512-4096 uniform-random token ids and 256 greedy
output tokens each.

A step is one iteration of the engine in steady state at that concurrency: every one of the 256
sequences produces a token — one request has just finished and its replacement's whole prompt is
prefilled in the same call as the 255 decode rows (ragged batch through the manifest's `prefill`
program). Inputs of each step are written from pinned host memory and the step's tokens are read back
to the host, through the package's public API (kern_b200.Runtime + kern_b200.Engine).

    python bench.py --gpus 1 --steps 16 --warmup 3
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...

Prints one JSON line (rank 0). `--impl reference` reports why the reference cannot run here.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

PUBLISHED_TOK_S = None   # the reference publishes no B200 number for this config (BASELINE.json `published` is empty)


def clocks_sampler(gpu: int, stop: threading.Event, out: list):
    q = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
        "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
    while not stop.is_set():
        try:
            r = subprocess.run(["nvidia-smi", f"--id={gpu}", f"--query-gpu={q}", "--format=csv,noheader,nounits"],
                               capture_output=True, text=True, timeout=5)
            parts = [x.strip() for x in r.stdout.strip().split(",")]
            if len(parts) >= 6:
                out.append(parts)
        except Exception:
            pass
        stop.wait(0.2)


def summarize_clocks(samples):
    if not samples:
        return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
    mhz = sorted(int(s[0]) for s in samples if s[0].isdigit())
    reasons = set()
    for s in samples:
        for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), s[2:6]):
            if v.lower().startswith("active"):
                reasons.add(name)
    return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": int(samples[0][1]) if samples[0][1].isdigit() else None,
            "reasons": sorted(reasons)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=16)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--concurrency", type=int, default=256)
    ap.add_argument("--layers", type=int, default=36, help="for quick functional checks only; the headline is 36")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--parallelism", default="dp", choices=["tp", "dp"],
                    help="N > 1: data-parallel replicas, the concurrency split between them (default: the higher "
                         "tok/s per box for a model that fits one GPU), or tensor parallel over one replicated batch "
                         "(lower latency per token)")
    ap.add_argument("--tp-unfused", action="store_true",
                    help="tensor parallel without the GEMM + reduce-scatter fusion (the all-reduce kernel pushes the partials "
                         "instead of the GEMM epilogue; A/B)")
    ap.add_argument("--profile", action="store_true", help="after the timed region, run one more step with per-call timing and print the cost by op to stderr")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a Rust workspace (maturin wheel) and no Rust toolchain is installed; its kernels are "
                          "prebuilt sm_103a cubins fetched from Hugging Face, which this box cannot reach"}))
        return 0

    import numpy as np
    import torch

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    steps, warmup = args.steps, max(3, args.warmup)

    from kern_b200.engine import Engine
    from kern_b200.models import dense
    from kern_b200.runtime import Runtime

    tp = world > 1 and args.parallelism == "tp"
    # tensor parallel: every rank is fed the whole batch; data parallel: replicas split the concurrent requests
    conc = args.concurrency if tp else args.concurrency // world
    out_len, p_lo, p_hi = 256, 512, 4096
    cfg = dense.DenseConfig(name="dense-8b", layers=args.layers, max_seqs=max(conc, 8), max_tokens=p_hi + conc + 64,
                            max_context=p_hi + out_len + 64, page_size=64, tp=world if tp else 1)
    torch.cuda.set_device(local)
    if tp:
        from kern_b200.models import dense_tp
        from kern_b200.parallel import group

        doc = dense_tp.build_manifest_tp(cfg, fused=not args.tp_unfused)
        rt = Runtime(doc, gpu=local, memory_fraction=0.90, topology=group.topology(doc["topology"]["groups"], rank, world))
        dense.load_random_weights(rt, cfg, seed=args.seed)
        group.start(rt)
    else:
        rt = Runtime(dense.build_manifest(cfg), gpu=local, memory_fraction=0.92)
        dense.load_random_weights(rt, cfg, seed=args.seed)
        rt.once()
    eng = Engine(rt)
    rng = np.random.default_rng(args.seed + (0 if tp else rank))   # tensor-parallel ranks replay the same requests

    def new_prompt():
        return rng.integers(0, cfg.vocab, int(rng.integers(p_lo, p_hi + 1))).tolist()

    # ---- bring the engine to steady state: `conc` live sequences at staggered ages ----
    seqs, last = [], []
    t0 = time.perf_counter()
    prefill_tokens = 0
    pending = []
    start_ages = rng.permutation([(i * out_len) // conc for i in range(conc)])   # evenly spread: steady state
    for i in range(conc):
        p = new_prompt()
        s = eng.open(len(p) + out_len + 8)
        s.age = int(start_ages[i])                 # tokens it has produced so far in its life
        pending.append((s, p))
        if sum(len(q) for _, q in pending) + p_hi > cfg.max_tokens - conc or i == conc - 1:
            toks = eng.step(pending)
            prefill_tokens += sum(len(q) for _, q in pending)
            for (s2, _), t in zip(pending, toks):
                seqs.append(s2)
                last.append(t[0])
            pending = []
    rt.synchronize()
    prefill_s = time.perf_counter() - t0
    # advance every sequence by its age so contexts look like a running server's
    ages = [s.age for s in seqs]
    for k in range(max(ages) if ages else 0):
        live = [(s, [last[i]]) for i, s in enumerate(seqs) if k < ages[i]]
        if not live:
            break
        # (decode program; untimed)
        idx = [i for i, s in enumerate(seqs) if k < ages[i]]
        toks = eng.step(live, eager=True)     # every batch size once: not worth a graph each
        for i, t in zip(idx, toks):
            last[i] = t[0]
    rt.check_error()

    def one_step(timed=False):
        # requests that have produced all their tokens finish; new ones take their places and are prefilled in
        # the same call as everyone else's decode rows
        fresh, rows = {}, 0
        for j in range(conc):
            if seqs[j].age >= out_len:
                eng.close(seqs[j])
                p = new_prompt()
                s = eng.open(len(p) + out_len + 8)
                s.age = 0
                seqs[j] = s
                fresh[j] = p
                rows += len(p)
        batch = [(seqs[i], fresh.get(i) or [last[i]]) for i in range(conc)]
        toks = eng.step(batch, timed=timed)
        for i, t in enumerate(toks):
            last[i] = t[0]
            seqs[i].age += 1
        return rows

    for _ in range(warmup):
        one_step()
    rt.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()

    samples, stop = [], threading.Event()
    th = threading.Thread(target=clocks_sampler, args=(local, stop, samples), daemon=True)
    th.start()
    stream = torch.cuda.ExternalStream(rt.stream, device=local)
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    h2d0, d2h0, launches = eng.h2d_bytes, eng.d2h_bytes, 0
    prompt_rows = 0
    wall0 = time.perf_counter()
    evs[0].record(stream)
    for k in range(steps):
        prompt_rows += one_step()
        launches += eng.last_launches
        evs[k + 1].record(stream)
    rt.synchronize()
    torch.cuda.synchronize()
    wall = time.perf_counter() - wall0
    stop.set()
    th.join(timeout=2)
    if world > 1:
        dist.barrier()
    step_ms = [evs[k].elapsed_time(evs[k + 1]) for k in range(steps)]
    dev_s = sum(step_ms) / 1e3
    rt.check_error()
    if args.profile and rank == 0:
        rows = one_step(timed=True)
        by_op = {}
        for label, op, ms, n in eng.last_times:
            e = by_op.setdefault(op, [0.0, 0, 0])
            e[0] += ms; e[1] += n; e[2] += 1
        total = sum(v[0] for v in by_op.values())
        print(f"# cost by op of one step ({rows} prompt rows + {conc} decode rows), eager, total {total:.2f} ms", file=sys.stderr)
        for op, (ms, n, calls) in sorted(by_op.items(), key=lambda kv: -kv[1][0]):
            print(f"#   {op:14s} {ms:8.3f} ms  {100 * ms / total:5.1f}%  calls {calls:4d}  launches {n}", file=sys.stderr)

    if world > 1:
        t = torch.tensor([dev_s, wall], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dev_s, wall = float(t[0]), float(t[1])
    total_tokens = conc * (1 if tp else world) * steps
    value = total_tokens / dev_s
    e2e = total_tokens / wall
    if rank == 0:
        sm = sorted(step_ms)
        line = {
            "metric": "output tok/s per box at fixed concurrency; p50 TTFT & TPOT", "value": round(value, 1), "unit": "tok/s",
            "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": round(dev_s / steps * 1e3, 3),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": (value / PUBLISHED_TOK_S) if PUBLISHED_TOK_S else None,
            "dtype": "bf16", "data": "synthetic (uniform-random token ids, random-init N(0,0.02) bf16 weights)",
            "config": {"model": "dense GQA 8B-class: 36L hidden 4096 32Q/8KV hd128 SwiGLU 12288 vocab 151936"
                       if args.layers == 36 else f"REDUCED {args.layers}-layer functional check (not a headline number)",
                       "global_batch": conc * (1 if tp else world), "seq_len": f"prompts {p_lo}-{p_hi} uniform, {out_len} outputs",
                       "parallelism": (f"tp{world}" if tp else f"dp{world}") if world > 1 else "tp1",
                       "step": "steady-state engine iteration: 1 finished request replaced (whole prompt prefilled) + decode rows, every live sequence emits a token",
                       "l2": "inputs larger than L2 (weights 15 GB + paged KV of all live sequences read every step)",
                       "mean_prompt_rows_per_step": round(prompt_rows / steps, 1)},
            "tpot_ms_p50": round(sm[len(sm) // 2], 3), "ttft_ms_p50": round(sm[len(sm) // 2], 3),
            "ttft_note": "a new request's prompt is prefilled inside the step it is admitted in, so its first token arrives one step after admission",
            "prefill_tok_s_warmup_wallclock": round(prefill_tokens / prefill_s, 1),
            "e2e": {"value": round(e2e, 1), "unit": "tok/s", "h2d_bytes_per_step": (eng.h2d_bytes - h2d0) // steps,
                    "d2h_bytes_per_step": (eng.d2h_bytes - d2h0) // steps},
            "gpu_launches": launches, "clocks": summarize_clocks(samples),
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
