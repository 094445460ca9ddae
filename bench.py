"""Headline benchmark: output tokens/s of the serving engine at fixed concurrency.

Config (b), the default: dense GQA 8B-class decoder (36 layers, hidden 4096, 32 Q / 8 KV heads of 128, SwiGLU 12288,
vocab 151936, bf16 random init), 256 concurrent requests with prompts of 512-4096 uniform-random token ids and 256
greedy output tokens each; N GPUs = tensor parallel over N ranks (sequence-parallel prefill rows, fused
GEMM + reduce-scatter and all-gather + GEMM kernels over NVLink peer memory).

The timed loop is the serving loop a user of the package runs: `kern_b200.serve.scheduler.Scheduler.step()` over a
`kern_b200.Engine` over a `kern_b200.Runtime` — admission, leases, prefix cache bookkeeping, bucketing, chunk budget,
the host-to-device copy of the step's inputs from pinned memory and the device-to-host read of its tokens are all
inside it. The system is held in steady state: 256 requests are live at staggered ages, so in every step one request
finishes and its replacement (submitted the moment the slot frees) is admitted and its whole prompt prefilled in the same
call as the other 255 requests' decode rows; every live sequence emits one token per step.

    python bench.py [--gpus 1] [--steps 256] [--warmup 3] [--config b]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P bench.py --gpus N ...

Prints one JSON line (rank 0). TTFT of a request = host clock from its submission to its first token being on the host;
TPOT = gap between consecutive tokens of a request (both p50 over the requests / tokens of the timed region).
`--impl reference` runs what of the reference can run on this machine (see baseline/README.md) or says why not.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import subprocess
import sys
import threading
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

PUBLISHED_TOK_S = None   # the reference publishes no B200 number for this config (BASELINE.json `published` is empty)
METRIC = "output tok/s per box at fixed concurrency; p50 TTFT & TPOT"


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


def pct(sorted_vals, q):
    if not sorted_vals:
        return None
    return sorted_vals[min(len(sorted_vals) - 1, int(q * len(sorted_vals)))]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256, help="timed steps (256 = every live sequence turns over once)")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="b", choices=["b", "c", "d", "e", "toy"],
                    help="b: dense GQA 8B-class at concurrency 256 (the headline); c: the hybrid 27B-class decoder under agent-style "
                         "traffic on one GPU; d: decode of a routed-experts decoder with the experts sharded over the GPUs "
                         "(fused dispatch / combine); e: pipelined prefill of 32k-token prompts, then decode, over the KDA + latent-attention + "
                         "routed-experts decoder, a stage per GPU; toy: the reference's own toy-paged package "
                         "(its manifest and cubin) served by this engine, the workload of the reference arm")
    ap.add_argument("--concurrency", type=int, default=256)
    ap.add_argument("--layers", type=int, default=36, help="for quick functional checks only; the headline is 36")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--parallelism", default="tp", choices=["tp", "dp"],
                    help="N > 1: tensor parallel over one batch (the configuration the metric names; default), or "
                         "data-parallel replicas with the concurrency split between them (reported for comparison only)")
    ap.add_argument("--tp-layout", default=None, choices=["sp", "sp-pull", "fused", "unfused"],
                    help="tensor-parallel ragged program: sequence-parallel rows (GEMM + reduce-scatter epilogue, reduce + norm on "
                         "own rows, normed rows pushed to every rank; default up to 4 GPUs, the sizes it has been measured at; "
                         "8 GPUs default to `fused`), the same with the all-gather pulled inside the next "
                         "GEMM, replicated rows with the GEMM epilogue pushing partials to the all-reduce, or replicated rows with a "
                         "plain GEMM and the all-reduce kernel pushing them (A/B)")
    ap.add_argument("--experts", default="mx", choices=["mx", "bf16"],
                    help="config d: MXFP4 expert weights with MXFP8 expert activations (the config's own formats), or bf16 experts")
    ap.add_argument("--profile", action="store_true", help="after the timed region, run one more step with per-call timing and print the cost by op to stderr")
    args = ap.parse_args()
    if args.tp_layout is None:
        args.tp_layout = "sp" if args.gpus <= 4 else "fused"

    if args.impl == "reference":
        from baseline import reference_arm

        return reference_arm.main(args)
    if args.config == "toy":
        from kern_b200.testing import bench_toy

        return bench_toy.main(args)
    if args.config == "c":
        from kern_b200.testing import bench_agent

        return bench_agent.main(args)
    if args.config == "e":
        # pipeline-parallel prefill of long prompts, then decode of the batch, a process per stage (torchrun ranks = stages)
        from kern_b200.parallel import pp_pipeline_check

        os.environ.setdefault("RANK", "0"); os.environ.setdefault("WORLD_SIZE", "1")
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1"); os.environ.setdefault("MASTER_PORT", "29571")
        return pp_pipeline_check.main(["--bench", "--json-line", "--model", "latent-48b-a3b", "--prompt", "32768", "--chunk", "2048",
                                       "--requests", str(max(1, min(args.concurrency, 4))), "--decode-steps", str(min(args.steps, 64)),
                                       "--timeout", "120"] + (["--layers", str(args.layers)] if args.layers != 36 else []))
    if args.config == "d":
        from kern_b200.testing import bench_ep

        return bench_ep.main(args)
    import numpy as np
    import torch

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")      # NCCL only carries the handshake and the final max over ranks
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    steps, warmup = args.steps, max(3, args.warmup)

    from kern_b200.engine import Engine
    from kern_b200.models import dense
    from kern_b200.runtime import Runtime
    from kern_b200.serve.scheduler import Request, Scheduler

    tp = world > 1 and args.parallelism == "tp"
    # tensor parallel: every rank is fed the whole batch; data parallel: replicas split the concurrent requests
    conc = args.concurrency if (tp or world == 1) else args.concurrency // world
    out_len, p_lo, p_hi = 256, 512, 4096
    cfg = dense.DenseConfig(name="dense-8b", layers=args.layers, max_seqs=max(conc, 8), max_tokens=p_hi + conc + 64,
                            max_context=p_hi + 2 * out_len + 64, page_size=64, tp=world if tp else 1)
    torch.cuda.set_device(local)
    if tp:
        from kern_b200.models import dense_tp
        from kern_b200.parallel import group

        doc = dense_tp.build_manifest_tp(cfg, fused=args.tp_layout != "unfused", sp=args.tp_layout.startswith("sp"),
                                         sp_push=args.tp_layout == "sp")
        rt = Runtime(doc, gpu=local, memory_fraction=0.90, topology=group.topology(doc["topology"]["groups"], rank, world))
        dense.load_random_weights(rt, cfg, seed=args.seed)
        group.start(rt)
    else:
        rt = Runtime(dense.build_manifest(cfg), gpu=local, memory_fraction=0.92)
        dense.load_random_weights(rt, cfg, seed=args.seed)
        rt.once()
    eng = Engine(rt)
    sch = Scheduler(eng, chunk=eng.rows_max, max_seqs=conc, prefix_cache=True, stats_every=1e9)
    rng = np.random.default_rng(args.seed + (0 if tp else rank))   # tensor-parallel ranks replay the same requests
    issued = [0]

    def new_request(max_tokens: int) -> Request:
        issued[0] += 1
        prompt = rng.integers(0, cfg.vocab, int(rng.integers(p_lo, p_hi + 1))).tolist()
        return Request(id=f"r{issued[0]}", prompt=prompt, max_tokens=max_tokens)

    # ---- bring the engine to steady state (untimed): `conc` live requests whose remaining lengths are 1..conc ----
    t0 = time.perf_counter()
    first = [new_request(2 * out_len) for _ in range(conc)]     # room in the lease for the tokens made while the others prefill
    for r in first:
        sch.submit(r)
    prefill_tokens = sum(len(r.prompt) for r in first)
    while any(r.fed < len(r.prompt) for r in first):
        sch.step()
    rt.synchronize()
    prefill_s = time.perf_counter() - t0
    remaining = rng.permutation(conc) + 1                        # one request ends in every step from here on
    for r, left in zip(first, remaining):
        r.max_tokens = len(r.out) + max(1, int(left) * out_len // conc)
    rt.check_error()

    live = {r.id: r for r in first}
    finished_in_region: list[Request] = []

    def one_step() -> int:
        """One scheduler step; every request that ends is replaced at once (closed loop). Returns the prompt rows fed."""
        before = sch.stats.prefill_tokens
        for r, _ in sch.step():
            if r.finished:
                live.pop(r.id, None)
                finished_in_region.append(r)
                nr = new_request(out_len)
                live[nr.id] = nr
                sch.submit(nr)
        return sch.stats.prefill_tokens - before

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
    finished_in_region.clear()
    region_t0 = time.monotonic()
    wall0 = time.perf_counter()
    evs[0].record(stream)
    for k in range(steps):
        prompt_rows += one_step()
        launches += eng.last_launches
        evs[k + 1].record(stream)
    rt.synchronize()
    torch.cuda.synchronize()
    wall = time.perf_counter() - wall0
    region_t1 = time.monotonic()
    stop.set()
    th.join(timeout=2)
    if world > 1:
        dist.barrier()
    step_ms = [evs[k].elapsed_time(evs[k + 1]) for k in range(steps)]
    dev_s = sum(step_ms) / 1e3
    rt.check_error()
    if args.profile:          # every rank runs the extra step (the ranks wait for one another); rank 0 prints
        eng_step = eng.step
        eng.step = lambda batch, **kw: eng_step(batch, timed=True, **{k: v for k, v in kw.items() if k != "timed"})
        rows = one_step()
        eng.step = eng_step
        by_op = {}
        for label, op, ms, n in eng.last_times:
            e = by_op.setdefault(op, [0.0, 0, 0])
            e[0] += ms; e[1] += n; e[2] += 1
        total = sum(v[0] for v in by_op.values())
        if rank == 0:
            print(f"# cost by op of one step ({rows} prompt rows + {conc} decode rows), eager, total {total:.2f} ms", file=sys.stderr)
            for op, (ms, n, calls) in sorted(by_op.items(), key=lambda kv: -kv[1][0]):
                print(f"#   {op:14s} {ms:8.3f} ms  {100 * ms / total:5.1f}%  calls {calls:4d}  launches {n}", file=sys.stderr)

    # per-request latencies of the timed region (host clock: they include the copies both ways and the scheduler)
    reqs = list(live.values()) + finished_in_region
    ttft = sorted(1e3 * (r.first_token_at - r.arrival) for r in reqs
                  if r.first_token_at is not None and region_t0 <= r.arrival and r.first_token_at <= region_t1)
    gaps = sorted(1e3 * (b - a) for r in reqs for a, b in zip(r.token_times, r.token_times[1:]) if a >= region_t0 and b <= region_t1)

    if world > 1:
        t = torch.tensor([dev_s, wall], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dev_s, wall = float(t[0]), float(t[1])
    replicas = 1 if (tp or world == 1) else world
    total_tokens = conc * replicas * steps
    value = total_tokens / dev_s
    e2e = total_tokens / wall
    if rank == 0:
        sm = sorted(step_ms)
        line = {
            "metric": METRIC, "value": round(value, 1), "unit": "tok/s",
            "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": round(dev_s / steps * 1e3, 3),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": (value / PUBLISHED_TOK_S) if PUBLISHED_TOK_S else None,
            "dtype": "bf16", "data": "synthetic (uniform-random token ids, random-init N(0,0.02) bf16 weights)",
            "config": {"model": "dense GQA 8B-class: 36L hidden 4096 32Q/8KV hd128 SwiGLU 12288 vocab 151936"
                       if args.layers == 36 else f"REDUCED {args.layers}-layer functional check (not a headline number)",
                       "global_batch": conc * replicas, "seq_len": f"prompts {p_lo}-{p_hi} uniform, {out_len} outputs",
                       "parallelism": (f"tp{world}" if tp else f"dp{world}") if world > 1 else "tp1",
                       "tp_layout": args.tp_layout if tp else None,
                       "step": "steady-state scheduler step: 1 finished request replaced (whole prompt prefilled) + decode rows, every live sequence emits a token",
                       "l2": "inputs larger than L2 (weights 15 GB + paged KV of all live sequences read every step)",
                       "mean_prompt_rows_per_step": round(prompt_rows / steps, 1)},
            "step_ms": {"p10": round(pct(sm, 0.10), 3), "p50": round(pct(sm, 0.50), 3), "p90": round(pct(sm, 0.90), 3),
                        "min": round(sm[0], 3), "max": round(sm[-1], 3),
                        "sha1": hashlib.sha1(",".join(f"{x:.3f}" for x in step_ms).encode()).hexdigest()[:16],
                        "first": [round(x, 3) for x in step_ms[:8]]},
            "ttft_ms_p50": round(pct(ttft, 0.5), 3) if ttft else None, "ttft_ms_p90": round(pct(ttft, 0.9), 3) if ttft else None,
            "ttft_requests": len(ttft),
            "tpot_ms_p50": round(pct(gaps, 0.5), 3) if gaps else None, "tpot_ms_p90": round(pct(gaps, 0.9), 3) if gaps else None,
            "latency_note": "TTFT: submission (the moment a slot frees) to first token on the host; TPOT: gap between a request's "
                            "consecutive tokens on the host; rank 0's clock",
            "timed_region_s": round(wall, 3),
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
