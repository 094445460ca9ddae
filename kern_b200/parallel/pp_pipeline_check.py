"""Pipelined prefill over a process per stage (`serve/pp_ranks.py`), checked against the uncut model and timed.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        -m kern_b200.parallel.pp_pipeline_check [--cpu] [--bench --model dense-8b --prompt 32768 --chunk 2048]
        [--stall-stage S --timeout 3]

Check: a dense decoder of 2 N layers cut into N stages; the head prefills several prompts in chunks, all chunks in
flight, then decodes a few steps through the same pipeline; every emitted token equals the uncut model's.
`--stall-stage S`: stage S stops serving after two items (a failure made on the host: it just stops calling); the
stage before it must end with a timeout error naming it, not hang. `--bench`: prompt tokens per second of one long
prompt through the pipeline (device time of the head's first issue to the last stage's token, max over ranks).
CPU ranks (`--cpu`) use gloo and the host-memory executor.
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import os
import sys
import time

import torch
import torch.distributed as dist


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--cpu", action="store_true")
    ap.add_argument("--bench", action="store_true")
    ap.add_argument("--model", default="dense-8b")
    ap.add_argument("--layers", type=int, default=0, help="bench: layers of the model (default: its own count)")
    ap.add_argument("--prompt", type=int, default=32768)
    ap.add_argument("--chunk", type=int, default=2048)
    ap.add_argument("--ahead", type=int, default=4)
    ap.add_argument("--stall-stage", type=int, default=-1)
    ap.add_argument("--timeout", type=float, default=60.0)
    ap.add_argument("--requests", type=int, default=1, help="bench: prompts prefilled one after the other (all chunks in flight)")
    ap.add_argument("--decode-steps", type=int, default=0, help="bench: decode steps of all the requests as one batch, after the prefill")
    ap.add_argument("--json-line", action="store_true", help="bench: print the benchmark driver's line (bench.py --config e)")
    a = ap.parse_args(argv)
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", 0))
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    if os.environ.get("KERN_LOG"):            # KERN_LOG=debug: every stage writes its `pp item` lines (serve/pp_timeline.py reads them)
        from ..utils.logline import setup_logging

        setup_logging()
    import datetime

    host_timeout = datetime.timedelta(seconds=max(30.0, 4 * a.timeout))
    if a.cpu:
        dist.init_process_group("gloo", timeout=host_timeout)
    else:
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    ctrl = dist.new_group(backend="gloo", timeout=host_timeout)                       # announcements: every stage
    report = dist.new_group(ranks=[0, world - 1], backend="gloo", timeout=datetime.timedelta(days=1)) if world > 1 else None
    from ..engine import Engine
    from ..models import dense
    from ..runtime import verify
    from ..serve import pp, pp_ranks

    build, load_random = dense.build_manifest, dense.load_random_weights
    if a.bench:
        from ..models import registry

        cfg, build, load_random, _make = registry.resolve(a.model, max_seqs=max(8, a.requests), max_tokens=a.chunk,
                                                          max_context=a.prompt + a.decode_steps + 64, page_size=64, layers=a.layers or None)
        tokens = a.requests * (a.prompt + a.decode_steps + 64) + 4 * a.chunk + 1024
    else:
        cfg = dataclasses.replace(dense.TINY if not a.cpu else dense.TOY, layers=2 * world, name="tiny-deep")
        tokens = cfg.page_size * 64
    doc = build(cfg)
    docs = pp.cut(doc, pp.layer_cuts(doc, world)) if world > 1 else [doc]
    proto = json.loads(verify(doc)[0].protocol(sampled=False))

    def load(d):
        if a.cpu:
            from ..cpu import CpuRuntime

            rt = CpuRuntime(d, weights=dense.random_weights(cfg, seed=0, std=0.05), tokens=tokens, slots=8)
        else:
            from ..runtime import Runtime

            rt = Runtime(d, gpu=local, tokens=tokens, slots=max(8, a.requests + 2))
            if a.bench:
                load_random(rt, cfg, seed=0)
            else:
                w = dense.random_weights(cfg, seed=0, std=0.05)
                rt.load_tensors(lambda name: w[name].to(f"cuda:{local}"))
        rt.once()
        return rt

    rt = load(docs[rank])
    pipe = pp_ranks.Pipeline(rt, docs, proto, data_pg=None, ctrl_pg=ctrl, report_pg=report, ahead=a.ahead, timeout=a.timeout, unit=cfg.page_size,
                             pages=tokens // cfg.page_size, slots=max(8, a.requests + 2) if a.bench else 8)
    dist.barrier()
    out = {"check": "pipeline_prefill", "stages": world, "ok": True}
    code = 0
    try:
        if rank != 0:
            if rank == a.stall_stage:
                for _ in range(2):                     # take two items, then stop answering (the process stays alive for a while)
                    pipe.stage.run(pipe._hear())
                time.sleep(3 * a.timeout)
                return 0
            n = pipe.serve()
            out["items"] = n
        else:
            g = torch.Generator().manual_seed(4)
            if a.bench:
                prompt = torch.randint(0, cfg.vocab, (a.prompt,), generator=g).tolist()
                warm = pipe.open(a.chunk * 2 + 8)
                pipe.prefill(warm, prompt[: a.chunk * 2], a.chunk)          # warm-up: two chunks through every stage
                warm.lease.release()
                prompts = [prompt] + [torch.randint(0, cfg.vocab, (a.prompt,), generator=g).tolist() for _ in range(a.requests - 1)]
                seqs = [pipe.open(a.prompt + a.decode_steps + 8) for _ in prompts]
                t0 = time.perf_counter()
                # every chunk of every prompt is announced before any token is read: the stages never wait for the head
                last = []
                for s, p in zip(seqs, prompts):
                    k = None
                    for i in range(0, len(p), a.chunk):
                        k = pipe.submit([(s, p[i:i + a.chunk])])
                    last.append(k)
                toks = [pipe.tokens(k)[0][0] for k in last]
                dt = time.perf_counter() - t0
                out.update({"bench": True, "model": cfg.name, "layers": cfg.layers, "prompt": a.prompt, "requests": a.requests,
                            "chunk": a.chunk, "ahead": a.ahead, "seconds": round(dt, 4),
                            "prompt_tok_s": round(a.requests * a.prompt / dt, 1), "first_token": toks[0]})
                if a.decode_steps:
                    t1 = time.perf_counter()
                    for _ in range(a.decode_steps):
                        k = pipe.submit([(s, [t]) for s, t in zip(seqs, toks)])
                        toks = [t[0] for t in pipe.tokens(k)]
                    dd = time.perf_counter() - t1
                    out.update({"decode_steps": a.decode_steps, "decode_seconds": round(dd, 4),
                                "decode_tok_s": round(a.requests * a.decode_steps / dd, 1), "tpot_ms": round(1e3 * dd / a.decode_steps, 3)})
            else:
                oracle = Engine(load(doc))
                prompts = [torch.randint(0, cfg.vocab, (n,), generator=g).tolist() for n in ((40, 7, 90) if not a.cpu else (21, 5, 30))]
                chunk = 16 if not a.cpu else 8
                seqs = [pipe.open(len(p) + 8) for p in prompts]
                oseqs = [oracle.open(len(p) + 8) for p in prompts]
                pending = []
                for s, p in zip(seqs, prompts):                              # every chunk of every prompt is announced before any token is read
                    last = None
                    for i in range(0, len(p), chunk):
                        last = pipe.submit([(s, p[i:i + chunk])])
                    pending.append(last)
                got = [pipe.tokens(k)[0][0] for k in pending]
                want = []
                for s, p in zip(oseqs, prompts):
                    t = None
                    for i in range(0, len(p), chunk):
                        t = oracle.step([(s, p[i:i + chunk])])
                    want.append(t[0][0])
                ok = got == want
                toks = got
                for _ in range(4):                                           # decode steps through the same pipeline
                    k = pipe.submit([(s, [t]) for s, t in zip(seqs, toks)])
                    nxt = [t[0] for t in pipe.tokens(k)]
                    ref = [t[0] for t in oracle.step([(s, [t]) for s, t in zip(oseqs, toks)])]
                    ok = ok and nxt == ref
                    toks = ref
                out.update({"ok": bool(ok), "items": pipe.k, "moved_bytes_stage0": pipe.stage.moved_bytes})
            pipe.stop()
    except pp_ranks.StageTimeout as e:
        out.update({"ok": False, "timeout": str(e), "stage": rank})
        code = 3
    if hasattr(rt, "check_error"):
        try:
            rt.check_error()
        except Exception as e:      # noqa: BLE001
            out.update({"ok": False, "device_error": str(e)})
            code = 1
    if rank == 0 and a.bench and a.json_line and out.get("ok"):
        total_s = out["seconds"] + out.get("decode_seconds", 0.0)
        print(json.dumps({
            "metric": "prompt tok/s through the pipeline (prefill of every request, all chunks in flight), then decode tok/s of the batch",
            "value": out["prompt_tok_s"], "unit": "tok/s", "n_gpus": world, "steps": a.requests * (-(-a.prompt // a.chunk)) + a.decode_steps,
            "warmup": 2, "ms_per_step": round(1e3 * total_s / max(1, a.requests * (-(-a.prompt // a.chunk)) + a.decode_steps), 3),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic (uniform-random token ids, random-init bf16 weights)",
            "config": {"model": (f"{cfg.name}: {cfg.layers} layers, KDA with every {cfg.full_every}-th layer latent attention, "
                                 f"{cfg.experts} routed experts top-{cfg.top_k}") if hasattr(cfg, "full_every") else f"{cfg.name}: {cfg.layers} layers",
                       "same_config": False,
                       "why": "config (e) names the K3 shape (hidden 7168, 384 experts, MXFP4) on eight stages with an expert-parallel decode "
                              "tier; this is the same layer pattern at the 48B-A3B size, bf16, prefill and decode through one pipeline of "
                              "N stage processes",
                       "requests": a.requests, "prompt": a.prompt, "chunk": a.chunk, "decode_steps": a.decode_steps,
                       "parallelism": f"pp{world}", "clock": "the head's wall clock from the first announced chunk to the last token read"},
            "prefill_seconds": out["seconds"], "decode_tok_s": out.get("decode_tok_s"), "tpot_ms_p50": out.get("tpot_ms"),
            "ttft_ms_p50": round(1e3 * out["seconds"] / a.requests, 1)}), flush=True)
    elif rank == 0 or code:
        print(json.dumps(out), flush=True)
    if code == 3:
        os._exit(3)            # the neighbours are gone or stuck: leave without the group's shutdown handshake
    if not out["ok"]:
        code = code or 1
    dist.barrier()
    dist.destroy_process_group()
    return code


if __name__ == "__main__":
    sys.exit(main())
