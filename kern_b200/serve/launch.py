"""Deployment shapes from a manifest and two numbers: `world` rank processes (one per GPU) in `tp`-sized groups.

  world == 1              the scheduler drives a local engine (no rank process)
  world == tp             one tensor-parallel group behind executors; the head schedules it
  world  > tp             world / tp replicas (each a rank or a tp group): a data-parallel tier, lockstep fan-out

The head owns no GPU: it keeps the pools' accounting, the prefix caches and the HTTP front; ranks connect, say Hello,
get the Table of peers, join, and then serve orders. A rank that cannot start fails the head at once; a rank that dies
later closes its control connection and the watch thread ends the head (fail fast).
Reference counterpart: crates/kern-serve/src/lib.rs:317-404 (dispatch by manifest shape and flags), executor.rs.
"""
from __future__ import annotations

import json
import logging
import multiprocessing as mp

from . import wire
from .dp import DpTier
from .executor import Executors, serve_rank
from .ranks import GroupEngine
from .scheduler import Scheduler
from .watch import Watch

log = logging.getLogger("kern.serve")


def _make_runtime(spec: dict, rank: int, world: int):
    """Runs in the rank process. spec: {manifest: dict, weights: path|None, model: name|None, cpu: bool, tokens, slots, tp}"""
    from ..parallel.group import topology

    doc = spec["manifest"]
    topo = topology(doc.get("topology", {}).get("groups", {}), rank, world) if doc.get("topology") else {}
    if spec.get("cpu"):
        from ..cpu import CpuRuntime

        rt = CpuRuntime(doc, weights=spec.get("weights"), tokens=spec.get("tokens") or 4096, slots=spec.get("slots", 0), topology=topo)
        rt.offer = lambda: {}
        rt.connect = lambda g, offers: None
        return rt
    from ..runtime import Runtime

    rt = Runtime(doc, weights=spec.get("weights"), gpu=rank % max(1, spec.get("gpus", world)), topology=topo,
                 tokens=spec.get("tokens") or 0, slots=spec.get("slots", 0))
    if spec.get("tensors"):          # a checkpoint handed over as tensors (tests, self-checks)
        dev = f"cuda:{rank % max(1, spec.get('gpus', world))}"
        rt.load_tensors(lambda name: spec["tensors"][name].to(dev))
    elif spec.get("model") and not spec.get("weights"):
        from ..models import registry

        cfg, _build, load, _make = registry.resolve(spec["model"], **spec.get("overrides", {}))
        load(rt, cfg)
    return rt


def _rank_main(addr, rank: int, world: int, spec: dict) -> None:
    from ..utils.logline import setup_logging

    setup_logging()
    serve_rank(tuple(addr), rank, world, lambda: _make_runtime(spec, rank, world))


def launch(spec: dict, world: int, tp: int = 1, chunk: int | None = None, max_seqs: int | None = None, timeout: float = 600.0,
           context: str = "spawn"):
    """-> (scheduler-like, executors, processes). The scheduler-like object has submit / step / idle / abort / metrics / stats."""
    from .. import _native

    m, errs = _native.verify(json.dumps(spec["manifest"]))
    if m is None:
        raise ValueError("manifest does not verify:\n  - " + "\n  - ".join(errs))
    try:
        protocol = json.loads(m.protocol())
    except ValueError:
        protocol = json.loads(m.protocol(sampled=False))
    lsock = wire.listen()
    addr = lsock.getsockname()
    ctx = mp.get_context(context)
    procs = [ctx.Process(target=_rank_main, args=(addr, q, world, spec), daemon=True) for q in range(world)]
    for p in procs:
        p.start()
    try:
        ex = Executors(lsock, world, {"tp": tp}, watch=Watch(), timeout=timeout)
    finally:
        lsock.close()
    unit = ex.hellos[0]["unit"]
    if world // tp > 1:
        sched = DpTier(ex, protocol, unit, tp=tp, chunk=chunk, max_seqs=max_seqs)
    else:
        sched = Scheduler(GroupEngine(ex, protocol, unit, tp=tp), chunk=chunk, max_seqs=max_seqs)
    log.info("serving world=%d tp=%d replicas=%d", world, tp, world // tp)
    return sched, ex, procs


# ---- pipeline parallel: the launching process is the head (stage 0), the other stages are processes of their own ----
def _pp_init(rank: int, world: int, port: int, cpu: bool, timeout: float):
    """Join the pipeline's process groups: data (NCCL, or gloo on CPU), announcements (gloo, every stage), reports (gloo,
    head and last stage)."""
    import datetime
    import os

    import torch
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    host_timeout = datetime.timedelta(seconds=max(30.0, 4 * timeout))
    if cpu:
        dist.init_process_group("gloo", timeout=host_timeout)
    else:
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{rank}"))
    ctrl = dist.new_group(backend="gloo", timeout=host_timeout)
    report = dist.new_group(ranks=[0, world - 1], backend="gloo", timeout=datetime.timedelta(days=1)) if world > 1 else None
    return ctrl, report


def _pp_pipeline(spec: dict, rank: int, world: int, ctrl, report, ahead: int, timeout: float):
    from . import pp, pp_ranks

    doc = spec["manifest"]
    docs = pp.cut(doc, pp.layer_cuts(doc, world)) if world > 1 else [doc]
    m, errs = __import__("kern_b200")._native.verify(json.dumps(doc))
    if m is None:
        raise ValueError("manifest does not verify:\n  - " + "\n  - ".join(errs))
    proto = json.loads(m.protocol(sampled=False))
    rt = _make_runtime(dict(spec, manifest=docs[rank], gpus=world), rank, 1)
    rt.once()
    unit = getattr(rt, "page_unit", None) or 1
    return pp_ranks.Pipeline(rt, docs, proto, data_pg=None, ctrl_pg=ctrl, report_pg=report, ahead=ahead, timeout=timeout,
                             unit=unit, pages=rt.pages, slots=rt.slots)


def _pp_stage_main(rank: int, world: int, port: int, spec: dict, ahead: int, timeout: float) -> None:
    from ..utils.logline import setup_logging

    setup_logging()
    import torch.distributed as dist

    ctrl, report = _pp_init(rank, world, port, bool(spec.get("cpu")), timeout)
    pipe = _pp_pipeline(spec, rank, world, ctrl, report, ahead, timeout)
    dist.barrier()
    n = pipe.serve()
    log.info("pipeline stage %d served %d items", rank, n)
    dist.barrier()
    dist.destroy_process_group()


def launch_pp(spec: dict, stages: int, chunk: int | None = None, max_seqs: int | None = None, ahead: int = 4,
              timeout: float = 60.0, context: str = "spawn"):
    """A pipeline of `stages` processes, one per GPU, over the manifest cut at layer boundaries: THIS process becomes
    the head (stage 0, GPU 0: it owns the pool, packs items and runs the scheduler), stages 1.. are spawned. Prompt
    chunks follow one another through the stages (up to `ahead` unreported items); the crossing buffers travel by NCCL
    p2p on side streams. -> (scheduler, pipeline, processes); `shutdown_pp` ends it.
    Reference counterpart: crates/kern-serve/src/lib.rs:317-404 (a manifest with `cut` and --pp starts head and stages),
    pp/head.rs, pp/stage.rs."""
    import socket

    import torch.distributed as dist

    from . import pp_ranks

    with socket.socket() as sk:
        sk.bind(("127.0.0.1", 0))
        port = sk.getsockname()[1]
    ctx = mp.get_context(context)
    procs = [ctx.Process(target=_pp_stage_main, args=(q, stages, port, spec, ahead, timeout), daemon=True) for q in range(1, stages)]
    for p in procs:
        p.start()
    ctrl, report = _pp_init(0, stages, port, bool(spec.get("cpu")), timeout)
    pipe = _pp_pipeline(spec, 0, stages, ctrl, report, ahead, timeout)
    dist.barrier()
    sched = Scheduler(pp_ranks.HeadEngine(pipe), chunk=chunk, max_seqs=max_seqs, prefix_cache=False)
    log.info("serving a pipeline of %d stages", stages)
    return sched, pipe, procs


def shutdown_pp(pipe, procs) -> None:
    import torch.distributed as dist

    pipe.stop()
    dist.barrier()
    dist.destroy_process_group()
    for p in procs:
        p.join(10)
        if p.is_alive():
            p.terminate()


def shutdown(ex, procs) -> None:
    if ex.watch:
        ex.watch.stop()
    ex.close()
    for p in procs:
        p.join(5)
        if p.is_alive():
            p.terminate()


def _pp_selftest(argv=None) -> int:
    """`python -m kern_b200.serve.launch --stages S [--cpu]`: a small dense decoder served by a pipeline of S stage
    processes under the scheduler (long prompts in chunks, several requests, decode steps), compared token for token
    with the same requests on one engine. Prints one JSON line."""
    import argparse
    import dataclasses

    import torch

    from ..engine import Engine
    from ..models import dense
    from .scheduler import Request

    ap = argparse.ArgumentParser()
    ap.add_argument("--stages", type=int, default=2)
    ap.add_argument("--cpu", action="store_true")
    a = ap.parse_args(argv)
    cfg = dataclasses.replace(dense.TOY if a.cpu else dense.TINY, layers=2 * a.stages, name="tiny-deep")
    weights = dense.random_weights(cfg, seed=0, std=0.05)
    doc = dense.build_manifest(cfg)
    tokens = cfg.page_size * 48
    if a.cpu:
        from ..cpu import CpuRuntime

        one = CpuRuntime(doc, weights=weights, tokens=tokens)
    else:
        from ..runtime import Runtime

        one = Runtime(doc, gpu=0, tokens=tokens)
        one.load_tensors(lambda name: weights[name].to("cuda:0"))
    one.once()
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(1, cfg.vocab, (n,), generator=g).tolist() for n in (40, 7, 23, 3)]
    chunk = 16

    def serve(sched):
        reqs = [Request(id=str(i), prompt=p, max_tokens=5) for i, p in enumerate(prompts)]
        for r in reqs:
            sched.submit(r)
        for _ in range(2000):
            if sched.idle():
                break
            sched.step()
        return [r.out for r in reqs], sched.idle()

    want, _ = serve(Scheduler(Engine(one), chunk=chunk, max_seqs=3, prefix_cache=False))
    spec = {"manifest": doc, "cpu": a.cpu, "tokens": tokens, "weights": weights if a.cpu else None}
    if not a.cpu:
        spec["tensors"] = weights
    sched, pipe, procs = launch_pp(spec, a.stages, chunk=chunk, max_seqs=3, timeout=30.0)
    try:
        got, idle = serve(sched)
    finally:
        shutdown_pp(pipe, procs)
    ok = got == want and idle and all(not p.is_alive() for p in procs)
    print(json.dumps({"check": "pipeline_under_scheduler", "stages": a.stages, "ok": ok, "items": pipe.k,
                      "requests": len(prompts), "tokens": sum(map(len, got))}), flush=True)
    return 0 if ok else 1


if __name__ == "__main__":
    raise SystemExit(_pp_selftest())
