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

    gpu = spec["gpu_of_rank"][rank] if spec.get("gpu_of_rank") else rank % max(1, spec.get("gpus", world))
    rt = Runtime(doc, weights=spec.get("weights"), gpu=gpu, topology=topo, tokens=spec.get("tokens") or 0, slots=spec.get("slots", 0))
    if spec.get("tensors"):          # a checkpoint handed over as tensors (tests, self-checks)
        dev = f"cuda:{gpu}"
        rt.load_tensors(lambda name: spec["tensors"][name].to(dev))
    elif spec.get("model") and not spec.get("weights"):
        from ..models import registry

        cfg, _build, load, _make = registry.resolve(spec["model"], **spec.get("overrides", {}))
        load(rt, cfg)
    return rt


def _rank_main(addr, rank: int, world: int, spec: dict) -> None:
    from ..utils.logline import setup_logging

    setup_logging()
    serve_rank(tuple(addr), rank, world, lambda: _make_runtime(spec, rank, world), export_pools=bool(spec.get("export_pools")))


def launch(spec: dict, world: int, tp: int = 1, chunk: int | None = None, max_seqs: int | None = None, timeout: float = 600.0,
           context: str = "spawn", by_position: bool = False, engine_only: bool = False):
    """-> (scheduler-like, executors, processes). The scheduler-like object has submit / step / idle / abort / metrics / stats.
    `by_position`: the group is a decode context-parallel group (a member manifest that deals positions over its ranks);
    `engine_only`: return the group's engine instead of a scheduler (a decode tier drives it itself)."""
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
        # the groups the manifest names (a tensor-parallel decoder: {"tp": n}; a context-parallel member: {"dcp": n})
        groups = dict(spec["manifest"].get("topology", {}).get("groups", {})) or {"tp": tp}
        ex = Executors(lsock, world, groups, watch=Watch(), timeout=timeout)
    finally:
        lsock.close()
    unit = ex.hellos[0]["unit"]
    if engine_only:
        return GroupEngine(ex, protocol, unit, tp=tp, by_position=by_position), ex, procs
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


# ---- prefill / decode disaggregation: this process is the prefill tier, the decode tier a process on its own GPU ----
def _pd_decode_main(addr, spec: dict, gpu: int, max_seqs: int | None, stop_ids: tuple) -> None:
    from ..engine import Engine
    from ..utils.logline import setup_logging
    from . import pd_serve

    setup_logging()
    rt = _make_runtime(dict(spec, gpus=1 << 30), gpu, 1)          # `gpu` is the device index itself
    rt.once()
    eng = Engine(rt)
    sock = wire.connect(tuple(addr))
    max_seq = eng.pool.total_pages * rt.page_unit
    wire.send(sock, pd_serve.hello_of(rt, spec["manifest"], max_seq, handles=rt.export_states()))
    calls = pd_serve.decode_loop(sock, eng, max_seqs=max_seqs, stop_ids=stop_ids)
    if hasattr(rt, "check_error"):
        rt.check_error()
    log.info("decode tier made %d decode calls", calls)


def launch_pd(spec: dict, decode_spec: dict | None = None, chunk: int | None = None, max_seqs: int | None = None,
              decode_max_seqs: int | None = None, stop_ids: tuple = (), prefill_gpu: int = 0, decode_gpu: int = 1,
              timeout: float = 600.0, context: str = "spawn", decode_gpus: list[int] | None = None, dealer=None,
              front: bool = False):
    """Prefill and decode on two GPUs: THIS process is the prefill tier (its own runtime, pool, prefix cache and
    scheduler on `prefill_gpu`), the decode tier is a spawned process on `decode_gpu` that exports its pools; a prompt's
    pages and slot are pushed into the seats the decode tier granted (device copies over NVLink) and the request goes
    on there. `decode_spec`: the decode tier's own spec (capacity, slots; default: `spec`). With `spec["cpu"]` both
    tiers are host-memory executors in this process (the decode tier a thread), the frames still travel over a socket.
    `decode_gpus` (two or more): the decode tier is a group of rank processes, one per listed GPU, whose manifest
    (`decode_spec["manifest"]`) deals every sequence's positions over the members (decode context parallelism); its head
    (seats, steps, accounting) is a thread of this process; `dealer`: how the prompt's rows reach the members when a
    state's pages are not token-contiguous (`pd_serve`). `front`: the prefill scheduler runs on a head thread and the
    returned object only relays (`front.Front`), so decode tokens are not held behind a prefill step.
    -> (scheduler-like prefill tier, worker). `shutdown_pd` ends it.
    Reference counterpart: crates/kern-serve/src/lib.rs:317-404 (tiers by flags), pd/handoff.rs, pd/decoder.rs."""
    import threading

    from ..engine import Engine
    from . import pd_serve

    dspec = decode_spec or spec
    lsock = wire.listen()
    addr = lsock.getsockname()
    pools = None
    if decode_gpus and len(decode_gpus) > 1:
        from . import pd

        n = len(decode_gpus)
        d_eng, ex, procs = launch(dict(dspec, export_pools=True, gpu_of_rank=list(decode_gpus)), world=n, tp=n, timeout=timeout,
                                  context=context, by_position=True, engine_only=True)
        unit = ex.hellos[0]["unit"]
        hello = pd.pools_message(dspec["manifest"], unit, n, d_eng.pool.total_pages * unit * n)
        hello["members"] = [h["pools"] for h in ex.hellos]

        def g_main():
            sock = wire.connect(tuple(addr))
            wire.send(sock, {"hello": hello})
            pd_serve.decode_loop(sock, d_eng, max_seqs=decode_max_seqs, stop_ids=stop_ids, idle_wait=0.02)
            sock.close()

        thread = threading.Thread(target=g_main, daemon=True, name="kern-decode-group")
        worker = _DecodeGroup(thread, ex, procs)
    elif spec.get("cpu"):
        d_rt = _make_runtime(dspec, 0, 1)
        d_rt.once()
        d_eng = Engine(d_rt)
        pools = d_rt.export_states()

        def d_main():
            sock = wire.connect(tuple(addr))
            wire.send(sock, pd_serve.hello_of(d_rt, dspec["manifest"], d_eng.pool.total_pages * d_rt.page_unit))
            pd_serve.decode_loop(sock, d_eng, max_seqs=decode_max_seqs, stop_ids=stop_ids, idle_wait=0.02)
            sock.close()

        worker = threading.Thread(target=d_main, daemon=True, name="kern-decode-tier")
    else:
        ctx = mp.get_context(context)
        worker = ctx.Process(target=_pd_decode_main, args=(addr, dspec, decode_gpu, decode_max_seqs, tuple(stop_ids)), daemon=True)
    worker.start()
    try:
        rt = _make_runtime(dict(spec, gpus=1 << 30), prefill_gpu, 1)
        rt.once()
        lsock.settimeout(timeout)
        sock = wire.accept(lsock)
    finally:
        lsock.close()
    sched = Scheduler(Engine(rt), chunk=chunk, max_seqs=max_seqs)
    tier = pd_serve.connect_tiers(sched, rt, spec["manifest"], sock, pools=pools, timeout=timeout, dealer=dealer, front=front)
    log.info("serving a prefill tier on gpu %d and a decode tier on gpu %d", prefill_gpu, decode_gpu)
    return tier, worker


class _DecodeGroup:
    """A decode group's head thread with its rank processes, behind the start / join / is_alive of a worker."""

    def __init__(self, thread, ex, procs):
        self.thread, self.ex, self.procs = thread, ex, procs

    def start(self) -> None:
        self.thread.start()

    def join(self, timeout: float | None = None) -> None:
        self.thread.join(timeout)
        shutdown(self.ex, self.procs)

    def is_alive(self) -> bool:
        return self.thread.is_alive() or any(p.is_alive() for p in self.procs)


def shutdown_pd(tier, worker) -> None:
    tier.close()
    worker.join(10)
    if worker.is_alive() and hasattr(worker, "terminate"):
        worker.terminate()


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
    with the same requests on one engine; `--pd`: the same requests through a prefill tier and a decode tier on two
    GPUs (`--cpu`: two host-memory executors). Prints one JSON line."""
    import argparse
    import dataclasses

    import torch

    from ..engine import Engine
    from ..models import dense
    from .scheduler import Request

    ap = argparse.ArgumentParser()
    ap.add_argument("--stages", type=int, default=2)
    ap.add_argument("--pd", action="store_true", help="a prefill tier and a decode tier instead of a pipeline")
    ap.add_argument("--dcp", type=int, default=0, help="with --pd: the decode tier is a context-parallel group of this many ranks")
    ap.add_argument("--front", action="store_true", help="with --pd: the prefill scheduler on a head thread (serve/front.py)")
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
    if a.pd:
        # the decode tier holds two sequences at a time: later requests wait for a seat (Busy, then a grant)
        if a.dcp > 1:
            # a decode group that deals positions over its members; its ranks go round the GPUs of the box (rank 0 shares
            # GPU 0 with the prefill tier when there are no more GPUs than ranks)
            from ..models import dense_dcp

            n_gpu = max(1, torch.cuda.device_count())
            first = 1 if n_gpu > a.dcp else 0
            dspec = dict(spec, manifest=dense_dcp.build_manifest_dcp(cfg, a.dcp), tokens=cfg.page_size * 8)
            tier, worker = launch_pd(spec, dspec, chunk=chunk, max_seqs=3, decode_max_seqs=2, timeout=120.0, front=a.front,
                                     decode_gpus=[(first + i) % n_gpu for i in range(a.dcp)], dealer=dense_dcp.dealer(cfg))
        else:
            tier, worker = launch_pd(spec, dict(spec, tokens=cfg.page_size * 8), chunk=chunk, max_seqs=3, decode_max_seqs=2, timeout=60.0,
                                     front=a.front)
        try:
            got, idle = serve(tier)
            served = tier.metrics()
        finally:
            shutdown_pd(tier, worker)
        flat = lambda xs: [t for x in xs for t in x]
        agree = sum(int(x == y) for x, y in zip(flat(got), flat(want)))
        # a context-parallel group merges partial attention in another order: the first token of every request (the prefill
        # tier's) is exact, the decode tier's may differ where two logits are within rounding of each other
        exact = got == want if a.dcp <= 1 else ([g[:1] for g in got] == [w[:1] for w in want] and agree >= 0.85 * len(flat(want)))
        ok = exact and idle and not worker.is_alive()
        print(json.dumps({"check": "prefill_decode_tiers_under_scheduler", "ok": ok, "requests": len(prompts), "decode_ranks": max(1, a.dcp),
                          "tokens": sum(map(len, got)), "tokens_agree": agree,
                          "prefix_cache_entries": served["prefix_cache"]["entries"]}), flush=True)
        return 0 if ok else 1
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
