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
    if spec.get("model") and not spec.get("weights"):
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


def shutdown(ex, procs) -> None:
    if ex.watch:
        ex.watch.stop()
    ex.close()
    for p in procs:
        p.join(5)
        if p.is_alive():
            p.terminate()
