"""Pipeline parallelism with a process per stage: the manifest is cut into N stage manifests, rank s loads stage s on
its own GPU, and every call walks the ranks in order — a stage runs its part, pushes the workspaces that cross the cut
straight into the next stage's exported landing buffers (device copies over NVLink, `Runtime.push_bytes`), and tells
the next rank to go. The last stage emits the tokens. Checked against the uncut model on the last rank's GPU.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 -m kern_b200.parallel.pp_check

Every rank computes the same fills from the same sequence bookkeeping (the pool is a pure function of the same asks), so
only activations and one go-ahead per boundary travel. Reference: crates/kern-serve/src/pp/stage.rs:41-192,
crates/kern-manifest/src/cut.rs:79-282, crates/kern-run/examples/pp_chain.
"""
from __future__ import annotations

import argparse
import json
import sys
import os

import numpy as np
import torch
import torch.distributed as dist


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=5)
    a = ap.parse_args(argv)
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    from .. import fills
    from ..engine import Engine
    from ..models import dense
    from ..runtime import Runtime, verify
    from ..serve import pp

    import dataclasses

    cfg = dense.TINY if world <= 2 else dataclasses.replace(dense.TINY, layers=2 * world, name="tiny-deep")
    doc = dense.build_manifest(cfg)
    stages = pp.cut(doc, pp.layer_cuts(doc, world))
    weights = dense.random_weights(cfg, seed=0, std=0.05)
    dev = torch.device(f"cuda:{local}")
    rt = Runtime(stages[rank], gpu=local, tokens=cfg.page_size * 64, slots=8)
    rt.load_tensors(lambda name: weights[name].to(dev))
    rt.once()
    # what crosses into this stage: its exported buffers that the previous stage holds — written there, or relayed (a
    # table made in the first stage that a later stage reads travels through every stage in between as an input)
    prev = stages[rank - 1]["buffers"] if rank else {}
    landing = [n for n, x in stages[rank]["buffers"].items() if x.get("export") and n in prev and not prev[n].get("fill")]
    handles = [None] * world
    dist.all_gather_object(handles, rt.export_buffers(landing))
    nxt = {n: rt._rt.import_region(h) for n, h in handles[rank + 1].items()} if rank + 1 < world else {}
    proto = json.loads(verify(doc)[0].protocol(sampled=False))
    from .. import _native

    unit = cfg.page_size
    row_pages = min((t["width"] * t["stride"] // unit for t in proto["page_tables"]), default=0)
    pool = _native.Pool(unit, cfg.page_size * 64 // unit, 8, row_pages)      # the same asks on every rank: the same ids
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(0, cfg.vocab, (n,), generator=g).tolist() for n in (40, 7, 90)]
    leases = [pool.lease(len(p) + a.steps + 1) for p in prompts]
    lengths = [0] * len(prompts)
    # the oracle: the uncut model on the last rank
    oracle = None
    if rank == world - 1:
        full = Runtime(doc, gpu=local, tokens=cfg.page_size * 64, slots=8)
        full.load_tensors(lambda name: weights[name].to(dev))
        full.once()
        oracle = Engine(full)
        oseqs = [oracle.open(len(p) + a.steps + 1) for p in prompts]
    np_of = {"i32": np.int32, "i64": np.int64, "f32": np.float32}
    ok, moved = True, 0
    feed = prompts
    for it in range(a.steps + 1):
        entries = [fills.Entry(length=lengths[i], new=feed[i], pages=leases[i].pages, slot=leases[i].slot,
                               slots=leases[i].slots_of(lengths[i], lengths[i] + len(feed[i])), sampling=fills.Sampling())
                   for i in range(len(prompts))]
        call = fills.build(proto, unit, entries)
        bufs = stages[rank]["buffers"]
        for name, (dtype, col) in call.columns.items():
            if name in bufs and bufs[name]["kind"] == "input":
                rt.write(name, np.ascontiguousarray(col.astype(np_of[dtype])))
        if rank > 0:
            dist.recv(torch.zeros(1, device=dev), src=rank - 1)         # the previous stage's push has landed
            # the receive is only enqueued on torch's stream; the runtime issues on its own stream, so the host waits
            # for the signal itself before it launches (a graph replay is otherwise quick enough to overtake it)
            torch.cuda.current_stream().synchronize()
        rt.issue(call.program, {k: v for k, v in call.vars.items() if k in stages[rank]["vars"]})
        if rank + 1 < world:
            vmax = {k: v["max"] for k, v in stages[rank + 1]["vars"].items()}
            for name, ptr in nxt.items():
                n = pp._bytes_for(stages[rank + 1]["buffers"][name], call.vars, vmax)
                rt.push_bytes(name, ptr, n)
                moved += n
            rt.synchronize()
            dist.send(torch.ones(1, device=dev), dst=rank + 1)
        toks = torch.zeros(len(prompts), dtype=torch.int64, device=dev)
        if rank == world - 1:
            rt.synchronize()
            rt.check_error()
            ef = next(f for f in proto["fills"] if f["name"] == call.forward["emits"])
            got = np.asarray(rt.read(ef["name"], call.groups * ef["width"])).reshape(call.groups, ef["width"])[:, 0]
            want = [t[0] for t in oracle.step(list(zip(oseqs, feed)))]
            if got.tolist() != want and ok:
                print(json.dumps({"check": "pipeline_process_per_stage", "first_mismatch_call": it, "got": got.tolist(),
                                  "want": want}), file=sys.stderr, flush=True)
            ok = ok and got.tolist() == want
            toks = torch.tensor(want, dtype=torch.int64, device=dev)
        dist.broadcast(toks, src=world - 1)
        for i in range(len(prompts)):
            lengths[i] += len(feed[i])
        feed = [[int(t)] for t in toks.tolist()]
    flag = torch.tensor([int(ok)], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    mv = torch.tensor([moved], dtype=torch.int64, device=dev)
    dist.all_reduce(mv)
    if rank == 0:
        print(json.dumps({"check": "pipeline_process_per_stage", "stages": world, "calls": a.steps + 1,
                          "crossing_bytes": int(mv.item()), "ok": bool(flag.item())}), flush=True)
    dist.barrier()
    dist.destroy_process_group()
    return 0 if flag.item() else 1


if __name__ == "__main__":
    raise SystemExit(main())
