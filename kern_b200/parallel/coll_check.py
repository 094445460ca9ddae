"""The `extern:nccl_*` launches of a manifest, checked on N ranks (one process per GPU under `torch.distributed.run`,
or N gloo ranks on CPU with `--cpu`): all-reduce f32, all-gather bf16, reduce-scatter f32 and all-to-all i32 over a
`tp` group, eager and as one captured program; prints one JSON line per check.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 -m kern_b200.parallel.coll_check

Reference: crates/kern-runtime/src/nccl.rs:190 (what each collective moves), examples/cross_collective.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def manifest(world: int, n_max: int) -> dict:
    buf = lambda dt, n, kind: {"dtype": dt, "shape": [n], "kind": kind}
    op = lambda entry, a, b: {"params": [f"in buffer<{a}>", f"out buffer<{b}>", "i64", "i32"],
                              "impl": {"launches": [{"entry": entry}]}}
    call = lambda o, x, y: {"op": o, "args": [{"buf": x}, {"buf": y}, {"var": "n"}, {"rank": "tp"}]}
    calls = [call("ar", "ar_x", "ar_y"), call("ag", "ag_x", "ag_y"), call("rs", "rs_x", "rs_y"), call("a2a", "aa_x", "aa_y")]
    return {"schema_version": 7, "model": "collectives", "topology": {"groups": {"tp": world}},
            "vars": {"n": {"max": n_max, "axis": "rows"}}, "states": {}, "modules": {},
            "buffers": {"ar_x": buf("f32", n_max, "input"), "ar_y": buf("f32", n_max, "output"),
                        "ag_x": buf("bf16", n_max, "input"), "ag_y": buf("bf16", n_max * world, "output"),
                        "rs_x": buf("f32", n_max * world, "input"), "rs_y": buf("f32", n_max, "output"),
                        "aa_x": buf("i32", n_max * world, "input"), "aa_y": buf("i32", n_max * world, "output")},
            "ops": {"ar": op("extern:nccl_allreduce_f32", "f32", "f32"), "ag": op("extern:nccl_allgather_bf16", "bf16", "bf16"),
                    "rs": op("extern:nccl_reducescatter_f32", "f32", "f32"), "a2a": op("extern:nccl_alltoall_i32", "i32", "i32")},
            "programs": {"step": {"calls": calls}, "captured": {"batch": {"groups": 1, "rows": "n"}, "graph": True, "calls": calls}}}


def inputs(rank: int, world: int, n: int, rep: int, device):
    g = lambda r: torch.Generator().manual_seed(1000 * rep + r)
    ar = lambda r: torch.randn(n, generator=g(r))
    ag = lambda r: torch.randn(n, generator=g(r + 50)).to(torch.bfloat16)
    rs = lambda r: torch.randn(n * world, generator=g(r + 100))
    aa = lambda r: torch.randint(-1000, 1000, (n * world,), generator=g(r + 150), dtype=torch.int32)
    mine = {"ar_x": ar(rank), "ag_x": ag(rank), "rs_x": rs(rank), "aa_x": aa(rank)}
    want = {"ar_y": sum(ar(r) for r in range(world)),
            "ag_y": torch.cat([ag(r) for r in range(world)]),
            "rs_y": sum(rs(r) for r in range(world))[rank * n:(rank + 1) * n],
            "aa_y": torch.cat([aa(p)[rank * n:(rank + 1) * n] for p in range(world)])}
    return {k: v.to(device) for k, v in mine.items()}, {k: v.to(device) for k, v in want.items()}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--cpu", action="store_true", help="gloo ranks and the host-memory executor")
    ap.add_argument("--sizes", type=int, nargs="+", default=[1, 1000, 1 << 16])
    a = ap.parse_args(argv)
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    from . import group

    doc = manifest(world, max(a.sizes))
    if a.cpu:
        from ..cpu import CpuRuntime

        if world > 1:
            dist.init_process_group("gloo")
        rt, device = CpuRuntime(doc, topology={"tp": (rank, world)}), "cpu"
    else:
        from ..runtime import Runtime

        torch.cuda.set_device(local)
        if world > 1:
            dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
        rt, device = Runtime(doc, gpu=local, topology={"tp": (rank, world)}), f"cuda:{local}"
        if world > 1:
            group.start(rt)
    results = []
    for program in ("step", "captured"):
        for rep, n in enumerate(a.sizes):
            mine, want = inputs(rank, world, n, rep + (10 if program == "captured" else 0), device)
            for name, t in mine.items():
                rt.tensor(name)[: t.numel()] = t
            if not a.cpu:
                torch.cuda.synchronize()
            rt.run(program, {"n": n})
            ok = True
            for name, t in want.items():
                got = rt.tensor(name)[: t.numel()]
                close = torch.equal(got, t) if t.dtype in (torch.int32, torch.bfloat16) else torch.allclose(got, t, rtol=1e-5, atol=1e-5)
                ok = ok and bool(close)
            flag = torch.tensor([int(ok)], device=device)
            if world > 1:
                dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            results.append({"program": program, "n": n, "ok": bool(flag.item())})
    if rank == 0:
        print(json.dumps({"check": "collective_externs", "world": world, "backend": "gloo" if a.cpu else "nccl",
                          "results": results}), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0 if all(r["ok"] for r in results) else 1


if __name__ == "__main__":
    raise SystemExit(main())
