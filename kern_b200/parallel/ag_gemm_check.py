"""The all-gather fused into the tensor-core GEMM, checked and timed on N ranks (one process per GPU):
every rank holds its slice of the rows, one kernel pulls the other slices over NVLink while it multiplies, and the
product must equal the GEMM over all rows. Timed against the two-step form (NCCL all-gather, then the plain GEMM).

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 -m kern_b200.parallel.ag_gemm_check --time

Reference: docs/multi-gpu.md:495-528 (per layer: nccl_allgather_bf16, then the projections).
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def manifest(world: int, rows_max: int, n: int, k: int) -> dict:
    from ..models import common as C

    bufs = {"w": {"dtype": "bf16", "shape": [n, k], "kind": "input"},
            "c": {"dtype": "bf16", "shape": ["rows", n], "kind": "output"},
            "error": {"dtype": "i32", "shape": [1], "kind": "output"}}
    bufs.update(C.ag_gemm_buffers(rows_max, k, world, alternate=True))
    B = lambda name: {"buf": name}
    args = lambda g: [B(g), B(g + "_peers"), B("w"), B("c"), B("ag.bar"), B("ag.bar_peers"), B("ag.bar_epoch"),
                      B("ag.blocks"), B("ag.cta_epochs"), B("error"), {"var": "rows"}]
    call = {"op": "ag_gemm", "args": args("ag.g")}
    # the layout a decoder uses: consecutive calls switch between two row buffers, and the barrier that opens call k + 1
    # is what tells everyone that call k's pulls are over, so nothing follows the GEMM
    pair = [{"op": "ag_gemm_open", "args": args("ag.g")}, {"op": "ag_gemm_open", "args": args("ag.g1")}]
    return {"schema_version": 7, "model": "ag-gemm-check", "vars": {"rows": {"max": rows_max, "axis": "rows"}},
            "topology": {"groups": {"tp": world}}, "states": {}, "buffers": bufs,
            "modules": C.modules_for(["ag_gemm", "tp_allreduce_norm"]),
            "ops": {"ag_gemm": C.ag_gemm_op(n, k, world), "ag_gemm_open": C.ag_gemm_op(n, k, world, closing_barrier=False)},
            "programs": {"step": {"calls": [call]},
                         "step_graph": {"batch": {"groups": 1, "rows": "rows"}, "graph": True, "calls": [call]},
                         "pair_graph": {"batch": {"groups": 1, "rows": "rows"}, "graph": True, "calls": pair * 2}}}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, nargs="+", default=[128, 1024, 256, 2048], help="rows per rank (multiples of 128)")
    ap.add_argument("--n", type=int, default=3072)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--time", action="store_true")
    a = ap.parse_args(argv)
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device(f"cuda:{local}")
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    from ..runtime import Runtime
    from . import group

    rows_max = max(a.rows) * world
    rt = Runtime(manifest(world, rows_max, a.n, a.k), gpu=local, topology={"tp": (rank, world)})
    group.start(rt)          # a group of one still fills its peer tables (with its own addresses)
    g = torch.Generator().manual_seed(9)
    w = (torch.randn(a.n, a.k, generator=g) * 0.05).to(torch.bfloat16).to(dev)
    rt.tensor("w").copy_(w)
    G = rt.tensor("ag.g")
    results = []
    G1 = rt.tensor("ag.g1")
    for it, tr in enumerate(a.rows + a.rows[:2] + a.rows[:1]):
        program = "step" if it < len(a.rows) else ("step_graph" if it < len(a.rows) + 2 else "pair_graph")
        T = tr * world
        slices = [(torch.randn(tr, a.k, generator=torch.Generator().manual_seed(100 * it + r)) * 0.5).to(torch.bfloat16) for r in range(world)]
        G[:T].fill_(float("nan"))                              # what is not pulled stays NaN and poisons the product
        G[rank * tr:(rank + 1) * tr].copy_(slices[rank].to(dev))
        if program == "pair_graph":
            G1[:T].fill_(float("nan"))
            G1[rank * tr:(rank + 1) * tr].copy_(slices[rank].to(dev))
        torch.cuda.synchronize()
        rt.run(program, {"rows": T})
        rt.check_error()
        got = rt.tensor("c")[:T].float()
        want = torch.cat(slices).to(dev).float() @ w.float().t()
        err = float((got - want).abs().max())
        ok = torch.tensor([int(err < 0.06 and bool(torch.isfinite(got).all()))], device=dev)
        if world > 1:
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        results.append({"rows_per_rank": tr, "program": program, "max_abs_err": round(err, 4), "ok": bool(ok.item())})
    line = {"check": "allgather_gemm_fused", "world": world, "n": a.n, "k": a.k, "results": results}
    if a.time:
        from ..ops import gemm as GM

        times = []
        stream = torch.cuda.ExternalStream(rt.stream)
        for tr in a.rows:
            T = tr * world
            mine = (torch.randn(tr, a.k, device=dev) * 0.5).to(torch.bfloat16)
            G[rank * tr:(rank + 1) * tr].copy_(mine)
            torch.cuda.synchronize()

            def fused():
                rt.issue("step_graph", {"rows": T})

            G1 = rt.tensor("ag.g1")
            G1[rank * tr:(rank + 1) * tr].copy_(mine)
            torch.cuda.synchronize()

            def alternating():          # four GEMMs per replay, two row buffers, no closing barrier
                rt.issue("pair_graph", {"rows": T})

            full = torch.empty(T, a.k, dtype=torch.bfloat16, device=dev)
            out = torch.empty(T, a.n, dtype=torch.bfloat16, device=dev)

            def two_step():
                if world > 1:
                    dist.all_gather_into_tensor(full, mine)
                else:
                    full.copy_(mine)
                GM.gemm(full, w, out=out)

            row = {"rows_per_rank": tr}
            for name, fn, st, per in (("fused_us", fused, stream, 1), ("fused_alternating_us", alternating, stream, 4),
                                      ("allgather_then_gemm_us", two_step, torch.cuda.current_stream(), 1)):
                for _ in range(3):
                    fn()
                torch.cuda.synchronize()
                if world > 1:
                    dist.barrier()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(st)
                for _ in range(20):
                    fn()
                e1.record(st)
                torch.cuda.synchronize()
                t = torch.tensor([e0.elapsed_time(e1) / 20 / per * 1e3], device=dev)
                if world > 1:
                    dist.all_reduce(t, op=dist.ReduceOp.MAX)
                row[name] = round(float(t), 1)
            rt.check_error()
            times.append(row)
        line["times_max_over_ranks"] = times
        line["note"] = "fused = barrier + all-gather GEMM + barrier in one captured program; the two-step form is NCCL all-gather + the plain tcgen05 GEMM"
    if rank == 0:
        print(json.dumps(line), flush=True)
    allok = all(r["ok"] for r in results)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0 if allok else 1


if __name__ == "__main__":
    raise SystemExit(main())
