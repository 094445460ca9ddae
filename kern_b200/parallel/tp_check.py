"""Self-check of the tensor-parallel path on N GPUs of one box (one process per GPU):

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        -m kern_b200.parallel.tp_check [--rows 8 300] [--time]

1. the fused peer all-reduce + residual + RMSNorm kernel against exact small-integer sums (one-shot and
   two-shot modes, eager and replayed from a CUDA graph);
2. the tensor-parallel dense decoder (tiny shape) against the same model on one GPU: prefill and decode logits;
3. with --time: the kernel's device time (max over ranks) for decode-sized and prefill-sized messages.

Every rank prints nothing but rank 0's JSON lines; exit code 0 means every check held.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist


def check_allreduce(rt, rank, world, rows_list, hidden, iters_graph=3):
    """Drive the manifest's allreduce_norm op alone through a tiny one-op manifest."""
    results = []
    for rows in rows_list:
        torch.manual_seed(1234)          # same on every rank
        parts = torch.randint(-3, 4, (world, rows, hidden), device="cuda").to(torch.bfloat16)
        x0 = torch.randint(-2, 3, (rows, hidden), device="cuda").to(torch.bfloat16)
        w = (torch.randint(1, 3, (hidden,), device="cuda")).to(torch.bfloat16)
        want_x = (parts.float().sum(0) + x0.float())
        want_xn = want_x * torch.rsqrt(want_x.pow(2).mean(-1, keepdim=True) + 1e-6) * w.float()
        for replay in (False, True):
            rt.tensor("part")[:rows] = parts[rank]
            rt.tensor("x")[:rows] = x0
            rt.tensor("w")[:] = w
            torch.cuda.synchronize()
            dist.barrier()
            if replay:
                for _ in range(iters_graph):      # the same graph replayed: the epoch lives on the device
                    rt.tensor("x")[:rows] = x0
                    torch.cuda.synchronize()
                    dist.barrier()
                    rt.run("step_graph", {"tokens": rows})
            else:
                rt.run("step", {"tokens": rows})
            rt.check_error()
            got_x, got_xn = rt.tensor("x")[:rows].float(), rt.tensor("xn")[:rows].float()
            ok = torch.equal(got_x, want_x) and torch.allclose(got_xn, want_xn, rtol=2e-2, atol=2e-2)
            results.append({"rows": rows, "graph": replay, "ok": bool(ok)})
            dist.barrier()
    return results


def allreduce_manifest(hidden, world, rows_max, lamport=False):
    from ..models import common as C

    bufs = {"part": {"dtype": "bf16", "shape": ["tokens", hidden], "kind": "input"},
            "x": {"dtype": "bf16", "shape": ["tokens", hidden], "kind": "inout", "export": True},
            "x_peers": {"dtype": "u64", "shape": [world], "kind": "peer", "of": "x", "group": "tp"},
            "xn": {"dtype": "bf16", "shape": ["tokens", hidden], "kind": "output"},
            "w": {"dtype": "bf16", "shape": [hidden], "kind": "input"},
            "error": {"dtype": "i32", "shape": [1], "kind": "output"}}
    bufs.update(C.tp_buffers(hidden, world, rows_max, lamport=lamport))
    B = lambda n: {"buf": n}
    call = {"op": "allreduce_norm", "args": [B("part"), B("x"), B("x_peers"), B("xn"), B("w"), B("tp.comm"), B("tp.comm_peers"),
                                             B("tp.flags"), B("tp.flags_peers"), B("tp.epochs"), B("error"), {"var": "tokens"}] +
            ([B("tp.lamport"), B("tp.lamport_peers"), B("tp.lamport_epochs")] if lamport else [])}
    return {"schema_version": 7, "model": "tp-allreduce-check",
            "vars": {"tokens": {"max": rows_max, "axis": "rows"}},
            "topology": {"groups": {"tp": world}}, "states": {}, "buffers": bufs,
            "modules": C.modules_for(["tp_allreduce_norm"] + (["misc"] if lamport else [])),
            "ops": {"allreduce_norm": C.tp_allreduce_norm_op(hidden, 1e-6, world, rows_max, lamport=lamport),
                    **({"lamport_init": C.tp_lamport_init_op(hidden, world)} if lamport else {})},
            "programs": {"step": {"calls": [call]},
                         **({"init": {"once": True, "calls": [{"op": "lamport_init", "args": [B("tp.lamport")]}]}} if lamport else {}),
                         # sixteen back-to-back calls in one graph: the per-call device time without launch gaps
                         "burst16": {"batch": {"groups": 1, "rows": "tokens"}, "graph": True, "calls": [call] * 16},
                         "step_graph": {"batch": {"groups": 1, "rows": "tokens"}, "graph": True, "calls": [call]}}}


def allgather_manifest(world, slot_bytes):
    from ..models import common as C

    bufs = {"x": {"dtype": "u8", "shape": [slot_bytes], "kind": "input"},
            "y": {"dtype": "u8", "shape": [world, slot_bytes], "kind": "output"},
            "error": {"dtype": "i32", "shape": [1], "kind": "output"}}
    bufs.update(C.tp_allgather_buffers(world, slot_bytes))
    B = lambda n: {"buf": n}
    call = {"op": "allgather", "args": [B("x"), B("y"), B("ag.sym"), B("ag.sym_peers"), B("ag.flags"), B("ag.flags_peers"),
                                        B("ag.epochs"), B("error"), {"var": "bytes"}]}
    return {"schema_version": 7, "model": "tp-allgather-check", "vars": {"bytes": {"max": slot_bytes}},
            "topology": {"groups": {"tp": world}}, "states": {}, "buffers": bufs,
            "modules": C.modules_for(["tp_allreduce_norm"]), "ops": {"allgather": C.tp_allgather_op(world, slot_bytes)},
            "programs": {"step": {"calls": [call]}, "burst16": {"calls": [call] * 16}}}


def check_allgather(rank, world, local, sizes=(16, 4096, 1 << 20), time_it=False):
    from ..runtime import Runtime
    from . import group

    slot = max(sizes)
    rt = Runtime(allgather_manifest(world, slot), gpu=local, topology={"tp": (rank, world)})
    group.start(rt)
    out = []
    for n in sizes:
        for rep in range(3):                 # parities alternate; the third call reuses the first one's buffer
            x = ((torch.arange(n, device="cuda") * 7 + rank * 31 + rep) % 251).to(torch.uint8)
            rt.tensor("x")[:n] = x
            torch.cuda.synchronize()
            dist.barrier()
            rt.run("step", {"bytes": n})
            rt.check_error()
            y = rt.tensor("y").view(-1)[: world * n].view(world, n)
            want = torch.stack([((torch.arange(n, device="cuda") * 7 + r * 31 + rep) % 251).to(torch.uint8) for r in range(world)])
            out.append({"bytes": n, "rep": rep, "ok": bool(torch.equal(y, want))})
            dist.barrier()
    times = []
    if time_it:
        stream = torch.cuda.ExternalStream(rt.stream)
        for n in sizes:
            for _ in range(3):
                rt.run("burst16", {"bytes": n})
            dist.barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record(stream)
            for _ in range(20):
                rt.issue("burst16", {"bytes": n})
            b.record(stream)
            rt.synchronize()
            t = torch.tensor([a.elapsed_time(b) / 320 * 1e3], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            times.append({"bytes_per_rank": n, "us_max_over_ranks": round(float(t), 2)})
    return out, times


def check_model(rank, world, fused=True, sp=False, sp_push=True):
    """`sp`: the ragged program in the sequence-parallel layout (scatter epilogue, reduce + norm on own rows, all-gather
    GEMM), with calls of several 128-row blocks, a ragged tail, and a second ragged call after decode steps."""
    from ..engine import Engine
    from ..models import dense, dense_tp
    from ..runtime import Runtime
    from . import group

    cfg = dense.DenseConfig(name="tiny-tp", vocab=512, hidden=256, layers=2, heads=8, kv_heads=max(2, world),
                            head_dim=64, intermediate=512 * world // 2, rope_theta=10000.0, page_size=16,
                            max_tokens=640 if sp else 256, max_seqs=8, max_context=512 if sp else 256, tp=world)
    weights = dense.random_weights(cfg, seed=0, std=0.05)
    doc = dense_tp.build_manifest_tp(cfg, fused=fused, sp=sp, sp_push=sp_push)
    # canary bands around every allocation, the exported ones included: the scatter epilogues and the pushes of the
    # peers write into this rank's memory, and a write past a region's end would land in its band
    rt = Runtime(doc, gpu=torch.cuda.current_device(), topology=group.topology(doc["topology"]["groups"], rank, world),
                 tokens=cfg.page_size * (160 if sp else 64), guard_bands=True)
    rt.load_tensors(lambda name: weights[name].cuda())
    group.start(rt)
    eng = Engine(rt)
    oracle = dense.DenseOracle(cfg, weights, device="cuda")
    torch.manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab, (n,)).tolist() for n in ((300, 5, 181) if sp else (37, 5, 80))]
    seqs = [eng.open(len(p) + 40) for p in prompts]
    caches = [oracle.new_cache() for _ in prompts]
    first = eng.step(list(zip(seqs, prompts)))
    worst = 0.0
    logits = rt.tensor("logits")[:3].float()
    for i, (p, c) in enumerate(zip(prompts, caches)):
        worst = max(worst, float((logits[i] - oracle.forward(p, c)[-1]).abs().max()))
    toks = [f[0] for f in first]
    for _ in range(4):
        refs = [oracle.forward([t], c)[-1] for t, c in zip(toks, caches)]
        nxt = eng.step([(s, [t]) for s, t in zip(seqs, toks)])
        logits = rt.tensor("logits")[:3].float()
        for i in range(3):
            worst = max(worst, float((logits[i] - refs[i]).abs().max()))
        toks = [n[0] for n in nxt]
    if sp:
        # a second and a third ragged call (the staging parity alternates): new sequences next to decode rows of the old
        for lens in ((70, 33), (129,)):
            more = [torch.randint(0, cfg.vocab, (n,)).tolist() for n in lens]
            new_seqs = [eng.open(len(p) + 8) for p in more]
            new_caches = [oracle.new_cache() for _ in more]
            refs = [oracle.forward([t], c)[-1] for t, c in zip(toks, caches)] + [oracle.forward(p, c)[-1] for p, c in zip(more, new_caches)]
            nxt = eng.step([(s_, [t]) for s_, t in zip(seqs, toks)] + list(zip(new_seqs, more)))
            logits = rt.tensor("logits")[:len(refs)].float()
            for i, r in enumerate(refs):
                worst = max(worst, float((logits[i] - r).abs().max()))
            toks = [n[0] for n in nxt[:3]]
            for s_ in new_seqs:
                eng.close(s_)
    rt.check_error()
    torch.distributed.barrier() if world > 1 else None      # every rank's writes into this rank's memory are done
    bad = rt.check_guards()
    return {"model_max_logit_diff": round(worst, 4), "ok": worst < 0.12 and not bad, "graphs": rt.graphs, "sp": sp,
            "guard_bands_overwritten": bad}


def check_moe(rank, world):
    """Expert-parallel MoE decoder (attention by heads, experts by ranges) against the one-GPU fp32 oracle."""
    import dataclasses

    from ..engine import Engine
    from ..models import moe, moe_ep
    from ..runtime import Runtime
    from . import group

    cfg = dataclasses.replace(moe.TINY_MOE, name="tiny-moe-ep", heads=8, kv_heads=max(2, world), experts=16, top_k=4, tp=world)
    weights = moe.random_weights(cfg, seed=0, std=0.05)
    doc = moe_ep.build_manifest_ep(cfg)
    rt = Runtime(doc, gpu=torch.cuda.current_device(), topology=group.topology(doc["topology"]["groups"], rank, world),
                 tokens=cfg.page_size * 64)
    rt.load_tensors(lambda name: weights[name].cuda())
    group.start(rt)
    eng = Engine(rt)
    oracle = moe.MoeOracle(cfg, weights, device="cuda")
    torch.manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab, (n,)).tolist() for n in (37, 5, 80)]
    seqs = [eng.open(120) for _ in prompts]
    caches = [oracle.new_cache() for _ in prompts]
    first = eng.step(list(zip(seqs, prompts)))
    diffs = []
    logits = rt.tensor("logits")[:3].float()
    for i, (p, c) in enumerate(zip(prompts, caches)):
        diffs.append((logits[i] - oracle.forward(p, c)[-1]).abs())
    toks = [f[0] for f in first]
    for _ in range(4):
        refs = [oracle.forward([t], c)[-1] for t, c in zip(toks, caches)]
        nxt = eng.step([(s, [t]) for s, t in zip(seqs, toks)])
        logits = rt.tensor("logits")[:3].float()
        diffs += [(logits[i] - refs[i]).abs() for i in range(3)]
        toks = [n[0] for n in nxt]
    rt.check_error()
    worst, mean = max(float(d.max()) for d in diffs), max(float(d.mean()) for d in diffs)
    return {"moe_max_logit_diff": round(worst, 4), "moe_mean_logit_diff": round(mean, 4), "ok": worst < 0.3 and mean < 0.05}


def time_allreduce(rt, world, rows_list, iters=20):
    out = []
    stream = torch.cuda.ExternalStream(rt.stream)
    for rows in rows_list:
        for _ in range(3):
            rt.run("burst16", {"tokens": rows})
        dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record(stream)
        for _ in range(iters):
            rt.issue("burst16", {"tokens": rows})
        b.record(stream)
        rt.synchronize()
        t = torch.tensor([a.elapsed_time(b) / (16 * iters) * 1e3], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        out.append({"rows": rows, "us_max_over_ranks": round(float(t), 2)})
    return out


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, nargs="*", default=[1, 8, 64, 65, 300, 1000])
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--time", action="store_true")
    ap.add_argument("--skip-model", action="store_true")
    ap.add_argument("--no-lamport", action="store_true", help="decode-sized all-reduce through flags instead of the flagless one-shot")
    ap.add_argument("--moe", action="store_true", help="also check the expert-parallel MoE decoder")
    ap.add_argument("--unfused", action="store_true", help="the model check without the GEMM + reduce-scatter fusion")
    ap.add_argument("--sp", action="store_true", help="also check the decoder with the sequence-parallel ragged program")
    ap.add_argument("--only-sp", action="store_true", help="run the sequence-parallel decoder check alone")
    args = ap.parse_args(argv)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    from ..runtime import Runtime
    from . import group

    if args.only_sp:
        from . import group as _g   # noqa: F401
        ok_all = True
        for push in (True, False):
            m = check_model(rank, world, sp=True, sp_push=push)
            ok_all &= m["ok"]
            if rank == 0:
                print(json.dumps({"check": "tp_model_sp", "world": world, "all_gather": "push" if push else "pull", **m}))
        flag = torch.tensor([int(ok_all)], device="cuda")
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        dist.destroy_process_group()
        return 0 if int(flag) else 1
    rows_max = max(args.rows + [4096 if args.time else 1])
    rt = Runtime(allreduce_manifest(args.hidden, world, rows_max, lamport=not args.no_lamport), gpu=local,
                 topology={"tp": (rank, world)})
    group.start(rt)
    ok = True
    res = check_allreduce(rt, rank, world, args.rows, args.hidden)
    ok &= all(r["ok"] for r in res)
    if rank == 0:
        print(json.dumps({"check": "allreduce_residual_norm", "world": world, "results": res}))
    if args.time:
        t = time_allreduce(rt, world, [1, 8, 16, 32, 64, 256, 1024, 4096])
        if rank == 0:
            print(json.dumps({"check": "allreduce_time", "hidden": args.hidden, "world": world, "lamport": not args.no_lamport,
                              "results": t}))
    ag, ag_t = check_allgather(rank, world, local, time_it=args.time)
    ok &= all(r["ok"] for r in ag)
    if rank == 0:
        print(json.dumps({"check": "allgather", "world": world, "ok": all(r["ok"] for r in ag), "times": ag_t}))
    if not args.skip_model:
        m = check_model(rank, world, fused=not args.unfused)
        ok &= m["ok"]
        if rank == 0:
            print(json.dumps({"check": "tp_model", "world": world, "fused_gemm_reduce_scatter": not args.unfused, **m}))
    if args.sp and not args.skip_model:
        m = check_model(rank, world, sp=True)
        ok &= m["ok"]
        if rank == 0:
            print(json.dumps({"check": "tp_model_sp", "world": world, **m}))
    if args.moe:
        e = check_moe(rank, world)
        ok &= e["ok"]
        if rank == 0:
            print(json.dumps({"check": "ep_moe_model", "world": world, **e}))
    flag = torch.tensor([int(ok)], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    dist.destroy_process_group()
    return 0 if int(flag) else 1


if __name__ == "__main__":
    sys.exit(main())
