"""Expert parallelism over sharded tokens, checked on N ranks (one process per GPU): every rank holds its own tokens and
1/N of the experts. One captured program per layer call:

    all-gather of the expert ids (NCCL built-in)  ->  barrier  ->  plan over all tokens, own experts only
    ->  dispatch = the gather pulls exactly the needed rows out of the home ranks' activation buffers (NVLink peer loads)
    ->  grouped tcgen05 GEMM + SwiGLU  ->  grouped GEMM
    ->  combine = every result row is pushed into its slot on the token's home rank (NVLink peer stores)  ->  barrier
    ->  the home rank weighs its k slots

The result must equal the dense evaluation of the same mixture (every expert's weights are generated from one seed on
every rank). Timed against the replicated layout (`models/moe_ep.py`: every rank sees all tokens, partial sums all-reduced).

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 -m kern_b200.parallel.ep_check --time

Reference: docs/roadmap.md:13-16,63 (all-to-all dispatch / combine around the routed GEMMs), docs/serve.md:402-453.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def manifest(world: int, rows_max: int, hidden: int, inter: int, experts: int, k: int) -> dict:
    """`rows_max`: tokens per rank. Experts are dealt in contiguous ranges of experts / world."""
    from ..models import common as C

    assert experts % world == 0
    e_n = experts // world
    T = rows_max * world
    max_tiles = T * k // C.BM + e_n
    buf = lambda dt, shape, kind="workspace", **kw: {"dtype": dt, "shape": shape, "kind": kind, **kw}
    peer = lambda of: {"dtype": "u64", "shape": [world], "kind": "peer", "of": of, "group": "ep"}
    bufs = {
        "ep.x": buf("bf16", [rows_max, hidden], "inout", export=True), "ep.x_peers": peer("ep.x"),
        "ep.ret": buf("bf16", [rows_max, k, hidden], "inout", export=True), "ep.ret_peers": peer("ep.ret"),
        "ep.bar": buf("u32", [32], "carry", export=True), "ep.bar_peers": peer("ep.bar"), "ep.bar_epoch": buf("u32", [1], "carry"),
        "ids": buf("i32", ["rows", k], "input"), "w": buf("f32", ["rows", k], "input"), "iota": buf("i32", ["rows", k], "input"),
        "ids_all": buf("i32", [T, k]), "perm": buf("i32", [T, k]), "offsets": buf("i32", [e_n + 1]), "tiles": buf("i32", [max_tiles, 4]),
        "tile_count": buf("i32", [1]), "n_rows": buf("i32", [1]),
        "xp": buf("bf16", [T * k, hidden]), "act": buf("bf16", [T * k, inter]), "y": buf("bf16", [T * k, hidden]),
        "w1": buf("bf16", [e_n, 2 * inter, hidden], "input"), "w2": buf("bf16", [e_n, hidden, inter], "input"),
        "out": buf("bf16", ["rows", hidden], "output"), "error": buf("i32", [1], "output"),
    }
    L = lambda module, entry, block, grid, lp, args, **kw: {"module": module, "entry": entry, "block": block, "grid": grid,
                                                            "params": lp, "args": args, **kw}
    all_entries = {"mul": ["rows", world * k]}
    ops = {}
    ops["ids_allgather"] = {"params": ["in buffer<i32>", "out buffer<i32>", "i64", "i32"],
                            "impl": {"launches": [{"entry": "extern:nccl_allgather_i32"}]}}
    ops["barrier"] = {"params": ["inout buffer<u32>", "in buffer<u64>", "inout buffer<u32>", "out buffer<i32>"], "impl": {"launches": [L(
        "tp_allreduce_norm", "kern_peer_barrier", [32, 1, 1], [1, 1, 1],
        ["inout buffer<u32>", "in buffer<u64>", "inout buffer<u32>", "out buffer<i32>", "i32", "i32", "i64"],
        [{"param": 0}, {"param": 1}, {"param": 2}, {"param": 3}, {"rank": "ep"}, {"i32": world}, {"i64": 2_000_000_000}])]}}
    ops["plan"] = {"params": ["in buffer<i32>", "out buffer<i32>", "out buffer<i32>", "out buffer<i32>", "out buffer<i32>",
                              "out buffer<i32>", "i32", "out buffer<i32>"], "impl": {"launches": [L(
        "moe", "kern_moe_plan", [1024, 1, 1], [1, 1, 1],
        ["in buffer<i32>", "out buffer<i32>", "out buffer<i32>", "out buffer<i32>", "out buffer<i32>", "out buffer<i32>", "i32",
         "i32", "i32", "i32", "i32", "out buffer<i32>", "i32", "i32"],
        [{"param": 0}, {"param": 1}, {"param": 2}, {"param": 3}, {"param": 4}, {"param": 5}, {"param": 6}, {"i32": 0},
         {"i32": e_n}, {"i32": C.BM}, {"i32": max_tiles}, {"param": 7}, {"rank": "ep"}, {"i32": e_n}], shared_mem=2 * e_n * 4)]}}
    ops["dispatch"] = {"params": ["in buffer<u64>", "in buffer<i32>", "out buffer<bf16>", "i32", "i32"], "impl": {"launches": [L(
        "moe", "kern_moe_gather_peers_bf16", [128, 1, 1], [all_entries, 1, 1],
        ["in buffer<u64>", "in buffer<i32>", "out buffer<bf16>", "i32", "i32", "i32", "i32"],
        [{"param": 0}, {"param": 1}, {"param": 2}, {"param": 3}, {"i32": k}, {"i32": hidden}, {"param": 4}])]}}

    def routed(n, kk, epi):
        bn = 128 if n >= 128 else 64
        out_cols = n // 2 if epi == "swiglu" else n
        a_map = {"pack": {"size": 128, "fields": [{"at": 0, "tensormap": {
            "param": 0, "dtype": "bf16", "dims": [kk, 0], "strides": [kk * 2], "box": [C.BK, C.BM], "swizzle": 128, "l2_promotion": 256}}]}}
        b_map = {"pack": {"size": 128, "fields": [{"at": 0, "tensormap": {
            "param": 1, "dtype": "bf16", "dims": [kk, n, e_n], "strides": [kk * 2, n * kk * 2],
            "box": [C.BK, bn // 2 if epi == "swiglu" else bn, 1], "swizzle": 128, "l2_promotion": 256}}]}}
        return {"params": ["in buffer<bf16>", "in buffer<bf16>", "out buffer<bf16>", "in buffer<i32>", "in buffer<i32>", "i32",
                           "out buffer<i32>"], "impl": {"launches": [L(
            "moe", f"kern_moe_gemm_bf16{'_swiglu' if epi == 'swiglu' else ''}_n{bn}", [192, 1, 1], [C.SMS, 1, 1],
            ["bytes<128>", "bytes<128>", "out buffer<bf16>", "in buffer<i32>", "in buffer<i32>", "i32", "i32", "i32", "i32",
             "out buffer<i32>"],
            [a_map, b_map, {"param": 2}, {"param": 3}, {"param": 4}, {"param": 5}, {"i32": n}, {"i32": kk}, {"i32": out_cols},
             {"param": 6}], shared_mem=C.gemm_smem(bn))]}}

    ops["fc1"] = routed(2 * inter, hidden, "swiglu")
    ops["fc2"] = routed(hidden, inter, "store")
    ops["return"] = {"params": ["in buffer<bf16>", "in buffer<i32>", "in buffer<u64>", "i32", "i32"], "impl": {"launches": [L(
        "moe", "kern_moe_return_bf16", [128, 1, 1], [all_entries, 1, 1],
        ["in buffer<bf16>", "in buffer<i32>", "in buffer<u64>", "i32", "i32", "i32", "i32"],
        [{"param": 0}, {"param": 1}, {"param": 2}, {"param": 3}, {"i32": k}, {"i32": hidden}, {"param": 4}])]}}
    ops["combine"] = {"params": ["in buffer<bf16>", "in buffer<i32>", "in buffer<f32>", "out buffer<bf16>"], "impl": {"launches": [L(
        "moe", "kern_moe_combine_bf16", [128, 1, 1], ["rows", 1, 1],
        ["in buffer<bf16>", "in buffer<i32>", "in buffer<f32>", "i64", "out buffer<bf16>", "i32", "i32", "i32", "i32"],
        [{"param": 0}, {"param": 1}, {"param": 2}, {"i64": 0}, {"param": 3}, {"i32": C.I32_MAX}, {"i32": k}, {"i32": hidden},
         {"i32": 0}])]}}
    B = lambda n: {"buf": n}
    E = lambda x: {"expr": x}
    bar = {"op": "barrier", "args": [B("ep.bar"), B("ep.bar_peers"), B("ep.bar_epoch"), B("error")]}
    calls = [
        {"op": "ids_allgather", "label": "ids", "args": [B("ids"), B("ids_all"), E({"mul": ["rows", k]}), {"rank": "ep"}]},
        dict(bar, label="bar_open"),
        {"op": "plan", "label": "plan", "args": [B("ids_all"), B("perm"), B("offsets"), B("tiles"), B("tile_count"), B("n_rows"),
                                                 E(all_entries), B("error")]},
        {"op": "dispatch", "label": "dispatch", "args": [B("ep.x_peers"), B("perm"), B("xp"), E(all_entries), {"var": "rows"}]},
        {"op": "fc1", "label": "fc1", "args": [B("xp"), B("w1"), B("act"), B("tiles"), B("tile_count"), E(all_entries), B("error")]},
        {"op": "fc2", "label": "fc2", "args": [B("act"), B("w2"), B("y"), B("tiles"), B("tile_count"), E(all_entries), B("error")]},
        {"op": "return", "label": "return", "args": [B("y"), B("perm"), B("ep.ret_peers"), E(all_entries), {"var": "rows"}]},
        dict(bar, label="bar_close"),
        {"op": "combine", "label": "combine", "args": [B("ep.ret"), B("iota"), B("w"), B("out")]},
    ]
    return {"schema_version": 7, "model": "ep-all-to-all-check", "vars": {"rows": {"max": rows_max, "axis": "rows"}},
            "topology": {"groups": {"ep": world}}, "states": {}, "buffers": bufs,
            "modules": C.modules_for(["moe", "tp_allreduce_norm"]), "ops": ops,
            "programs": {"step": {"calls": calls},
                         "step_graph": {"batch": {"groups": 1, "rows": "rows"}, "graph": True, "calls": calls}}}


def manifest_fused(world: int, rows_max: int, hidden: int, inter: int, experts: int, k: int, bn: int | None = None,
                   mx: bool = False) -> dict:
    """The same layer with the dispatch inside FC1 and the combine inside FC2 (`moe.cu`, the `kern_ep_*` entries): five
    launches, no barrier kernel, no NCCL call. `rows_max`: tokens per rank. `mx`: MXFP4 expert weights and MXFP8
    activations (`gemm_mx.cu`): a sixth launch quantises this rank's rows once, and e4m3 rows cross NVLink."""
    from ..models import common as C
    from ..models import moe_ep

    assert experts % world == 0 and hidden % 8 == 0
    e_n = experts // world
    buf = lambda dt, shape, kind="workspace", **kw: {"dtype": dt, "shape": shape, "kind": kind, **kw}
    if mx:
        from ..ops.gemm_mx import atom_bytes

        bufs = {
            "x": buf("bf16", ["rows", hidden], "input"),
            "ids": buf("i32", ["rows", k], "input"), "w": buf("f32", ["rows", k], "input"),
            "w1": buf("u8", [e_n, 2 * inter, hidden // 2], "input"), "sf1": buf("u8", [e_n, atom_bytes(2 * inter, hidden)], "input"),
            "w2": buf("u8", [e_n, hidden, inter // 2], "input"), "sf2": buf("u8", [e_n, atom_bytes(hidden, inter)], "input"),
            "out": buf("bf16", ["rows", hidden], "output"), "error": buf("i32", [1], "output"),
            **moe_ep.ep_fused_buffers_mx(world, rows_max, hidden, inter, e_n, k),
        }
        ops = moe_ep.ep_fused_ops_mx(world, rows_max, hidden, inter, e_n, k, "rows", bn=bn)
        calls = moe_ep.ep_fused_calls("ids", "w", "x", "w1", "w2", "out", "rows", mx=("sf1", "sf2"))
        return {"schema_version": 7, "model": "ep-fused-mx-check", "vars": {"rows": {"max": rows_max, "axis": "rows"}},
                "topology": {"groups": {"ep": world}}, "states": {}, "buffers": bufs,
                "modules": C.modules_for(["moe", "gemm_mx"]), "ops": ops,
                "programs": {"step": {"calls": calls},
                             "step_graph": {"batch": {"groups": 1, "rows": "rows"}, "graph": True, "calls": calls}}}
    bufs = {
        "ep.x": buf("bf16", [rows_max, hidden], "inout", export=True),
        "ids": buf("i32", ["rows", k], "input"), "w": buf("f32", ["rows", k], "input"),
        "w1": buf("bf16", [e_n, 2 * inter, hidden], "input"), "w2": buf("bf16", [e_n, hidden, inter], "input"),
        "out": buf("bf16", ["rows", hidden], "output"), "error": buf("i32", [1], "output"),
        **moe_ep.ep_fused_buffers(world, rows_max, hidden, inter, e_n, k, "ep.x"),
    }
    ops = moe_ep.ep_fused_ops(world, rows_max, hidden, inter, e_n, k, "rows", bn=bn)
    calls = moe_ep.ep_fused_calls("ids", "w", "ep.x", "w1", "w2", "out", "rows")
    return {"schema_version": 7, "model": "ep-fused-check", "vars": {"rows": {"max": rows_max, "axis": "rows"}},
            "topology": {"groups": {"ep": world}}, "states": {}, "buffers": bufs,
            "modules": C.modules_for(["moe"]), "ops": ops,
            "programs": {"step": {"calls": calls},
                         "step_graph": {"batch": {"groups": 1, "rows": "rows"}, "graph": True, "calls": calls}}}


def check_model(rank: int, world: int, dev, traffic: int | None = None, mx: bool = False) -> dict:
    """The MoE decoder with tokens sharded over the group (`models/moe_ep.py::build_manifest_ep_sharded`): every rank
    serves its own prompts, the routed layers are the fused kernels; logits against the one-GPU fp32 oracle. `mx`: the
    decoder with MXFP4 experts; its logits against the one-GPU manifest of the same block-scaled checkpoint on this
    GPU (the same quantisation points, so only the order of the sums differs)."""
    import dataclasses

    from ..engine import Engine
    from ..models import moe, moe_ep
    from ..runtime import Runtime
    from . import group

    cfg = dataclasses.replace(moe.TINY_MOE, name="tiny-moe-eps", experts=16, top_k=4)
    weights = moe.random_weights(cfg, seed=0, std=0.05)
    if mx:
        cfg = dataclasses.replace(cfg, name="tiny-moe-eps-mx", mx_experts=True, moe_intermediate=128)
        weights = moe.mx_checkpoint(cfg, moe.random_weights(cfg, seed=0, std=0.05))
    doc = moe_ep.build_manifest_ep_sharded(cfg, world)
    rt = Runtime(doc, gpu=dev.index, topology=group.topology(doc["topology"]["groups"], rank, world), tokens=cfg.page_size * 64)
    rt.load_tensors(lambda name: weights[name].to(dev))
    group.start(rt)
    eng = Engine(rt)
    g = torch.Generator().manual_seed(100 + (rank if traffic is None else traffic))     # every rank has its own traffic
    prompts = [torch.randint(0, cfg.vocab, (int(n),), generator=g).tolist() for n in torch.randint(3, 90, (3,), generator=g)]
    seqs = [eng.open(140) for _ in prompts]
    if mx:
        ref_rt = Runtime(moe.build_manifest(cfg), gpu=dev.index, tokens=cfg.page_size * 64)
        ref_rt.load_tensors(lambda name: weights[name].to(dev))
        ref_rt.once()
        ref = Engine(ref_rt)
        rseqs = [ref.open(140) for _ in prompts]

        def want(batch):
            ref.step(list(zip(rseqs, batch)))
            ref_rt.check_error()
            return ref_rt.tensor("logits")[:3].float().clone()
    else:
        oracle = moe.MoeOracle(cfg, weights, device="cuda")
        caches = [oracle.new_cache() for _ in prompts]
        want = lambda batch: torch.stack([oracle.forward(p, c)[-1] for p, c in zip(batch, caches)])
    refs = want(prompts)
    first = eng.step(list(zip(seqs, prompts)))
    diffs = [(rt.tensor("logits")[:3].float() - refs).abs()]
    toks = [f[0] for f in first]
    for _ in range(4):                                                   # the same number of steps on every rank
        refs = want([[t] for t in toks])
        nxt = eng.step([(s, [t]) for s, t in zip(seqs, toks)])
        diffs.append((rt.tensor("logits")[:3].float() - refs).abs())
        toks = [n[0] for n in nxt]
    rt.check_error()
    worst, mean = max(float(d.max()) for d in diffs), max(float(d.mean(-1).max()) for d in diffs)
    # bf16 against the fp32 oracle with std 0.05 weights: the mean difference sits at 0.01-0.05 depending on the prompts
    ok = torch.tensor([int(worst < 0.3 and mean < 0.08)], device=dev)
    if world > 1:
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    mine = torch.tensor([worst, mean], device=dev)
    every = [torch.zeros_like(mine) for _ in range(world)]
    if world > 1:
        dist.all_gather(every, mine)
    else:
        every = [mine]
    return {"max_logit_diff": round(worst, 4), "mean_logit_diff": round(mean, 4), "graphs": rt.graphs, "ok": bool(ok.item()),
            "by_rank": [[round(float(x[0]), 4), round(float(x[1]), 4)] for x in every]}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, nargs="+", default=[8, 200, 64], help="tokens per rank")
    ap.add_argument("--hidden", type=int, default=1024)
    ap.add_argument("--inter", type=int, default=512)
    ap.add_argument("--experts", type=int, default=16)
    ap.add_argument("--top-k", type=int, default=4)
    ap.add_argument("--time", action="store_true")
    ap.add_argument("--fused", action="store_true", help="dispatch inside FC1, combine inside FC2 (five launches per layer)")
    ap.add_argument("--mx", action="store_true", help="with --fused: MXFP4 expert weights, MXFP8 activations (block-scaled tcgen05 GEMMs)")
    ap.add_argument("--bn", type=int, default=None, choices=[64, 128, 256], help="tile width of the fused routed GEMMs (default: by row count)")
    ap.add_argument("--traffic", type=int, default=None, help="the model check with the prompts rank N of a larger group would get")
    ap.add_argument("--model", action="store_true", help="also run the MoE decoder with sharded tokens and fused routed layers")
    a = ap.parse_args(argv)
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device(f"cuda:{local}")
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    from ..runtime import Runtime
    from . import group

    h, I, E, k = a.hidden, a.inter, a.experts, a.top_k
    e_n = E // world
    rows_max = max(a.rows)
    doc = manifest_fused(world, rows_max, h, I, E, k, bn=a.bn, mx=a.mx) if a.fused else manifest(world, rows_max, h, I, E, k)
    xname = "x" if a.fused and a.mx else "ep.x"
    rt = Runtime(doc, gpu=local, topology={"ep": (rank, world)},
                 guard_bands=True)      # canary bands around every allocation: the peers' adds and stores land in this rank's memory
    group.start(rt)
    g = torch.Generator().manual_seed(21)
    w1 = (torch.randn(E, 2 * I, h, generator=g) * 0.05).to(torch.bfloat16)       # [gate rows ; up rows] per expert
    w2 = (torch.randn(E, h, I, generator=g) * 0.05).to(torch.bfloat16)
    if a.fused and a.mx:
        from ..ops import gemm_mx as G
        from ..ops import moe as M

        mine = slice(rank * e_n, (rank + 1) * e_n)
        q1, s1, q2, s2 = M.prepare_expert_weights_mx(w1[mine].to(dev).float(), w2[mine].to(dev).float())
        for name, t in (("w1", q1), ("sf1", s1), ("w2", q2), ("sf2", s2)):
            rt.tensor(name).copy_(t.reshape(rt.tensor(name).shape))
        # the statement: every expert's weights through MXFP4 and back, activations through MXFP8 before each GEMM
        w1d = torch.stack([G.dequant_mxfp4(*G.quantize_mxfp4_torch(w1[e].to(dev).float())) for e in range(E)])
        w2d = torch.stack([G.dequant_mxfp4(*G.quantize_mxfp4_torch(w2[e].to(dev).float())) for e in range(E)])
        q8 = lambda t: G.dequant_mxfp8(*G.quantize_mxfp8_torch(t))
    else:
        rt.tensor("w1").copy_(w1[rank * e_n:(rank + 1) * e_n].to(dev))
        rt.tensor("w2").copy_(w2[rank * e_n:(rank + 1) * e_n].to(dev))
        w1d, w2d = w1.to(dev).float(), w2.to(dev).float()
        q8 = None
    results = []
    for it, tr in enumerate(a.rows + a.rows[:1]):
        program = "step_graph" if it >= len(a.rows) else "step"
        gi = torch.Generator().manual_seed(300 + it)
        xs = [(torch.randn(tr, h, generator=gi) * 0.5).to(torch.bfloat16) for _ in range(world)]
        ids = [torch.stack([torch.randperm(E, generator=gi)[:k] for _ in range(tr)]).to(torch.int32) for _ in range(world)]
        ws = [torch.rand(tr, k, generator=gi) for _ in range(world)]
        rt.tensor(xname)[:tr].copy_(xs[rank].to(dev))
        rt.tensor("ids").view(-1)[: tr * k].copy_(ids[rank].reshape(-1).to(dev))
        rt.tensor("w").view(-1)[: tr * k].copy_(ws[rank].reshape(-1).to(dev))
        if not a.fused:
            rt.tensor("iota").view(-1)[: tr * k].copy_(torch.arange(tr * k, dtype=torch.int32, device=dev))
            rt.tensor("ep.ret").fill_(float("nan"))        # a slot nobody returns to would poison the sum
        torch.cuda.synchronize()
        rt.run(program, {"rows": tr})
        rt.check_error()
        got = rt.tensor("out")[:tr].float()
        x = xs[rank].to(dev).float()
        if q8 is not None:
            x = q8(x)
        want = torch.zeros(tr, h, device=dev)
        for t in range(tr):
            for j in range(k):
                e = int(ids[rank][t, j])
                gu = w1d[e] @ x[t]
                act = torch.nn.functional.silu(gu[:I]) * gu[I:]
                act = q8(act[None])[0] if q8 is not None else act.to(torch.bfloat16).float()
                want[t] += float(ws[rank][t, j]) * (w2d[e] @ act).to(torch.bfloat16).float()
        err = float((got - want).abs().max())
        tol = 0.05 * max(1.0, float(want.abs().max()))
        ok = torch.tensor([int(err < tol and bool(torch.isfinite(got).all()))], device=dev)
        if world > 1:
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        results.append({"rows_per_rank": tr, "program": program, "max_abs_err": round(err, 4), "ok": bool(ok.item())})
    if world > 1:
        dist.barrier()
    bad = rt.check_guards()
    results.append({"guard_bands_overwritten": bad, "ok": not bad})
    line = {"check": ("expert_parallel_fused_mx" if a.mx else "expert_parallel_fused") if a.fused else "expert_parallel_all_to_all", "world": world, "experts": E, "top_k": k, "hidden": h, "results": results}
    if a.time:
        stream = torch.cuda.ExternalStream(rt.stream)
        times = []
        for tr in a.rows:
            for _ in range(3):
                rt.issue("step_graph", {"rows": tr})
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(20):
                rt.issue("step_graph", {"rows": tr})
            e1.record(stream)
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1) / 20 * 1e3], device=dev)
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            times.append({"rows_per_rank": tr, "layer_us_max_over_ranks": round(float(t), 1)})
        rt.check_error()
        line["times"] = times
        # cost by call of the largest size: eager, an event between calls, median of 5 (waits for peers included)
        tr = max(a.rows)
        samples = []
        for _ in range(6):
            if world > 1:
                dist.barrier()
            samples.append(rt.issue_timed("step", {"rows": tr}))
        rt.check_error()
        by = {}
        for smp in samples[1:]:
            for label, op, ms, _ in smp:
                by.setdefault(label, []).append(ms * 1e3)
        line["by_call_us"] = {"rows_per_rank": tr, **{l: round(sorted(v)[len(v) // 2], 1) for l, v in by.items()}}
    if rank == 0:
        print(json.dumps(line), flush=True)
    model_ok = True
    if a.model:
        m = check_model(rank, world, dev, a.traffic, mx=a.mx)
        model_ok = m["ok"]
        if rank == 0:
            print(json.dumps({"check": "expert_parallel_sharded_decoder" + ("_mx" if a.mx else ""), "world": world, **m}), flush=True)
    allok = all(r["ok"] for r in results) and model_ok
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0 if allok else 1


if __name__ == "__main__":
    raise SystemExit(main())
