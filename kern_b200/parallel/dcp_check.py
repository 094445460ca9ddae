"""Decode context parallelism across GPUs, checked on N ranks (`torch.distributed.run`, one process per GPU): the
positions of every sequence are dealt round-robin (position p lives on member p % N at local index p / N), every rank
runs the paged decode attention over its own pages and leaves un-normalised partials (o, m, l), the partials are
all-gathered over NVLink and merged once; the result must equal attention over the whole context.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 -m kern_b200.parallel.dcp_check

Reference: crates/kern-pool/src/deal.rs:26-156 (the dealing), docs/pool.md:199-211; the reference merges the partial
softmax inside its attention kernels' callers the same way (log-sum-exp merge).
"""
from __future__ import annotations

import argparse
import json
import os

import numpy as np
import torch
import torch.distributed as dist


def check_model(rank: int, world: int, local: int, steps: int = 6, cpu: bool = False) -> dict:
    """The dense decoder as a context-parallel decode group: every rank prefills the prompts on a whole-context
    runtime of its own (the stand-in for a prefill tier), deals the KV rows to its member pool, and the group decodes;
    logits are compared step by step with the whole-context runtime decoding the same tokens."""
    from ..engine import Engine
    from .. import fills
    from ..models import dense, dense_dcp
    from ..ops import attention as A
    from ..runtime import Runtime
    from . import group

    cfg = dense.TINY
    dev = torch.device("cpu" if cpu else f"cuda:{local}")
    weights = dense.random_weights(cfg, seed=0, std=0.05)
    if cpu:       # gloo ranks and the host-memory executor: the same manifests, PyTorch statements per kernel
        from ..cpu import CPU_KERNELS, CpuRuntime

        full = CpuRuntime(dense.build_manifest(cfg), weights=weights, tokens=cfg.page_size * 64)
        rt = CpuRuntime(dense_dcp.build_manifest_dcp(cfg, world), weights=weights, tokens=cfg.page_size * 64,
                        topology={"dcp": (rank, world)})
        full.once()
        rt.once()
    else:
        full = Runtime(dense.build_manifest(cfg), gpu=local, tokens=cfg.page_size * 64, slots=8)
        full.load_tensors(lambda name: weights[name].to(dev))
        full.once()
        rt = Runtime(dense_dcp.build_manifest_dcp(cfg, world), gpu=local, topology={"dcp": (rank, world)},
                     tokens=cfg.page_size * 64, slots=8)
        rt.load_tensors(lambda name: weights[name].to(dev))
        if world > 1:
            group.start(rt)
        else:
            rt.once()
    eng = Engine(full)
    member = Engine(rt)          # its fills and readers; pages are assigned by hand below
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, cfg.vocab, (n,), generator=g).tolist() for n in (45, 3, 130, 17)]
    seqs = [eng.open(len(p) + steps + 2) for p in prompts]
    first = eng.step(list(zip(seqs, prompts)))
    toks = [f[0] for f in first]
    # member pages: each sequence gets enough local pages for its share of (prompt + steps), ids from 1
    page, W = cfg.page_size, cfg.table_width
    local_pages, nxt = [], 1
    for p in prompts:
        n = -(-(-(-(len(p) + steps + 2) // world)) // page) + 1
        local_pages.append(list(range(nxt, nxt + n)))
        nxt += n
    src_table = torch.zeros(len(prompts), W, dtype=torch.int32, device=dev)
    dst_table = torch.zeros(len(prompts), W, dtype=torch.int32, device=dev)
    for i, s in enumerate(seqs):
        pg = list(s.lease.pages)
        src_table[i, : len(pg)] = torch.tensor(pg, dtype=torch.int32)
        dst_table[i, : len(local_pages[i])] = torch.tensor(local_pages[i], dtype=torch.int32)
    lens = torch.tensor([len(p) for p in prompts], dtype=torch.int32, device=dev)
    for i in range(cfg.layers):
        if cpu:
            CPU_KERNELS["kern_deal_rows_bf16"]((1, len(prompts), 1), full.states[f"kv.l{i}"], rt.states[f"kv.l{i}"], src_table,
                                               dst_table, lens, len(prompts), W, W, cfg.kv_heads, cfg.head_dim, page, rank,
                                               world, 0, None)
        else:
            full.synchronize()
            A.deal_rows(full.tensor(f"kv.l{i}"), rt.tensor(f"kv.l{i}"), src_table, dst_table, lens, cfg.kv_heads, cfg.head_dim,
                        page, rank, world)
    if not cpu:
        torch.cuda.synchronize()
    # The decode calls are staged by the serving host's own code (`serve/ranks.py`, a by-position group): it leases every
    # member its share of each sequence, and builds the member's item with its own page table and dealt slots. The
    # member pools it keeps account of are the ones filled above, so its leases must name the same pages.
    from types import SimpleNamespace

    from ..serve.ranks import Ranks

    ranks = Ranks(member.p, member.unit, [nxt + 4] * world, [8] * world, tp=world, by_position=True)
    seqs_g = []
    for i, p in enumerate(prompts):
        gl = ranks.lease(0, len(p) + steps + 2)
        seqs_g.append(SimpleNamespace(lease=gl, length=len(p), sampling=seqs[i].sampling))
    mine = [list(sg.lease.members[rank].pages) for sg in seqs_g]
    # re-deal into the pages the host's leases name (the hand-made tables above only sized the pool)
    dst_table.zero_()
    for i, pg in enumerate(mine):
        dst_table[i, : len(pg)] = torch.tensor(pg, dtype=torch.int32)
    for i in range(cfg.layers):
        if cpu:
            CPU_KERNELS["kern_deal_rows_bf16"]((1, len(prompts), 1), full.states[f"kv.l{i}"], rt.states[f"kv.l{i}"], src_table,
                                               dst_table, lens, len(prompts), W, W, cfg.kv_heads, cfg.head_dim, page, rank,
                                               world, 0, None)
        else:
            A.deal_rows(full.tensor(f"kv.l{i}"), rt.tensor(f"kv.l{i}"), src_table, dst_table, lens, cfg.kv_heads, cfg.head_dim,
                        page, rank, world)
    if not cpu:
        torch.cuda.synchronize()
    worst, agree = 0.0, 0
    for _ in range(steps):
        ref_next = eng.step([(s, [t]) for s, t in zip(seqs, toks)])
        ref_logits = full.tensor("logits")[: len(prompts)].float().clone()
        staged = ranks.stage(0, [(sg, [t]) for sg, t in zip(seqs_g, toks)])
        item = ranks.item_for(staged, rank)
        for name, (dtype, col) in item["rows"].items():
            member._write(name, dtype, np.asarray(col))
        rt.issue(item["program"], item["vars"])
        got_next = member.read_tokens(staged.call.forward, staged.call.groups)[: len(prompts)]
        if not cpu:
            rt.check_error()
        logits = rt.tensor("logits")[: len(prompts)].float()
        worst = max(worst, float((logits - ref_logits).abs().max()))
        agree += sum(int(a[0] == b[0]) for a, b in zip(got_next, ref_next))
        toks = [n[0] for n in ref_next]
        for sg in seqs_g:
            sg.length += 1
    return {"check": "dcp_model", "world": world, "steps": steps, "max_logit_diff": round(worst, 4),
            "tokens_agree": agree, "of": steps * len(prompts), "ok": worst < 0.1}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", action="store_true", help="also run the dense decoder as a context-parallel decode group")
    ap.add_argument("--lens", type=int, nargs="+", default=[1, 3, 64, 65, 300, 777, 4099])
    ap.add_argument("--splits", type=int, default=2)
    ap.add_argument("--time", action="store_true")
    ap.add_argument("--cpu", action="store_true", help="gloo ranks and the host-memory executor (the model check only)")
    a = ap.parse_args(argv)
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    if a.cpu:
        if world > 1:
            dist.init_process_group("gloo")
        ml = check_model(rank, world, local, cpu=True)
        okm = torch.tensor([int(ml["ok"])])
        if world > 1:
            dist.all_reduce(okm, op=dist.ReduceOp.MIN)
        ml["ok"] = bool(okm.item())
        if rank == 0:
            print(json.dumps(dict(ml, backend="gloo")), flush=True)
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return 0 if ml["ok"] else 1
    torch.cuda.set_device(local)
    dev = torch.device(f"cuda:{local}")
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    from ..ops import attention as A
    from ..ops.launcher import Kernels

    hq, hk, d, page = 16, 4, 128, 16
    lens, seqs, splits = a.lens, len(a.lens), a.splits
    g = torch.Generator(device="cpu").manual_seed(11)              # the same tensors on every rank
    bf = lambda t: t.to(torch.bfloat16).to(dev)
    q = bf(torch.randn(seqs, hq * d, generator=g))
    ks = [bf(torch.randn(l, hk, d, generator=g)) for l in lens]
    vs = [bf(torch.randn(l, hk, d, generator=g)) for l in lens]
    seq_lens = torch.tensor(lens, dtype=torch.int32, device=dev)
    local_lens = A.dcp_local_lens(seq_lens, rank, world)
    want_local = [len(range(rank, l, world)) for l in lens]
    lens_ok = local_lens.tolist() == want_local
    # this rank's pool: its share of every sequence, packed into its own pages
    pages_needed = sum(-(-n // page) for n in want_local) + 1
    pool = torch.zeros(pages_needed, 2, hk, page, d, dtype=torch.bfloat16, device=dev)
    table = torch.zeros(seqs, max(1, max(-(-n // page) for n in want_local)), dtype=torch.int32, device=dev)
    nxt = 1
    for s in range(seqs):
        kk, vv = ks[s][rank::world], vs[s][rank::world]
        for p in range(-(-want_local[s] // page)):
            table[s, p] = nxt
            lo, hi = p * page, min(want_local[s], (p + 1) * page)
            pool[nxt, 0, :, : hi - lo] = kk[lo:hi].transpose(0, 1)
            pool[nxt, 1, :, : hi - lo] = vv[lo:hi].transpose(0, 1)
            nxt += 1
    out = torch.empty(seqs, hq * d, dtype=torch.bfloat16, device=dev)
    n_o, n_ml = seqs * hq * splits * d, seqs * hq * splits * 2
    all_o = torch.empty(world * n_o, dtype=torch.float32, device=dev)
    all_ml = torch.empty(world * n_ml, dtype=torch.float32, device=dev)

    def step():
        ws = A.new_partials(seqs, hq, d, splits, dev)          # neutral slots: an empty share stays (m = -inf, l = 0)
        A.paged_attention(q, pool, table, local_lens, hq, out=out, splits=splits, workspace=ws, partial=(0, splits))
        if world > 1:
            dist.all_gather_into_tensor(all_o, ws[0])
            dist.all_gather_into_tensor(all_ml, ws[1])
        else:
            all_o.copy_(ws[0]); all_ml.copy_(ws[1])
        A.merge_rank_partials(all_o, all_ml, out, seqs, hq, d, splits, world)

    step()
    torch.cuda.synchronize()
    Kernels.get(dev).check_error()
    worst = 0.0
    for s, l in enumerate(lens):
        ref = A.attention_reference(q[s:s + 1].view(1, hq, d), ks[s], vs[s], torch.tensor([l - 1], device=dev))
        worst = max(worst, float((out[s:s + 1].float() - ref).abs().max()))
    ok = torch.tensor([int(lens_ok and worst < 2e-2)], device=dev)
    line = {"check": "decode_context_parallel", "world": world, "lens": lens, "max_abs_err": round(worst, 5)}
    if a.time:
        for _ in range(3):
            step()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0.record()
        for _ in range(20):
            step()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / 20 * 1e3], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        line["us_per_step_max_over_ranks"] = round(float(t), 1)
    if world > 1:
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    line["ok"] = bool(ok.item())
    if rank == 0:
        print(json.dumps(line), flush=True)
    if a.model:
        ml = check_model(rank, world, local)
        okm = torch.tensor([int(ml["ok"])], device=dev)
        if world > 1:
            dist.all_reduce(okm, op=dist.ReduceOp.MIN)
        ml["ok"] = bool(okm.item())
        line["ok"] = line["ok"] and ml["ok"]
        if rank == 0:
            print(json.dumps(ml), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0 if line["ok"] else 1


if __name__ == "__main__":
    raise SystemExit(main())
