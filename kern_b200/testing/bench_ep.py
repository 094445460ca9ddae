"""`bench.py --config d`: decode of a routed-experts decoder whose experts are sharded over the GPUs of the box.

Every rank serves its own share of the concurrent sequences (attention, norms, router and head whole on every rank: data
parallel) and holds 1/N of every layer's experts; each routed layer is the fused pair of kernels — dispatch inside FC1,
combine inside FC2 (`models/moe_ep.py::build_manifest_ep_sharded`, `csrc/kernels/sm100/moe.cu`). The ranks step in
lockstep. The timed step is one decode call of every rank (CUDA-graph replay) at a fixed context; the figure is the
whole box's output tokens per second, device-timed, max over ranks.

The model is the 30B-A3B routed decoder of `models/moe.py` (48 layers, hidden 2048, 128 experts top-8, GQA attention),
random init, with the expert formats of the benchmark's config (d) — MXFP4 expert weights, MXFP8 expert activations, the
block-scaled pair of `gemm_mx.cu` (`--experts bf16`: bf16 experts) — but not its shape: the MLA decoder with 256 experts
of hidden 7168 needs four GPUs or more even at MXFP4, and this repo has no decoder of that layer pattern (three dense
layers, a shared expert); the line says so (`"same_config": false`).
Reference shape: docs/serve.md:402-453 (EP decode tier), docs/roadmap.md:13-16.
"""
from __future__ import annotations

import dataclasses
import json
import os


def main(args) -> int:
    import torch

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(local)
    dev = torch.device(f"cuda:{local}")
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)
    from ..engine import Engine
    from ..models import moe, moe_ep
    from ..parallel import group
    from ..runtime import Runtime

    steps, warmup = args.steps, max(3, args.warmup)
    ctx = 4096
    conc = min(args.concurrency, 128 * world)          # one GPU holds the whole model: room for 128 sequences at this context
    per_rank = max(1, conc // world)
    mx = getattr(args, "experts", "mx") == "mx"
    cfg = dataclasses.replace(moe.MOE_30B, layers=args.layers if args.layers != 36 else moe.MOE_30B.layers,
                              max_seqs=max(per_rank, 8), max_tokens=max(per_rank, 256), max_context=ctx + steps + warmup + 72,
                              page_size=64, mx_experts=mx)
    doc = moe_ep.build_manifest_ep_sharded(cfg, world)
    topo = group.topology(doc["topology"]["groups"], rank, world)
    rt = Runtime(doc, gpu=local, topology=topo, tokens=per_rank * (cfg.max_context + 64), memory_fraction=0.92)
    if mx:
        # random nibbles under a block scale of 2^-7: e2m1 values of rms 2.9 become weights of rms 0.02
        moe.load_random_weights(rt, dataclasses.replace(cfg, mx_experts=False), seed=0, skip=lambda n: ".mlp.experts." in n)
        g = torch.Generator(device=dev).manual_seed(7 + rank)
        for name, b in doc["buffers"].items():
            if b["kind"] == "weight" and b["dtype"] == "u8":
                t = rt.tensor(name)
                if name.endswith((".sf1", ".sf2")):
                    t.fill_(120)
                else:
                    t.view(-1).copy_(torch.randint(0, 256, (t.numel(),), generator=g, device=dev, dtype=torch.uint8))
    else:
        moe.load_random_weights(rt, cfg, seed=0)
    group.start(rt)
    eng = Engine(rt)
    seqs = [eng.open(cfg.max_context - 8) for _ in range(per_rank)]
    for s in seqs:              # a context that is already there (its cache content is whatever the pool holds: the step's cost is the same)
        s.length = ctx
        s.tokens = [1] * ctx
    toks = [[1 + (i % 1000)] for i in range(per_rank)]
    stream = torch.cuda.ExternalStream(rt.stream)

    def one():
        nonlocal toks
        out = eng.step(list(zip(seqs, toks)))
        toks = [[o[0]] for o in out]

    launches0 = 0
    for _ in range(warmup):
        one()
    rt.check_error()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    launches0 = rt.launches_total
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(steps):
        one()
    e1.record(stream)
    torch.cuda.synchronize()
    rt.check_error()
    t = torch.tensor([e0.elapsed_time(e1)], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.barrier()
    ms = float(t) / steps
    line = {
        "metric": "output tok/s per box at fixed concurrency (decode steps at a fixed context)", "value": round(per_rank * world / ms * 1e3, 1),
        "unit": "tok/s", "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": round(ms, 3), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16; routed experts MXFP4 weights x MXFP8 activations (config d's formats)" if mx else "bf16",
        "data": "synthetic (random-init N(0,0.02) bf16 weights" + (", expert weights random MXFP4 nibbles under 2^-7 block scales" if mx else "") +
                ", contexts already in the cache, greedy tokens fed back)",
        "config": {"model": f"routed-experts decoder 30B-A3B: {cfg.layers}L hidden 2048 32Q/4KV hd128, 128 experts top-8 (intermediate 768)",
                   "same_config": False,
                   "why": "config (d) names an MLA decoder with 256 experts of hidden 7168 (61 layers, three of them dense, a shared "
                          "expert): that layer pattern is not built here and its weights need four GPUs or more even at MXFP4; "
                          "the expert formats and the fused expert-parallel kernels are the config's",
                   "experts": "mxfp4 x mxfp8" if mx else "bf16",
                   "concurrency": per_rank * world, "context": ctx, "parallelism": f"ep{world} (attention data parallel)",
                   "routed_layer": "dispatch inside FC1, combine inside FC2: " + ("six" if mx else "five") + " launches, no NCCL call"},
        "tpot_ms_p50": round(ms, 3), "gpu_launches": int(rt.launches_total - launches0), "graphs": rt.graphs,
    }
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    return 0
