"""A decoder cut into pipeline stages and served as a chain: `cut` splits the manifest at layer boundaries, every stage
is a runtime of its own (here in one process, in host memory with `--cpu` or on GPUs 0..S-1), activations cross the
cuts, and the chain emits exactly the tokens of the uncut model.

    python examples/python/pp_chain.py --cpu [--stages 2]

Prints one JSON line. For a process per stage with overlapped NCCL transfers see
`python -m torch.distributed.run ... -m kern_b200.parallel.pp_pipeline_check`.
Reference counterpart: crates/kern-run/examples/pp_chain.rs.
"""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--cpu", action="store_true")
    ap.add_argument("--stages", type=int, default=2)
    ap.add_argument("--model", default="toy", choices=["toy", "tiny"])
    a = ap.parse_args()
    import torch

    from kern_b200.engine import Engine
    from kern_b200.models import dense
    from kern_b200.serve import pp
    from kern_b200.serve.scheduler import Request, Scheduler

    cfg = dense.TOY if a.model == "toy" else dense.TINY
    weights = dense.random_weights(cfg, seed=2, std=0.08)
    doc = dense.build_manifest(cfg)
    at = pp.layer_cuts(doc, a.stages)
    stage_docs = pp.cut(doc, at)
    if a.cpu:
        from kern_b200.cpu import CpuRuntime

        mk = lambda d, i: CpuRuntime(d, weights=weights, tokens=cfg.page_size * 24)
        transfer = None
    else:
        from kern_b200.runtime import Runtime

        n_gpu = torch.cuda.device_count()

        def mk(d, i):
            rt = Runtime(d, gpu=i % n_gpu, tokens=cfg.page_size * 24)
            rt.load_tensors(lambda name: weights[name].to(f"cuda:{i % n_gpu}"))
            return rt

        transfer = pp.device_transfer
    stages = [mk(d, i) for i, d in enumerate(stage_docs)]
    whole = mk(doc, 0)
    for rt in stages + [whole]:
        rt.once()
    pipe = pp.PipelineEngine(stages, whole.protocol, transfer=transfer) if transfer else pp.PipelineEngine(stages, whole.protocol)
    torch.manual_seed(0)
    prompts = [torch.randint(1, cfg.vocab, (n,)).tolist() for n in (13, 30, 4)]
    outs = []
    for eng in (Engine(whole), pipe):
        sch = Scheduler(eng, chunk=16, max_seqs=3)
        reqs = [Request(id=str(i), prompt=p, max_tokens=5) for i, p in enumerate(prompts)]
        for r in reqs:
            sch.submit(r)
        sch.run_until_idle(500)
        outs.append([r.out for r in reqs])
    print(json.dumps({"example": "pp_chain", "stages": a.stages, "cut_at": at, "ok": outs[0] == outs[1],
                      "states_per_stage": [sorted(d["states"]) for d in stage_docs], "moved_bytes": pipe.moved_bytes}))
    return 0 if outs[0] == outs[1] else 1


if __name__ == "__main__":
    raise SystemExit(main())
