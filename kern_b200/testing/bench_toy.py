"""Serve a toy package of the reference's format — its manifest, its cubin, its weights file, unmodified — through this
package's runtime and scheduler, under the traffic `baseline/reference_arm.py` gives the reference's own Python engine:
all requests submitted at once, at most `concurrency` running, prompts of 512-2048 uniform-random byte tokens, 256
outputs each, no stop token. The two numbers differ only in the engine: same manifest, same kernels.

    python bench.py --config toy            (after `python baseline/install_ref.py --reference <upstream checkout>`)
"""
from __future__ import annotations

import json
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent.parent
PKG = ROOT / "baseline" / "_ref" / "toy_pkg"


def available() -> bool:
    return (PKG / "toy-paged.json").exists()


def oracle():
    """The reference's own statement of the toy arithmetic (tools/toy/model.py), loaded from the installed copy."""
    import importlib.util

    spec = importlib.util.spec_from_file_location("kern_ref_toy_model", ROOT / "baseline" / "_ref" / "tools" / "toy" / "model.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def check_against_oracle(reqs, doc: dict, limit: int) -> int:
    """Requests whose served tokens equal the oracle's greedy continuation (up to its end-of-sequence)."""
    model = oracle()
    ok = 0
    for r in reqs:
        want = model.generate(r.prompt, limit, doc)
        got = [t for t in r.out[:limit]]
        ok += got[:len(want)] == want and (len(want) == limit or (len(got) > len(want) and got[len(want)] == model.EOS))
    return ok


def run(concurrency: int = 256, requests: int | None = None, out_len: int = 256, seed: int = 0, gpu: int = 0,
        target: str = "toy-paged", verify: int = 6) -> dict:
    import numpy as np

    from ..engine import Engine
    from ..runtime import Runtime
    from ..serve.scheduler import Request, Scheduler

    requests = requests or 2 * concurrency
    rng = np.random.default_rng(seed)
    prompts = [rng.integers(0, 256, int(rng.integers(512, 2049))).tolist() for _ in range(requests)]
    capacity = (concurrency + 1) * (2048 + out_len + 64)
    rt = Runtime((PKG / f"{target}.json").read_text(), kernels=PKG / "kernels", weights=[PKG / "model" / "toy.safetensors"],
                 gpu=gpu, tokens=capacity, slots=concurrency + 1)
    rt.once()
    eng = Engine(rt)
    sch = Scheduler(eng, chunk=eng.rows_max, max_seqs=concurrency, prefix_cache=True, stats_every=1e9)
    warm = [Request(id=f"w{i}", prompt=p[:600], max_tokens=8) for i, p in enumerate(prompts[:4])]
    for r in warm:
        sch.submit(r)
    sch.run_until_idle(10000)
    rt.synchronize()
    launches0 = rt.launches_total
    reqs = [Request(id=f"r{i}", prompt=p, max_tokens=out_len) for i, p in enumerate(prompts)]
    t0 = time.monotonic()
    for r in reqs:
        r.arrival = t0
        sch.submit(r)
    steps0 = sch.stats.steps
    sch.run_until_idle(10_000_000)
    rt.synchronize()
    wall = time.monotonic() - t0
    rt.check_error()
    tokens = sum(len(r.out) for r in reqs)
    checked = reqs[:: max(1, len(reqs) // verify)][:verify] if verify else []
    exact = check_against_oracle(checked, rt.doc, out_len) if checked else 0
    ttft = sorted(r.first_token_at - t0 for r in reqs)
    gaps = sorted(b - a for r in reqs for a, b in zip(r.token_times, r.token_times[1:]))
    return {"output_tok_s": tokens / wall, "tokens": tokens, "wall_s": wall, "requests": requests, "concurrency": concurrency,
            "steps": sch.stats.steps - steps0, "gpu_launches": rt.launches_total - launches0,
            "ttft_ms_p50_all_submitted_at_t0": 1e3 * ttft[len(ttft) // 2], "tpot_ms_p50": 1e3 * gaps[len(gaps) // 2],
            "prefix_hit_tokens": sch.stats.prefix_hit_tokens, "oracle_checked": len(checked), "oracle_exact": exact}


def main(args) -> int:
    if not available():
        print(json.dumps({"config": "toy", "unavailable": "baseline/_ref/toy_pkg is missing: python baseline/install_ref.py --reference <checkout>"}))
        return 0
    conc = min(256, args.concurrency)
    res = run(conc, 2 * conc, 256, args.seed)
    print(json.dumps({
        "metric": "output tok/s at fixed concurrency", "value": round(res["output_tok_s"], 1), "unit": "tok/s", "n_gpus": 1,
        "higher_is_better": True, "impl": "ours", "data": "synthetic (uniform-random byte tokens)", "dtype": "i64 (exact integer model)",
        "config": {"model": "toy-paged package of the reference (its manifest + its toy.cu cubin for sm_100a), served by kern_b200",
                   "concurrency": conc, "requests": res["requests"], "seq_len": "prompts 512-2048 uniform, 256 outputs"},
        "ttft_ms_p50_all_submitted_at_t0": round(res["ttft_ms_p50_all_submitted_at_t0"], 2),
        "tpot_ms_p50": round(res["tpot_ms_p50"], 3), "wall_s": round(res["wall_s"], 2), "steps": res["steps"],
        "gpu_launches": res["gpu_launches"],
        "exact_vs_reference_oracle": f"{res['oracle_exact']}/{res['oracle_checked']} sampled requests equal tools/toy/model.py token for token"}))
    return 0
