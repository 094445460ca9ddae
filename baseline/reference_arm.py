"""The reference arm of bench.py: what of the upstream project can run on this machine, run unmodified.

What cannot run. The reference's engine is a Rust workspace whose Python package builds with maturin, and the
attention / routed-GEMM / FMHA kernels its model packages name are prebuilt sm_103a cubins fetched from Hugging Face.
With no Rust toolchain and no network, none of the benchmark's model configs can be executed by the reference here,
so for those this arm prints its `unavailable` line.

What can run, and is run. The reference ships a pure-Python consumer of its package format (examples/python:
manifest.py, executor.py, server.py — cuda-python, torch, safetensors, tokenizers only), the source of its exact
"toy" serving model (tools/kernels-src/toy.cu, plain nvcc) and the generator of complete toy packages
(tools/toy/gen.py). `baseline/install_ref.py` copies those files, unmodified, to baseline/_ref and runs the generator
for sm_100a. This arm then serves the `toy-paged` package with the reference's own continuous-batching `Engine` over
its own `Executor` and kernels (graph replay on), under the benchmark's traffic shape scaled to the package's limits
(256 concurrent requests, prompts 512-2048 uniform-random byte tokens, 256 outputs each), and reports output tok/s,
TTFT and TPOT. Nothing of kern_b200 is imported on this path. `bench.py --config toy` serves the same package — the
same manifest and the same cubin — through kern_b200's runtime and scheduler.
"""
from __future__ import annotations

import json
import os
import queue
import sys
import threading
import time
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF = HERE / "_ref"
PKG = REF / "toy_pkg"

WHY_MODELS = ("the reference's engine is a Rust workspace (maturin wheel) and no Rust toolchain is installed; the attention, "
              "routed-GEMM and FMHA kernels of its model packages are prebuilt sm_103a cubins fetched from Hugging Face, "
              "which this box cannot reach")


def toy_workload(seed: int, requests: int, p_lo: int = 512, p_hi: int = 2048):
    import numpy as np

    rng = np.random.default_rng(seed)
    return [rng.integers(0, 256, int(rng.integers(p_lo, p_hi + 1))).tolist() for _ in range(requests)]


def run_reference_toy(concurrency: int, requests: int, out_len: int, seed: int, gpu: int = 0) -> dict:
    """Serve the toy-paged package with the reference's own Python engine; all requests are submitted at once and at
    most `concurrency` run together (its admission), so a finished request is replaced at once."""
    sys.path.insert(0, str(REF / "examples" / "python"))
    import torch
    from tokenizers import Tokenizer

    from executor import Executor          # the reference's files, unmodified
    from manifest import Sampling
    from server import Engine

    prompts = toy_workload(seed, requests)
    capacity = (concurrency + 1) * (2048 + out_len + 64)
    rt = Executor(PKG / "toy-paged.json", PKG / "kernels", [PKG / "model" / "toy.safetensors"], capacity_tokens=capacity,
                  seq_slots=concurrency + 1, gpu=gpu)
    tok = Tokenizer.from_file(str(PKG / "model" / "tokenizer.json"))
    # warm-up: a few requests through the whole path (graph capture of the decode shapes it meets)
    eng = Engine(rt, tok, set(), concurrency, None, True)          # no stop tokens: every request makes out_len tokens
    warm = [eng.submit(p[:600], 8, Sampling()) for p in prompts[:4]]
    for r in warm:
        while r.out.get(timeout=120)[1] is None:
            pass
    torch.cuda.synchronize()
    t0 = time.monotonic()
    reqs = [eng.submit(p, out_len, Sampling()) for p in prompts]
    first: dict[int, float] = {}
    last: dict[int, float] = {}
    gaps: list[float] = []
    pending = set(range(len(reqs)))
    deadline = t0 + 1800
    while pending and time.monotonic() < deadline:
        idle = True
        for i in list(pending):
            try:
                while True:
                    _, fin = reqs[i].out.get_nowait()
                    now = time.monotonic()
                    idle = False
                    if i in last:
                        gaps.append(now - last[i])
                    else:
                        first[i] = now
                    last[i] = now
                    if fin is not None:
                        pending.discard(i)
                        break
            except queue.Empty:
                pass
        if idle:
            time.sleep(0.0005)
    wall = time.monotonic() - t0
    if pending:
        raise RuntimeError(f"{len(pending)} requests did not finish in 1800 s")
    tokens = sum(len(r.generated) for r in reqs)
    ttft = sorted(first[i] - t0 for i in first)
    gaps.sort()
    return {"output_tok_s": tokens / wall, "tokens": tokens, "wall_s": wall, "requests": requests,
            "ttft_ms_p50_all_submitted_at_t0": 1e3 * ttft[len(ttft) // 2],
            "tpot_ms_p50": 1e3 * gaps[len(gaps) // 2] if gaps else None}


def main(args) -> int:
    line = {"impl": "reference", "unavailable": WHY_MODELS, "same_config": False}
    if not (PKG / "toy-paged.json").exists():
        line["toy"] = "baseline/_ref is not installed (python baseline/install_ref.py)"
        print(json.dumps(line))
        return 0
    if int(os.environ.get("RANK", "0")) != 0:          # the reference's Python engine is a one-GPU program
        return 0
    try:
        import torch

        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device")
        conc = min(256, args.concurrency)
        res = run_reference_toy(conc, 2 * conc, 256, args.seed)
        line["ran"] = {
            "what": "the reference's examples/python Engine + Executor (unmodified) serving its toy-paged package "
                    "(tools/toy/gen.py, tools/kernels-src/toy.cu built with nvcc for sm_100a)",
            "metric": "output tok/s at fixed concurrency", "value": round(res["output_tok_s"], 1), "unit": "tok/s",
            "config": {"model": "toy-paged (4 KiB/token paged state, exact integer kernels)", "concurrency": conc,
                       "requests": res["requests"], "seq_len": "prompts 512-2048 uniform, 256 outputs", "n_gpus": 1},
            "ttft_ms_p50_all_submitted_at_t0": round(res["ttft_ms_p50_all_submitted_at_t0"], 2),
            "tpot_ms_p50": round(res["tpot_ms_p50"], 3) if res["tpot_ms_p50"] else None,
            "wall_s": round(res["wall_s"], 2), "ours": "python bench.py --config toy (same package through kern_b200)"}
    except Exception as e:      # the arm reports, it does not fail the bench
        line["toy_error"] = repr(e)[:400]
    print(json.dumps(line))
    return 0
