"""The counters sampler against the real driver on one GPU:

    python -m kern_b200.testing.counters_selftest [--seconds 1.5] [--period-ms 20]

Runs this repo's bf16 tcgen05 GEMM (4096 x 4096 x 4096) back to back for a while with `trace.Counters` sampling beside
it, then an idle stretch, and prints one JSON line: whether the device offers performance-monitoring samples, and the
median SM clock, power and SM / tensor / DRAM busy shares (per mille) under load and idle. Read-only towards the GPU's
settings. Reference counterpart: crates/kern-runtime/src/counters.rs:93-214.
"""
from __future__ import annotations

import argparse
import json
import statistics
import tempfile
import time


def main(argv=None) -> int:
    import pyarrow.parquet as pq
    import torch

    from .. import trace
    from ..ops.gemm import gemm

    ap = argparse.ArgumentParser()
    ap.add_argument("--seconds", type=float, default=1.5)
    ap.add_argument("--period-ms", type=float, default=20.0)
    a = ap.parse_args(argv)
    dev = torch.device("cuda:0")
    x = torch.randn(4096, 4096, device=dev).to(torch.bfloat16)
    w = torch.randn(4096, 4096, device=dev).to(torch.bfloat16)
    gemm(x, w)
    torch.cuda.synchronize()
    with tempfile.TemporaryDirectory() as d:
        rec = trace.Recorder(d)
        smp = trace.Counters(rec, gpu=0, period=a.period_ms / 1e3)
        smp.start()
        t0 = time.time()
        while time.time() - t0 < a.seconds:
            for _ in range(50):
                gemm(x, w)
            torch.cuda.synchronize()
        t_idle = time.time_ns()
        time.sleep(max(0.5, a.seconds / 2))
        smp.stop()
        smp.join(5)
        files = [p for p in rec.rotate() if ".counters." in p.name]
        t = pq.ParquetFile(files[0]).read().to_pydict() if files else {"t_ns": []}
    med = lambda xs: statistics.median(xs) if xs else None
    load = [i for i, ts in enumerate(t["t_ns"]) if ts < t_idle]
    idle = [i for i, ts in enumerate(t["t_ns"]) if ts >= t_idle + int(0.2e9)]
    pick = lambda col, idx: med([t[col][i] for i in idx]) if t["t_ns"] else None
    out = {"check": "counters_sampler", "samples": len(t["t_ns"]), "gpm": bool(smp.gpm), "dropped": rec.dropped,
           "load": {c: pick(c, load) for c in ("sm_mhz", "power_w", "gpu_util", "sm_active_pm", "tensor_active_pm", "dram_bw_pm")},
           "idle": {c: pick(c, idle) for c in ("sm_mhz", "power_w", "gpu_util", "sm_active_pm", "tensor_active_pm", "dram_bw_pm")}}
    out["ok"] = out["samples"] >= 10 and (not smp.gpm or (out["load"]["tensor_active_pm"] or 0) > (out["idle"]["tensor_active_pm"] or 0))
    print(json.dumps(out), flush=True)
    return 0 if out["ok"] else 1


if __name__ == "__main__":
    raise SystemExit(main())
