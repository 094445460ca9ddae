"""The smallest useful manifest: one var, one weight, one op (a row-wise RMSNorm from the package's kernels), one
program — built, verified, run and checked against PyTorch. It shows every step a larger model generator takes.

    python examples/python/minimal.py            # on a B200
    python examples/python/minimal.py --cpu      # the same manifest through the host-memory executor

Reference counterpart: examples/minimal.json, examples/python/run.py.
"""
import argparse
import json
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

from kern_b200.models import common as C      # noqa: E402
from kern_b200.runtime import verify          # noqa: E402


def manifest(width: int = 256, rows_max: int = 1024) -> dict:
    return {
        "schema_version": 7, "model": "minimal",
        "vars": {"tokens": {"max": rows_max}},
        "states": {},
        "buffers": {
            "x": {"dtype": "bf16", "shape": ["tokens", width], "kind": "input"},
            "w": {"dtype": "bf16", "shape": [width], "kind": "weight", "bind": [{"tensor": "norm.weight"}]},
            "y": {"dtype": "bf16", "shape": ["tokens", width], "kind": "output"},
        },
        "modules": C.modules_for(["norm_embed"]),      # name -> {source, sha256}: the runtime loads cubins by content
        "ops": {"norm": C.rms_norm_op(width, 1e-6)},
        "programs": {"step": {"calls": [{"op": "norm", "label": "norm", "args": [{"buf": "x"}, {"buf": "w"}, {"buf": "y"}]}]}},
    }


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--cpu", action="store_true")
    ap.add_argument("--print", action="store_true", help="print the manifest and stop")
    a = ap.parse_args()
    doc = manifest()
    if a.print:
        print(json.dumps(doc, indent=1))
        return 0
    m, diags = verify(doc)
    assert m is not None, diags
    weights = {"norm.weight": (1 + 0.1 * torch.randn(256)).to(torch.bfloat16)}
    if a.cpu:
        from kern_b200.cpu import CpuRuntime

        rt, dev = CpuRuntime(doc, weights=weights), "cpu"
    else:
        from kern_b200.runtime import Runtime

        rt, dev = Runtime(doc), "cuda"
        rt.load_tensors(lambda name: weights[name].cuda())
    rows = 37
    x = torch.randn(rows, 256, device=dev).to(torch.bfloat16)
    rt.tensor("x")[:rows] = x
    launches = rt.run("step", {"tokens": rows})
    y = rt.tensor("y")[:rows].float()
    xf = x.float()
    want = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6) * weights["norm.weight"].float().to(dev)
    err = float((y - want).abs().max())
    print(json.dumps({"rows": rows, "launches": launches, "max_abs_err": round(err, 5), "ok": err < 0.05}))
    return 0 if err < 0.05 else 1


if __name__ == "__main__":
    raise SystemExit(main())
