"""Run one program of any manifest on raw files: the gate for an op whose launch was lifted from another project.

    python -m kern_b200.testing.program_io --manifest probe.json [--kernels DIR] [--weights W.safetensors] --program attn \\
        --vars tokens=512 --in q=dump/q.bin --in kv=dump/kv.bin --out o=got/o.bin [--expect o=dump/out.bin[:atol]] [--cpu]

Every `--in NAME=FILE` fills a buffer (or a state) with the file's bytes from its start; the program runs once with the
vars; every `--out NAME=FILE` writes the buffer's bytes — as many as its shape holds at these vars — and every
`--expect NAME=FILE` compares them with a dump: byte for byte (the same cubin on the same bytes gives the same bytes; a
difference is a wrong field of the declaration), or within `atol` in the buffer's dtype. Prints one JSON line per
compared buffer and exits 1 on a difference. `--cpu` runs the manifest's ops through the host-memory executor (only the
package's own ops have host forms). Reference counterpart: crates/kern-run/examples/program_io.rs.
"""
from __future__ import annotations

import argparse
import json
from pathlib import Path

import numpy as np
import torch


def _pairs(items, what):
    out = {}
    for it in items or []:
        if "=" not in it:
            raise SystemExit(f"--{what} wants NAME=FILE, got `{it}`")
        k, v = it.split("=", 1)
        out[k] = v
    return out


def live_bytes(doc: dict, name: str, vars: dict[str, int], whole: int) -> int:
    """How many bytes of a buffer its shape holds at these vars (a dim that names a var takes the var's value)."""
    b = doc.get("buffers", {}).get(name)
    if b is None:
        return whole
    n = 1
    for d in b["shape"]:
        n *= d if isinstance(d, int) else vars.get(d, doc["vars"][d]["max"])
    es = {"bf16": 2, "f16": 2, "f32": 4, "i32": 4, "u32": 4, "i64": 8, "u64": 8, "u8": 1, "i8": 1, "fp8e4m3": 1}.get(b["dtype"], 1)
    return min(whole, n * es)


_TORCH = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32, "i32": torch.int32, "i64": torch.int64, "u8": torch.uint8}


def run(doc: dict, program: str, vars: dict[str, int], ins: dict[str, str], outs: dict[str, str], expects: dict[str, str],
        kernels=None, weights=None, cpu: bool = False) -> list[dict]:
    if cpu:
        from ..cpu import CpuRuntime

        rt = CpuRuntime(doc, weights=weights)
    else:
        from ..runtime import Runtime

        rt = Runtime(doc, kernels=kernels)
        if weights:
            rt.load_weights(weights)
    raw = lambda name: rt.tensor(name).contiguous().view(-1).view(torch.uint8)
    for name, path in ins.items():
        data = np.fromfile(path, dtype=np.uint8)
        dst = rt.tensor(name)
        flat = dst.view(-1).view(torch.uint8)
        if data.size > flat.numel():
            raise SystemExit(f"--in {name}: {path} holds {data.size} bytes, the buffer {flat.numel()}")
        flat[:data.size] = torch.from_numpy(data).to(flat.device)
    rt.run(program, vars)
    rt.synchronize()
    rt.check_error()
    results = []
    for name, path in outs.items():
        got = raw(name).cpu().numpy()
        got = got[:live_bytes(doc, name, vars, got.size)]
        Path(path).parent.mkdir(parents=True, exist_ok=True)
        got.tofile(path)
    for name, spec in expects.items():
        path, _, tol = spec.partition(":")
        got = raw(name).cpu()
        got = got[:live_bytes(doc, name, vars, got.numel())]
        want = torch.from_numpy(np.fromfile(path, dtype=np.uint8))
        rec = {"buffer": name, "bytes": int(got.numel()), "expected_bytes": int(want.numel())}
        n = min(got.numel(), want.numel())
        if tol:
            dt = _TORCH.get(doc["buffers"][name]["dtype"], torch.uint8)
            es = torch.empty(0, dtype=dt).element_size()
            a, b = got[:n - n % es].view(dt).float(), want[:n - n % es].view(dt).float()
            rec["max_abs_diff"] = float((a - b).abs().max()) if a.numel() else 0.0
            rec["ok"] = rec["max_abs_diff"] <= float(tol) and got.numel() == want.numel()
        else:
            diff = (got[:n] != want[:n]).nonzero()
            rec["first_difference_at"] = int(diff[0]) if diff.numel() else None
            rec["ok"] = diff.numel() == 0 and got.numel() == want.numel()
        results.append(rec)
    return results


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--manifest", required=True)
    ap.add_argument("--kernels", help="the directory that holds the manifest's modules (default: the package's own)")
    ap.add_argument("--weights")
    ap.add_argument("--program", required=True)
    ap.add_argument("--vars", action="append", default=[], help="NAME=VALUE (repeatable, or comma-separated)")
    ap.add_argument("--in", dest="ins", action="append")
    ap.add_argument("--out", dest="outs", action="append")
    ap.add_argument("--expect", action="append")
    ap.add_argument("--cpu", action="store_true")
    a = ap.parse_args(argv)
    doc = json.loads(Path(a.manifest).read_text())
    vars = {k: int(v) for item in a.vars for k, v in (kv.split("=") for kv in item.split(","))}
    results = run(doc, a.program, vars, _pairs(a.ins, "in"), _pairs(a.outs, "out"), _pairs(a.expect, "expect"),
                  kernels=a.kernels, weights=a.weights, cpu=a.cpu)
    for r in results:
        print(json.dumps(r))
    return 0 if all(r["ok"] for r in results) else 1


if __name__ == "__main__":
    raise SystemExit(main())
