"""The checked kernel build exercised on one GPU (run with KERN_B200_CHECKED=1 in the environment; it says so otherwise).

    KERN_B200_CHECKED=1 python -m kern_b200.testing.checked_selftest

1. A dense, a routed-experts and a hybrid (recurrent state slots) decoder each prefill and decode through the checked
   modules, twice: no access is refused, both runs give the same tokens, and the device error word stays clear.
2. A row gather whose source pointer comes from a table in device memory (the expert-parallel dispatch's peer table) is
   pointed at memory this runtime does not own — a tensor of another allocator, mapped and harmless to read: the
   checked kernel skips the access, the destination stays untouched, and `check_error` names the check site and the
   address. Pointed at the runtime's own buffer, the same launch copies the rows.

Prints one JSON line. Reference counterpart: docs/runtime.md (the KERN_CHECKED build of tools/kernels-src with per-access
bounds checks behind a define).
"""
from __future__ import annotations

import json


def gather_manifest(rows: int, hidden: int) -> dict:
    from ..models import common as C

    buf = lambda dt, shape, kind: {"dtype": dt, "shape": shape, "kind": kind}
    L = {"module": "moe", "entry": "kern_moe_gather_peers_bf16", "block": [128, 1, 1], "grid": [rows, 1, 1],
         "params": ["in buffer<u64>", "in buffer<i32>", "out buffer<bf16>", "i32", "i32", "i32", "i32"],
         "args": [{"param": 0}, {"param": 1}, {"param": 2}, {"i32": rows}, {"i32": 1}, {"i32": hidden}, {"i32": rows}]}
    return {"schema_version": 7, "model": "checked-gather", "vars": {}, "states": {},
            "buffers": {"table": buf("u64", [1], "input"), "perm": buf("i32", [rows], "input"), "x": buf("bf16", [rows, hidden], "inout"),
                        "out": buf("bf16", [rows, hidden], "output")},
            "modules": C.modules_for(["moe"]),
            "ops": {"gather": {"params": ["in buffer<u64>", "in buffer<i32>", "out buffer<bf16>"], "impl": {"launches": [L]}}},
            "programs": {"step": {"calls": [{"op": "gather", "args": [{"buf": "table"}, {"buf": "perm"}, {"buf": "out"}]}]},
                         "back": {"calls": [{"op": "gather", "args": [{"buf": "table"}, {"buf": "perm"}, {"buf": "x"}]}]}}}


def main() -> int:
    import numpy as np
    import torch

    from .. import _build
    from ..engine import Engine
    from ..models import dense, hybrid, moe
    from ..runtime import Runtime

    out = {"check": "checked_kernel_build", "checked_env": _build.checked()}
    if not _build.checked():
        out["ok"] = False
        out["why"] = "KERN_B200_CHECKED is not set: this process loads the normal build"
        print(json.dumps(out), flush=True)
        return 2
    ok = True
    # 1. whole decoders through the checked modules
    models = {}
    for name, mod, cfg in (("dense", dense, dense.TINY), ("moe", moe, moe.TINY_MOE), ("hybrid", hybrid, hybrid.TINY_HYBRID)):
        w = mod.random_weights(cfg, seed=0, std=0.05)
        runs = []
        for _ in range(2):
            rt = Runtime(mod.build_manifest(cfg), tokens=cfg.page_size * 32, slots=4)
            rt.load_tensors(lambda n: w[n].cuda())
            rt.once()
            eng = Engine(rt)
            runs.append(eng.generate(list(range(1, 40)), 6))
            rt.check_error()                     # raises if a checked access was refused
            checked = bool(rt._rt.checked)
            del eng, rt
        models[name] = {"checked_modules": checked, "tokens": runs[0], "repeatable": runs[0] == runs[1]}
        ok = ok and checked and runs[0] == runs[1]
    out["models"] = models
    # 2. a pointer the runtime does not own is refused; its own buffer is taken
    rows, hidden = 8, 256
    rt = Runtime(gather_manifest(rows, hidden))
    x = (torch.arange(rows * hidden, device="cuda").reshape(rows, hidden) % 251).to(torch.bfloat16)
    rt.tensor("x").copy_(x)
    rt.tensor("perm").copy_(torch.arange(rows, dtype=torch.int32, device="cuda"))
    foreign = x.clone()                          # the caching allocator's memory: mapped, not this runtime's
    rt.write("table", np.array([foreign.data_ptr()], dtype=np.uint64))
    rt.run("step", {})
    refused = ""
    try:
        rt.check_error()
    except RuntimeError as e:
        refused = str(e)
    untouched = bool((rt.tensor("out") == 0).all())
    rt.write("table", np.array([rt.region("x")[0]], dtype=np.uint64))
    rt.run("step", {})
    rt.check_error()
    copied = bool((rt.tensor("out") == x).all())
    out["foreign_pointer"] = {"refused": refused, "destination_untouched": untouched, "own_buffer_copied": copied}
    ok = ok and "check site 5" in refused and untouched and copied
    out["ok"] = ok
    print(json.dumps(out), flush=True)
    return 0 if ok else 1


if __name__ == "__main__":
    raise SystemExit(main())
