"""program_io: one program of a manifest on raw files, compared with a dump (through the host-memory executor here)."""
import importlib.util
import json
import sys
from pathlib import Path

import numpy as np
import torch

from kern_b200.testing import program_io

ROOT = Path(__file__).resolve().parents[1]


def _minimal():
    spec = importlib.util.spec_from_file_location("minimal_example", ROOT / "examples" / "python" / "minimal.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.manifest()


def test_runs_a_program_from_files_and_compares_with_a_dump(tmp_path):
    doc = _minimal()
    (tmp_path / "m.json").write_text(json.dumps(doc))
    rows, width = 37, 256
    x = torch.randn(rows, width).to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(width)).to(torch.bfloat16)
    x.view(torch.int16).numpy().tofile(tmp_path / "x.bin")
    w.view(torch.int16).numpy().tofile(tmp_path / "w.bin")
    xf = x.float()
    want = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6) * w.float()).to(torch.bfloat16)
    want.view(torch.int16).numpy().tofile(tmp_path / "want.bin")
    args = ["--manifest", str(tmp_path / "m.json"), "--program", "step", "--vars", f"tokens={rows}", "--in", f"x={tmp_path / 'x.bin'}",
            "--in", f"w={tmp_path / 'w.bin'}", "--out", f"y={tmp_path / 'got' / 'y.bin'}", "--cpu"]
    assert program_io.main(args + ["--expect", f"y={tmp_path / 'want.bin'}:0.02"]) == 0
    got = np.fromfile(tmp_path / "got" / "y.bin", dtype=np.uint8)
    assert got.size == rows * width * 2                                    # the rows these vars hold, not the buffer's maximum
    # byte for byte against its own output: equal; against a dump with one flipped byte: the place is named
    assert program_io.main(args + ["--expect", f"y={tmp_path / 'got' / 'y.bin'}"]) == 0
    bad = got.copy()
    bad[1001] ^= 0x40
    bad.tofile(tmp_path / "bad.bin")
    res = program_io.run(doc, "step", {"tokens": rows}, {"x": str(tmp_path / "x.bin"), "w": str(tmp_path / "w.bin")}, {},
                         {"y": str(tmp_path / "bad.bin")}, cpu=True)
    assert res == [{"buffer": "y", "bytes": rows * width * 2, "expected_bytes": rows * width * 2, "first_difference_at": 1001, "ok": False}]


def test_live_bytes_follow_the_vars():
    doc = _minimal()
    assert program_io.live_bytes(doc, "y", {"tokens": 3}, 1 << 30) == 3 * 256 * 2
    assert program_io.live_bytes(doc, "w", {"tokens": 3}, 512) == 512
    assert program_io.live_bytes(doc, "some_state", {}, 4096) == 4096
