"""Source-level guards over every file that ships: no TMA / bulk load with cluster multicast anywhere (a load whose
source may be another GPU's memory must never use it, and nothing here needs it), no batched-memcpy driver calls,
every spin-wait in a kernel is bounded."""
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
SOURCES = [p for pat in ("csrc/**/*.cu", "csrc/**/*.cuh", "csrc/**/*.hpp", "csrc/**/*.cpp", "kern_b200/**/*.py", "bench.py",
                         "__graft_entry__.py", "kern_vllm/*.py", "kern_sglang/*.py") for p in ROOT.glob(pat)]

MC = "multi" + "cast"
BANNED = [MC + "::cluster", r"\." + MC + r"\b", "SM90_TMA_LOAD_" + MC.upper(), r"SM100_TMA_\w*" + MC.upper(),
          "cudaMemcpy" + "BatchAsync", "cudaMemcpy3D" + "BatchAsync", "cuMemcpy" + "BatchAsync", "cuMemcpy3D" + "BatchAsync",
          r"__trap\s*\("]


def test_no_banned_tokens():
    assert len(SOURCES) > 40
    for p in SOURCES:
        text = p.read_text(errors="replace")
        for pat in BANNED:
            m = re.search(pat, text)
            assert m is None, f"{p.relative_to(ROOT)}: `{m.group(0)}` is not allowed in shipped sources"


def test_every_device_spin_has_a_limit():
    """A `while` that polls memory in a kernel file must sit next to a timeout / iteration limit."""
    for p in ROOT.glob("csrc/kernels/**/*.cu*"):
        lines = p.read_text().splitlines()
        for i, line in enumerate(lines):
            if re.search(r"while\s*\(.*(ld_acquire|ld_volatile|has_poison|try_wait|volatile)", line) or re.search(r"while\s*\(\s*true\s*\)", line):
                window = "\n".join(lines[max(0, i - 3): i + 12])
                assert re.search(r"timeout|globaltimer|limit|spins|iters|kMaxSpin", window), f"{p.name}:{i + 1}: unbounded wait"
