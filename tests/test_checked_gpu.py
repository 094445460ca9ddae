"""The checked kernel build (-DKERN_CHECKED, `kern_b200/kernels_checked/`): data-derived addresses are looked up in the
runtime's table of allocations before they are used. The build itself is checked without a GPU; on a GPU whole decoders
run through it, and a pointer the runtime does not own (another allocator's tensor: mapped, harmless) is refused."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_checked_build_has_every_module_under_its_own_hashes():
    from kern_b200 import _build

    if not os.path.exists(_build.NVCC):
        pytest.skip("no nvcc on this machine")
    normal = _build.build_kernels()
    checked = _build.build_kernels(checked_build=True)
    assert set(normal) == set(checked)
    # the modules with check sites differ; a define that changed nothing would leave the bytes alone
    for name in ("moe", "norm_embed", "attn_prep", "gdn", "gemm_mx"):
        assert normal[name]["sha256"] != checked[name]["sha256"], name
    assert _build.kernels_dir(True).name == "kernels_checked" and _build.kernels_dir(False).name == "kernels"


@pytest.mark.gpu
def test_checked_build_runs_models_and_refuses_a_foreign_pointer(cuda):
    p = subprocess.run([sys.executable, "-m", "kern_b200.testing.checked_selftest"], cwd=ROOT, capture_output=True, text=True, timeout=900,
                       env=dict(os.environ, KERN_B200_CHECKED="1", PYTHONPATH=ROOT))
    assert p.returncode == 0, (p.stdout[-3000:], p.stderr[-3000:])
    line = json.loads([l for l in p.stdout.splitlines() if l.startswith("{")][-1])
    assert line["ok"] and all(m["checked_modules"] and m["repeatable"] for m in line["models"].values()), line
    fp = line["foreign_pointer"]
    assert "check site 5" in fp["refused"] and fp["destination_untouched"] and fp["own_buffer_copied"], fp
