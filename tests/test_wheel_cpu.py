"""A wheel built from the tree is whole: version, entry points, every cubin under the hash its index pins, the native
files inside and none of them linked against a CUDA library."""
import subprocess
import sys
from pathlib import Path

import pytest

from kern_b200 import _build
from kern_b200.testing import check_wheel

ROOT = Path(__file__).resolve().parent.parent


def test_needed_reads_the_dynamic_section():
    so = _build.native_path()
    libs = check_wheel.needed(so.read_bytes())
    assert any(l.startswith("libc.so") for l in libs) and not any(l.startswith(("libcu", "libnv", "libnccl")) for l in libs)
    with pytest.raises(ValueError):
        check_wheel.needed(b"not an elf file at all")


@pytest.mark.timeout(600)
def test_built_wheel_passes_its_self_check(tmp_path):
    p = subprocess.run([sys.executable, "-m", "pip", "wheel", str(ROOT), "--no-deps", "--no-build-isolation", "-w", str(tmp_path), "-q"],
                       capture_output=True, text=True, timeout=580)
    if p.returncode != 0 and "No module named pip" in p.stderr:
        pytest.skip("no pip in this interpreter")
    assert p.returncode == 0, p.stderr[-2000:]
    wheel = next(tmp_path.glob("kern_b200-*.whl"))
    assert not wheel.name.endswith("-none-any.whl")
    assert check_wheel.check(wheel) == []
    assert check_wheel.main([str(wheel)]) == 0
    # a wheel that lost a cubin is named
    import zipfile

    broken = tmp_path / wheel.name.replace("kern_b200-", "kern_b200-broken-")
    with zipfile.ZipFile(wheel) as src, zipfile.ZipFile(broken, "w") as dst:
        for item in src.infolist():
            if item.filename != "kern_b200/kernels/moe.cubin":
                dst.writestr(item, src.read(item.filename))
    assert any("moe.cubin is not in the wheel" in e for e in check_wheel.check(broken))
