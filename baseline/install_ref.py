"""Install what of the reference can run here into baseline/_ref (git-ignored), unmodified.

The prescribed install, `python -m pip install --no-index --no-build-isolation --find-links /opt/wheelhouse --target
baseline/_ref <reference>`, fails: the repository root is not a Python project, and its Python package
(crates/kern-py) builds with maturin from Rust sources. What does run without Rust is copied as files: the pure-Python
manifest consumer (examples/python), the C++ one (examples/cpp), the toy package generator (tools/toy) and the kernel
sources it compiles (tools/kernels-src). Then the reference's own generator builds its toy packages for sm_100a with
nvcc (cross-compiles without a GPU).

    python baseline/install_ref.py [--reference /path/to/reference]
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
PARTS = ["examples/python", "examples/cpp", "tools/toy", "tools/kernels-src", "LICENSE"]


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("KERN_REFERENCE_DIR", ""))
    a = ap.parse_args()
    src = Path(a.reference)
    if not a.reference or not src.is_dir():
        print("pass --reference (or set KERN_REFERENCE_DIR) to the upstream checkout", file=sys.stderr)
        return 2
    dst = HERE / "_ref"
    for part in PARTS:
        s, d = src / part, dst / part
        if not s.exists():
            continue
        d.parent.mkdir(parents=True, exist_ok=True)
        if s.is_dir():
            shutil.copytree(s, d, dirs_exist_ok=True)
        else:
            shutil.copy2(s, d)
    env = dict(os.environ, PATH=os.environ.get("PATH", "") + ":/usr/local/cuda/bin")
    subprocess.run([sys.executable, str(dst / "tools" / "toy" / "gen.py"), "--out", str(dst / "toy_pkg"), "--sm", "sm_100a"],
                   check=True, env=env)
    print("installed:", dst)
    return 0


if __name__ == "__main__":
    sys.exit(main())
