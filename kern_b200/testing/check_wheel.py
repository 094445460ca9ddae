"""Prove a built wheel is whole, without a GPU and without installing it:

    pip wheel . --no-deps --no-build-isolation -w dist/ && python -m kern_b200.testing.check_wheel dist/kern_b200-*.whl

- the version in the wheel's metadata is the package's (`kern_b200.__version__`);
- the console script and both engine plugins' entry points are declared, and the plugin packages are inside;
- every kernel source of the tree has its cubin in the wheel, `kernels/index.json` names exactly those, and each cubin's
  bytes hash to the sha256 the index pins (the identity a manifest's module carries);
- the native module, the `kern` and `kern-run` binaries, the no-alloc host library and the capture library are inside;
- no native file links a CUDA or NVIDIA library (`DT_NEEDED` read straight out of the ELF dynamic section): the runtime
  opens the driver, NCCL and CUPTI at run time, so the wheel imports on a machine that has none of them.

`check(path) -> [findings]`; the command prints them and exits 1 if there are any.
Reference counterpart: scripts/check_wheel.sh, .github/workflows/release.yml:76-114.
"""
from __future__ import annotations

import hashlib
import json
import struct
import sys
import zipfile
from pathlib import Path

ENTRY_POINTS = {"console_scripts": {"kern": "kern_b200.cli:main"},
                "vllm.general_plugins": {"kern_b200": "kern_vllm:register"},
                "sglang.srt.plugins": {"kern_b200": "kern_sglang:register"}}


def needed(elf: bytes) -> list[str]:
    """The DT_NEEDED names of a 64-bit little-endian ELF file (empty for a static one)."""
    if elf[:4] != b"\x7fELF" or elf[4] != 2 or elf[5] != 1:
        raise ValueError("not a 64-bit little-endian ELF file")
    shoff, = struct.unpack_from("<Q", elf, 0x28)
    shentsize, shnum = struct.unpack_from("<HH", elf, 0x3A)
    sections = [struct.unpack_from("<IIQQQQIIQQ", elf, shoff + i * shentsize) for i in range(shnum)]
    out = []
    for (_name, kind, _flags, _addr, off, size, link, _info, _align, entsize) in sections:
        if kind != 6:                                   # SHT_DYNAMIC
            continue
        str_off = sections[link][4]
        for at in range(off, off + size, entsize or 16):
            tag, val = struct.unpack_from("<qQ", elf, at)
            if tag == 0:
                break
            if tag == 1:                                # DT_NEEDED
                end = elf.index(b"\0", str_off + val)
                out.append(elf[str_off + val:end].decode())
    return out


def _entry_points(text: str) -> dict[str, dict[str, str]]:
    out: dict[str, dict[str, str]] = {}
    group = None
    for line in text.splitlines():
        line = line.strip()
        if line.startswith("[") and line.endswith("]"):
            group = line[1:-1]
            out[group] = {}
        elif "=" in line and group is not None:
            k, v = line.split("=", 1)
            out[group][k.strip()] = v.strip()
    return out


def check(wheel: str | Path) -> list[str]:
    from .. import __version__, _build

    errs = []
    if Path(wheel).name.endswith("-none-any.whl"):
        errs.append("the wheel is tagged py3-none-any although it carries native files")
    with zipfile.ZipFile(wheel) as z:
        names = set(z.namelist())
        meta = next((n for n in names if n.endswith(".dist-info/METADATA")), None)
        if meta is None:
            return ["no METADATA in the wheel"]
        version = next((l.split(":", 1)[1].strip() for l in z.read(meta).decode().splitlines() if l.startswith("Version:")), None)
        if version != __version__:
            errs.append(f"the wheel says version {version}, the package {__version__}")
        ep_name = meta.replace("METADATA", "entry_points.txt")
        eps = _entry_points(z.read(ep_name).decode()) if ep_name in names else {}
        for group, want in ENTRY_POINTS.items():
            for k, v in want.items():
                if eps.get(group, {}).get(k) != v:
                    errs.append(f"entry point {group}: {k} = {v} is missing (has: {eps.get(group)})")
        for pkg in ("kern_b200", "kern_vllm", "kern_sglang", "kern_b200/serve", "kern_b200/models", "kern_b200/testing"):
            if f"{pkg}/__init__.py" not in names:
                errs.append(f"the wheel has no package {pkg}")
        # kernels: one cubin per source, pinned by the index
        idx_name = "kern_b200/kernels/index.json"
        index = json.loads(z.read(idx_name)) if idx_name in names else {}
        if not index:
            errs.append("kern_b200/kernels/index.json is missing")
        sources = {p.stem for p in _build.kernel_sources()}
        if set(index) != sources:
            errs.append(f"the index names {sorted(set(index) ^ sources)} differently from the kernel sources")
        for mod, e in sorted(index.items()):
            f = f"kern_b200/kernels/{e['source']}"
            if f not in names:
                errs.append(f"{f} is not in the wheel")
            elif hashlib.sha256(z.read(f)).hexdigest() != e["sha256"]:
                errs.append(f"{f} does not hash to the sha256 its index pins")
        # native files: present, and free of CUDA link-time dependencies
        native = [n for n in names if n.startswith("kern_b200/_native") and n.endswith(".so")]
        if not native:
            errs.append("the native module kern_b200/_native*.so is missing")
        for n in ("kern_b200/bin/kern", "kern_b200/bin/kern-run", "kern_b200/libattn_decode_noalloc.so", "kern_b200/libkern_capture.so"):
            if n not in names:
                errs.append(f"{n} is missing")
        for n in native + [x for x in ("kern_b200/bin/kern", "kern_b200/bin/kern-run", "kern_b200/libkern_capture.so") if x in names]:
            try:
                linked = [l for l in needed(z.read(n)) if l.startswith(("libcu", "libnv", "libnccl"))]
            except ValueError as e:
                errs.append(f"{n}: {e}")
                continue
            if linked:
                errs.append(f"{n} links {', '.join(linked)}: the runtime opens those at run time instead")
    return errs


def main(argv=None) -> int:
    argv = sys.argv[1:] if argv is None else argv
    if len(argv) != 1:
        print("usage: python -m kern_b200.testing.check_wheel WHEEL")
        return 2
    errs = check(argv[0])
    for e in errs:
        print("wheel:", e)
    print(f"{argv[0]}: {'ok' if not errs else f'{len(errs)} findings'}")
    return 1 if errs else 0


if __name__ == "__main__":
    raise SystemExit(main())
