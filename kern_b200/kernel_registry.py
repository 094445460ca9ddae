"""The kernel registry: what the build produced, as families with variants and measured picks, with a content-addressed
store beside it.

    family    one kernel source (`csrc/kernels/sm100/<name>.cu`): one parameter ABI per entry, however it is built
    variant   one artifact of a family: its sha256 (the identity a manifest's module pins), the entries it defines, the
              defines it was built with (`normal`: none; `checked`: -DKERN_CHECKED) and the toolchain line
    pick      a measured choice for one (op, workload shape): which variant — or which entry of it — `kern bench` found
              best, with the bench's report kept in the store as the evidence; never recorded without a report

`document(name)` regenerates a family's document from the tree (sources and cubins) and the picks of
`kernel_index/picks.toml` (the one committed part: a cubin's hash depends on the build, a measured choice does not);
`write_all()` writes `kernel_index/<family>.toml`; `check()` is the offline check a CI runs: every document parses
and is named after its family, every sha256 is 64 hex characters and names one variant across all families, every
variant's bytes in the tree hash to its sha, every entry a variant lists exists in its family's source, every pick names a
variant and an entry that exist and a report that is in the store, and every document is normalised (regenerating it
changes nothing). The store is `$KERN_B200_CACHE/blobs/<sha256>` (default `~/.cache/kern_b200`): bytes are written once
under their hash and never replaced.

    python -m kern_b200 kernels                   # sha256 and file of every module of the build in use
    python -m kern_b200 kernels index             # (re)write kernel_index/*.toml
    python -m kern_b200 kernels check             # the offline check; exit 1 with one line per finding
    python -m kern_b200 kernels pick moe ep_fc2 "rows>192" normal report.json --entry kern_ep_fc2_bf16_combine_n256
    python -m kern_b200 kernels import their.cubin their-family [--entry NAME ...] [--capture launches.jsonl] [--origin URL@COMMIT]
    python -m kern_b200 kernels land manifest.json DIR   # every pinned module into DIR, by content (store, then own build)

Reference counterpart: tools/kernels/index.py (families, variants, picks), pick.py, store.py, check.py, docs/registry.md.
"""
from __future__ import annotations

import datetime
import hashlib
import json
import os
import platform
import re
import tomllib
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
INDEX = ROOT / "kernel_index"
HEX64 = re.compile(r"^[0-9a-f]{64}$")
MACRO_ENTRY = re.compile(r"^\s*(KERN_\w+_ENTRY)\((\w+)", re.M)
FLAVOURS = {"normal": ("kernels", []), "checked": ("kernels_checked", ["KERN_CHECKED"])}


# ---- the store ---------------------------------------------------------------------------------------------------
def cache_dir() -> Path:
    env = os.environ.get("KERN_B200_CACHE")
    return Path(env) if env else Path.home() / ".cache" / "kern_b200"


def blob_path(sha256: str) -> Path:
    return cache_dir() / "blobs" / sha256


def report_path(sha256: str) -> Path:
    """A pick's bench report beside the index (small JSON, committed with the pick it proves)."""
    return INDEX / "reports" / f"{sha256}.json"


def put(path: str | Path, beside_index: bool = False) -> str:
    """Copy a file into the store under its sha256 (written once, never replaced); returns the sha. `beside_index`: also
    under `kernel_index/reports/`, where a pick's evidence travels with the repository."""
    data = Path(path).read_bytes()
    sha = hashlib.sha256(data).hexdigest()
    for dst in [blob_path(sha)] + ([report_path(sha)] if beside_index else []):
        if not dst.exists():
            dst.parent.mkdir(parents=True, exist_ok=True)
            tmp = dst.with_suffix(".tmp")
            tmp.write_bytes(data)
            tmp.replace(dst)
    return sha


# ---- documents -----------------------------------------------------------------------------------------------------
def _name_after(text: str, at: int) -> str | None:
    """The function name after `... void `, past a launch-bounds attribute and its (possibly nested) parentheses."""
    while True:
        m = re.match(r"\s*(__launch_bounds__|__attribute__)\s*\(", text[at:])
        if not m:
            break
        at += m.end() - 1
        depth = 0
        while True:
            depth += {"(": 1, ")": -1}.get(text[at], 0)
            at += 1
            if depth == 0:
                break
    nm = re.match(r"\s*(\w+)\s*\(", text[at:])
    return nm.group(1) if nm else None


_PRE: dict[tuple, str | None] = {}


def _preprocessed(source: Path) -> str | None:
    """`nvcc -E` of a kernel source (cached by path and mtime); None where there is no compiler."""
    import subprocess

    from . import _build

    key = (str(source), source.stat().st_mtime_ns)
    if key not in _PRE:
        try:
            p = subprocess.run([_build.NVCC, *_build.ARCH, "-std=c++17", "-E", "-I", str(_build.KSRC), str(source)],
                               capture_output=True, text=True, timeout=120)
            # keep what comes from the kernel sources themselves: the toolkit's headers declare no entry of ours
            _PRE[key] = p.stdout if p.returncode == 0 else None
        except (OSError, subprocess.SubprocessError):
            _PRE[key] = None
    return _PRE[key]


def entries_of(source: Path) -> list[str]:
    """The `extern "C" __global__` names a source defines, directly or through its KERN_*_ENTRY(name, ...) macros."""
    from . import _build

    text = _preprocessed(source)
    if text is not None:
        # the compiler's own expansion: every macro-made name is spelled out, included sources are inlined
        names = set()
        for m in re.finditer(r'extern\s+"C"\s+__attribute__\(\(global\)\)\s+void\s+|extern\s+"C"\s+__global__\s+void\s+', text):
            nm = _name_after(text, m.end())
            if nm:
                names.add(nm)
        return sorted(names)
    text = source.read_text().replace("\\\n", " ")          # no compiler here: macro bodies on one line, names by pattern
    names = set()
    for m in re.finditer(r'extern\s+"C"\s+__global__\s+void\s+', text):
        nm = _name_after(text, m.end())
        if nm:
            names.add(nm)
    macros = set(re.findall(r"#define\s+(KERN_\w+_ENTRY)\(", text))
    names |= {n for m, n in MACRO_ENTRY.findall(text) if m in macros}
    names.discard("name")                      # the macro definitions' own placeholder
    for inc in re.findall(r'#include\s+"([\w.]+\.cu)"', text):            # a module built on another source's body
        if f"KERN_{Path(inc).stem.split('_')[0].upper()}_NO_ENTRIES" in text or "_NO_ENTRIES" in text:
            continue
        names |= set(entries_of(_build.KSRC / inc))
    return sorted(names)


def families() -> list[str]:
    from . import _build

    return [p.stem for p in _build.kernel_sources()]


PICKS = INDEX / "picks.toml"          # the measured choices: the one part of the index that is not a build output


def load(name: str) -> dict:
    path = INDEX / f"{name}.toml"
    return tomllib.loads(path.read_text()) if path.exists() else {}


def load_picks() -> list[dict]:
    return list(tomllib.loads(PICKS.read_text()).get("pick", [])) if PICKS.exists() else []


def _write_picks(picks: list[dict]) -> None:
    INDEX.mkdir(exist_ok=True)
    q = json.dumps
    lines = ["# measured choices of a variant (and entry) for an op on a workload shape; each carries its bench report's sha256"]
    for p in sorted(picks, key=lambda p: (p["family"], p["op"], p["shape"])):
        lines += ["", "[[pick]]"] + [f"{k} = {q(p[k])}" for k in ("family", "op", "shape", "variant", "entry", "report", "measured") if k in p]
    PICKS.write_text("\n".join(lines) + "\n")


def document(name: str) -> dict:
    from . import _build

    src = _build.KSRC / f"{name}.cu"
    doc = {"family": {"name": name, "kind": "handwritten", "sm": "sm_100a", "source": f"csrc/kernels/sm100/{name}.cu",
                      "toolchain": "nvcc " + " ".join(_build.ARCH + [f for f in _build.NVCC_FLAGS if f not in ("-Xptxas", "-v")])},
           "variant": [], "pick": [{k: v for k, v in p.items() if k != "family"} for p in load_picks() if p.get("family") == name]}
    entries = entries_of(src)
    for flavour, (sub, defines) in FLAVOURS.items():
        cubin = _build.PKG / sub / f"{name}.cubin"
        if cubin.exists():
            doc["variant"].append({"name": flavour, "sha256": hashlib.sha256(cubin.read_bytes()).hexdigest(), "entries": entries,
                                   "defines": defines, "file": f"kern_b200/{sub}/{name}.cubin"})
    return doc


def _toml(doc: dict) -> str:
    q = json.dumps
    lines = ["[family]"] + [f"{k} = {q(v)}" for k, v in doc["family"].items()]
    for v in doc["variant"]:
        lines += ["", "[[variant]]"] + [f"{k} = {q(v[k])}" for k in ("name", "sha256", "entries", "defines", "file")]
    for p in doc.get("pick", []):
        lines += ["", "[[pick]]"] + [f"{k} = {q(p[k])}" for k in ("op", "shape", "variant", "entry", "report", "measured") if k in p]
    return "\n".join(lines) + "\n"


def write_all() -> list[Path]:
    INDEX.mkdir(exist_ok=True)
    out = []
    for name in families():
        path = INDEX / f"{name}.toml"
        path.write_text(_toml(document(name)))
        out.append(path)
    return out


def pick(family: str, op: str, shape: str, variant: str, report: str | Path, entry: str | None = None, measured: str | None = None) -> dict:
    """Record that `variant` (and `entry` of it) is the measured choice for `op` on `shape`; the report goes to the store."""
    doc = document(family)
    v = next((x for x in doc["variant"] if x["name"] == variant), None)
    if v is None:
        raise ValueError(f"family `{family}` has no variant `{variant}` (has: {', '.join(x['name'] for x in doc['variant'])})")
    if entry is not None and entry not in v["entries"]:
        raise ValueError(f"variant `{variant}` of `{family}` defines no entry `{entry}`")
    if not Path(report).exists():
        raise ValueError(f"a pick is never recorded without its bench report: {report} does not exist")
    sha = put(report, beside_index=True)
    rec = {"op": op, "shape": shape, "variant": variant, "report": sha,
           "measured": measured or f"{datetime.date.today().isoformat()} {platform.node()}"}
    if entry is not None:
        rec["entry"] = entry
    _write_picks([p for p in load_picks() if (p.get("family"), p["op"], p["shape"]) != (family, op, shape)] + [dict(rec, family=family)])
    INDEX.mkdir(exist_ok=True)
    (INDEX / f"{family}.toml").write_text(_toml(document(family)))
    return rec


def picked(family: str, op: str, shape: str) -> dict | None:
    """The recorded choice for (op, shape), for a generator that wants the measured variant instead of its own rule."""
    return next((p for p in load_picks() if (p.get("family"), p["op"], p["shape"]) == (family, op, shape)), None)


def check(require_reports: bool = True) -> list[str]:
    errs, seen = [], {}
    known = set(families())
    for path in sorted(p for p in INDEX.glob("*.toml") if p != PICKS) if INDEX.exists() else []:
        try:
            doc = tomllib.loads(path.read_text())
        except tomllib.TOMLDecodeError as e:
            errs.append(f"{path.name}: does not parse: {e}")
            continue
        name = doc.get("family", {}).get("name")
        if name != path.stem:
            errs.append(f"{path.name}: the family inside is `{name}`")
            continue
        if name not in known:
            errs.append(f"{path.name}: no source csrc/kernels/sm100/{name}.cu")
            continue
        fresh = document(name)
        if _toml(fresh) != path.read_text():
            errs.append(f"{path.name}: not what the tree regenerates (run `kern kernels index`)")
        names = set()
        for v in doc.get("variant", []):
            names.add(v["name"])
            if not HEX64.match(v.get("sha256", "")):
                errs.append(f"{path.name}: variant `{v['name']}`: sha256 is not 64 hex characters")
                continue
            if v["sha256"] in seen and seen[v["sha256"]] != (name, v["name"]):
                errs.append(f"{path.name}: variant `{v['name']}` has the sha256 of {seen[v['sha256']]}")
            seen[v["sha256"]] = (name, v["name"])
            f = ROOT / v.get("file", "")
            if not f.exists() or hashlib.sha256(f.read_bytes()).hexdigest() != v["sha256"]:
                errs.append(f"{path.name}: variant `{v['name']}`: {v.get('file')} does not hash to its sha256")
            missing = [e for e in v.get("entries", []) if e not in entries_of(ROOT / doc["family"]["source"])]
            if missing:
                errs.append(f"{path.name}: variant `{v['name']}` lists entries its source does not define: {', '.join(missing)}")
        for p in doc.get("pick", []):
            what = f"pick {p.get('op')} on {p.get('shape')}"
            v = next((x for x in doc.get("variant", []) if x["name"] == p.get("variant")), None)
            if v is None:
                errs.append(f"{path.name}: {what}: no variant `{p.get('variant')}`")
            elif p.get("entry") and p["entry"] not in v.get("entries", []):
                errs.append(f"{path.name}: {what}: variant `{v['name']}` has no entry `{p['entry']}`")
            if not HEX64.match(p.get("report", "")):
                errs.append(f"{path.name}: {what}: carries no report")
            elif require_reports and not (blob_path(p["report"]).exists() or report_path(p["report"]).exists()):
                errs.append(f"{path.name}: {what}: report {p['report'][:12]} is neither beside the index nor in the store ({cache_dir()})")
    for p in load_picks():
        if p.get("family") not in known:
            errs.append(f"picks.toml: pick {p.get('op')} on {p.get('shape')}: no family `{p.get('family')}`")
    for name in sorted(known - {p.stem for p in (INDEX.glob("*.toml") if INDEX.exists() else [])}):
        errs.append(f"kernel_index/{name}.toml is missing (run `kern kernels index`)")
    return errs + check_imported()


# ---- kernels that were not built here ------------------------------------------------------------------------------
IMPORTED = INDEX / "imported"      # committed: the hash of somebody else's cubin does not depend on this tree's build


def entries_from_capture(capture_file: str | Path, sha256: str) -> list[str]:
    """The symbols a captured process launched out of the module with this hash (`kern_b200/capture.py`)."""
    from . import capture

    cap = capture.Capture(capture.load(capture_file))
    return sorted({r["symbol"] for r in cap.launches if r.get("module") == sha256})


def entries_from_driver(path: str | Path) -> list[str]:
    """Every entry of a cubin, enumerated by the driver after loading it (needs a GPU; nothing is disassembled)."""
    from . import _native

    dev = _native.Device(0)
    return sorted(dev.entries(dev.load_module(Path(path).read_bytes())))


def import_cubin(path: str | Path, family: str, entries: list[str] | None = None, capture_file: str | Path | None = None,
                 origin: str | None = None) -> dict:
    """Register a cubin that another project built: its bytes go into the store under their sha256 and
    `kernel_index/imported/<family>.toml` records the hash, the size, the entries and where it came from (`origin`: the
    upstream URL and commit, as the importer states it). The entries come from `entries`, else from a capture of a
    process that launched the module, else from the driver on a machine with a GPU. Importing another build of the same
    family adds a variant; importing the same bytes again changes nothing.
    Reference counterpart: tools/kernels/import_cubin.py (which lists entries with an external dump tool)."""
    if not re.fullmatch(r"[a-z0-9][a-z0-9_\-]*", family):
        raise ValueError(f"family `{family}`: lower-case letters, digits, `_` and `-`")
    if family in families():
        raise ValueError(f"`{family}` is a family of this tree's own sources")
    sha = put(path)
    if not entries and capture_file:
        entries = entries_from_capture(capture_file, sha)
        if not entries:
            raise ValueError(f"the capture holds no launch out of a module with sha256 {sha[:12]}…")
    if not entries:
        try:
            entries = entries_from_driver(path)
        except Exception as e:
            raise ValueError(f"no entries given, no capture, and the driver could not list them ({e})") from None
    doc_path = IMPORTED / f"{family}.toml"
    doc = tomllib.loads(doc_path.read_text()) if doc_path.exists() else {"family": {"name": family, "kind": "imported"}, "variant": []}
    if not any(v["sha256"] == sha for v in doc["variant"]):
        doc["variant"].append({"name": f"v{len(doc['variant'])}", "sha256": sha, "entries": sorted(entries), "bytes": Path(path).stat().st_size,
                               "file": Path(path).name, "origin": origin or "", "imported": datetime.date.today().isoformat()})
    q = json.dumps
    lines = ["[family]"] + [f"{k} = {q(v)}" for k, v in doc["family"].items()]
    for v in doc["variant"]:
        lines += ["", "[[variant]]"] + [f"{k} = {q(v[k])}" for k in ("name", "sha256", "entries", "bytes", "file", "origin", "imported")]
    IMPORTED.mkdir(parents=True, exist_ok=True)
    doc_path.write_text("\n".join(lines) + "\n")
    return doc


def imported() -> dict[str, dict]:
    return {p.stem: tomllib.loads(p.read_text()) for p in sorted(IMPORTED.glob("*.toml"))} if IMPORTED.exists() else {}


def module_decl(family: str, variant: str | None = None) -> dict:
    """The `modules` entry a manifest carries for an imported family: {"source", "sha256"} (the last variant by default)."""
    doc = imported().get(family)
    if doc is None:
        raise KeyError(f"no imported family `{family}`")
    v = doc["variant"][-1] if variant is None else next(x for x in doc["variant"] if x["name"] == variant)
    return {"source": v["file"], "sha256": v["sha256"]}


def check_imported() -> list[str]:
    errs, seen = [], {}
    for name, doc in imported().items():
        if doc.get("family", {}).get("name") != name or doc["family"].get("kind") != "imported":
            errs.append(f"imported/{name}.toml: the family inside is `{doc.get('family', {}).get('name')}` of kind `{doc.get('family', {}).get('kind')}`")
        if not doc.get("variant"):
            errs.append(f"imported/{name}.toml: no variant")
        for v in doc.get("variant", []):
            if not HEX64.match(v.get("sha256", "")):
                errs.append(f"imported/{name}.toml: variant `{v.get('name')}`: sha256 is not 64 hex characters")
                continue
            if v["sha256"] in seen:
                errs.append(f"imported/{name}.toml: variant `{v['name']}` has the sha256 of {seen[v['sha256']]}")
            seen[v["sha256"]] = (name, v["name"])
            if not v.get("entries"):
                errs.append(f"imported/{name}.toml: variant `{v['name']}` lists no entry")
            blob = blob_path(v["sha256"])
            if blob.exists() and hashlib.sha256(blob.read_bytes()).hexdigest() != v["sha256"]:
                errs.append(f"imported/{name}.toml: variant `{v['name']}`: the store's blob does not hash to its name")
    return errs


def land(manifest: dict, into: str | Path) -> tuple[list[str], list[str]]:
    """Put every module a manifest pins into the directory a runtime is pointed at, by content: a file under `into` that
    already hashes to the pin stays; otherwise the bytes come from the store, else from this package's own kernels. File
    names are labels (the runtime finds modules by hash), so a landed file is named `<module>-<sha12>.cubin`.
    -> (landed files, modules nowhere to be found). Reference counterpart: tools/extract_kernels.sh, tools/kernels/store.py."""
    from . import _build

    into = Path(into)
    into.mkdir(parents=True, exist_ok=True)
    have = {hashlib.sha256(p.read_bytes()).hexdigest() for p in into.glob("*.cubin")}
    own = {}
    for sub, _ in FLAVOURS.values():
        for p in (_build.PKG / sub).glob("*.cubin"):
            own.setdefault(hashlib.sha256(p.read_bytes()).hexdigest(), p)
    landed, missing = [], []
    for name, mod in sorted(manifest.get("modules", {}).items()):
        sha = mod.get("sha256", "")
        if sha in have:
            continue
        src = blob_path(sha) if blob_path(sha).exists() else own.get(sha)
        if src is None:
            missing.append(f"{name} ({mod.get('source')}, {sha[:12]}…)")
            continue
        data = src.read_bytes()
        if hashlib.sha256(data).hexdigest() != sha:
            missing.append(f"{name}: {src} does not hash to its name")
            continue
        dst = into / f"{name}-{sha[:12]}.cubin"
        dst.write_bytes(data)
        have.add(sha)
        landed.append(dst.name)
    return landed, missing
