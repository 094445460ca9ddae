"""From a running program's launches to a manifest: read what `libkern_capture.so` wrote and turn it into facts.

    CUDA_INJECTION64_PATH=$(python -c 'import kern_b200.capture as c; print(c.library())') KERN_CAPTURE_DIR=cap ./program
    kern capture lift cap/pid*/launches.jsonl --symbol fwd_prepare [--names names.txt] [--all]
    kern capture mine cap/pid*/launches.jsonl [--tokens 7,64,512] [--json facts.json]

`lift` turns one captured launch into an op skeleton of the manifest format: the launch's `params` (`bytes<n>` for a
descriptor or a struct, `buffer<u8>` for a pointer, `i32` / `i64` / `f32` / `u8` for scalars) and `args`, with every
tensor-map descriptor spelled out (dtype, dims, strides, box, swizzle, L2 promotion) at the byte where it sits and every
struct as a `pack` of the fields that are not zero. Every distinct (allocation, offset) a launch points at becomes one
interface parameter of the op; the `pointers` table beside the skeleton says which is which (`@A+0x60000`: allocation A,
byte offset), and `--names` (lines of `name pointer`, printed by the launcher) replaces the letters by names — a letter
is an address, not a guess at what a parameter should be. `--all` prints one skeleton per shape variant of the symbol,
which shows the numbers that move with the shape; those become vars in the hand-written generator.

`mine` works on a whole serving run: it cuts the launches into windows at time gaps and into forward passes at the
bursts of the most frequent kernel, names a call site by (symbol, occurrence within its pass), and then
  - classifies every pointer by how its (allocation, offset) behaves: the same in every pass but different between the
    call sites of a symbol -> a weight; the same in every pass and at every site -> a state or an input; changing
    between passes -> workspace;
  - fits every grid axis and scalar that varies to the closed set {t, a*t, ceil(t/d), ceil(a*t/d), a*ceil(t/d)} (+ a
    constant), t being the pass's token count (given with `--tokens`, or taken from the scalar that most sites agree on).
It prints a report and, with `--json`, writes every fact; it does not write a manifest.

Reference counterpart: tools/kernel-capture/lift.py, tools/mine_capture.py, tools/kernel-capture/README.md.
"""
from __future__ import annotations

import argparse
import json
import math
import struct
import sys
from collections import Counter, defaultdict
from pathlib import Path

TMAP_DTYPES = {0: "u8", 1: "u16", 2: "u32", 3: "i32", 4: "u64", 5: "i64", 6: "f16", 7: "f32", 9: "bf16", 11: "tf32",
               13: "u4packed", 14: "u4"}
SWIZZLE = {0: 0, 1: 32, 2: 64, 3: 128}
L2 = {0: 0, 1: 64, 2: 128, 3: 256}


def library() -> Path:
    """The injection library's path (built on demand)."""
    from . import _build

    return _build.build_capture()


def load(path: str | Path) -> list[dict]:
    out = []
    with open(path) as f:
        for n, line in enumerate(f, 1):
            line = line.strip()
            if not line:
                continue
            try:
                out.append(json.loads(line))
            except json.JSONDecodeError:
                if n == 1:
                    raise ValueError(f"{path}: not a capture file")
                break                                   # a process that was killed leaves a cut last line
    return out


class Capture:
    """The records of one process, indexed: launches in order, descriptors by id."""

    def __init__(self, records: list[dict]):
        self.records = records
        self.launches = [r for r in records if r.get("kind") == "launch"]
        self.maps = {r["id"]: r for r in records if r.get("kind") == "tensormap"}
        self.modules = [r for r in records if r.get("kind") == "module"]

    def of_symbol(self, text: str) -> list[dict]:
        return [r for r in self.launches if text in r["symbol"]]


# ---------------------------------------------------------------- lift

def _letters():
    n = 0
    while True:
        s, k = "", n
        while True:
            s = chr(ord("A") + k % 26) + s
            k = k // 26 - 1
            if k < 0:
                break
        yield s
        n += 1


def _scalar(data: bytes) -> tuple[str, dict]:
    """A 1-, 4- or 8-byte parameter as (type, arg). Four bytes read as f32 when that is the likelier reading: the integer
    is huge while the float is a plain number."""
    if len(data) == 1:
        return "u8", {"u8": data[0]}
    if len(data) == 4:
        i, = struct.unpack("<i", data)
        f, = struct.unpack("<f", data)
        if abs(i) > (1 << 23) and math.isfinite(f) and 1e-8 < abs(f) < 1e8:
            return "f32", {"f32": float(f"{f:.9g}")}
        return "i32", {"i32": i}
    i, = struct.unpack("<q", data)
    return "i64", {"i64": i}


class _Interface:
    """The op's interface while a launch is lifted: one `buffer<u8>` per distinct (allocation, offset)."""

    def __init__(self, names: dict[int, str] | None):
        self.names, self.letters = names or {}, _letters()
        self.alloc_name: dict[int, str] = {}
        self.index: dict[tuple[int, int], int] = {}
        self.pointers: list[str] = []
        self.allocations: dict[str, dict] = {}

    def param(self, base: int, offset: int, nbytes: int | None) -> int:
        key = (base, offset)
        if key not in self.index:
            if base not in self.alloc_name:
                self.alloc_name[base] = self.names.get(base) or next(self.letters)
                self.allocations[self.alloc_name[base]] = {"base": hex(base), "bytes": nbytes}
            exact = self.names.get(base + offset) if offset else None      # a named view inside an allocation
            self.index[key] = len(self.pointers)
            self.pointers.append(f"@{exact}+0x0" if exact else f"@{self.alloc_name[base]}+{hex(offset)}")
        return self.index[key]


def _tensormap(t: dict, iface: _Interface, allocs: list[tuple[int, int]]) -> tuple[dict, list[str]]:
    addr = int(t["address"], 16)
    base, nbytes = next(((b, n) for b, n in allocs if b <= addr < b + n), (addr, None))
    decl = {"param": iface.param(base, addr - base, nbytes), "dtype": TMAP_DTYPES.get(t["dtype"], f"?{t['dtype']}"),
            "dims": t["dims"], "strides": t["strides"], "box": t["box"], "swizzle": SWIZZLE.get(t["swizzle"], t["swizzle"]),
            "l2_promotion": L2.get(t["l2_promotion"], t["l2_promotion"])}
    if t.get("oob_fill"):
        decl["oob_nan"] = True
    notes = []
    if any(e != 1 for e in t.get("elem_strides", [])):
        notes.append(f"element strides {t['elem_strides']} (the manifest format has none: the descriptor cannot be declared as is)")
    if t.get("interleave"):
        notes.append(f"interleave {t['interleave']}")
    if addr != base:
        notes.append(f"the descriptor starts {addr - base} bytes into its allocation: bind that view")
    return decl, notes


def lift(rec: dict, cap: Capture, names: dict[int, str] | None = None) -> dict:
    """One launch record -> {"op": {"params", "impl": {"launches": [launch]}}, "pointers", "allocations", "notes"}."""
    iface = _Interface(names)
    allocs = sorted({(int(p["base"], 16), p["bytes"]) for prm in rec["params"] for p in prm.get("pointers", [])})
    allocs += [(int(r["ptr"], 16), r["bytes"]) for r in cap.records if r.get("kind") == "alloc"]
    params, args, notes = [], [], []
    for prm in rec["params"]:
        data = bytes.fromhex(prm["hex"])
        ptrs = {p["at"]: p for p in prm.get("pointers", [])}
        maps = {m["at"]: cap.maps[m["id"]] for m in prm.get("tensormaps", []) if m["id"] in cap.maps}
        size = prm["size"]
        if size == 8 and 0 in ptrs:
            p = ptrs[0]
            params.append("inout buffer<u8>")
            args.append({"param": iface.param(int(p["base"], 16), p["offset"], p["bytes"])})
            continue
        if size in (1, 4, 8) and not maps:
            kind, arg = _scalar(data)
            params.append(kind)
            args.append(arg)
            continue
        fields, covered = [], set()
        for at, t in sorted(maps.items()):
            decl, why = _tensormap(t, iface, allocs)
            fields.append({"at": at, "tensormap": decl})
            notes += [f"param {prm['index']} +{at}: {w}" for w in why]
            covered.update(range(at, at + 128))
        for at, p in sorted(ptrs.items()):
            if at not in covered:
                fields.append({"at": at, "param": iface.param(int(p["base"], 16), p["offset"], p["bytes"])})
                covered.update(range(at, at + 8))
        for at in range(0, size - size % 4, 4):
            if at in covered or data[at:at + 4] == b"\0\0\0\0":
                continue
            fields.append({"at": at, **_scalar(data[at:at + 4])[1]})
        for at in range(size - size % 4, size):
            if data[at]:
                fields.append({"at": at, "u8": data[at]})
        params.append(f"bytes<{size}>")
        args.append({"pack": {"size": size, "fields": sorted(fields, key=lambda f: f["at"])}})
    launch = {"module": rec.get("module") or "?", "entry": rec["symbol"], "grid": rec["grid"], "block": rec["block"],
              "shared_mem": rec["smem"], "params": params, "args": args}
    if rec.get("cluster"):
        launch["cluster"] = rec["cluster"]
    if rec.get("cooperative"):
        notes.append("a cooperative launch: its blocks wait on one another, so the grid must fit the device at once")
    if rec.get("module") is None:
        notes.append("the launch's module was not seen loading (a module of the runtime's own registration): pin it by the file's sha256")
    return {"op": {"params": ["inout buffer<u8>"] * len(iface.pointers), "impl": {"launches": [launch]}},
            "pointers": {str(i): p for i, p in enumerate(iface.pointers)}, "allocations": iface.allocations,
            "attrs": rec.get("attrs", {}), "notes": notes}


def variant_key(rec: dict) -> tuple:
    """What makes two launches of a symbol the same shape: geometry and every byte that is not a pointer."""
    masked = []
    for prm in rec["params"]:
        data = bytearray.fromhex(prm["hex"])
        for p in prm.get("pointers", []):
            data[p["at"]:p["at"] + 8] = b"\0" * 8
        for m in prm.get("tensormaps", []):
            data[m["at"]:m["at"] + 128] = b"\0" * 128
        masked.append(bytes(data))
    return (rec["symbol"], tuple(rec["grid"]), tuple(rec["block"]), rec["smem"], tuple(masked))


def variants(launches: list[dict]) -> list[tuple[dict, int]]:
    """The first launch of every distinct shape, with how often the shape occurs."""
    seen: dict[tuple, list] = {}
    for r in launches:
        seen.setdefault(variant_key(r), [r, 0])[1] += 1
    return [(r, n) for r, n in seen.values()]


def read_names(path: str | Path) -> dict[int, str]:
    out = {}
    for line in Path(path).read_text().split("\n"):
        parts = line.split()
        if len(parts) == 2:
            out[int(parts[1], 16)] = parts[0]
    return out


# ---------------------------------------------------------------- mine

def windows(launches: list[dict], gap_ms: float = 5.0) -> list[list[dict]]:
    """Cut where the process launched nothing for `gap_ms`: requests and warm-up runs fall apart there."""
    out, cur = [], []
    for r in launches:
        if cur and r["t_ns"] - cur[-1]["t_ns"] > gap_ms * 1e6:
            out.append(cur)
            cur = []
        cur.append(r)
    if cur:
        out.append(cur)
    return out


def forwards(window: list[dict], core: str, burst_gap: int = 25) -> list[list[dict]]:
    """Cut a window into forward passes. The core kernel (the most frequent one: it runs in every layer) shows up as one
    dense burst per pass. A symbol that occurs exactly once per burst, before it, starts a pass (the earliest such symbol
    is taken); without one, a pass ends as many launches after its burst as the window's last pass does."""
    at = [i for i, r in enumerate(window) if r["symbol"] == core]
    if not at:
        return []
    bursts = [[at[0]]]
    for i in at[1:]:
        if i - bursts[-1][-1] > burst_gap:
            bursts.append([])
        bursts[-1].append(i)
    if len(bursts) == 1:
        return [window]
    counts = Counter(r["symbol"] for r in window)
    first_seen = {}
    for i, r in enumerate(window):
        first_seen.setdefault(r["symbol"], i)
    for sym in sorted((s for s, n in counts.items() if n == len(bursts) and s != core), key=first_seen.get):
        where = [i for i, r in enumerate(window) if r["symbol"] == sym]
        ends = [b[-1] for b in bursts]
        if all(w < b[0] for w, b in zip(where, bursts)) and all(w > e for w, e in zip(where[1:], ends)):
            return [window[a:b] for a, b in zip(where, where[1:] + [len(window)])]
    tail = len(window) - 1 - bursts[-1][-1]
    cuts = [0] + [min(len(window), b[-1] + tail + 1) for b in bursts]
    return [window[a:b] for a, b in zip(cuts, cuts[1:]) if b > a]


def sites(forward: list[dict]) -> dict[tuple[str, int], dict]:
    """Call sites of one pass: (symbol, how many launches of the symbol came before it in the pass)."""
    seen, out = Counter(), {}
    for r in forward:
        out[(r["symbol"], seen[r["symbol"]])] = r
        seen[r["symbol"]] += 1
    return out


def _ceil_div(a: int, b: int) -> int:
    return -(-a // b)


def fit(samples: list[tuple[int, int]], divisors=None, factors=None) -> list[dict]:
    """Every expression of the closed set that reproduces all (t, value) samples, simplest first:
    const, t, a*t, ceil(t/d), ceil(a*t/d), a*ceil(t/d). More than one answer means the samples do not tell them apart:
    capture another token count."""
    divisors = divisors or [2 ** i for i in range(1, 17)] + [48, 96, 192, 384, 768]
    factors = factors or list(range(2, 65)) + [128, 256]
    ts = {t for t, _ in samples}
    out = []
    if len({v for _, v in samples}) == 1:
        return [{"kind": "const", "value": samples[0][1]}]
    if len(ts) < 2:
        return []
    if all(v == t for t, v in samples):
        out.append({"kind": "t"})
    for a in factors:
        if all(v == a * t for t, v in samples):
            out.append({"kind": "mul", "a": a})
    for d in divisors:
        if all(v == _ceil_div(t, d) for t, v in samples):
            out.append({"kind": "ceil_div", "d": d})
    if not out:
        for d in divisors:
            for a in factors:
                if all(v == _ceil_div(a * t, d) for t, v in samples) and math.gcd(a, d) == 1:
                    out.append({"kind": "ceil_div_mul", "a": a, "d": d})
                if all(v == a * _ceil_div(t, d) for t, v in samples):
                    out.append({"kind": "mul_ceil_div", "a": a, "d": d})
    return out[:8]


def expr_text(e: dict) -> str:
    k = e["kind"]
    return {"const": lambda: str(e["value"]), "t": lambda: "t", "mul": lambda: f"{e['a']}*t", "ceil_div": lambda: f"ceil(t/{e['d']})",
            "ceil_div_mul": lambda: f"ceil({e['a']}*t/{e['d']})", "mul_ceil_div": lambda: f"{e['a']}*ceil(t/{e['d']})"}[k]()


def _scalars(rec: dict) -> dict[str, int]:
    """Every number of a launch that could depend on the shape: grid axes, dynamic shared bytes, and the 4-byte words of
    the parameters that are neither pointers nor descriptors."""
    out = {f"grid.{'xyz'[i]}": g for i, g in enumerate(rec["grid"])}
    out["smem"] = rec["smem"]
    for prm in rec["params"]:
        data = bytes.fromhex(prm["hex"])
        skip = set()
        for p in prm.get("pointers", []):
            skip.update(range(p["at"], p["at"] + 8))
        for m in prm.get("tensormaps", []):
            skip.update(range(m["at"], m["at"] + 128))
        for at in range(0, len(data) - len(data) % 4, 4):
            if at not in skip:
                out[f"p{prm['index']}+{at}"] = struct.unpack_from("<i", data, at)[0]
    return out


def _pointers(rec: dict, maps: dict) -> dict[str, tuple]:
    out = {}
    for prm in rec["params"]:
        for p in prm.get("pointers", []):
            out[f"p{prm['index']}+{p['at']}"] = (p["base"], p["offset"])
        for m in prm.get("tensormaps", []):
            if m["id"] in maps:
                out[f"p{prm['index']}+{m['at']}:map"] = ("map", maps[m["id"]]["address"])
    return out


def mine(cap: Capture, gap_ms: float = 5.0, tokens: list[int] | None = None, min_launches: int = 20, burst_gap: int = 25) -> dict:
    if not cap.launches:
        return {"error": "the capture holds no launches"}
    core = Counter(r["symbol"] for r in cap.launches).most_common(1)[0][0]
    wins = [w for w in windows(cap.launches, gap_ms)]
    passes = [f for w in wins if len(w) >= min_launches for f in forwards(w, core, burst_gap)]
    dropped = sum(len(w) for w in wins if len(w) < min_launches)
    if not passes:
        return {"error": f"no window of {min_launches} launches or more", "core": core, "windows": len(wins)}
    # passes of one launch sequence are one class; the largest class is analysed
    classes: dict[tuple, list[int]] = defaultdict(list)
    for i, f in enumerate(passes):
        classes[tuple(r["symbol"] for r in f)].append(i)
    members = max(classes.values(), key=len)
    chosen = [passes[i] for i in members]
    site_maps = [sites(f) for f in chosen]
    keys = list(site_maps[0])
    scalars = {k: [_scalars(sm[k]) for sm in site_maps] for k in keys}

    # the token count of every pass: given, or the varying vector that most sites carry
    given = None
    if tokens is not None:
        if len(tokens) != len(passes):
            return {"error": f"--tokens names {len(tokens)} passes, the capture has {len(passes)}"}
        given = [tokens[i] for i in members]
    votes = Counter()
    for k in keys:
        for name in scalars[k][0]:
            vec = tuple(s.get(name) for s in scalars[k])
            if len(set(vec)) > 1 and all(isinstance(v, int) and v > 0 for v in vec):
                votes[vec] += 1
    t_vec = tuple(given) if given else (votes.most_common(1)[0][0] if votes else None)

    exprs, unexplained = {}, []
    for k in keys:
        for name in scalars[k][0]:
            vec = [s.get(name) for s in scalars[k]]
            if len(set(vec)) <= 1 or t_vec is None:
                continue
            found = fit(list(zip(t_vec, vec)))
            label = f"{k[0]}#{k[1]} {name}"
            if found:
                exprs[label] = found
            else:
                unexplained.append({"site": label, "values": vec})

    # pointers
    ptrs = {k: [_pointers(sm[k], cap.maps) for sm in site_maps] for k in keys}
    by_symbol: dict[tuple[str, str], dict[int, tuple | None]] = defaultdict(dict)
    for k in keys:
        for name in ptrs[k][0]:
            ids = [p.get(name) for p in ptrs[k]]
            by_symbol[(k[0], name)][k[1]] = ids[0] if len(set(ids)) == 1 else None
    pointer_class = {}
    for (sym, name), per_site in sorted(by_symbol.items()):
        stable = [v for v in per_site.values() if v is not None]
        if len(stable) < len(per_site):
            kind = "workspace"
        elif len(chosen) < 2:
            kind = "fixed (one pass: cannot tell a weight from workspace)"
        elif len(per_site) == 1:
            kind = "fixed (one call site: a weight or a state)"
        elif len(set(stable)) == 1:
            kind = "state or input (the same at every call site)"
        elif len(set(stable)) == len(stable):
            kind = "weight (fixed, one per call site)"
        else:
            kind = f"fixed, {len(set(stable))} distinct over {len(stable)} call sites (shared weights or per-group state)"
        pointer_class[f"{sym} {name}"] = {"class": kind, "sites": len(per_site)}
    return {"core": core, "windows": len(wins), "passes": len(passes), "classes": len(classes), "analysed_passes": members,
            "launches_per_pass": len(chosen[0]), "dropped_launches": dropped, "tokens": list(t_vec) if t_vec else None,
            "tokens_from": "given" if given else ("the vector most sites carry" if t_vec else None),
            "expressions": exprs, "unexplained": unexplained, "pointers": pointer_class,
            "modules": sorted({r["sha256"] for r in cap.modules})}


def report(facts: dict) -> str:
    if "error" in facts:
        return "mine: " + facts["error"]
    lines = [f"core kernel: {facts['core']}",
             f"{facts['windows']} windows, {facts['passes']} forward passes in {facts['classes']} launch-sequence classes; analysed "
             f"{len(facts['analysed_passes'])} passes of {facts['launches_per_pass']} launches ({facts['dropped_launches']} launches in short windows dropped)",
             f"tokens per pass: {facts['tokens']} ({facts['tokens_from']})", "", "expressions (t = tokens):"]
    short = lambda s: s if len(s) <= 100 else s[:60] + "…" + s[-36:]
    for label, found in facts["expressions"].items():
        also = f"   also: {', '.join(expr_text(e) for e in found[1:])}" if len(found) > 1 else ""
        lines.append(f"  {short(label)} = {expr_text(found[0])}{also}")
    for u in facts["unexplained"]:
        lines.append(f"  {short(u['site'])} = ?  values {u['values']}")
    lines += ["", "pointers:"]
    for label, c in facts["pointers"].items():
        lines.append(f"  {short(label)}: {c['class']} [{c['sites']} sites]")
    return "\n".join(lines)


# ---------------------------------------------------------------- command

def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="kern capture", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)
    sub.add_parser("path", help="print the injection library's path")
    lp = sub.add_parser("lift", help="one launch -> an op skeleton")
    lp.add_argument("file")
    lp.add_argument("--symbol", required=True, help="text the kernel's symbol contains")
    lp.add_argument("--names", help="a file of `name pointer` lines")
    lp.add_argument("--all", action="store_true", help="one skeleton per shape variant")
    lp.add_argument("--nth", type=int, default=0, help="which launch of the symbol (default the first)")
    mp = sub.add_parser("mine", help="passes, pointer classes, expressions")
    mp.add_argument("file")
    mp.add_argument("--gap-ms", type=float, default=5.0)
    mp.add_argument("--tokens", help="token counts of the passes in order, comma-separated")
    mp.add_argument("--min-launches", type=int, default=20, help="windows with fewer launches are start-up noise")
    mp.add_argument("--burst-gap", type=int, default=25, help="launches between two core launches that end a pass's burst")
    mp.add_argument("--json", dest="json_out")
    a = ap.parse_args(argv)
    if a.cmd == "path":
        print(library())
        return 0
    cap = Capture(load(a.file))
    if a.cmd == "lift":
        found = cap.of_symbol(a.symbol)
        if not found:
            print(f"no launch whose symbol contains `{a.symbol}`; symbols: {sorted({r['symbol'] for r in cap.launches})[:20]}", file=sys.stderr)
            return 1
        names = read_names(a.names) if a.names else None
        picked = variants(found) if a.all else [(found[min(a.nth, len(found) - 1)], len(found))]
        for rec, n in picked:
            out = lift(rec, cap, names)
            out["launches_of_this_shape" if a.all else "launches_of_this_symbol"] = n
            print(json.dumps(out, indent=1))
        return 0
    facts = mine(cap, a.gap_ms, [int(x) for x in a.tokens.split(",")] if a.tokens else None, a.min_launches, a.burst_gap)
    print(report(facts))
    if a.json_out:
        Path(a.json_out).write_text(json.dumps(facts, indent=1))
    return 1 if "error" in facts else 0


if __name__ == "__main__":
    raise SystemExit(main())
