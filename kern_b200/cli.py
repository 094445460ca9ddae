"""The `kern` command: verify / cut / kernels / run / test / bench / workload / server.

    python -m kern_b200 verify model/manifest.json
    python -m kern_b200 cut model/manifest.json --at 40,80 --out stages/
    python -m kern_b200 run --manifest m.json --weights ckpt/ --prompt-ids 1,2,3 --steps 16 [--cpu]
    python -m kern_b200 test A.json B.json --weights ckpt/ [--cpu]        (exit 0 PASS / 1 FAIL / 2 INCONCLUSIVE)
    python -m kern_b200 bench --manifest m.json --weights ckpt/ [--workload w.toml]
    python -m kern_b200 server --manifest m.json --weights ckpt/ --port 8000

Flags override the `[targets.<name>]` of a `kern.toml` found by walking up from the working directory
(`gpu`, `capacity`, `[targets.x]{manifest,reference,kernels,weights,tokenizer}`, `[test]`, `[run]`).
Reference: crates/kern-run/src/bin/kern.rs:32-333, crates/kern-run/src/config.rs:40-159.
"""
from __future__ import annotations

import argparse
import json
import statistics
import sys
import time
import tomllib
from pathlib import Path


# ---- kern.toml ---------------------------------------------------------------------------------------
_TOP = {"gpu", "capacity", "targets", "kernels", "test", "run"}
_TARGET = {"manifest", "reference", "kernels", "weights", "tokenizer"}


def find_config(start: Path | None = None) -> tuple[Path | None, dict]:
    d = (start or Path.cwd()).resolve()
    for p in [d, *d.parents]:
        f = p / "kern.toml"
        if f.exists():
            cfg = tomllib.loads(f.read_text())
            unknown = set(cfg) - _TOP
            if unknown:
                raise SystemExit(f"{f}: unknown field(s) {sorted(unknown)}")
            for name, t in cfg.get("targets", {}).items():
                bad = set(t) - _TARGET
                if bad:
                    raise SystemExit(f"{f}: target `{name}`: unknown field(s) {sorted(bad)}")
            return f, cfg
    return None, {}


def resolve(args, cfg_path, cfg) -> None:
    """flag > target > default."""
    t = cfg.get("targets", {}).get(getattr(args, "target", None) or "", {})
    base = cfg_path.parent if cfg_path else Path.cwd()
    for key in ("manifest", "weights", "kernels", "tokenizer"):
        if getattr(args, key, None) is None and key in t:
            setattr(args, key, str(base / t[key]))
    if getattr(args, "gpu", None) is None:
        args.gpu = cfg.get("gpu", 0)
    if getattr(args, "capacity", None) is None:
        args.capacity = cfg.get("capacity", 0)


def make_runtime(args, manifest=None):
    manifest = manifest or args.manifest
    model = getattr(args, "model", None)
    if model and not manifest:
        from .models import registry

        over = {k: getattr(args, k, None) or None for k in ("layers", "max_tokens", "max_seqs", "max_context")}
        cfg, build, load, make = registry.resolve(model, **over)
        doc = build(cfg)
        # state slots only for models with per-sequence state: a lease that holds a slot makes its checkpoints usable
        # at their exact length only, which would cost a slot-free model most of its prefix-cache hits
        slots = (getattr(cfg, "max_seqs", 0) or 8) if any(s.get("bytes_per_seq") for s in doc["states"].values()) else 0
        if args.cpu:
            from .cpu import CpuRuntime

            rt = CpuRuntime(doc, weights=make(cfg), tokens=args.capacity or 4096, slots=slots)
        else:
            from .runtime import Runtime

            rt = Runtime(doc, kernels=args.kernels, gpu=args.gpu, tokens=args.capacity or 0, slots=slots)
            load(rt, cfg)
        rt.once()
        return rt
    if args.cpu:
        from .cpu import CpuRuntime

        rt = CpuRuntime(manifest, weights=_weights_path(args.weights), tokens=args.capacity or 4096, slots=getattr(args, "max_seqs", 0) or 0)
    else:
        from .runtime import Runtime

        rt = Runtime(manifest, kernels=args.kernels, weights=args.weights, gpu=args.gpu, tokens=args.capacity or 0,
                     slots=getattr(args, "max_seqs", 0) or 0)
    rt.once()
    return rt


def _weights_path(w):
    if w is None:
        return None
    p = Path(w)
    if p.is_dir():
        files = sorted(p.glob("*.safetensors"))
        if len(files) != 1:
            from .models.common import read_safetensors

            out = {}
            for f in files:
                out.update(read_safetensors(f))
            return out
        return files[0]
    return p


# ---- subcommands --------------------------------------------------------------------------------------
def cmd_verify(args) -> int:
    from . import _native

    text = Path(args.manifest).read_text()
    t0 = time.perf_counter()
    m, errs = _native.verify(text)
    ms = (time.perf_counter() - t0) * 1e3
    if m is None:
        print(f"{args.manifest}: {len(errs)} problem(s)")
        for e in errs:
            print("  -", e)
        return 1
    print(f"{args.manifest}: verified in {ms:.2f} ms (model `{m.model}`)")
    try:
        p = json.loads(m.protocol())
    except ValueError:
        try:
            p = json.loads(m.self_hosted().protocol(sampled=False))
            print("  (hosted or stage manifest: checked without a token output)")
        except ValueError as e:
            print(f"  no serving protocol: {e}")
            return 0
    print(f"  rows: `{p['rows']['var']}` <= {p['rows']['max']}   groups: `{p['groups']['var']}` <= {p['groups']['max']}"
          + (f"   ranks: `{p['ranks']['var']}`" if p.get("ranks") else "") + (f"   context: `{p['context']['var']}`" if p.get("context") else ""))
    for f in p["fills"]:
        ax = f["axis"] if isinstance(f["axis"], str) else f"[{f['axis']['fixed']}]"
        print(f"  fill {f['fill']:12s} {f['name']}  {f['dtype']} over {ax}" + (f" x{f['width']}" if f["width"] != 1 else ""))
    for t in p["page_tables"]:
        print(f"  page table {t['name']} [{p['groups']['var']}, {t['width']}] -> {t['state']} (page of {t['stride']})")
    for t in p["line_tables"]:
        print(f"  line table {t['name']} lines={t['lines']} -> {t['state']}")
    for f in p["forwards"]:
        print(f"  forward {f['name']}: up to {f['groups']} groups x {f['rows']} rows" + (f", emits {f['emits']}" if f["emits"] else "")
              + (f" (count {f['count']})" if f["count"] else "") + (", graph" if f["graph"] else ""))
    for name in p["once"]:
        print(f"  once {name}")
    for name in p["derive"]:
        print(f"  derive {name}")
    return 0


def cmd_cut(args) -> int:
    from . import _native

    m, errs = _native.verify(Path(args.manifest).read_text())
    if m is None:
        print("\n".join(errs))
        return 1
    try:
        stages = m.cut([int(x) for x in args.at.split(",")])
    except ValueError as e:
        print(e)
        return 1
    out = Path(args.out)
    out.mkdir(parents=True, exist_ok=True)
    whole = json.loads(m.to_json())
    for i, s in enumerate(stages):
        doc = json.loads(s.to_json())
        (out / f"stage{i}.json").write_text(s.to_json())
        regions = lambda d, st: len({a.get("offset", 0) for p in d["programs"].values() for c in p["calls"] for a in c["args"] if a.get("state") == st})
        use = ", ".join(f"{st} {regions(doc, st)}/{regions(whole, st)}" for st in doc["states"])
        print(f"stage {i}: {sum(len(p['calls']) for p in doc['programs'].values())} calls, {len(doc['buffers'])} buffers, states [{use}]")
    return 0


def cmd_schema(args) -> int:
    from . import schema

    if args.validate:
        errs = schema.validate(json.loads(Path(args.validate).read_text()))
        for e in errs:
            print("error:", e)
        return 1 if errs else 0
    if args.write:
        print(schema.write_golden())
        return 0
    if args.check:
        ok = schema.check_golden()
        print("schema/manifest-v7.schema.json is " + ("up to date" if ok else "STALE: run `python -m kern_b200 schema --write` and commit the diff"))
        return 0 if ok else 1
    sys.stdout.write(schema.text())
    return 0


def cmd_gate(args) -> int:
    """The serving scenarios (`testing/gate.py`) against a model target; fresh engines come from the same flags."""
    from .engine import Engine
    from .testing.gate import Gate

    first = make_runtime(args)
    p = first.protocol
    page = first.page_unit
    vocab = args.vocab or 256
    for b in first.doc["buffers"].values():
        if b.get("fill") == "token" and "domain" in b and "max" in b["domain"]:
            vocab = int(b["domain"]["max"]) + 1
    capacity = args.capacity or page * 24
    spare = [first]

    def make(tokens):
        if spare and tokens == capacity:
            return Engine(spare.pop())
        ns = argparse.Namespace(**vars(args))
        ns.capacity = tokens
        return Engine(make_runtime(ns))

    args.capacity = capacity
    results = Gate(make, vocab, page, capacity, seed=args.seed).run(args.only.split(",") if args.only else None)
    for r in results:
        print(r.line())
    bad = [r for r in results if not r.ok]
    print(f"{len(results) - len(bad)} of {len(results)} scenarios pass" + (f" (protocol rows {p['rows']['max']}, page {page})" if p else ""))
    return 1 if bad else 0


def cmd_kernels(args) -> int:
    """`kern kernels`: the modules of the build in use; `index` / `check` / `pick`: the kernel registry (`kernel_registry.py`)."""
    from .models.common import kernel_index

    what = getattr(args, "what", None)
    if what in (None, "list"):
        for name, e in sorted(kernel_index().items()):
            print(f"{e['sha256']}  {e['source']}")
        return 0
    from . import kernel_registry as R

    if what == "index":
        paths = R.write_all()
        print(f"{len(paths)} families -> {R.INDEX}")
        return 0
    if what == "check":
        errs = R.check(require_reports=not args.no_reports)
        for e in errs:
            print(e)
        print(f"{len([p for p in R.INDEX.glob('*.toml') if p != R.PICKS])} families, {len(R.load_picks())} picks, {len(errs)} findings")
        return 1 if errs else 0
    if what == "pick":
        if len(args.rest) != 5:
            print("usage: kern kernels pick <family> <op> <shape> <variant> <bench.json> [--entry NAME]")
            return 2
        family, op, shape, variant, report = args.rest
        try:
            rec = R.pick(family, op, shape, variant, report, entry=(args.entry or [None])[-1])
        except ValueError as e:
            print(e)
            return 1
        print(f"{family}: {op} on {shape} -> {variant}" + (f" / {rec['entry']}" if "entry" in rec else "") + f" (report @{rec['report'][:12]})")
        return 0
    if what == "import":
        if len(args.rest) != 2:
            print("usage: kern kernels import <cubin> <family> [--entry NAME ...] [--capture launches.jsonl] [--origin TEXT]")
            return 2
        try:
            doc = R.import_cubin(args.rest[0], args.rest[1], entries=args.entry, capture_file=args.capture, origin=args.origin)
        except ValueError as e:
            print(e)
            return 1
        v = doc["variant"][-1]
        print(f"{args.rest[1]}: {len(doc['variant'])} variant(s); {v['name']} @{v['sha256'][:12]} with {len(v['entries'])} entries")
        return 0
    if what == "land":
        if len(args.rest) != 2:
            print("usage: kern kernels land <manifest.json> <dir>")
            return 2
        landed, missing = R.land(json.loads(Path(args.rest[0]).read_text()), args.rest[1])
        for m in missing:
            print("missing:", m)
        print(f"{len(landed)} landed, {len(missing)} missing")
        return 1 if missing else 0
    print(f"unknown: kernels {what}")
    return 2


def _prompt_ids(args, tok=None):
    if args.prompt_ids:
        return [int(x) for x in args.prompt_ids.split(",")]
    from .serve.server import ByteTokenizer, HFTokenizer

    tok = HFTokenizer(args.tokenizer) if args.tokenizer else ByteTokenizer()
    return tok.encode(args.prompt or "hello")


def cmd_run(args) -> int:
    from .engine import Engine, Sampling

    rt = make_runtime(args)
    if hasattr(rt, "banner"):
        print(rt.banner(), file=sys.stderr)
    eng = Engine(rt)
    if getattr(args, "probe_dir", None):
        from .testing.probe import Probe

        eng.probe = Probe(args.probe_dir, args.probe_labels or "")
    prompt = _prompt_ids(args)
    t0 = time.perf_counter()
    toks = eng.generate(prompt, args.steps, chunk=args.chunk, sampling=Sampling(temperature=args.temperature, seed=args.seed))
    dt = time.perf_counter() - t0
    print(json.dumps({"prompt_tokens": len(prompt), "tokens": toks, "seconds": round(dt, 4), "tok_s": round(len(toks) / dt, 1)}))
    return 0


def cmd_e2e(args) -> int:
    """`kern test e2e-logits record --manifest M --out REC` writes a recording; `kern test e2e-logits --manifest M REC`
    judges this engine against it (exit 0 / 1)."""
    from .testing import e2e
    from .testing.abtest import EngineSide

    side = EngineSide(make_runtime(args))
    if args.record:
        vocab = max((b.get("domain", {}).get("max", 0) for b in side.doc["buffers"].values() if b.get("fill") == "token"), default=255) + 1
        qs = e2e.plan(args.seed, args.prompts, vocab, max_tokens=args.decode_steps)
        e2e.record(side, qs, source=side.doc["model"], chunk=args.chunk or 256, batch=args.batch).save(args.out)
        print(f"recorded {len(qs)} questions -> {args.out}")
        return 0
    rec = e2e.Recording.load(args.recording)
    text, code = e2e.summary(e2e.judge(rec, side, kl_limit=args.logit_kl, chunk=args.chunk or 256), noise_mean=rec.noise_mean)
    print(text)
    return code


def cmd_test(args) -> int:
    from .testing.abtest import EngineSide, run_test

    a = EngineSide(make_runtime(args, args.a))
    b = EngineSide(make_runtime(args, args.b))
    rep = run_test(a, b, seed=args.seed, prompts=args.prompts, decode_steps=args.decode_steps, logit_kl=args.logit_kl, chunk=args.chunk)
    print(rep.text())
    return rep.exit_code


def load_workload(path: str | None) -> dict:
    """Workload TOML: samples (12..256), seed, [[sweep]] of groups x (rows | chunk) x context with weights."""
    if path is None:
        return {"samples": 12, "seed": 0, "sweep": [{"groups": 1, "rows": 1, "context": 256, "weight": 1.0},
                                                     {"groups": 1, "chunk": 256, "context": 256, "weight": 1.0}]}
    w = tomllib.loads(Path(path).read_text())
    unknown = set(w) - {"samples", "seed", "sweep"}
    if unknown:
        raise SystemExit(f"{path}: unknown field(s) {sorted(unknown)}")
    if not 12 <= w.get("samples", 12) <= 256:
        raise SystemExit(f"{path}: samples must be 12..=256")
    return {"samples": w.get("samples", 12), "seed": w.get("seed", 0), "sweep": w.get("sweep", [])}


def cmd_bench(args) -> int:
    """Each sweep point: contexts built once, then `samples` timed calls of the forward program, each from the same
    pre-image (paged rows rewound, per-sequence states put back from a spare slot) and, on a GPU, behind an L2 flush and
    timed by CUDA events on the runtime's stream (graph programs replay their captured graph); min / p10 / p50 / p90 /
    max / cv and the raw samples.
    Reference counterpart: crates/kern-run/src/bench/mod.rs:1-17, crates/kern-runtime/src/profile.rs:30-150."""
    from .engine import Engine

    wl = load_workload(args.workload)
    if getattr(args, "candidate", None):
        return bench_candidate(args, wl)
    rt = make_runtime(args)
    report = bench_points(rt, wl, by_op=getattr(args, "by_op", False))
    if args.out:
        Path(args.out).write_text(json.dumps(report, indent=1))
    return 0


def bench_candidate(args, wl) -> int:
    """`--candidate FILE`: the candidate's ops are spliced over the manifest's (same interfaces), both are held to the
    same answers (the A/B test's verdict must be PASS), both are priced on the workload, and every sweep point says
    which implementation it would pick (the faster one when the gap exceeds both sides' spread)."""
    from . import _native
    from .testing.abtest import EngineSide, run_test

    base_text = Path(args.manifest).read_text()
    m, errs = _native.verify(base_text)
    if m is None:
        print("\n".join(errs))
        return 1
    try:
        spliced = m.splice(Path(args.candidate).read_text())
    except ValueError as e:
        print(e)
        return 1
    cand_text = spliced.to_json()
    a, b = make_runtime(args, base_text), make_runtime(args, cand_text)
    verdict = run_test(EngineSide(a), EngineSide(b), seed=wl["seed"], prompts=2, decode_steps=4, logit_kl=0.01, chunk=args.chunk or 256)
    print(f"held to outputs: {verdict.verdict}")
    if verdict.exit_code == 1:
        print(verdict.text())
        return 1
    ra, rb = bench_points(a, wl, quiet=True), bench_points(b, wl, quiet=True)
    picks = []
    for pa, pb in zip(ra["points"], rb["points"]):
        gap = pa["p50_ms"] - pb["p50_ms"]
        noise = max(pa["p90_ms"] - pa["p10_ms"], pb["p90_ms"] - pb["p10_ms"])
        pick = "candidate" if gap > noise else ("base" if -gap > noise else "either")
        picks.append({"groups": pa["groups"], "rows": pa["rows"], "context": pa["context"], "base_ms": pa["p50_ms"],
                      "candidate_ms": pb["p50_ms"], "pick": pick})
        print(json.dumps(picks[-1]))
    if args.out:
        Path(args.out).write_text(json.dumps({"version": 5, "held": verdict.verdict, "picks": picks}, indent=1))
    return 0


def _bench_device(rt):
    """On a GPU: (flush, events) — `flush(k)` writes a buffer larger than L2 so the next sample starts cold, `events()`
    records a start event on the runtime's stream and returns (start, end, stream). (None, None) on the host executor."""
    try:
        import torch

        if not (torch.cuda.is_available() and hasattr(rt, "stream") and hasattr(rt, "gpu")):
            return None, None
        dev = torch.device(f"cuda:{rt.gpu}")
        stream = torch.cuda.ExternalStream(rt.stream, device=dev)
        buf = torch.empty(192 << 20, dtype=torch.uint8, device=dev)

        def flush(k: int) -> None:
            with torch.cuda.stream(stream):
                buf.fill_(k & 0xFF)

        def events():
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            return a, b, stream

        return flush, events
    except Exception:
        return None, None


def bench_points(rt, wl, by_op: bool = False, quiet: bool = False) -> dict:
    from . import _native
    from .engine import Engine
    import numpy as np

    eng = Engine(rt)
    rng = np.random.default_rng(wl["seed"])
    report = {"version": 5, "points": []}
    for pt in wl["sweep"]:
        g, ctx = min(int(pt.get("groups", 1)), eng.groups_max), int(pt.get("context", 64))     # no more sequences than a call takes
        rows = min(int(pt.get("chunk", pt.get("rows", 1))), eng.rows_max // max(1, g))
        longest = min((t["width"] * t["stride"] for t in eng.page_tables), default=ctx)
        ctx = max(rows, min(ctx, longest))          # a context the manifest's page-table row can hold
        seqs = [eng.open(ctx) for _ in range(g)]
        if ctx > rows:
            pre = ctx - rows
            for i in range(0, pre, eng.rows_max // max(1, g)):
                n = min(eng.rows_max // max(1, g), pre - i)
                eng.step([(s, rng.integers(1, 200, n).tolist()) for s in seqs])
        # the pre-image of what a sample changes: paged rows are overwritten in place by the next sample (a slot is its
        # position), a per-sequence recurrent state is not — it is kept in a spare slot and put back before every sample
        shadows = []
        stateful = any(s.lease.slot >= 0 for s in seqs)
        try:
            for s in seqs:
                if s.lease.slot >= 0:
                    sh = eng.open(1)
                    shadows.append(sh)
                    rt.run_copies({"pages": [], "slot": (s.lease.slot, sh.lease.slot)})
        except _native.Denied:              # no spare slots for all of them: the samples run on from one another's state
            for sh in shadows:
                eng.close(sh)
            shadows = []
        pre_image = bool(shadows) or not stateful
        flush, events = _bench_device(rt)
        times, host_times = [], []
        for k in range(4 + wl["samples"]):                       # WARMUP = 4
            batch = [(s, rng.integers(1, 200, rows).tolist()) for s in seqs]
            for s, sh in zip(seqs, shadows):
                rt.run_copies({"pages": [], "slot": (sh.lease.slot, s.lease.slot)})
            if flush is not None:
                flush(k)                                         # every sample starts with a cold L2
            rt.synchronize()
            ev = events() if events is not None else None
            t0 = time.perf_counter()
            eng.step(batch)
            if ev is not None:
                ev[1].record(ev[2])
            rt.synchronize()
            host_ms = (time.perf_counter() - t0) * 1e3
            if k >= 4:
                host_times.append(host_ms)
                times.append(ev[0].elapsed_time(ev[1]) if ev is not None else host_ms)
            for s in seqs:                                       # rewind: every sample runs at the same context
                s.length -= rows
                del s.tokens[-rows:]
        for s in seqs + shadows:
            eng.close(s)
        raw = list(times)
        times.sort()
        q = lambda f: times[min(len(times) - 1, int(f * len(times)))]
        point = {"groups": g, "rows": rows, "context": ctx, "weight": pt.get("weight", 1.0), "min_ms": times[0], "p10_ms": q(0.1),
                 "p50_ms": q(0.5), "p90_ms": q(0.9), "max_ms": times[-1], "cv": statistics.pstdev(times) / max(1e-9, statistics.mean(times)),
                 "clock": "device" if events is not None else "host", "l2_flushed": flush is not None,
                 "pre_image": pre_image,
                 "host_p50_ms": sorted(host_times)[len(host_times) // 2], "samples_ms": [round(t, 4) for t in raw]}
        if by_op and hasattr(rt, "issue_timed"):
            # one more call of the same shape, eagerly, with an event between calls: the cost by op
            seqs2 = [eng.open(ctx) for _ in range(g)]
            if ctx > rows:
                pre = ctx - rows
                for i in range(0, pre, eng.rows_max // max(1, g)):
                    n = min(eng.rows_max // max(1, g), pre - i)
                    eng.step([(s, rng.integers(1, 200, n).tolist()) for s in seqs2])
            eng.step([(s, rng.integers(1, 200, rows).tolist()) for s in seqs2], timed=True)
            cost: dict[str, float] = {}
            for label, op, ms, _n in eng.last_times:
                cost[op] = cost.get(op, 0.0) + ms
            total = sum(cost.values()) or 1.0
            point["by_op"] = {op: round(ms / total, 4) for op, ms in sorted(cost.items(), key=lambda kv: -kv[1])}
            for s in seqs2:
                eng.close(s)
        report["points"].append(point)
        if not quiet:
            print(json.dumps(point))
    return report


def cmd_workload(args) -> int:
    """steps.parquet of a served run -> a weighted bench workload (buckets of groups x rows x context)."""
    import pyarrow.parquet as pq

    t = pq.ParquetFile(args.steps).read().to_pydict()      # the file alone: no partition columns from its path
    buckets: dict[tuple, float] = {}
    for g, r, c, ms in zip(t["groups"], t["rows"], t["context"], t.get("device_ms", [1.0] * len(t["groups"]))):
        key = (int(g), int(r), 1 << max(0, int(c) - 1).bit_length())
        buckets[key] = buckets.get(key, 0.0) + float(ms)
    total = sum(buckets.values()) or 1.0
    lines = [f"samples = {args.samples}", "seed = 0", ""]
    for (g, r, c), w in sorted(buckets.items(), key=lambda kv: -kv[1]):
        lines += ["[[sweep]]", f"groups = {g}", (f"rows = {r}" if r <= 16 else f"chunk = {r}"), f"context = {c}", f"weight = {w / total:.4f}", ""]
    Path(args.out).write_text("\n".join(lines))
    print(f"{len(buckets)} sweep points -> {args.out}")
    return 0


def cmd_server(args) -> int:
    import logging

    from .engine import Engine
    from .serve.scheduler import Scheduler
    from .serve.server import ByteTokenizer, HFTokenizer, Server
    from .utils.logline import setup_logging

    setup_logging()
    tok = HFTokenizer(args.tokenizer) if args.tokenizer else ByteTokenizer()
    if getattr(args, "pp", 1) > 1:
        # a pipeline of stage processes: this process is the head (stage 0), the manifest is cut at layer boundaries
        from .serve import launch

        if args.model:
            from .models import registry

            cfg, build, _load, _make = registry.resolve(args.model)
            doc = build(cfg)
        else:
            doc = json.loads(Path(args.manifest).read_text())
        spec = {"manifest": doc, "weights": args.weights, "model": args.model, "cpu": args.cpu, "tokens": args.capacity or 0,
                "slots": args.max_seqs or 0}
        sched, pipe, procs = launch.launch_pp(spec, args.pp, chunk=args.chunk, max_seqs=args.max_seqs or None)
        srv = Server(sched, tok, model_name=doc["model"], host=args.host, port=args.port, tool_parser=_tool_parser(args, doc))
        try:
            srv.serve_forever()
        finally:
            launch.shutdown_pp(pipe, procs)
        return 0
    if getattr(args, "pd", False):
        # prefill / decode disaggregation: this process is the prefill tier, the decode tier a process on its own GPU
        from .serve import launch

        if args.model:
            from .models import registry

            cfg, build, _load, _make = registry.resolve(args.model)
            doc = build(cfg)
        else:
            doc = json.loads(Path(args.manifest).read_text())
        spec = {"manifest": doc, "weights": args.weights, "model": args.model, "cpu": args.cpu, "tokens": args.capacity or 0,
                "slots": args.max_seqs or 0}
        dspec = dict(spec, tokens=args.decode_capacity or spec["tokens"])
        extra = {}
        if args.dcp > 1:
            # the decode tier is a context-parallel group: positions dealt over --dcp ranks on GPUs decode-gpu, decode-gpu + 1, ..
            from .models import dense, dense_dcp

            if not args.model or not isinstance(cfg, dense.DenseConfig):
                raise SystemExit("--dcp needs --model of the dense family (the member manifest is generated from its config)")
            dspec["manifest"] = dense_dcp.build_manifest_dcp(cfg, args.dcp)
            extra = {"decode_gpus": [args.decode_gpu + i for i in range(args.dcp)], "dealer": dense_dcp.dealer(cfg)}
        tier, worker = launch.launch_pd(spec, dspec, chunk=args.chunk, max_seqs=args.max_seqs or None, prefill_gpu=args.gpu or 0,
                                        decode_gpu=args.decode_gpu, front=True, **extra)
        srv = Server(tier, tok, model_name=doc["model"], host=args.host, port=args.port, tool_parser=_tool_parser(args, doc))
        try:
            srv.serve_forever()
        finally:
            launch.shutdown_pd(tier, worker)
        return 0
    if args.world > 1:
        # rank processes (one per GPU) behind this head: one tensor-parallel group, or a data-parallel tier of them
        from .serve import launch

        if args.model:
            from .models import registry

            cfg, build, _load, make = registry.resolve(args.model)
            if args.tp > 1:
                import dataclasses

                from .models import dense_tp

                doc = dense_tp.build_manifest_tp(dataclasses.replace(cfg, tp=args.tp))
            else:
                doc = build(cfg)
        else:
            doc = json.loads(Path(args.manifest).read_text())
        spec = {"manifest": doc, "weights": args.weights, "model": args.model, "cpu": args.cpu, "tokens": args.capacity or 0,
                "slots": args.max_seqs or 0}
        sched, ex, procs = launch.launch(spec, world=args.world, tp=args.tp, chunk=args.chunk, max_seqs=args.max_seqs or None)
        srv = Server(sched, tok, model_name=doc["model"], host=args.host, port=args.port, tool_parser=_tool_parser(args, doc))
        try:
            srv.serve_forever()
        finally:
            launch.shutdown(ex, procs)
        return 0
    rt = make_runtime(args)
    eng, rec, sampler = trace_setup(args, Engine(rt))
    sched = Scheduler(eng, chunk=args.chunk, max_seqs=args.max_seqs or None, rows=args.rows)
    srv = Server(sched, tok, model_name=rt.doc["model"], host=args.host, port=args.port, recorder=rec,
                 tool_parser=_tool_parser(args, rt.doc))
    logging.getLogger("kern.serve").info("listening host=%s port=%d model=%s", args.host, srv.port, rt.doc["model"])
    try:
        srv.serve_forever()
    finally:
        if sampler is not None:
            sampler.stop()
        if rec is not None:
            rec.rotator.stop()
            rec.close()
    return 0


def _tool_parser(args, doc: dict) -> str:
    """--tool-call-parser when it says more than `auto`, else the manifest's `chat.tool_parser`, else recognition by syntax."""
    from .serve.chat import select_parser

    return select_parser(getattr(args, "tool_call_parser", None), (doc.get("chat") or {}).get("tool_parser"))


def trace_setup(args, engine, nvml=None):
    """--trace-dir: every step of the engine goes to <dir>/date=../rank=0/*.steps.parquet (device and host time, shape,
    launches); --trace-sample N: every N-th step runs eagerly with an event between calls, its cost by call goes to
    *.kernels.parquet; --trace-pm-us P: a sampler thread writes clocks, power and the SM / tensor / DRAM busy shares to
    *.counters.parquet every P microseconds (at least 50). POST /kern/trace/rotate closes the files in use.
    -> (engine to schedule, recorder | None, sampler | None).
    Reference counterpart: crates/kern-serve/src/lib.rs:118-137 (--trace, --trace-dir, --trace-pm-us)."""
    if not getattr(args, "trace_dir", None):
        return engine, None, None
    from . import trace

    doc = getattr(getattr(engine, "rt", None), "doc", None) or {}
    rec = trace.Recorder(args.trace_dir, rank=0, comm=trace.comm_ops(doc))
    eng = trace.TracedEngine(engine, rec, sample_every=getattr(args, "trace_sample", 0) or 0)
    rec.rotator = trace.Rotator(rec)              # files close at every quarter hour of the wall clock
    rec.rotator.start()
    sampler = None
    pm = getattr(args, "trace_pm_us", 0) or 0
    if pm and (nvml is not None or not getattr(args, "cpu", False)):
        sampler = trace.Counters(rec, gpu=getattr(args, "gpu", None) or 0, period=max(50, pm) / 1e6, nvml=nvml)
        sampler.start()
    return eng, rec, sampler


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="kern", description="manifest-driven inference engine for B200")
    sub = ap.add_subparsers(dest="cmd", required=True)

    def common(p, manifest=True):
        if manifest:
            p.add_argument("--manifest")
        p.add_argument("--target", help="a [targets.<name>] of kern.toml")
        p.add_argument("--weights"); p.add_argument("--kernels"); p.add_argument("--tokenizer")
        p.add_argument("--gpu", type=int); p.add_argument("--capacity", type=int, help="token capacity of the paged states")
        p.add_argument("--cpu", action="store_true", help="run on the host-memory executor instead of a GPU")
        p.add_argument("--chunk", type=int); p.add_argument("--max-seqs", type=int, default=0)
        p.add_argument("--model", help="a built-in model family with random-init weights instead of --manifest/--weights")
        p.add_argument("--layers", type=int); p.add_argument("--max-tokens", type=int); p.add_argument("--max-context", type=int)

    v = sub.add_parser("verify"); v.add_argument("manifest")
    c = sub.add_parser("cut"); c.add_argument("manifest"); c.add_argument("--at", required=True); c.add_argument("--out", required=True)
    kn = sub.add_parser("kernels")
    kn.add_argument("what", nargs="?", choices=["list", "index", "check", "pick", "import", "land"])
    kn.add_argument("rest", nargs="*", help="pick: <family> <op> <shape> <variant> <bench.json>")
    kn.add_argument("--entry", action="append", help="pick: the entry of the variant that was measured best; import: an entry of the cubin (repeatable)")
    kn.add_argument("--capture", help="import: a capture file whose launches name the module's entries")
    kn.add_argument("--origin", help="import: where the cubin came from (URL and commit)")
    kn.add_argument("--no-reports", action="store_true", help="check: do not require the picks' reports to be in the local store")
    gt = sub.add_parser("gate", help="the serving scenarios every model target must pass"); common(gt)
    gt.add_argument("--only", help="comma-separated scenario names"); gt.add_argument("--seed", type=int, default=0)
    gt.add_argument("--vocab", type=int, help="token id range when the manifest declares no domain")
    sc = sub.add_parser("schema", help="the JSON Schema of the manifest wire format")
    sc.add_argument("--check", action="store_true", help="compare with the committed schema/manifest-v7.schema.json; exit 1 on a difference")
    sc.add_argument("--write", action="store_true", help="rewrite the committed file")
    sc.add_argument("--validate", help="a manifest to check against the schema (shape only; `verify` does the rest)")
    r = sub.add_parser("run"); common(r)
    r.add_argument("--prompt"); r.add_argument("--prompt-ids"); r.add_argument("--steps", type=int, default=16)
    r.add_argument("--temperature", type=float, default=0.0); r.add_argument("--seed", type=int, default=0)
    r.add_argument("--probe-dir", help="dump what the calls named by --probe-labels wrote, step by step, into this directory")
    r.add_argument("--probe-labels", help="comma-separated call labels (or label suffixes), e.g. l0.attn_out,head")
    t = sub.add_parser("test"); t.add_argument("a"); t.add_argument("b"); common(t, manifest=False)
    t.add_argument("--seed", type=int, default=0); t.add_argument("--prompts", type=int, default=4)
    t.add_argument("--decode-steps", type=int, default=8); t.add_argument("--logit-kl", type=float, default=0.01)
    e = sub.add_parser("e2e-logits", help="record an engine's answers, or judge an engine against a recording")
    common(e); e.add_argument("recording", nargs="?"); e.add_argument("--record", action="store_true"); e.add_argument("--out")
    e.add_argument("--seed", type=int, default=0); e.add_argument("--prompts", type=int, default=8)
    e.add_argument("--batch", type=int, default=4, help="--record: the noise of a question is measured along its own tokens alone, in batches of this many and of half as many")
    e.add_argument("--decode-steps", type=int, default=16); e.add_argument("--logit-kl", type=float, default=0.01)
    b = sub.add_parser("bench"); common(b); b.add_argument("--workload"); b.add_argument("--out")
    b.add_argument("--by-op", action="store_true", help="add each point's cost by op (one eager call with an event between calls)")
    b.add_argument("--candidate", help="a candidate (modules + ops) to splice over the manifest and price against it")
    w = sub.add_parser("workload"); w.add_argument("steps"); w.add_argument("--out", required=True); w.add_argument("--samples", type=int, default=32)
    s = sub.add_parser("server"); common(s)
    s.add_argument("--host", default="127.0.0.1"); s.add_argument("--port", type=int, default=8000); s.add_argument("--rows", type=int)
    s.add_argument("--world", type=int, default=1, help="rank processes (one per GPU)")
    s.add_argument("--tp", type=int, default=1, help="ranks per tensor-parallel group; world / tp groups form a data-parallel tier")
    s.add_argument("--pp", type=int, default=1, help="pipeline stages (one process per GPU; this process is the head): the manifest is cut at layer boundaries")
    s.add_argument("--tool-call-parser", default="auto", help="auto | none | hermes | qwen3_coder: how chat completions with `tools` get structured tool_calls (auto: the manifest's chat.tool_parser, else by syntax)")
    s.add_argument("--trace-dir", help="record every step (and sampled steps by call, and counters) as Parquet files under this directory")
    s.add_argument("--trace-sample", type=int, default=0, help="with --trace-dir: every N-th step runs eagerly with per-call device times")
    s.add_argument("--trace-pm-us", type=int, default=0, help="with --trace-dir: sample clocks, power and SM / tensor / DRAM busy shares every this many microseconds (>= 50)")
    s.add_argument("--pd", action="store_true", help="prefill/decode disaggregation: this process prefills (on --gpu), a decode process on --decode-gpu takes every request over with its first token")
    s.add_argument("--dcp", type=int, default=1, help="with --pd: the decode tier is a context-parallel group of this many ranks (dense family)")
    s.add_argument("--decode-gpu", type=int, default=1); s.add_argument("--decode-capacity", type=int, help="token capacity of the decode tier's paged states")
    cp = sub.add_parser("capture", help="lift | mine | path: from a program's captured launches to manifest facts (kern_b200/capture.py)")
    cp.add_argument("rest", nargs=argparse.REMAINDER)
    args = ap.parse_args(argv)
    if args.cmd == "capture":
        from . import capture

        return capture.main(args.rest)
    if args.cmd in ("run", "test", "bench", "server", "e2e-logits", "gate"):
        path, cfg = find_config()
        resolve(args, path, cfg)
        if args.cmd != "test" and not args.manifest and not getattr(args, "model", None):
            ap.error("--manifest, --model or a --target of kern.toml is required")
    return {"verify": cmd_verify, "cut": cmd_cut, "kernels": cmd_kernels, "schema": cmd_schema, "gate": cmd_gate, "run": cmd_run, "test": cmd_test, "bench": cmd_bench,
            "workload": cmd_workload, "server": cmd_server, "e2e-logits": cmd_e2e}[args.cmd](args)


if __name__ == "__main__":
    sys.exit(main())
