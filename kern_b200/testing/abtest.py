"""`kern test`: is manifest B the same function as manifest A?

Four stages, pure logic over a `Side` (something that can stage inputs, run a program and read buffers
— a GPU runtime, the CPU executor, or a fake in tests):

  DIFF   static: per-op change (interface / impl / added / removed) and the call lists of each program
         aligned by longest common subsequence into spans of changed calls;
  TAP    a seeded workload (random tokens from the token domain; prefill lengths half uniform, half on a
         structural boundary: page +-1, chunk +-1, the rows limit) run on A and on B from the same inputs;
         every buffer either side wrote is compared (count of differing elements, max ULP, max abs, NaN on one
         side only, +-0), logits rows by KL(A || B), argmax agreement, A's margin, rank of A's argmax in B,
         top-20 overlap;
  NOISE  A replayed against itself: the floor below which a difference is not evidence;
  PERF   per-program wall time of both sides.

Verdict ladder (first match): FAIL an output outside its declared domain -> FAIL an argmax flip whose row KL
exceeds --logit-kl -> INCONCLUSIVE a changed program the driver cannot feed -> PASS bit-identical -> PASS
value-identical (only +-0 differs) -> PASS logits bit-identical -> PASS logit evidence (every row KL within
the limit) -> PASS within the noise floor -> INCONCLUSIVE. Exit codes 0 / 1 / 2.

Reference: crates/kern-test/src/{lib,diff,harness,replay,compare,workload,report}.rs, docs/test.md:438-573.
"""
from __future__ import annotations

import json
import math
import time
from dataclasses import dataclass, field

import numpy as np

from .. import _native

PASS, FAIL, INCONCLUSIVE = "PASS", "FAIL", "INCONCLUSIVE"
EXIT = {PASS: 0, FAIL: 1, INCONCLUSIVE: 2}
TOP = 20


# ---- workload --------------------------------------------------------------------------------------
class Rng:
    """splitmix64: the same seed gives the same workload on every machine."""

    def __init__(self, seed: int):
        self.s = seed & 0xFFFFFFFFFFFFFFFF

    def next(self) -> int:
        self.s = (self.s + 0x9E3779B97F4A7C15) & 0xFFFFFFFFFFFFFFFF
        z = self.s
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & 0xFFFFFFFFFFFFFFFF
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & 0xFFFFFFFFFFFFFFFF
        return z ^ (z >> 31)

    def below(self, n: int) -> int:
        return self.next() % max(1, n)


def prefill_length(rng: Rng, rows_max: int, page: int, chunk: int) -> int:
    """Half the time uniform in [1, rows_max]; otherwise a structural boundary."""
    if rng.below(2) == 0:
        return 1 + rng.below(rows_max)
    cands = [page - 1, page, page + 1, chunk - 1, chunk, chunk + 1, rows_max, 2 * page + 1]
    cands = [c for c in cands if 1 <= c <= rows_max]
    return cands[rng.below(len(cands))]


# ---- DIFF ------------------------------------------------------------------------------------------
def op_changes(a: dict, b: dict) -> dict[str, str]:
    out = {}
    for name in sorted(set(a["ops"]) | set(b["ops"])):
        if name not in b["ops"]:
            out[name] = "removed"
        elif name not in a["ops"]:
            out[name] = "added"
        elif a["ops"][name]["params"] != b["ops"][name]["params"]:
            out[name] = "interface"
        elif _impl_key(a, name) != _impl_key(b, name):
            out[name] = "impl"
    return out


def _impl_key(doc: dict, op: str) -> str:
    """An implementation is its launches with each module replaced by the bytes it pins."""
    impl = json.loads(json.dumps(doc["ops"][op]["impl"]))
    for l in impl["launches"]:
        if "module" in l:
            l["module"] = doc["modules"].get(l["module"], {}).get("sha256", l["module"])
    return json.dumps(impl, sort_keys=True)


def align(a: list, b: list) -> list[tuple[int | None, int | None]]:
    """LCS alignment of two call lists (by op + args): pairs (i, j), (i, None) removed, (None, j) added."""
    ka = [json.dumps({"op": c["op"], "args": c["args"]}, sort_keys=True) for c in a]
    kb = [json.dumps({"op": c["op"], "args": c["args"]}, sort_keys=True) for c in b]
    n, m = len(ka), len(kb)
    dp = [[0] * (m + 1) for _ in range(n + 1)]
    for i in range(n - 1, -1, -1):
        for j in range(m - 1, -1, -1):
            dp[i][j] = dp[i + 1][j + 1] + 1 if ka[i] == kb[j] else max(dp[i + 1][j], dp[i][j + 1])
    out, i, j = [], 0, 0
    while i < n and j < m:
        if ka[i] == kb[j]:
            out.append((i, j)); i += 1; j += 1
        elif dp[i + 1][j] >= dp[i][j + 1]:
            out.append((i, None)); i += 1
        else:
            out.append((None, j)); j += 1
    out += [(k, None) for k in range(i, n)] + [(None, k) for k in range(j, m)]
    return out


def spans(a: dict, b: dict) -> dict[str, list[dict]]:
    """Per program both sides have: maximal runs of calls that differ (unaligned, or aligned to a changed op)."""
    changed = op_changes(a, b)
    out = {}
    for p in sorted(set(a["programs"]) & set(b["programs"])):
        pairs = align(a["programs"][p]["calls"], b["programs"][p]["calls"])
        cur, res = None, []
        for i, j in pairs:
            same = i is not None and j is not None and a["programs"][p]["calls"][i]["op"] not in changed
            if same:
                if cur:
                    res.append(cur); cur = None
                continue
            cur = cur or {"a": [], "b": []}
            if i is not None:
                cur["a"].append(i)
            if j is not None:
                cur["b"].append(j)
        if cur:
            res.append(cur)
        out[p] = res
    return out


def write_set(doc: dict, program: str, calls: list[int] | None = None) -> set[str]:
    """Buffers a program (or some of its calls) writes, by the ops' declared directions."""
    out = set()
    for k, c in enumerate(doc["programs"][program]["calls"]):
        if calls is not None and k not in calls:
            continue
        for arg, p in zip(c["args"], doc["ops"][c["op"]]["params"]):
            if "buf" in arg and (p.startswith("out ") or p.startswith("inout ")):
                out.add(arg["buf"])
    return out


# ---- compare ---------------------------------------------------------------------------------------
@dataclass
class Cmp:
    n: int = 0
    n_diff: int = 0
    max_ulp: int = 0
    max_abs: float = 0.0
    nan_only_one_side: int = 0
    signed_zero: int = 0

    @property
    def identical(self) -> bool:
        return self.n_diff == 0

    @property
    def value_identical(self) -> bool:
        return self.n_diff == self.signed_zero and self.nan_only_one_side == 0


def compare_bytes(dtype: str, a: bytes, b: bytes) -> Cmp:
    c = Cmp()
    va, vb = np.array(_native.decode_values(dtype, a)), np.array(_native.decode_values(dtype, b))
    c.n = len(va)
    es = len(a) // max(1, c.n)
    ra = np.frombuffer(a, dtype=np.uint8).reshape(c.n, es) if c.n else np.zeros((0, 1), np.uint8)
    rb = np.frombuffer(b, dtype=np.uint8).reshape(c.n, es) if c.n else np.zeros((0, 1), np.uint8)
    diff = (ra != rb).any(axis=1)
    c.n_diff = int(diff.sum())
    if c.n_diff == 0:
        return c
    na, nb = np.isnan(va), np.isnan(vb)
    c.nan_only_one_side = int((na ^ nb).sum())
    c.signed_zero = int(((va == 0) & (vb == 0) & diff).sum())
    both = diff & ~na & ~nb
    if both.any():
        c.max_abs = float(np.abs(va[both] - vb[both]).max())
        idx = np.nonzero(both)[0][:4096]                       # ULP on a sample: it is a report figure, not the verdict
        c.max_ulp = max(int(_native.ulp_distance(dtype, ra[i].tobytes(), rb[i].tobytes())) for i in idx)
    return c


def logit_stats(a: np.ndarray, b: np.ndarray) -> dict:
    """One logits row each: KL(A || B) in nats, argmax agreement, A's top-1/top-2 margin, rank of A's argmax in B,
    overlap of the top-20 sets."""
    a, b = a.astype(np.float64), b.astype(np.float64)
    la = a - (np.log(np.exp(a - a.max()).sum()) + a.max())
    lb = b - (np.log(np.exp(b - b.max()).sum()) + b.max())
    pa = np.exp(la)
    kl = float((pa * (la - lb)).sum())
    ia, ib = int(a.argmax()), int(b.argmax())
    top2 = np.partition(a, -2)[-2:]
    order_b = np.argsort(-b, kind="stable")
    ta, tb = set(np.argsort(-a, kind="stable")[:TOP].tolist()), set(order_b[:TOP].tolist())
    return {"kl": max(kl, 0.0), "agree": ia == ib, "margin": float(top2.max() - top2.min()),
            "rank_in_b": int(np.nonzero(order_b == ia)[0][0]), "top_overlap": len(ta & tb)}


# ---- sides -------------------------------------------------------------------------------------------
class EngineSide:
    """A Side over any runtime with the Runtime interface (GPU or CPU)."""

    def __init__(self, rt, logits: str | None = None):
        from ..engine import Engine

        self.rt = rt
        self.doc = rt.doc
        self.eng = Engine(rt)
        self.logits = logits or next((n for n in ("logits",) if n in rt.doc["buffers"]), None)

    def free_run(self, prompts: list[list[int]], steps: int, chunk: int):
        """Greedy generation of every prompt alone; returns tokens, per-step logits rows and timings."""
        outs, rows, t_prefill, t_decode = [], [], 0.0, 0.0
        for p in prompts:
            seq = self.eng.open(len(p) + steps)
            t0 = time.perf_counter()
            got = None
            for i in range(0, len(p), chunk):
                got = self.eng.step([(seq, p[i:i + chunk])])
            self.rt.synchronize()
            t_prefill += time.perf_counter() - t0
            toks = [got[0][0]]
            rows.append(self._logits_row())
            t0 = time.perf_counter()
            while len(toks) < steps:
                toks.append(self.eng.step([(seq, [toks[-1]])])[0][0])
                rows.append(self._logits_row())
            self.rt.synchronize()
            t_decode += time.perf_counter() - t0
            self.eng.close(seq)
            outs.append(toks)
        return outs, rows, {"prefill_s": t_prefill, "decode_s": t_decode}

    def forced_run(self, prompts, forced: list[list[int]], chunk: int):
        """Teacher-forced along another side's tokens: logits rows at the same positions."""
        rows = []
        for p, toks in zip(prompts, forced):
            seq = self.eng.open(len(p) + len(toks))
            for i in range(0, len(p), chunk):
                self.eng.step([(seq, p[i:i + chunk])])
            rows.append(self._logits_row())
            for t in toks[:-1]:
                self.eng.step([(seq, [t])])
                rows.append(self._logits_row())
            self.eng.close(seq)
        return rows

    def batched_forced_run(self, prompts, forced: list[list[int]], chunk: int, batch: int):
        """Teacher-forced like `forced_run`, but the decode steps of up to `batch` sequences run as one call: the same
        positions through other batch shapes (other tiles, other reduction orders). Rows per prompt, as `forced_run`
        returns them flattened."""
        rows: list[list] = [[] for _ in prompts]
        for g0 in range(0, len(prompts), max(1, batch)):
            idx = list(range(g0, min(len(prompts), g0 + max(1, batch))))
            seqs = {i: self.eng.open(len(prompts[i]) + len(forced[i])) for i in idx}
            for i in idx:
                for c in range(0, len(prompts[i]), chunk):
                    self.eng.step([(seqs[i], prompts[i][c:c + chunk])])
                rows[i].append(self._logits_row())
            for t in range(max(len(forced[i]) for i in idx) - 1):
                live = [i for i in idx if t < len(forced[i]) - 1]
                self.eng.step([(seqs[i], [forced[i][t]]) for i in live])
                for j, i in enumerate(live):
                    rows[i].append(self._logits_row(j))
            for i in idx:
                self.eng.close(seqs[i])
        return rows

    def _logits_row(self, j: int = 0):
        if self.logits is None:
            return None
        t = self.rt.tensor(self.logits)
        return t[j].float().cpu().numpy().copy()

    def snapshot(self, names) -> dict[str, bytes]:
        out = {}
        for n in names:
            if n in self.doc["buffers"]:
                t = self.rt.tensor(n)
                out[n] = t.contiguous().view(-1).view(__import__("torch").uint8).cpu().numpy().tobytes()
        return out


# ---- span-local replay ---------------------------------------------------------------------------------
def read_set(doc: dict, program: str, calls: list[int]) -> set[str]:
    """Buffers the given calls of a program read, by the ops' declared directions."""
    out = set()
    for k in calls:
        c = doc["programs"][program]["calls"][k]
        for arg, p in zip(c["args"], doc["ops"][c["op"]]["params"]):
            if "buf" in arg and (p.startswith("in ") or p.startswith("inout ")):
                out.add(arg["buf"])
    return out


def _buffer_bytes(doc: dict, name: str) -> tuple:
    b = doc["buffers"].get(name)
    return None if b is None else (b["dtype"], tuple(b["shape"]))


class DeltaImages:
    """Images of buffers, by (key, name), kept as deltas: a buffer's first image in full, every later one as the 64-byte
    blocks that differ from the image before it (most of a workspace does not change between two looks at it, and a
    recording of every span of every step in full would be many times the model's activations). `get` rebuilds an
    image by applying the deltas in order from the last image it rebuilt (the replay asks in recording order, so each
    `get` applies one delta); any earlier key is rebuilt from the buffer's first image.
    Reference: crates/kern-test/src/harness.rs:130-220 (delta snapshots, changed blocks)."""

    BLOCK = 64

    def __init__(self):
        self._chain: dict[str, list] = {}          # name -> [(key, None, full image) | (key, block indices, block bytes)]
        self._last: dict[str, "torch.Tensor"] = {}  # name -> the latest image put (what the next delta is against)
        self._cursor: dict[str, tuple[int, "torch.Tensor"]] = {}      # name -> (position in the chain, image there)
        self.full_bytes = 0                        # what whole images would have taken
        self.kept_bytes = 0                        # what is kept

    def put(self, key, name: str, img) -> None:
        import torch

        img = img.contiguous().view(-1).view(torch.uint8)
        self.full_bytes += img.numel()
        prev = self._last.get(name)
        if prev is None or prev.numel() != img.numel():
            self._chain.setdefault(name, []).append((key, None, img.clone()))
            self.kept_bytes += img.numel()
        else:
            n, B = img.numel(), self.BLOCK
            whole = n // B * B
            changed = (img[:whole].view(-1, B) != prev[:whole].view(-1, B)).any(1).nonzero().flatten()
            blocks = img[:whole].view(-1, B)[changed].clone()
            tail = img[whole:].clone()             # the odd bytes at the end travel whole
            self._chain[name].append((key, changed.to(torch.int32), (blocks, tail)))
            self.kept_bytes += blocks.numel() + tail.numel() + 4 * changed.numel()
        self._last[name] = img.clone()

    def get(self, key, name: str):
        chain = self._chain[name]
        at = next((i for i, e in enumerate(chain) if e[0] == key), None)
        if at is None:
            raise KeyError((key, name))
        pos, img = self._cursor.get(name, (-1, None))
        if pos > at or img is None:
            pos, img = -1, None
        while pos < at:
            pos += 1
            _k, idx, payload = chain[pos]
            if idx is None:
                img = payload.clone()
            else:
                blocks, tail = payload
                whole = img.numel() // self.BLOCK * self.BLOCK
                if idx.numel():
                    img[:whole].view(-1, self.BLOCK)[idx.long()] = blocks
                if tail.numel():
                    img[whole:] = tail
        self._cursor[name] = (pos, img)
        return img.clone()

    def has(self, key, name: str) -> bool:
        return any(e[0] == key for e in self._chain.get(name, []))


class SpanTap:
    """An engine probe (``Engine.probe``) that runs a program in call ranges around its changed spans.

    Recording side (A): before each span it keeps images of the buffers the span reads — on both sides — and after the
    span the buffers it writes. Replaying side (B): it runs its own calls up to the span, puts A's images of the same
    step into the buffers its span reads, runs only the span, and compares what the span wrote with what A's span
    wrote. A difference is then pinned to the span that made it, from identical inputs, instead of being read off the
    end of a free run where earlier differences have piled up. Paged / per-sequence states are not imaged: along
    forced tokens they differ only where an earlier span's outputs already did, which that span's line shows.
    Reference: crates/kern-test/src/harness.rs:46-220 (frontier snapshots), replay.rs."""

    def __init__(self, mine: dict, other: dict, spans_by_program: dict, side: str, store: dict, results: list | None = None):
        self.doc, self.other, self.side, self.store = mine, other, side, store
        self.images: DeltaImages = store.setdefault("__images__", DeltaImages())      # shared by the two sides' taps
        self.results = results if results is not None else []
        self.spans = {p: [sp for sp in ss if sp["a"] and sp["b"]] for p, ss in spans_by_program.items()}
        self.step = 0

    def _shared(self, names) -> list[str]:
        return sorted(n for n in names if _buffer_bytes(self.doc, n) is not None and
                      _buffer_bytes(self.doc, n) == _buffer_bytes(self.other, n))

    @staticmethod
    def _image(rt, names) -> dict:
        import torch

        if hasattr(rt, "synchronize"):
            rt.synchronize()
        return {n: rt.tensor(n).contiguous().view(-1).view(torch.uint8).cpu().clone() for n in names}

    def run(self, rt, program: str, vars: dict, tag: str) -> int:
        import torch

        calls = self.doc["programs"][program]["calls"]
        key_step = (program, tuple(sorted(vars.items())), self.step)
        self.step += 1
        lo, n = 0, 0
        for k, sp in enumerate(self.spans.get(program, [])):
            mine = sp["a"] if self.side == "a" else sp["b"]
            theirs_doc_calls = sp["b"] if self.side == "a" else sp["a"]
            first, last = mine[0], mine[-1] + 1
            reads = self._shared(read_set(self.doc, program, mine) | read_set(self.other, program, theirs_doc_calls))
            writes = self._shared(write_set(self.doc, program, mine) & write_set(self.other, program, theirs_doc_calls))
            n += rt.issue_range(program, vars, lo, first)
            key = key_step + (k,)
            if self.side == "a":
                self.store[key] = {"in": list(reads), "out": list(writes)}
                for name, img in self._image(rt, reads).items():
                    self.images.put(key + ("in",), name, img)
                n += rt.issue_range(program, vars, first, last)
                for name, img in self._image(rt, writes).items():
                    self.images.put(key + ("out",), name, img)
            else:
                rec = self.store.get(key)
                if rec is None:
                    self.results.append({"program": program, "span": k, "step": key_step[2], "skipped": "A recorded no such step"})
                    n += rt.issue_range(program, vars, first, last)
                else:
                    if hasattr(rt, "synchronize"):
                        rt.synchronize()
                    for name in rec["in"]:
                        t = rt.tensor(name)
                        t.view(-1).view(torch.uint8).copy_(self.images.get(key + ("in",), name).to(t.device))
                    n += rt.issue_range(program, vars, first, last)
                    got = self._image(rt, writes)
                    for name in writes:
                        want = self.images.get(key + ("out",), name)
                        c = compare_bytes(self.doc["buffers"][name]["dtype"], want.numpy().tobytes(), got[name].numpy().tobytes())
                        self.results.append({"program": program, "span": k, "step": key_step[2], "buffer": name,
                                             "identical": c.identical, "value_identical": c.value_identical,
                                             "differing": c.n_diff, "max_abs": c.max_abs, "max_ulp": c.max_ulp})
            lo = last
        n += rt.issue_range(program, vars, lo, len(calls))
        return n


def replay_spans(side_a: "EngineSide", side_b: "EngineSide", work: list[list[int]], forced: list[list[int]], chunk: int) -> list[dict]:
    """Run the workload on A recording span images, then on B (teacher-forced along `forced`, A's tokens) replaying
    every changed span from A's images. Returns one line per (program, span, step, buffer)."""
    sp = spans(side_a.doc, side_b.doc)
    if not any(x["a"] and x["b"] for ss in sp.values() for x in ss):
        return []
    store, results = {}, []
    side_a.eng.probe = SpanTap(side_a.doc, side_b.doc, sp, "a", store)
    try:
        side_a.forced_run(work, forced, chunk)
    finally:
        side_a.eng.probe = None
    side_b.eng.probe = SpanTap(side_b.doc, side_a.doc, sp, "b", store, results)
    try:
        side_b.forced_run(work, forced, chunk)
    finally:
        side_b.eng.probe = None
    img = store["__images__"]
    if results:
        results[0]["snapshot_bytes"] = {"whole_images": img.full_bytes, "kept_as_deltas": img.kept_bytes}
    return results


# ---- report ------------------------------------------------------------------------------------------
@dataclass
class Report:
    lines: list[str] = field(default_factory=list)
    verdict: str = INCONCLUSIVE
    reason: str = ""
    facts: dict = field(default_factory=dict)

    def add(self, line: str) -> None:
        self.lines.append(line)

    def text(self) -> str:
        return "\n".join(self.lines + [f"{self.verdict}: {self.reason}"])

    @property
    def exit_code(self) -> int:
        return EXIT[self.verdict]


def run_test(side_a: EngineSide, side_b: EngineSide, seed: int = 0, prompts: int = 4, decode_steps: int = 8,
             logit_kl: float = 0.01, chunk: int | None = None) -> Report:
    rep = Report()
    a, b = side_a.doc, side_b.doc
    # DIFF
    changes = op_changes(a, b)
    sp = spans(a, b)
    rep.facts["op_changes"] = changes
    rep.facts["spans"] = {p: len(s) for p, s in sp.items()}
    for name, how in changes.items():
        rep.add(f"diff op {name}: {how}")
    for p, s in sp.items():
        if s:
            rep.add(f"diff program {p}: {len(s)} span(s) of changed calls")
    for p in sorted(set(a["programs"]) ^ set(b["programs"])):
        rep.add(f"diff program {p}: only on one side")
    pa, pb = side_a.eng.p, side_b.eng.p
    if pa["rows"]["max"] != pb["rows"]["max"] or {f["fill"] for f in pa["fills"]} != {f["fill"] for f in pb["fills"]}:
        rep.verdict, rep.reason = INCONCLUSIVE, "the two manifests are driven differently (rows bound or fills differ); the same workload cannot feed both"
        return rep
    # TAP
    rng = Rng(seed)
    rows_max = min(pa["rows"]["max"], pb["rows"]["max"])
    page = side_a.eng.unit
    chunk = chunk or rows_max
    tok_fill = next(f for f in pa["fills"] if f["fill"] == "token")
    dom = a["buffers"][tok_fill["name"]].get("domain", {})
    lo, hi = int(dom.get("min", 0)), int(dom.get("max", 255))
    cap = min(rows_max, side_a.eng.pool.total_pages * page - decode_steps - 1,
              min((t["width"] * t["stride"] for t in pa["page_tables"]), default=rows_max) - decode_steps - 1)
    work = [[lo + rng.below(hi - lo + 1) for _ in range(prefill_length(rng, max(1, cap), page, chunk))] for _ in range(prompts)]
    rep.add(f"tap workload seed={seed} prompts={[len(w) for w in work]} decode_steps={decode_steps}")
    out_a, rows_a, perf_a = side_a.free_run(work, decode_steps, chunk)
    out_b, rows_b, perf_b = side_b.free_run(work, decode_steps, chunk)
    out_a2, rows_a2, _ = side_a.free_run(work, decode_steps, chunk)          # NOISE: A against itself
    forced_b = side_b.forced_run(work, out_a, chunk) if out_a != out_b else rows_b
    # domain check of outputs
    for toks in out_b:
        for t in toks:
            if not (lo <= t <= hi):
                rep.verdict, rep.reason = FAIL, f"B emitted token {t}, outside the declared domain [{lo}, {hi}]"
                return rep
    same_tokens = out_a == out_b
    rep.add(f"tap tokens {'identical' if same_tokens else 'differ'} over {sum(map(len, out_a))} generated tokens")
    have_logits = rows_a and rows_a[0] is not None and forced_b and forced_b[0] is not None
    stats, noise = [], []
    if have_logits:
        stats = [logit_stats(x, y) for x, y in zip(rows_a, forced_b)]
        noise = [logit_stats(x, y) for x, y in zip(rows_a, rows_a2)]
        worst = max(stats, key=lambda s: s["kl"])
        rep.add(f"logits rows={len(stats)} max_kl={worst['kl']:.3e} argmax_agree={sum(s['agree'] for s in stats)}/{len(stats)} "
                f"min_top{TOP}_overlap={min(s['top_overlap'] for s in stats)}")
        rep.add(f"noise max_kl={max(s['kl'] for s in noise):.3e}")
        rep.facts["max_kl"] = worst["kl"]
    # REPLAY: every changed span of B from A's images of the same step
    span_lines = replay_spans(side_a, side_b, work, out_a, chunk) if any(sp.values()) else []
    rep.facts["span_replay"] = span_lines
    by_span: dict = {}
    for l in span_lines:
        if "buffer" in l:
            by_span.setdefault((l["program"], l["span"]), []).append(l)
    for (prog, k), ls in sorted(by_span.items()):
        worst_l = max(ls, key=lambda l: (not l["value_identical"], l["max_abs"]))
        how = "bit-identical" if all(l["identical"] for l in ls) else (
            "value-identical" if all(l["value_identical"] for l in ls) else
            f"differs: {worst_l['buffer']} max_abs={worst_l['max_abs']:.3e} max_ulp={worst_l['max_ulp']} at step {worst_l['step']}")
        rep.add(f"replay program {prog} span {k}: {len(ls)} comparisons from A's images, {how}")
    bit_identical = have_logits and all(np.array_equal(x, y) for x, y in zip(rows_a, forced_b))
    rep.add(f"perf A prefill {perf_a['prefill_s'] * 1e3:.2f} ms decode {perf_a['decode_s'] * 1e3:.2f} ms | "
            f"B prefill {perf_b['prefill_s'] * 1e3:.2f} ms decode {perf_b['decode_s'] * 1e3:.2f} ms")
    rep.facts["perf"] = {"a": perf_a, "b": perf_b}
    # verdict ladder
    if have_logits:
        flips = [s for s in stats if not s["agree"] and s["kl"] > logit_kl]
        if flips:
            rep.verdict, rep.reason = FAIL, f"{len(flips)} argmax flip(s) with row KL above {logit_kl} (worst {max(f['kl'] for f in flips):.3e})"
            return rep
    if not changes and not any(sp.values()) and same_tokens and (bit_identical or not have_logits):
        rep.verdict, rep.reason = PASS, "bit-identical (and no structural difference)"
    elif same_tokens and bit_identical:
        rep.verdict, rep.reason = PASS, "logits bit-identical"
    elif have_logits and all(s["kl"] <= logit_kl for s in stats):
        rep.verdict, rep.reason = PASS, f"logit evidence: every row KL <= {logit_kl}; flips within the limit are ties"
    elif have_logits and noise and max(s["kl"] for s in stats) <= max(s["kl"] for s in noise) * 1.5 + 1e-12:
        rep.verdict, rep.reason = PASS, "within the noise floor of A against itself"
    elif not have_logits and same_tokens:
        rep.verdict, rep.reason = PASS, "tokens identical (the manifest exposes no logits buffer)"
    else:
        rep.verdict, rep.reason = INCONCLUSIVE, "differences above the noise floor without a logits verdict"
    return rep
