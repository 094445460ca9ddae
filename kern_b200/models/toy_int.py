"""The exact integer model: manifests, the host twin of its arithmetic, and the CPU statements of its kernels.

A served token has one right value, decided by what the sequence's KV slots (and state line) hold; see
csrc/kernels/sm100/toy_int.cu. ``generate(ids, n, lined)`` is the twin every serving test compares against.
Two manifests: ``paged`` (KV pages only) and ``stateful`` (pages + a per-sequence line), each with a ragged
``prefill`` and a graph-replayed ``decode``. Reference counterpart of the idea: tools/toy/gen.py, tools/toy/model.py.
"""
from __future__ import annotations

import numpy as np
import torch

from . import common as C

M = (1 << 64) - 1
WORDS, LINE, EOS, EOS_EVERY, VOCAB = 32, 8, 256, 80, 256
K_LINE = 0xD6E8FEB86659FD93


def fmix(x: int) -> int:
    x ^= x >> 33
    x = (x * 0xFF51AFD7ED558CCD) & M
    x ^= x >> 33
    x = (x * 0xC4CEB9FE1A85EC53) & M
    return x ^ (x >> 33)


def mark(t: int, p: int, w: int) -> int:
    return fmix(((t * 0x9FB21C651E98DF25) & M) ^ ((p * 0xA24BAED4963EE407) & M) ^ (((w + 1) * 0x8CB92BA72F3D8DD7) & M))


def rotl(x: int, k: int) -> int:
    k &= 63
    return ((x << k) | (x >> (64 - k))) & M if k else x


def slot_sum(t: int, p: int) -> int:
    return sum(rotl(mark(t, p, w), (p + w) & 63) for w in range(WORDS)) & M


def next_of(s: int) -> int:
    return EOS if (s >> 57) % EOS_EVERY == 0 else s & 255


def generate(ids: list[int], max_tokens: int, lined: bool = False) -> list[int]:
    """The greedy continuation of `ids`: up to `max_tokens` tokens; end-of-sequence ends it and is not returned."""
    s, c = 0, 0
    for p, t in enumerate(ids):
        s = (s + slot_sum(t, p)) & M
        c = rotl(c, 11) ^ mark(t, p, 0xFFFF)
    out, n = [], len(ids)
    for _ in range(max_tokens):
        t = next_of((s + (c if lined else 0)) & M)
        if t == EOS:
            break
        out.append(t)
        s = (s + slot_sum(t, n)) & M
        c = rotl(c, 11) ^ mark(t, n, 0xFFFF)
        n += 1
    return out


def build_manifest(lined: bool = False, page_size: int = 16, max_tokens: int = 128, max_seqs: int = 8,
                   max_context: int = 256, name: str | None = None, per_sequence_prefill: bool = False) -> dict:
    """`per_sequence_prefill` (paged form only): the ragged program takes one sequence per call and only appends — it
    emits nothing, and the first step is fed the prompt's last token — the shape of the reference's paged packages
    (tools/toy/gen.py:107-113)."""
    W = -(-max_context // page_size)
    B = lambda n: {"buf": n}
    bufs = {
        "token_ids": {"dtype": "i64", "shape": ["tokens"], "kind": "input", "fill": "token", "domain": {"min": 0, "max": 255}},
        "positions": {"dtype": "i64", "shape": ["tokens"], "kind": "input", "fill": "position",
                      "domain": {"min": 0, "max": max_context - 1}},
        "slot_mapping": {"dtype": "i64", "shape": ["tokens"], "kind": "input", "fill": "slot", "domain": {"index_into": "kv"}},
        "seq_lens": {"dtype": "i32", "shape": ["seqs"], "kind": "input", "fill": "seq_len"},
        "cu_seqlens": {"dtype": "i32", "shape": [max_seqs + 1], "kind": "input", "fill": "cu_seqlens"},
        "block_table": {"dtype": "i32", "shape": ["seqs", W], "kind": "input", "domain": {"index_into": "kv", "stride": page_size}},
        "next_token": {"dtype": "i64", "shape": ["seqs"], "kind": "output", "fill": "tokens"},
        "error": {"dtype": "i32", "shape": [1], "kind": "output", "fill": "error"},
    }
    states = {"kv": {"bytes_per_token": WORDS * 8}}
    if lined:
        states["line"] = {"bytes_per_seq": LINE * 8}
        bufs["lines"] = {"dtype": "i32", "shape": [1, "seqs"], "kind": "input", "domain": {"index_into": "line"}}
    ops = {
        "append": {"params": ["in buffer<i64>", "in buffer<i64>", "in buffer<i64>", "inout state", "out buffer<i32>"],
                   "impl": {"launches": [{"module": "toy_int", "entry": "toy_append", "block": [WORDS, 1, 1], "grid": ["tokens", 1, 1],
                                          "params": ["in buffer<i64>", "in buffer<i64>", "in buffer<i64>", "inout state", "i32", "i64",
                                                     "out buffer<i32>"],
                                          "args": [{"param": 0}, {"param": 1}, {"param": 2}, {"param": 3}, {"i32": C.I32_MAX},
                                                   {"i64": C.I64_MAX}, {"param": 4}]}]}},
    }

    def predict_op(ragged: bool):
        iface = ["in state", "in buffer<i32>", "in buffer<i32>"]
        lp = list(iface)
        args = [{"param": 0}, {"param": 1}, {"param": 2}]
        if lined:
            iface += ["in buffer<i32>", "in state"]
            lp += ["in buffer<i32>", "in state"]
            args += [{"param": 3}, {"param": 4}]
        else:
            lp += ["i64", "i64"]
            args += [{"i64": 0}, {"i64": 0}]
        if ragged:
            iface.append("in buffer<i32>")
            lp.append("in buffer<i32>")
            args.append({"param": len(iface) - 1})
        else:
            lp.append("i64")
            args.append({"i64": 0})
        iface.append("out buffer<i64>")
        lp += ["out buffer<i64>", "i32", "i32", "i32"]
        args += [{"param": len(iface) - 1}, {"i32": C.I32_MAX}, {"i32": W}, {"i32": page_size}]
        return {"params": iface, "impl": {"launches": [{"module": "toy_int", "entry": "toy_predict", "block": [256, 1, 1],
                                                        "grid": ["seqs", 1, 1], "params": lp, "args": args}]}}

    def fold_op(ragged: bool):
        iface = ["in buffer<i64>", "in buffer<i64>"] + (["in buffer<i32>"] if ragged else []) + ["in buffer<i32>", "inout state"]
        lp = ["in buffer<i64>", "in buffer<i64>", "in buffer<i32>" if ragged else "i64", "in buffer<i32>", "inout state", "i32", "i32"]
        n = len(iface)
        args = [{"param": 0}, {"param": 1}, {"param": 2} if ragged else {"i64": 0}, {"param": n - 2}, {"param": n - 1},
                {"i32": C.I32_MAX}, {"i32": 1}]
        return {"params": iface, "impl": {"launches": [{"module": "toy_int", "entry": "toy_fold", "block": [32, 1, 1],
                                                        "grid": ["seqs", 1, 1], "params": lp, "args": args}]}}

    ops["predict_p"], ops["predict_d"] = predict_op(True), predict_op(False)
    if lined:
        ops["fold_p"], ops["fold_d"] = fold_op(True), fold_op(False)

    def calls(prefill: bool) -> list[dict]:
        out = [{"op": "append", "args": [B("token_ids"), B("positions"), B("slot_mapping"), {"state": "kv"}, B("error")]}]
        if lined:
            cu = [B("cu_seqlens")] if prefill else []
            out.append({"op": "fold_p" if prefill else "fold_d",
                        "args": [B("token_ids"), B("positions"), *cu, B("lines"), {"state": "line"}]})
        pa = [{"state": "kv"}, B("block_table"), B("seq_lens")] + ([B("lines"), {"state": "line"}] if lined else [])
        out.append({"op": "predict_p" if prefill else "predict_d",
                    "args": pa + ([B("cu_seqlens")] if prefill else []) + [B("next_token")]})
        return out

    prefill = {"batch": {"groups": max_seqs, "rows": "tokens"}, "calls": calls(True)}
    if per_sequence_prefill:
        assert not lined
        prefill = {"batch": {"groups": 1, "rows": "tokens"}, "calls": calls(True)[:1]}
        ops.pop("predict_p")
        bufs.pop("cu_seqlens")
    return {"schema_version": 7, "model": name or ("toy-int-stateful" if lined else "toy-int-paged"),
            "vars": {"tokens": {"max": max_tokens, "axis": "rows"}, "seqs": {"max": max_seqs, "axis": "groups"}},
            "states": states, "buffers": bufs, "modules": C.modules_for(["toy_int"]), "ops": ops,
            "programs": {"prefill": prefill,
                         "decode": {"batch": {"groups": max_seqs, "rows": 1}, "graph": True, "calls": calls(False)}}}


# ---- CPU statements ------------------------------------------------------------------------------------
def _u64(t: torch.Tensor) -> np.ndarray:
    return t.numpy().view(np.uint64)


def _k_append(g, tokens, positions, slots, kv, rows, kv_slots, err):
    words = _u64(kv.view(torch.int64)) if kv.dtype != torch.int64 else _u64(kv)
    for r in range(g[0]):
        s = int(slots[r])
        if s < 0:
            continue
        for w in range(WORDS):
            words[s * WORDS + w] = mark(int(tokens[r]), int(positions[r]), w)


def _k_fold(g, tokens, positions, cu, lines, state, seqs, rows_per_seq):
    words = _u64(state.view(torch.int64))
    for s in range(g[0]):
        line = int(lines[s])
        if line <= 0:
            continue
        r0, r1 = (int(cu[s]), int(cu[s + 1])) if isinstance(cu, torch.Tensor) else (s * rows_per_seq, (s + 1) * rows_per_seq)
        c = int(words[line * LINE])
        for r in range(r0, r1):
            c = rotl(c, 11) ^ mark(int(tokens[r]), int(positions[r]), 0xFFFF)
        for i in range(LINE):
            words[line * LINE + i] = c ^ ((i * K_LINE) & M)


def _k_predict(g, kv, table, seq_lens, lines, state, cu, nxt, seqs, max_pages, page):
    words = _u64(kv.view(torch.int64))
    for s in range(g[0]):
        L = int(seq_lens[s])
        if isinstance(cu, torch.Tensor) and int(cu[s + 1]) == int(cu[s]):
            L = 0
        S = 0
        for p in range(L):
            slot = int(table[s * max_pages + p // page]) * page + p % page
            for w in range(WORDS):
                S = (S + rotl(int(words[slot * WORDS + w]), (p + w) & 63)) & M
        if isinstance(lines, torch.Tensor):
            line = int(lines[s])
            lw = _u64(state.view(torch.int64))
            c = int(lw[line * LINE])
            for i in range(1, LINE):
                if int(lw[line * LINE + i]) ^ ((i * K_LINE) & M) != c:
                    c = (~c) & M
            if line > 0:
                S = (S + c) & M
        nxt[s] = 0 if L <= 0 else next_of(S)


def register_cpu() -> None:
    from .. import cpu

    cpu.register("toy_append", _k_append)
    cpu.register("toy_fold", _k_fold)
    cpu.register("toy_predict", _k_predict)


register_cpu()
