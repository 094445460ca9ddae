"""Speculative decoding as a manifest: a target decoder and a small draft decoder in one runtime, one pool, and a
`round` program (a fixed block of R rows per sequence, captured as one CUDA graph) that drafts, verifies and counts
on the device. Speculation is not a schema concept — it is a program with rows > 1 and a `count` output.

round (rows R = k + 1, the host stages the anchor token of every sequence in all R rows, with the R next positions
and slots):
  chain step j = 0..k : the draft runs one row per sequence at position base + j on token (j == 0 ? anchor : d[j-1]),
                        appends its own KV there, and proposes d[j] (the last step only writes KV: its proposal is unused)
  verify              : ids = [anchor, d[0..k-1]]; the target runs all R rows causally; row j predicts what follows id j
  accept              : a = longest prefix of d reproduced by verify; count = a + 1; tokens = verify[0..a]
Rollback is free: a paged slot is its position, rejected rows are overwritten by the next round. `prefill` and
`decode` run the draft alongside the target so its KV cache always holds the same tokens.
Reference shape: docs/spec-decode.md:9-66; tools/kernels-src/spec_round.cu, markov_rows.cu.
"""
from __future__ import annotations

import copy
import dataclasses

from . import common as C
from . import dense

SHARED = ("token_ids", "positions", "slot_mapping", "seq_lens", "cu_seqlens", "block_table", "error")


def _rename(doc: dict, prefix: str, keep=SHARED) -> dict:
    """Every buffer (but the shared inputs), state and op of a manifest under `prefix`; weights bind `draft.<tensor>`."""
    d = copy.deepcopy(doc)
    nb = lambda n: n if n in keep else prefix + n
    bufs = {}
    for n, b in d["buffers"].items():
        if n in keep:
            continue
        b = dict(b)
        for seg in b.get("bind", []):
            seg["tensor"] = "draft." + seg["tensor"]
        if (b.get("domain") or {}).get("index_into"):
            b["domain"]["index_into"] = prefix + b["domain"]["index_into"]
        bufs[prefix + n] = b
    d["buffers"] = bufs
    d["states"] = {prefix + n: s for n, s in d["states"].items()}
    d["ops"] = {prefix + n: o for n, o in d["ops"].items()}
    for p in d["programs"].values():
        for c in p["calls"]:
            c["op"] = prefix + c["op"]
            if "label" in c:
                c["label"] = prefix + c["label"]
            c["args"] = [dict(a) for a in c["args"]]       # a generator may share one arg object between calls
            for a in c["args"]:
                if "buf" in a:
                    a["buf"] = nb(a["buf"])
                elif "state" in a:
                    a["state"] = prefix + a["state"]
    return d


def _swap(calls: list[dict], mapping: dict[str, str]) -> list[dict]:
    out = copy.deepcopy(calls)
    for c in out:
        c["args"] = [dict(a) for a in c["args"]]
        for a in c["args"]:
            if a.get("buf") in mapping:
                a["buf"] = mapping[a["buf"]]
    return out


def draft_config(target: dense.DenseConfig, layers: int = 1, hidden: int | None = None) -> dense.DenseConfig:
    """A shallow decoder over the same vocabulary, pages and limits as the target."""
    h = hidden or target.hidden
    return dataclasses.replace(target, name=target.name + "-draft", layers=layers, hidden=h,
                               heads=max(1, h // target.head_dim), kv_heads=max(1, min(target.kv_heads, h // target.head_dim)),
                               intermediate=max(16, (h * 3) // 16 * 16))


def build_manifest(target: dense.DenseConfig, draft: dense.DenseConfig | None = None, k: int = 4) -> dict:
    draft = draft or draft_config(target)
    assert draft.vocab == target.vocab and draft.page_size == target.page_size and draft.max_context == target.max_context
    R = k + 1
    S, T = target.max_seqs, target.max_tokens
    assert S * R <= T, "a round of every sequence must fit the rows of a call"
    doc = dense.build_manifest(target)
    dd = _rename(dense.build_manifest(draft), "d.")
    doc["model"] = f"{target.name}+spec{k}"
    doc["buffers"].update(dd["buffers"])
    doc["states"].update(dd["states"])
    doc["ops"].update(dd["ops"])
    B = lambda n: {"buf": n}
    err = B("error")
    bufs, ops = doc["buffers"], doc["ops"]
    h, d, hq, hk, W = target.hidden, target.head_dim, target.heads, target.kv_heads, target.table_width

    # the draft shadows prefill and decode (all layers, no head): its KV cache follows the target's
    is_head = lambda c: c["op"] in ("d.norm_last", "d.lm_head", "d.pick", "d.last_row")
    for prog in ("prefill", "decode"):
        doc["programs"][prog]["calls"] += [c for c in dd["programs"][prog]["calls"] if not is_head(c)]
    doc["programs"]["load"]["calls"] += dd["programs"]["load"]["calls"]
    bufs.pop("d.last")
    ops.pop("d.last_row")
    bufs["d.next_token"] = {"dtype": "i64", "shape": ["seqs"], "kind": "workspace"}     # a proposal, not an answer

    # ---- round ----
    for name, dt in (("c.tok", "i64"), ("c.pos", "i64"), ("c.slot", "i64")):
        bufs[name] = {"dtype": dt, "shape": ["seqs"], "kind": "workspace"}
    bufs["c.lens"] = {"dtype": "i32", "shape": ["seqs"], "kind": "workspace"}
    bufs["anchor"] = {"dtype": "i64", "shape": ["seqs"], "kind": "workspace"}
    bufs["drafts"] = {"dtype": "i64", "shape": ["seqs", R], "kind": "workspace"}
    bufs["ids"] = {"dtype": "i64", "shape": ["tokens"], "kind": "workspace"}
    bufs["verify"] = {"dtype": "i64", "shape": ["tokens"], "kind": "workspace"}
    bufs["logits_r"] = {"dtype": "bf16", "shape": [S * R, target.vocab], "kind": "workspace"}
    bufs["round_tokens"] = {"dtype": "i64", "shape": ["seqs", R], "kind": "output", "fill": "tokens"}
    bufs["round_count"] = {"dtype": "i32", "shape": ["seqs"], "kind": "output", "fill": "count"}

    def small(entry, lp, args, grid, block=(128, 1, 1), module="spec"):
        return {"module": module, "entry": entry, "block": list(block), "grid": grid, "params": lp, "args": args}

    # these three run a thread per sequence in blocks of 128: the real sequence count is an argument (interface: [.., n, seqs])
    ops["column"] = {"params": ["in buffer<i64>", "out buffer<i64>", "i32", "i32"], "impl": {"launches": [small(
        "kern_spec_column_i64", ["in buffer<i64>", "out buffer<i64>", "i32", "i32", "i32"],
        [{"param": 0}, {"param": 1}, {"param": 3}, {"i32": R}, {"param": 2}], [{"ceil_div": ["seqs", 128]}, 1, 1])]}}
    ops["lens"] = {"params": ["in buffer<i32>", "out buffer<i32>", "i32", "i32"], "impl": {"launches": [small(
        "kern_spec_lens", ["in buffer<i32>", "out buffer<i32>", "i32", "i32"],
        [{"param": 0}, {"param": 1}, {"param": 3}, {"param": 2}], [{"ceil_div": ["seqs", 128]}, 1, 1])]}}
    ops["chain"] = {"params": ["in buffer<i64>", "inout buffer<i64>", "i32", "i32"], "impl": {"launches": [small(
        "kern_spec_chain", ["in buffer<i64>", "inout buffer<i64>", "i32", "i32", "i32"],
        [{"param": 0}, {"param": 1}, {"param": 3}, {"param": 2}, {"i32": R}], [{"ceil_div": ["seqs", 128]}, 1, 1])]}}
    ops["splice"] = {"params": ["in buffer<i64>", "in buffer<i64>", "out buffer<i64>"], "impl": {"launches": [small(
        "kern_spec_splice", ["in buffer<i64>", "in buffer<i64>", "out buffer<i64>", "i32", "i32", "i32", "i64"],
        [{"param": 0}, {"param": 1}, {"param": 2}, {"i32": C.I32_MAX}, {"i32": R}, {"i32": R}, {"i64": 0}], ["seqs", 1, 1],
        block=(32, 1, 1))]}}
    ops["accept"] = {"params": ["in buffer<i64>", "in buffer<i64>", "out buffer<i32>", "out buffer<i64>"], "impl": {"launches": [small(
        "kern_spec_accept", ["in buffer<i64>", "in buffer<i64>", "out buffer<i32>", "out buffer<i64>", "i64", "i64", "i32", "i32",
                             "i32", "i32", "i32"],
        [{"param": 0}, {"param": 1}, {"param": 2}, {"param": 3}, {"i64": 0}, {"i64": 0}, {"i32": C.I32_MAX}, {"i32": R}, {"i32": R},
         {"i32": 0}, {"i32": 0}], ["seqs", 1, 1], block=(32, 1, 1))]}}
    ops["attn_verify"] = C.attn_decode_op(hq, hk, d, target.page_size, W, target.qkv_dim, S, rows=R)
    ops["lm_head_rows"] = C.gemm_op(target.vocab, h, rows_max=S * R)
    ops["pick_rows"] = C.argmax_op(target.vocab, rows_var="tokens")

    # a chain step has one row per sequence while the round's call has R: the draft's decode ops once more with the
    # row count taken from `seqs` (grids, `when` ranges, scratch shapes, row arguments)
    import json as _json

    used = {c["op"] for c in dd["programs"]["decode"]["calls"]}
    for name in used:
        ops["dc." + name[2:]] = _json.loads(_json.dumps(dd["ops"][name]).replace('"tokens"', '"seqs"'))
    chain_map = {"token_ids": "c.tok", "positions": "c.pos", "slot_mapping": "c.slot", "seq_lens": "c.lens"}
    step = _swap(dd["programs"]["decode"]["calls"], chain_map)        # the draft's whole decode step, head included
    for c in step:
        c["op"] = "dc." + c["op"][2:]
        for a in c["args"]:
            if a.get("var") == "tokens":
                a["var"] = "seqs"
    for name in ("d.lm_head", "d.norm_last", "d.pick"):      # only the chain runs the draft's head
        ops.pop(name)
    ops["zero_i64"] = {"params": ["out buffer<i64>"], "impl": {"launches": [small(
        "kern_fill_i64", ["out buffer<i64>", "i64", "i64"], [{"param": 0}, {"i64": S * R}, {"i64": 0}], [8, 1, 1],
        block=(256, 1, 1), module="misc")]}}
    calls = [{"op": "column", "label": "anchor", "args": [B("token_ids"), B("anchor"), {"i32": 0}, {"var": "seqs"}]},
             {"op": "zero_i64", "label": "drafts0", "args": [B("drafts")]}]
    for j in range(R):
        src = B("anchor") if j == 0 else None
        if j == 0:
            calls.append({"op": "column", "label": f"c{j}.tok", "args": [B("token_ids"), B("c.tok"), {"i32": 0}, {"var": "seqs"}]})
        else:
            calls.append({"op": "column", "label": f"c{j}.tok", "args": [B("drafts"), B("c.tok"), {"i32": j - 1}, {"var": "seqs"}]})
        calls += [{"op": "column", "label": f"c{j}.pos", "args": [B("positions"), B("c.pos"), {"i32": j}, {"var": "seqs"}]},
                  {"op": "column", "label": f"c{j}.slot", "args": [B("slot_mapping"), B("c.slot"), {"i32": j}, {"var": "seqs"}]},
                  {"op": "lens", "label": f"c{j}.lens", "args": [B("seq_lens"), B("c.lens"), {"i32": R - 1 - j}, {"var": "seqs"}]}]
        for c in copy.deepcopy(step):
            c["label"] = f"c{j}." + c.get("label", c["op"])
            calls.append(c)
        calls.append({"op": "chain", "label": f"c{j}.keep", "args": [B("d.next_token"), B("drafts"), {"i32": j}, {"var": "seqs"}]})
    calls.append({"op": "splice", "label": "splice", "args": [B("anchor"), B("drafts"), B("ids")]})
    # verify: the target's decode step over R rows per sequence
    verify = []
    for c in copy.deepcopy(doc["programs"]["decode"]["calls"]):
        if c["op"].startswith("d.") or c["op"] in ("norm_last", "lm_head", "pick"):
            continue
        if c["op"] == "attn_decode":
            c["op"] = "attn_verify"
        c["args"] = [dict(a) for a in c["args"]]
        for a in c["args"]:
            if a.get("buf") == "token_ids":
                a["buf"] = "ids"
        c["label"] = "v." + c.get("label", c["op"])
        verify.append(c)
    calls += verify
    calls += [{"op": "norm", "label": "v.final_norm", "args": [B("x"), B("w.norm"), B("xn")]},
              {"op": "lm_head_rows", "label": "v.lm_head", "args": [B("xn"), B("w.head"), B("logits_r"), {"var": "tokens"}, err]},
              {"op": "pick_rows", "label": "v.argmax", "args": [B("logits_r"), B("verify")]},
              {"op": "accept", "label": "accept", "args": [B("drafts"), B("verify"), B("round_count"), B("round_tokens")]}]
    doc["programs"]["round"] = {"batch": {"groups": S, "rows": R}, "graph": True, "calls": calls}
    doc["modules"] = C.modules_for(["norm_embed", "gemm_bf16", "attn_prep", "attn_paged", "misc", "sampling", "spec"])
    return doc


def random_weights(target: dense.DenseConfig, draft: dense.DenseConfig | None = None, seed: int = 0, std: float = 0.02,
                   draft_from_target: bool = False):
    """Target weights plus `draft.`-prefixed draft weights. `draft_from_target`: the draft is a copy of the target's first
    layers (a draft that often agrees, for tests of the accept path)."""
    draft = draft or draft_config(target)
    w = dense.random_weights(target, seed=seed, std=std)
    if draft_from_target:
        assert draft.hidden == target.hidden and draft.heads == target.heads and draft.intermediate == target.intermediate
        dw = {n: t for n, t in w.items() if not n.startswith("model.layers.") or int(n.split(".")[2]) < draft.layers}
    else:
        dw = dense.random_weights(draft, seed=seed + 1, std=std)
    w.update({"draft." + n: t for n, t in dw.items()})
    return w


# ---- CPU statements of the round's glue kernels --------------------------------------------------------
def _register_cpu() -> None:
    from .. import cpu

    def column(g, src, dst, seqs, stride, col):
        dst[:seqs] = src[: seqs * stride].view(seqs, stride)[:, col]

    def lens(g, src, out, seqs, delta):
        n = seqs
        v = src[:n]
        out[:n] = ((v > 0) * (v - delta).clamp(min=0)).to(out.dtype)

    def chain(g, nxt, drafts, seqs, col, stride):
        n = seqs
        drafts[: n * stride].view(n, stride)[:, col] = nxt[:n]

    def splice(g, anchor, drafts, ids, seqs, block, dstride, mask):
        n = g[0]
        rows = ids[: n * block].view(n, block)
        rows[:, 0] = anchor[:n]
        rows[:, 1:] = drafts[: n * dstride].view(n, dstride)[:, : block - 1] if hasattr(drafts, "view") else mask

    def accept(g, drafts, verify, count, emitted, line_in, line_adv, seqs, block, dstride, line_rows, seqs_max):
        n = g[0]
        d, v = drafts[: n * dstride].view(n, dstride), verify[: n * block].view(n, block)
        em = emitted[: n * block].view(n, block)
        for i in range(n):
            a = 0
            while a < block - 1 and int(d[i, a]) == int(v[i, a]):
                a += 1
            count[i] = a + 1
            em[i] = 0
            em[i, : a + 1] = v[i, : a + 1]

    cpu.register("kern_spec_column_i64", column)
    cpu.register("kern_spec_lens", lens)
    cpu.register("kern_spec_chain", chain)
    cpu.register("kern_spec_splice", splice)
    cpu.register("kern_spec_accept", accept)


_register_cpu()
