"""The MoE decoder over a rank group: attention tensor-parallel by heads, experts expert-parallel — rank r keeps experts
[r E/n, (r+1) E/n) and computes their share of every token of the replicated batch; the shares meet in the same fused
all-reduce + residual + RMSNorm that closes the attention block. No all-to-all: at decode sizes the token rows are small
next to the expert weights, so every rank routes every token and runs only its own experts.
Reference shape: docs/roadmap.md:13-16 (EP decode as gather, local experts, reduce).
"""
from __future__ import annotations

from . import common as C
from . import dense_tp
from .moe import MoeConfig, _moe_ops


def build_manifest_ep(cfg: MoeConfig, lamport: bool = True) -> dict:
    n = cfg.tp
    assert n >= 2 and cfg.experts % n == 0
    # the attention half (and the dense MLP's wiring, replaced below) comes from the tensor-parallel dense generator
    doc = dense_tp.build_manifest_tp(cfg, fused=False, lamport=lamport)
    doc["model"] = f"{cfg.name}-ep{n}"
    bufs, ops = doc["buffers"], doc["ops"]
    h, I, E, k, T = cfg.hidden, cfg.moe_intermediate, cfg.experts, cfg.top_k, cfg.max_tokens
    el = E // n
    for name in ("gate_up", "down_proj"):
        ops.pop(name)
    bufs.pop("act")
    ops.update(_moe_ops(cfg, 0, el, ep_group="tp", accumulate=False))
    max_tiles = T * k // C.BM + el
    bufs["moe.logits"] = {"dtype": "f32", "shape": ["tokens", E], "kind": "workspace"}
    bufs["moe.ids"] = {"dtype": "i32", "shape": ["tokens", k], "kind": "workspace"}
    bufs["moe.w"] = {"dtype": "f32", "shape": ["tokens", k], "kind": "workspace"}
    bufs["moe.perm"] = {"dtype": "i32", "shape": ["tokens", k], "kind": "workspace"}
    bufs["moe.offsets"] = {"dtype": "i32", "shape": [el + 1], "kind": "workspace"}
    bufs["moe.tiles"] = {"dtype": "i32", "shape": [max_tiles, 4], "kind": "workspace"}
    bufs["moe.tile_count"] = {"dtype": "i32", "shape": [1], "kind": "workspace"}
    bufs["moe.rows"] = {"dtype": "i32", "shape": [1], "kind": "workspace"}
    bufs["moe.x"] = {"dtype": "bf16", "shape": ["tokens", k, h], "kind": "workspace"}
    bufs["moe.act"] = {"dtype": "bf16", "shape": ["tokens", k, I], "kind": "workspace"}
    bufs["moe.y"] = {"dtype": "bf16", "shape": ["tokens", k, h], "kind": "workspace"}
    B = lambda name: {"buf": name}
    err = B("error")
    ranked = lambda fmt: {"group": "tp", "tensors": [fmt(r) for r in range(n)]}
    for i in range(cfg.layers):
        p = f"model.layers.{i}.mlp."
        for name in (f"w.l{i}.gu", f"w.l{i}.down"):
            bufs.pop(name)
        bufs[f"w.l{i}.router"] = {"dtype": "bf16", "shape": [E, h], "kind": "weight", "bind": [{"tensor": p + "gate.weight"}]}
        bufs[f"w.l{i}.w1"] = {"dtype": "bf16", "shape": [el, 2 * I, h], "kind": "weight",
                              "bind": [{"tensor": ranked(lambda r, j=j, part=part: p + f"experts.{r * el + j}.{part}_proj.weight")}
                                       for j in range(el) for part in ("gate", "up")]}
        bufs[f"w.l{i}.w2"] = {"dtype": "bf16", "shape": [el, h, I], "kind": "weight",
                              "bind": [{"tensor": ranked(lambda r, j=j: p + f"experts.{r * el + j}.down_proj.weight")} for j in range(el)]}

    def moe_calls(i: int) -> list[dict]:
        l = f"l{i}."
        ent = {"expr": {"mul": ["tokens", k]}}
        return [
            {"op": "moe_router", "label": l + "router", "args": [B("xn"), B(f"w.l{i}.router"), B("moe.logits"), {"var": "tokens"}, err]},
            {"op": "moe_route", "label": l + "route", "args": [B("moe.logits"), B("moe.ids"), B("moe.w"), {"var": "tokens"}]},
            {"op": "moe_plan", "label": l + "plan", "args": [B("moe.ids"), B("moe.perm"), B("moe.offsets"), B("moe.tiles"),
                                                             B("moe.tile_count"), B("moe.rows"), ent, err]},
            {"op": "moe_gather", "label": l + "gather", "args": [B("xn"), B("moe.perm"), B("moe.x"), ent]},
            {"op": "moe_fc1", "label": l + "fc1", "args": [B("moe.x"), B(f"w.l{i}.w1"), B("moe.act"), B("moe.tiles"), B("moe.tile_count"), ent, err]},
            {"op": "moe_fc2", "label": l + "fc2", "args": [B("moe.act"), B(f"w.l{i}.w2"), B("moe.y"), B("moe.tiles"), B("moe.tile_count"), ent, err]},
            {"op": "moe_combine", "label": l + "combine", "args": [B("moe.y"), B("moe.perm"), B("moe.w"), B("part")]},   # this rank's share
        ]

    for prog in ("prefill", "decode"):
        out = []
        for c in doc["programs"][prog]["calls"]:
            lbl = c.get("label", "")
            if lbl.endswith(".gate_up"):
                out += moe_calls(int(lbl[1:lbl.index(".")]))
            elif lbl.endswith(".down"):
                continue
            else:
                out.append(c)
        doc["programs"][prog]["calls"] = out
    mods = list(doc["modules"]) + ["moe"]
    doc["modules"] = C.modules_for([m for m in mods if m != "gemv_bf16"])
    return doc
