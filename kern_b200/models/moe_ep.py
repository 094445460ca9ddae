"""The MoE decoder over a rank group: attention tensor-parallel by heads, experts expert-parallel — rank r keeps experts
[r E/n, (r+1) E/n) and computes their share of every token of the replicated batch; the shares meet in the same fused
all-reduce + residual + RMSNorm that closes the attention block. No all-to-all: at decode sizes the token rows are small
next to the expert weights, so every rank routes every token and runs only its own experts.
Reference shape: docs/roadmap.md:13-16 (EP decode as gather, local experts, reduce).
"""
from __future__ import annotations

import dataclasses

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


# ---- expert parallel over sharded tokens: every rank runs its own sequences (attention data-parallel), experts by ranges ----

EP_WIDE_FROM = 192      # rows of this rank from which the routed GEMMs take 256-wide tiles


def ep_fused_buffers(world: int, rows_max: int, hidden: int, inter: int, e_n: int, k: int, x: str, group: str = "ep") -> dict:
    """Buffers of the fused dispatch / combine kernels (`moe.cu`, `kern_ep_*`). `x`: the name of the activation buffer
    the experts read (exported here, with its peer table `<x>_peers`); `rows_max`: tokens per rank."""
    T = rows_max * world
    max_tiles = T * k // C.BM + e_n
    max_rows = max_tiles * C.BM                  # every expert's rows start on a 128-row boundary
    buf = lambda dt, shape, kind="workspace", **kw: {"dtype": dt, "shape": shape, "kind": kind, **kw}
    peer = lambda of: {"dtype": "u64", "shape": [world], "kind": "peer", "of": of, "group": group}
    return {
        x + "_peers": peer(x),
        "ep.ids_all": buf("i32", [T, k], "carry", export=True), "ep.ids_peers": peer("ep.ids_all"),
        "ep.ready": buf("u32", [world], "carry", export=True), "ep.ready_peers": peer("ep.ready"),
        "ep.pub_epoch": buf("u32", [1], "carry"),
        "ep.ret": buf("bf16", [rows_max, k, hidden], "carry", export=True), "ep.ret_peers": peer("ep.ret"),
        "ep.done": buf("u32", [world], "carry", export=True), "ep.done_peers": peer("ep.done"),
        "ep.state": buf("u32", [2], "carry"), "ep.blocks": buf("u32", [max_tiles], "carry"),
        "ep.cta_epochs": buf("u32", [C.SMS], "carry"),
        "ep.perm": buf("i32", [T, k]), "ep.offsets": buf("i32", [e_n + 1]), "ep.tiles": buf("i32", [max_tiles, 4]),
        "ep.tile_count": buf("i32", [1]), "ep.n_rows": buf("i32", [1]), "ep.src_tok": buf("i32", [max_rows]),
        "ep.row_choice": buf("i32", [max_rows]),
        "ep.xp": buf("bf16", [max_rows, hidden], "carry"), "ep.act": buf("bf16", [max_rows, inter]),
    }


def ep_fused_ops(world: int, rows_max: int, hidden: int, inter: int, e_n: int, k: int, rows_var: str, group: str = "ep",
                 accumulate: bool = False, timeout_ns: int = 2_000_000_000, bn: int | None = None) -> dict:
    """The five ops of a fused expert-parallel layer. Interfaces:
    ep_publish [ids, ids_peers, ready_peers, pub_epoch, rows];
    ep_plan [ids_all, perm, offsets, tiles, tile_count, n_rows, src_tok, row_choice, ready, pub_epoch, err];
    ep_fc1 [xp, w1, act, tiles, tile_count, x_peers, src_tok, blocks, cta_epochs, err];
    ep_fc2 [act, w2, tiles, tile_count, ret_peers, src_tok, row_choice, state, done_peers, err];
    ep_finalize [ret, w, out, done, state, err] (`accumulate`: out += the experts' weighted sum, else out = it)."""
    T = rows_max * world
    max_tiles = T * k // C.BM + e_n
    max_rows = max_tiles * C.BM
    L = lambda module, entry, block, grid, lp, args, **kw: {"module": module, "entry": entry, "block": block, "grid": grid,
                                                            "params": lp, "args": args, **kw}
    P = lambda i: {"param": i}
    rank = {"rank": group}
    ops = {}
    ops["ep_publish"] = {"params": ["in buffer<i32>", "in buffer<u64>", "in buffer<u64>", "inout buffer<u32>", "i32"],
                         "impl": {"launches": [L(
        "moe", "kern_ep_publish", [1024, 1, 1], [1, 1, 1],
        ["in buffer<i32>", "in buffer<u64>", "in buffer<u64>", "inout buffer<u32>", "i32", "i32", "i32", "i32", "i32"],
        [P(0), P(1), P(2), P(3), P(4), {"i32": rows_max}, {"i32": k}, rank, {"i32": world}])]}}
    # the table and flag words the peers write into are `inout` here: their writers are other ranks' kernels
    ops["ep_plan"] = {"params": ["inout buffer<i32>", "out buffer<i32>", "out buffer<i32>", "out buffer<i32>", "out buffer<i32>",
                                 "out buffer<i32>", "out buffer<i32>", "out buffer<i32>", "inout buffer<u32>", "in buffer<u32>",
                                 "out buffer<i32>"], "impl": {"launches": [L(
        "moe", "kern_moe_plan_ep", [1024, 1, 1], [1, 1, 1],
        ["inout buffer<i32>", "out buffer<i32>", "out buffer<i32>", "out buffer<i32>", "out buffer<i32>", "out buffer<i32>",
         "out buffer<i32>", "out buffer<i32>", "inout buffer<u32>", "in buffer<u32>"] + ["i32"] * 6 +
        ["out buffer<i32>", "i32", "i32", "i64"],
        [P(i) for i in range(10)] + [{"i32": T * k}, {"i32": k}, {"i32": e_n}, {"i32": C.BM}, {"i32": max_tiles}, {"i32": max_rows},
                                     P(10), rank, {"i32": world}, {"i64": timeout_ns}], shared_mem=2 * e_n * 4)]}}

    def maps(kk, n, swiglu, bn):
        a_map = {"pack": {"size": 128, "fields": [{"at": 0, "tensormap": {
            "param": 0, "dtype": "bf16", "dims": [kk, 0], "strides": [kk * 2], "box": [C.BK, C.BM], "swizzle": 128, "l2_promotion": 256}}]}}
        b_map = {"pack": {"size": 128, "fields": [{"at": 0, "tensormap": {
            "param": 1, "dtype": "bf16", "dims": [kk, n, e_n], "strides": [kk * 2, n * kk * 2],
            "box": [C.BK, bn // 2 if swiglu else bn, 1], "swizzle": 128, "l2_promotion": 256}}]}}
        return a_map, b_map

    # 128-wide tiles keep every SM streaming expert weights at decode sizes; 256-wide tiles are the faster tensor-core
    # shape once every expert has several row tiles (measured at 2 ranks, hidden 7168 / intermediate 2048: 758 against
    # 1002 us per layer at 1024 tokens per rank). `bn` fixes one width; None picks by this rank's row count.
    def widths(n: int) -> list[tuple[int, dict | None]]:
        small = 128 if n >= 128 else 64
        if bn is not None:
            return [(min(bn, small) if bn < 256 or n < 256 else 256, None)]
        if n < 256 or rows_max <= EP_WIDE_FROM:
            return [(small, None)]
        return [(small, {"var": rows_var, "max": EP_WIDE_FROM}), (256, {"var": rows_var, "min": EP_WIDE_FROM + 1})]

    def with_when(launch: dict, when: dict | None) -> dict:
        if when is not None:
            launch["when"] = when
        return launch

    fc1 = []
    for bn1, when in widths(2 * inter):
        a1, b1 = maps(hidden, 2 * inter, True, bn1)
        fc1.append(with_when(L(
            "moe", f"kern_ep_fc1_bf16_swiglu_n{bn1}", [320, 1, 1], [C.SMS, 1, 1],
            ["bytes<128>", "bytes<128>", "out buffer<bf16>", "in buffer<i32>", "in buffer<i32>", "i32", "i32", "i32", "i32",
             "out buffer<i32>", "in buffer<u64>", "inout buffer<bf16>", "in buffer<i32>", "inout buffer<u32>", "inout buffer<u32>",
             "i32", "i32", "i32", "i32"],
            [a1, b1, P(2), P(3), P(4), {"i32": max_rows}, {"i32": 2 * inter}, {"i32": hidden}, {"i32": inter}, P(9), P(5), P(0), P(6),
             P(7), P(8), {"i32": rows_max}, {"i32": max_tiles}, rank, {"i32": world}], shared_mem=C.gemm_smem(bn1)), when))
    ops["ep_fc1"] = {"params": ["inout buffer<bf16>", "in buffer<bf16>", "out buffer<bf16>", "in buffer<i32>", "in buffer<i32>",
                                "in buffer<u64>", "in buffer<i32>", "inout buffer<u32>", "inout buffer<u32>", "out buffer<i32>"],
                     "impl": {"launches": fc1}}
    fc2 = []
    for bn2, when in widths(hidden):
        a2, b2 = maps(inter, hidden, False, bn2)
        fc2.append(with_when(L(
            "moe", f"kern_ep_fc2_bf16_combine_n{bn2}", [192, 1, 1], [C.SMS, 1, 1],
            ["bytes<128>", "bytes<128>", "in buffer<i32>", "in buffer<i32>", "i32", "i32", "i32", "out buffer<i32>", "in buffer<u64>",
             "in buffer<i32>", "in buffer<i32>", "inout buffer<u32>", "in buffer<u64>", "i32", "i32", "i32", "i32"],
            [a2, b2, P(2), P(3), {"i32": max_rows}, {"i32": hidden}, {"i32": inter}, P(9), P(4), P(5), P(6), P(7), P(8),
             {"i32": rows_max}, {"i32": k}, rank, {"i32": world}],
            shared_mem=C.gemm_smem(bn2) + 20480), when))     # + the epilogue's row staging
    ops["ep_fc2"] = {"params": ["in buffer<bf16>", "in buffer<bf16>", "in buffer<i32>", "in buffer<i32>", "in buffer<u64>",
                                "in buffer<i32>", "in buffer<i32>", "inout buffer<u32>", "in buffer<u64>", "out buffer<i32>"],
                     "impl": {"launches": fc2}}
    odir = "inout" if accumulate else "out"
    ops["ep_finalize"] = {"params": ["inout buffer<bf16>", "in buffer<f32>", f"{odir} buffer<bf16>", "inout buffer<u32>",
                                     "in buffer<u32>", "out buffer<i32>"], "impl": {"launches": [L(
        "moe", "kern_ep_finalize", [128, 1, 1], [rows_var, 1, 1],
        ["inout buffer<bf16>", "in buffer<f32>", f"{odir} buffer<bf16>", "i64", "inout buffer<u32>", "in buffer<u32>",
         "out buffer<i32>", "i32", "i32", "i32", "i32", "i64", "i32"],
        [P(0), P(1), P(2), {"i64": 0}, P(3), P(4), P(5), {"i32": C.I32_MAX}, {"i32": k}, {"i32": hidden}, {"i32": world},
         {"i64": timeout_ns}, {"i32": int(accumulate)}])]}}
    return ops


def mx_smem(bn: int) -> int:
    """Shared memory of a block-scaled GEMM CTA (gemm_mx.cu::MxCfg)."""
    stages = 4 if bn == 256 else 6
    return 1024 + stages * (128 * 128 + bn * 128 + (2048 if bn == 256 else 1024)) + 256


def ep_fused_buffers_mx(world: int, rows_max: int, hidden: int, inter: int, e_n: int, k: int, group: str = "ep") -> dict:
    """Buffers of the block-scaled form of the fused layer: the home rank's quantised rows and row-major scales are what
    the peers pull (exported), the expert-sorted operands are e4m3 bytes with scale atoms."""
    from ..ops.gemm_mx import atom_bytes

    assert hidden % 128 == 0 and inter % 128 == 0, "block-scaled experts need hidden and intermediate multiples of 128"
    bufs = ep_fused_buffers(world, rows_max, hidden, inter, e_n, k, "ep.q8", group)
    max_rows = bufs["ep.src_tok"]["shape"][0]
    buf = lambda dt, shape, kind="workspace", **kw: {"dtype": dt, "shape": shape, "kind": kind, **kw}
    peer = lambda of: {"dtype": "u64", "shape": [world], "kind": "peer", "of": of, "group": group}
    bufs.update({
        "ep.q8": buf("u8", [rows_max, hidden], "carry", export=True),
        "ep.sf8": buf("u8", [rows_max, hidden // 32], "carry", export=True), "ep.sf8_peers": peer("ep.sf8"),
        "ep.xp": buf("u8", [max_rows, hidden], "carry"), "ep.sfp": buf("u8", [atom_bytes(max_rows, hidden)], "carry"),
        "ep.act": buf("u8", [max_rows, inter]), "ep.sfact": buf("u8", [atom_bytes(max_rows, inter)]),
    })
    return bufs


def ep_fused_ops_mx(world: int, rows_max: int, hidden: int, inter: int, e_n: int, k: int, rows_var: str, group: str = "ep",
                    accumulate: bool = False, timeout_ns: int = 2_000_000_000, bn: int | None = None) -> dict:
    """The fused layer with MXFP4 expert weights and MXFP8 activations (gemm_mx.cu, the `kern_ep_*_mxfp8_mxfp4_*`
    entries): publish, plan and finalize are the bf16 form's; the home rank quantises its rows once (`ep_quant`), FC1
    pulls e4m3 rows and scale words from the home ranks, FC2 stores bf16 rows into the home ranks' slots. Interfaces:
    ep_quant [x, q8, sf8, rows];
    ep_fc1 [xp, w1, act, tiles, tile_count, q8_peers, src_tok, blocks, cta_epochs, err, sfp, sf1, sfact, sf8_peers];
    ep_fc2 [act, w2, tiles, tile_count, ret_peers, src_tok, row_choice, state, done_peers, err, sfact, sf2]."""
    from ..ops.gemm_mx import atom_bytes

    ops = ep_fused_ops(world, rows_max, hidden, inter, e_n, k, rows_var, group, accumulate, timeout_ns, bn)
    T = rows_max * world
    max_tiles = T * k // C.BM + e_n
    max_rows = max_tiles * C.BM
    L = lambda module, entry, block, grid, lp, args, **kw: {"module": module, "entry": entry, "block": block, "grid": grid,
                                                            "params": lp, "args": args, **kw}
    P = lambda i: {"param": i}
    rank = {"rank": group}
    ops["ep_quant"] = {"params": ["in buffer<bf16>", "out buffer<u8>", "out buffer<u8>", "i32"], "impl": {"launches": [L(
        "gemm_mx", "kern_quant_mxfp8_rows", [128, 1, 1], [rows_var, 1, 1],
        ["in buffer<bf16>", "out buffer<u8>", "out buffer<u8>", "i32", "i32", "i32"],
        [P(0), P(1), P(2), P(3), {"i32": hidden}, {"i32": hidden}])]}}

    def maps(kk, n, bn_):
        a_map = {"pack": {"size": 128, "fields": [{"at": 0, "tensormap": {
            "param": 0, "dtype": "u8", "dims": [kk, 0], "strides": [kk], "box": [128, C.BM], "swizzle": 128, "l2_promotion": 256}}]}}
        b_map = {"pack": {"size": 128, "fields": [{"at": 0, "tensormap": {
            "param": 1, "dtype": "u4", "dims": [kk, n, e_n], "strides": [kk // 2, n * kk // 2],
            "box": [128, bn_, 1], "swizzle": 128, "l2_promotion": 256}}]}}
        return a_map, b_map

    def widths(n: int) -> list[tuple[int, dict | None]]:
        if bn is not None:
            return [(256 if bn == 256 and n % 256 == 0 else 128, None)]
        if n % 256 != 0 or rows_max <= EP_WIDE_FROM:
            return [(128, None)]
        return [(128, {"var": rows_var, "max": EP_WIDE_FROM}), (256, {"var": rows_var, "min": EP_WIDE_FROM + 1})]

    def with_when(launch: dict, when: dict | None) -> dict:
        if when is not None:
            launch["when"] = when
        return launch

    fc1 = []
    for bn1, when in widths(2 * inter):
        a1, b1 = maps(hidden, 2 * inter, bn1)
        fc1.append(with_when(L(
            "gemm_mx", f"kern_ep_fc1_mxfp8_mxfp4_swiglu_mxfp8_n{bn1}", [320, 1, 1], [C.SMS, 1, 1],
            ["bytes<128>", "bytes<128>", "inout buffer<u8>", "in buffer<u8>", "out buffer<u8>", "i32", "i32", "i32", "i32",
             "out buffer<i32>", "in buffer<i32>", "in buffer<i32>", "i64", "out buffer<u8>", "in buffer<u64>", "in buffer<u64>",
             "inout buffer<u8>", "in buffer<i32>", "inout buffer<u32>", "inout buffer<u32>", "i32", "i32", "i32"],
            [a1, b1, P(10), P(11), P(2), {"i32": max_rows}, {"i32": 2 * inter}, {"i32": hidden}, {"i32": inter}, P(9), P(3), P(4),
             {"i64": atom_bytes(2 * inter, hidden)}, P(12), P(5), P(13), P(0), P(6), P(7), P(8), {"i32": rows_max},
             {"i32": max_tiles}, {"i32": world}], shared_mem=mx_smem(bn1)), when))
    ops["ep_fc1"] = {"params": ["inout buffer<u8>", "in buffer<u8>", "out buffer<u8>", "in buffer<i32>", "in buffer<i32>",
                                "in buffer<u64>", "in buffer<i32>", "inout buffer<u32>", "inout buffer<u32>", "out buffer<i32>",
                                "inout buffer<u8>", "in buffer<u8>", "out buffer<u8>", "in buffer<u64>"],
                     "impl": {"launches": fc1}}
    fc2 = []
    for bn2, when in widths(hidden):
        a2, b2 = maps(inter, hidden, bn2)
        fc2.append(with_when(L(
            "gemm_mx", f"kern_ep_fc2_mxfp8_mxfp4_combine_n{bn2}", [192, 1, 1], [C.SMS, 1, 1],
            ["bytes<128>", "bytes<128>", "in buffer<u8>", "in buffer<u8>", "i32", "i32", "i32", "out buffer<i32>", "in buffer<i32>",
             "in buffer<i32>", "i64", "in buffer<u64>", "in buffer<i32>", "in buffer<i32>", "inout buffer<u32>", "in buffer<u64>",
             "i32", "i32", "i32", "i32"],
            [a2, b2, P(10), P(11), {"i32": max_rows}, {"i32": hidden}, {"i32": inter}, P(9), P(2), P(3),
             {"i64": atom_bytes(hidden, inter)}, P(4), P(5), P(6), P(7), P(8), {"i32": rows_max}, {"i32": k}, rank, {"i32": world}],
            shared_mem=mx_smem(bn2) + 20480), when))     # + the epilogue's row staging
    ops["ep_fc2"] = {"params": ["in buffer<u8>", "in buffer<u8>", "in buffer<i32>", "in buffer<i32>", "in buffer<u64>",
                                "in buffer<i32>", "in buffer<i32>", "inout buffer<u32>", "in buffer<u64>", "out buffer<i32>",
                                "in buffer<u8>", "in buffer<u8>"],
                     "impl": {"launches": fc2}}
    return ops


def ep_fused_calls(ids: str, w: str, x: str, w1: str, w2: str, out: str, rows_var: str, label: str = "",
                   mx: tuple[str, str] | None = None) -> list[dict]:
    """The five calls of one fused layer: routing of this rank's rows in `ids` / `w`, activations in the exported `x`,
    this rank's expert weights `w1` / `w2`, the experts' weighted sum into `out`."""
    B = lambda n: {"buf": n}
    err = B("error")
    if mx is not None:
        # `mx`: the scale atoms of w1 and of w2. The rows are quantised before the publish: a peer that has seen this
        # rank's ready word may pull them.
        sf1, sf2 = mx
        calls = ep_fused_calls(ids, w, "ep.q8", w1, w2, out, rows_var, label)
        calls.insert(0, {"op": "ep_quant", "label": label + "quant", "args": [B(x), B("ep.q8"), B("ep.sf8"), {"var": rows_var}]})
        calls[3]["args"] += [B("ep.sfp"), B(sf1), B("ep.sfact"), B("ep.sf8_peers")]
        calls[4]["args"] += [B("ep.sfact"), B(sf2)]
        return calls
    return [
        {"op": "ep_publish", "label": label + "publish", "args": [B(ids), B("ep.ids_peers"), B("ep.ready_peers"), B("ep.pub_epoch"),
                                                                  {"var": rows_var}]},
        {"op": "ep_plan", "label": label + "plan", "args": [B("ep.ids_all"), B("ep.perm"), B("ep.offsets"), B("ep.tiles"),
                                                            B("ep.tile_count"), B("ep.n_rows"), B("ep.src_tok"), B("ep.row_choice"),
                                                            B("ep.ready"), B("ep.pub_epoch"), err]},
        {"op": "ep_fc1", "label": label + "fc1", "args": [B("ep.xp"), B(w1), B("ep.act"), B("ep.tiles"), B("ep.tile_count"),
                                                          B(x + "_peers"), B("ep.src_tok"), B("ep.blocks"), B("ep.cta_epochs"), err]},
        {"op": "ep_fc2", "label": label + "fc2", "args": [B("ep.act"), B(w2), B("ep.tiles"), B("ep.tile_count"), B("ep.ret_peers"),
                                                          B("ep.src_tok"), B("ep.row_choice"), B("ep.state"), B("ep.done_peers"), err]},
        {"op": "ep_finalize", "label": label + "finalize", "args": [B("ep.ret"), B(w), B(out), B("ep.done"), B("ep.state"), err]},
    ]


def build_manifest_ep_sharded(cfg: MoeConfig, world: int) -> dict:
    """The MoE decoder with tokens sharded over an expert-parallel group: every rank serves its own sequences (attention,
    norms, router and head are whole on every rank: data parallel), rank r keeps experts [r E/n, (r+1) E/n), and every
    routed layer is the fused pair of kernels — dispatch inside FC1, combine inside FC2. The ranks step in lockstep: a
    layer's kernels wait for every rank's publish and done words. `cfg.max_tokens` is the rows per rank.
    `cfg.mx_experts`: MXFP4 expert weights and MXFP8 expert activations (the block-scaled pair of `gemm_mx.cu`)."""
    from . import moe

    assert world >= 1 and cfg.experts % world == 0
    doc = moe.build_manifest(dataclasses.replace(cfg, mx_experts=False) if getattr(cfg, "mx_experts", False) else cfg)
    doc["model"] = f"{cfg.name}-ep{world}-sharded"
    doc.setdefault("topology", {}).setdefault("groups", {})["ep"] = world
    bufs, ops = doc["buffers"], doc["ops"]
    h, I, E, k, T = cfg.hidden, cfg.moe_intermediate, cfg.experts, cfg.top_k, cfg.max_tokens
    el = E // world
    for name in ("moe_plan", "moe_gather", "moe_fc1", "moe_fc2", "moe_combine"):
        ops.pop(name)
    for name in ("moe.perm", "moe.offsets", "moe.tiles", "moe.tile_count", "moe.rows", "moe.x", "moe.act", "moe.y"):
        bufs.pop(name)
    mx = bool(getattr(cfg, "mx_experts", False))
    if mx:
        from ..ops.gemm_mx import atom_bytes

        bufs.update(ep_fused_buffers_mx(world, T, h, I, el, k))
        ops.update(ep_fused_ops_mx(world, T, h, I, el, k, "tokens", accumulate=True))
    else:
        bufs["xn"]["export"] = True
        bufs.update(ep_fused_buffers(world, T, h, I, el, k, "xn"))
        ops.update(ep_fused_ops(world, T, h, I, el, k, "tokens", accumulate=True))
    ranked = lambda fmt: {"group": "ep", "tensors": [fmt(r) for r in range(world)]}
    mine = {"group": "ep", "ranges": [[r * el, (r + 1) * el] for r in range(world)]}
    for i in range(cfg.layers):
        p = f"model.layers.{i}.mlp."
        if mx:
            # this rank's range of the stacked block-scaled tensors (`moe.mx_checkpoint`)
            for name, shape, tensor in ((f"w.l{i}.w1", [el, 2 * I, h // 2], "experts.w1_mxfp4"),
                                        (f"w.l{i}.sf1", [el, atom_bytes(2 * I, h)], "experts.w1_scales"),
                                        (f"w.l{i}.w2", [el, h, I // 2], "experts.w2_mxfp4"),
                                        (f"w.l{i}.sf2", [el, atom_bytes(h, I)], "experts.w2_scales")):
                bufs[name] = {"dtype": "u8", "shape": shape, "kind": "weight", "bind": [{"tensor": p + tensor, "rows": mine}]}
            continue
        bufs[f"w.l{i}.w1"] = {"dtype": "bf16", "shape": [el, 2 * I, h], "kind": "weight",
                              "bind": [{"tensor": ranked(lambda r, j=j, part=part: p + f"experts.{r * el + j}.{part}_proj.weight")}
                                       for j in range(el) for part in ("gate", "up")]}
        bufs[f"w.l{i}.w2"] = {"dtype": "bf16", "shape": [el, h, I], "kind": "weight",
                              "bind": [{"tensor": ranked(lambda r, j=j: p + f"experts.{r * el + j}.down_proj.weight")} for j in range(el)]}
    drop = (".plan", ".gather", ".fc1", ".fc2")
    for prog in doc["programs"].values():
        out = []
        for c in prog["calls"]:
            lbl = c.get("label", "")
            if lbl.endswith(drop):
                continue
            if lbl.endswith(".combine"):
                i = int(lbl[1:lbl.index(".")])
                out += ep_fused_calls("moe.ids", "moe.w", "xn", f"w.l{i}.w1", f"w.l{i}.w2", "x", "tokens", label=f"l{i}.ep_",
                                      mx=(f"w.l{i}.sf1", f"w.l{i}.sf2") if mx else None)
            else:
                out.append(c)
        prog["calls"] = out
    return C.ensure_modules(doc)
