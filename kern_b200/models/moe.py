"""Mixture-of-experts decoder (GQA attention + routed SwiGLU experts, the Qwen3-MoE / DeepSeek-style MLP): manifest
generator, synthetic checkpoint, oracle, and the CPU statements of the MoE kernels.

A layer's MLP is: router GEMM (f32 logits) -> top-k routing -> plan (expert-sorted rows + the M-tile table) -> gather
-> routed GEMM with SwiGLU epilogue -> routed GEMM -> weighted combine accumulated into the residual. Under expert
parallelism a rank keeps experts [e_lo, e_hi) and computes its share of every token; the shares meet in the
tensor-parallel all-reduce.
Reference shape: the routed batched GEMMs and routing tables of kernel_index/trtllm_bmm_*.toml, tools/kernels-src/topk_row.cu.
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass

import torch
import torch.nn.functional as F

from . import common as C
from . import dense


@dataclass
class MoeConfig(dense.DenseConfig):
    experts: int = 128
    top_k: int = 8
    moe_intermediate: int = 768
    scoring: str = "softmax"          # softmax | sigmoid
    routed_scale: float = 1.0
    mx_experts: bool = False          # expert weights MXFP4 (e2m1 + UE8M0 per 32), expert activations MXFP8


TOY_MOE = MoeConfig(name="toy-moe", vocab=256, hidden=64, layers=2, heads=4, kv_heads=2, head_dim=16, intermediate=128,
                    rope_theta=10000.0, page_size=16, max_tokens=64, max_seqs=4, max_context=64, experts=8, top_k=2,
                    moe_intermediate=32)
TINY_MOE = MoeConfig(name="tiny-moe", vocab=512, hidden=256, layers=2, heads=4, kv_heads=2, head_dim=64, intermediate=512,
                     rope_theta=10000.0, page_size=16, max_tokens=256, max_seqs=8, max_context=256, experts=16, top_k=4,
                     moe_intermediate=128)
MOE_30B = MoeConfig(name="moe-30b-a3b", vocab=151936, hidden=2048, layers=48, heads=32, kv_heads=4, head_dim=128,
                    intermediate=6144, qk_norm=True, experts=128, top_k=8, moe_intermediate=768)


def weight_names(cfg: MoeConfig) -> dict[str, tuple[int, ...]]:
    out = {n: s for n, s in dense.weight_names(cfg).items() if ".mlp." not in n}
    h, I = cfg.hidden, cfg.moe_intermediate
    for i in range(cfg.layers):
        p = f"model.layers.{i}.mlp."
        out[p + "gate.weight"] = (cfg.experts, h)
        for e in range(cfg.experts):
            out[p + f"experts.{e}.gate_proj.weight"] = (I, h)
            out[p + f"experts.{e}.up_proj.weight"] = (I, h)
            out[p + f"experts.{e}.down_proj.weight"] = (h, I)
    return out


def random_weights(cfg: MoeConfig, seed: int = 0, device: str = "cpu", std: float = 0.02) -> dict[str, torch.Tensor]:
    g = torch.Generator(device=device).manual_seed(seed)
    out = {}
    for name, shape in weight_names(cfg).items():
        if name.endswith("norm.weight"):
            t = 1.0 + 0.1 * torch.randn(shape, generator=g, device=device)
        elif name.endswith("mlp.gate.weight"):
            t = 10 * std * torch.randn(shape, generator=g, device=device)       # a router with opinions
        else:
            t = std * torch.randn(shape, generator=g, device=device)
        out[name] = t.to(torch.bfloat16)
    return out


def load_random_weights(rt, cfg: MoeConfig, seed: int = 0, std: float = 0.02, skip=None) -> None:
    """`skip(name)`: checkpoint tensors the caller fills itself (buffers that bind only such tensors are left alone)."""
    shapes = weight_names(cfg)
    order = {n: i for i, n in enumerate(shapes)}

    def provider(name: str) -> torch.Tensor:
        dev = rt.tensor(next(iter(rt.doc["buffers"]))).device
        g = torch.Generator(device=dev).manual_seed(seed * 1000003 + order[name])
        scale = 1.0 if name.endswith("norm.weight") else (10 * std if name.endswith("mlp.gate.weight") else std)
        t = torch.randn(shapes[name], generator=g, device=dev) * (0.1 if name.endswith("norm.weight") else scale)
        return ((1.0 + t) if name.endswith("norm.weight") else t).to(torch.bfloat16)

    rt.load_tensors(provider, skip=skip)


def _moe_ops(cfg: MoeConfig, e_lo: int, e_n: int, ep_group: str | None = None, accumulate: bool = True) -> dict:
    """`ep_group`: the rank of that group shifts the expert range by e_n per rank (expert parallel). `accumulate`: the
    combine adds into its output (a residual) instead of overwriting it (a partial sum for an all-reduce)."""
    h, I, E, k, T = cfg.hidden, cfg.moe_intermediate, cfg.experts, cfg.top_k, cfg.max_tokens
    max_tiles = T * k // C.BM + e_n
    L = lambda module, entry, block, grid, lp, args, **kw: {"module": module, "entry": entry, "block": block, "grid": grid,
                                                            "params": lp, "args": args, **kw}
    ops = {}
    ops["moe_router"] = C.gemm_op(E, h, epilogue="f32", rows_max=T)
    ops["moe_route"] = {"params": ["in buffer<f32>", "out buffer<i32>", "out buffer<f32>", "i32"], "impl": {"launches": [L(
        "moe", "kern_moe_route_f32", [128, 1, 1], [{"ceil_div": ["tokens", 4]}, 1, 1],
        ["in buffer<f32>", "i64", "out buffer<i32>", "out buffer<f32>", "i32", "i32", "i32", "i32", "i32", "f32", "i32"],
        [{"param": 0}, {"i64": 0}, {"param": 1}, {"param": 2}, {"param": 3}, {"i32": E}, {"i32": k},
         {"i32": 1 if cfg.scoring == "softmax" else 0}, {"i32": 1}, {"f32": cfg.routed_scale}, {"i32": E}])]}}
    # `tokens` bounds the entries through the grid-free loop: the kernel is told tokens * k by the `entries` arg
    ops["moe_plan"] = {"params": ["in buffer<i32>", "out buffer<i32>", "out buffer<i32>", "out buffer<i32>", "out buffer<i32>",
                                  "out buffer<i32>", "i32", "out buffer<i32>"], "impl": {"launches": [L(
        "moe", "kern_moe_plan", [1024, 1, 1], [1, 1, 1],
        ["in buffer<i32>", "out buffer<i32>", "out buffer<i32>", "out buffer<i32>", "out buffer<i32>", "out buffer<i32>", "i32",
         "i32", "i32", "i32", "i32", "out buffer<i32>", "i32", "i32"],
        [{"param": 0}, {"param": 1}, {"param": 2}, {"param": 3}, {"param": 4}, {"param": 5}, {"param": 6}, {"i32": e_lo},
         {"i32": e_lo + e_n}, {"i32": C.BM}, {"i32": max_tiles}, {"param": 7},
         {"rank": ep_group} if ep_group else {"i32": 0}, {"i32": e_n if ep_group else 0}], shared_mem=2 * e_n * 4)]}}
    ops["moe_gather"] = {"params": ["in buffer<bf16>", "in buffer<i32>", "out buffer<bf16>", "i32"], "impl": {"launches": [L(
        "moe", "kern_moe_gather_bf16", [128, 1, 1], [{"mul": ["tokens", k]}, 1, 1],
        ["in buffer<bf16>", "in buffer<i32>", "out buffer<bf16>", "i32", "i32", "i32"],
        [{"param": 0}, {"param": 1}, {"param": 2}, {"param": 3}, {"i32": k}, {"i32": h}])]}}

    def routed(n, kk, epi):
        bn = 128 if n >= 128 else 64
        out_cols = n // 2 if epi == "swiglu" else n
        a_map = {"pack": {"size": 128, "fields": [{"at": 0, "tensormap": {
            "param": 0, "dtype": "bf16", "dims": [kk, 0], "strides": [kk * 2], "box": [C.BK, C.BM], "swizzle": 128, "l2_promotion": 256}}]}}
        b_map = {"pack": {"size": 128, "fields": [{"at": 0, "tensormap": {
            "param": 1, "dtype": "bf16", "dims": [kk, n, e_n], "strides": [kk * 2, n * kk * 2],
            "box": [C.BK, bn // 2 if epi == "swiglu" else bn, 1], "swizzle": 128, "l2_promotion": 256}}]}}
        return {"params": ["in buffer<bf16>", "in buffer<bf16>", "out buffer<bf16>", "in buffer<i32>", "in buffer<i32>", "i32",
                           "out buffer<i32>"], "impl": {"launches": [L(
            "moe", f"kern_moe_gemm_bf16{'_swiglu' if epi == 'swiglu' else ''}_n{bn}", [192, 1, 1], [C.SMS, 1, 1],
            ["bytes<128>", "bytes<128>", "out buffer<bf16>", "in buffer<i32>", "in buffer<i32>", "i32", "i32", "i32", "i32",
             "out buffer<i32>"],
            [a_map, b_map, {"param": 2}, {"param": 3}, {"param": 4}, {"param": 5}, {"i32": n}, {"i32": kk}, {"i32": out_cols},
             {"param": 6}], shared_mem=C.gemm_smem(bn))]}}

    ops["moe_fc1"] = routed(2 * I, h, "swiglu")
    ops["moe_fc2"] = routed(h, I, "store")
    ops["moe_combine"] = {"params": ["in buffer<bf16>", "in buffer<i32>", "in buffer<f32>",
                                     ("inout" if accumulate else "out") + " buffer<bf16>"], "impl": {"launches": [L(
        "moe", "kern_moe_combine_bf16", [128, 1, 1], ["tokens", 1, 1],
        ["in buffer<bf16>", "in buffer<i32>", "in buffer<f32>", "i64", ("inout" if accumulate else "out") + " buffer<bf16>",
         "i32", "i32", "i32", "i32"],
        [{"param": 0}, {"param": 1}, {"param": 2}, {"i64": 0}, {"param": 3}, {"i32": C.I32_MAX}, {"i32": k}, {"i32": h},
         {"i32": int(accumulate)}])]}}
    return ops


def mx_rows_bound(tokens: int, k: int, experts: int) -> int:
    """Rows of the expert-sorted buffers when every expert's rows start on a 128-row boundary."""
    return (-(-tokens * k // C.BM) + experts) * C.BM


def _moe_mx_ops(cfg: MoeConfig, e_n: int) -> dict:
    """The block-scaled form of the routed experts (csrc/kernels/sm100/gemm_mx.cu): aligned plan, gather fused with the
    MXFP8 quantiser, FC1 = MXFP8 x MXFP4 with the SwiGLU + MXFP8 epilogue, FC2 = MXFP8 x MXFP4 -> bf16."""
    from ..ops.gemm_mx import atom_bytes

    h, I, k, T = cfg.hidden, cfg.moe_intermediate, cfg.top_k, cfg.max_tokens
    rows = mx_rows_bound(T, k, e_n)
    L = lambda module, entry, block, grid, lp, args, **kw: {"module": module, "entry": entry, "block": block, "grid": grid,
                                                            "params": lp, "args": args, **kw}
    ops = {}
    ops["moe_gather_q"] = {"params": ["in buffer<bf16>", "in buffer<i32>", "out buffer<u8>", "out buffer<u8>", "i32"], "impl": {"launches": [L(
        "gemm_mx", "kern_moe_gather_quant_mxfp8", [128, 1, 1], [{"mul": ["tokens", k]}, 1, 1],
        ["in buffer<bf16>", "in buffer<i32>", "out buffer<u8>", "out buffer<u8>", "i32", "i32", "i32"],
        [{"param": 0}, {"param": 1}, {"param": 2}, {"param": 3}, {"param": 4}, {"i32": k}, {"i32": h}])]}}

    def routed(n, kk, swiglu):
        bn = 256 if n % 256 == 0 else 128
        a_map = {"pack": {"size": 128, "fields": [{"at": 0, "tensormap": {
            "param": 0, "dtype": "u8", "dims": [kk, 0], "strides": [kk], "box": [128, C.BM], "swizzle": 128, "l2_promotion": 256}}]}}
        b_map = {"pack": {"size": 128, "fields": [{"at": 0, "tensormap": {
            "param": 1, "dtype": "u4", "dims": [kk, n, e_n], "strides": [kk // 2, n * kk // 2],
            "box": [128, bn, 1], "swizzle": 128, "l2_promotion": 256}}]}}
        out_t = "out buffer<u8>" if swiglu else "out buffer<bf16>"
        iface = ["in buffer<u8>", "in buffer<u8>", "in buffer<u8>", "in buffer<u8>", out_t, "in buffer<i32>", "in buffer<i32>",
                 "out buffer<i32>"] + (["out buffer<u8>"] if swiglu else [])
        stages = 4 if bn == 256 else 6
        smem = 1024 + stages * (128 * 128 + bn * 128 + (2048 if bn == 256 else 1024)) + 256
        entry = f"kern_moe_gemm_mxfp8_mxfp4{'_swiglu_mxfp8' if swiglu else ''}_n{bn}"
        return {"params": iface, "impl": {"launches": [L(
            "gemm_mx", entry, [192, 1, 1], [C.SMS, 1, 1],
            ["bytes<128>", "bytes<128>", "in buffer<u8>", "in buffer<u8>", out_t, "i32", "i32", "i32", "i32", "out buffer<i32>",
             "in buffer<i32>", "in buffer<i32>", "i64", "out buffer<u8>" if swiglu else "i64"],
            [a_map, b_map, {"param": 2}, {"param": 3}, {"param": 4}, {"i32": rows}, {"i32": n}, {"i32": kk},
             {"i32": n // 2 if swiglu else n}, {"param": 7}, {"param": 5}, {"param": 6}, {"i64": atom_bytes(n, kk)},
             {"param": 8} if swiglu else {"i64": 0}], shared_mem=smem)]}}

    ops["moe_fc1"] = routed(2 * I, h, True)
    ops["moe_fc2"] = routed(h, I, False)
    return ops


def build_manifest(cfg: MoeConfig) -> dict:
    """The dense decoder's manifest with every layer's MLP replaced by the routed experts."""
    doc = dense.build_manifest(cfg)
    doc["model"] = cfg.name
    return moeify(doc, cfg, ["norm_embed", "gemm_bf16", "attn_prep", "attn_paged", "misc", "sampling", "moe"])


def moeify(doc: dict, cfg, modules: list[str]) -> dict:
    """Replace the dense MLP of every layer of `doc` by routed experts. The document follows the decoder builders'
    naming: calls labelled `l<i>.gate_up` / `l<i>.down`, weights `w.l<i>.gu` / `w.l<i>.down`, rows `xn` -> `x`.
    `cfg` brings hidden, layers, max_tokens, experts, top_k, moe_intermediate, scoring and routed_scale."""
    bufs, ops = doc["buffers"], doc["ops"]
    h, I, E, k, T = cfg.hidden, cfg.moe_intermediate, cfg.experts, cfg.top_k, cfg.max_tokens
    mx = bool(getattr(cfg, "mx_experts", False))
    for name in ("gate_up", "down_proj"):
        ops.pop(name)
    bufs.pop("act")
    ops.update(_moe_ops(cfg, 0, E))
    max_tiles = T * k // C.BM + E
    if mx:
        from ..ops.gemm_mx import atom_bytes

        assert h % 128 == 0 and I % 128 == 0, "block-scaled experts need hidden and intermediate multiples of 128"
        ops.update(_moe_mx_ops(cfg, E))
        ops["moe_plan"]["impl"]["launches"][0]["entry"] = "kern_moe_plan_aligned"
        ops.pop("moe_gather")
        rows = mx_rows_bound(T, k, E)
    bufs["moe.logits"] = {"dtype": "f32", "shape": ["tokens", E], "kind": "workspace"}
    bufs["moe.ids"] = {"dtype": "i32", "shape": ["tokens", k], "kind": "workspace"}
    bufs["moe.w"] = {"dtype": "f32", "shape": ["tokens", k], "kind": "workspace"}
    bufs["moe.perm"] = {"dtype": "i32", "shape": ["tokens", k], "kind": "workspace"}
    bufs["moe.offsets"] = {"dtype": "i32", "shape": [E + 1], "kind": "workspace"}
    bufs["moe.tiles"] = {"dtype": "i32", "shape": [max_tiles, 4], "kind": "workspace"}
    bufs["moe.tile_count"] = {"dtype": "i32", "shape": [1], "kind": "workspace"}
    bufs["moe.rows"] = {"dtype": "i32", "shape": [1], "kind": "workspace"}
    if mx:
        bufs["moe.x"] = {"dtype": "u8", "shape": [rows, h], "kind": "workspace"}
        bufs["moe.sfx"] = {"dtype": "u8", "shape": [atom_bytes(rows, h)], "kind": "workspace"}
        bufs["moe.act"] = {"dtype": "u8", "shape": [rows, I], "kind": "workspace"}
        bufs["moe.sfact"] = {"dtype": "u8", "shape": [atom_bytes(rows, I)], "kind": "workspace"}
        bufs["moe.y"] = {"dtype": "bf16", "shape": [rows, h], "kind": "workspace"}
    else:
        bufs["moe.x"] = {"dtype": "bf16", "shape": ["tokens", k, h], "kind": "workspace"}
        bufs["moe.act"] = {"dtype": "bf16", "shape": ["tokens", k, I], "kind": "workspace"}
        bufs["moe.y"] = {"dtype": "bf16", "shape": ["tokens", k, h], "kind": "workspace"}
    B = lambda n: {"buf": n}
    err = B("error")
    for i in range(cfg.layers):
        p = f"model.layers.{i}.mlp."
        for name in (f"w.l{i}.gu", f"w.l{i}.down"):
            bufs.pop(name)
        bufs[f"w.l{i}.router"] = {"dtype": "bf16", "shape": [E, h], "kind": "weight", "bind": [{"tensor": p + "gate.weight"}]}
        if mx:
            # the packed form of a block-scaled checkpoint: nibbles and scale atoms per layer, experts stacked
            # (`mx_checkpoint` writes it from bf16 expert weights)
            bufs[f"w.l{i}.w1"] = {"dtype": "u8", "shape": [E, 2 * I, h // 2], "kind": "weight", "bind": [{"tensor": p + "experts.w1_mxfp4"}]}
            bufs[f"w.l{i}.sf1"] = {"dtype": "u8", "shape": [E, atom_bytes(2 * I, h)], "kind": "weight", "bind": [{"tensor": p + "experts.w1_scales"}]}
            bufs[f"w.l{i}.w2"] = {"dtype": "u8", "shape": [E, h, I // 2], "kind": "weight", "bind": [{"tensor": p + "experts.w2_mxfp4"}]}
            bufs[f"w.l{i}.sf2"] = {"dtype": "u8", "shape": [E, atom_bytes(h, I)], "kind": "weight", "bind": [{"tensor": p + "experts.w2_scales"}]}
            continue
        bufs[f"w.l{i}.w1"] = {"dtype": "bf16", "shape": [E, 2 * I, h], "kind": "weight",
                              "bind": [{"tensor": p + f"experts.{e}.{n}_proj.weight"} for e in range(E) for n in ("gate", "up")]}
        bufs[f"w.l{i}.w2"] = {"dtype": "bf16", "shape": [E, h, I], "kind": "weight",
                              "bind": [{"tensor": p + f"experts.{e}.down_proj.weight"} for e in range(E)]}

    def moe_calls(i: int) -> list[dict]:
        l = f"l{i}."
        if mx:
            return [
                {"op": "moe_router", "label": l + "router", "args": [B("xn"), B(f"w.l{i}.router"), B("moe.logits"), {"var": "tokens"}, err]},
                {"op": "moe_route", "label": l + "route", "args": [B("moe.logits"), B("moe.ids"), B("moe.w"), {"var": "tokens"}]},
                {"op": "moe_plan", "label": l + "plan", "args": [B("moe.ids"), B("moe.perm"), B("moe.offsets"), B("moe.tiles"),
                                                                 B("moe.tile_count"), B("moe.rows"), {"expr": {"mul": ["tokens", k]}}, err]},
                {"op": "moe_gather_q", "label": l + "gather", "args": [B("xn"), B("moe.perm"), B("moe.x"), B("moe.sfx"),
                                                                       {"expr": {"mul": ["tokens", k]}}]},
                {"op": "moe_fc1", "label": l + "fc1", "args": [B("moe.x"), B(f"w.l{i}.w1"), B("moe.sfx"), B(f"w.l{i}.sf1"), B("moe.act"),
                                                               B("moe.tiles"), B("moe.tile_count"), err, B("moe.sfact")]},
                {"op": "moe_fc2", "label": l + "fc2", "args": [B("moe.act"), B(f"w.l{i}.w2"), B("moe.sfact"), B(f"w.l{i}.sf2"), B("moe.y"),
                                                               B("moe.tiles"), B("moe.tile_count"), err]},
                {"op": "moe_combine", "label": l + "combine", "args": [B("moe.y"), B("moe.perm"), B("moe.w"), B("x")]},
            ]
        return [
            {"op": "moe_router", "label": l + "router", "args": [B("xn"), B(f"w.l{i}.router"), B("moe.logits"), {"var": "tokens"}, err]},
            {"op": "moe_route", "label": l + "route", "args": [B("moe.logits"), B("moe.ids"), B("moe.w"), {"var": "tokens"}]},
            {"op": "moe_plan", "label": l + "plan", "args": [B("moe.ids"), B("moe.perm"), B("moe.offsets"), B("moe.tiles"),
                                                             B("moe.tile_count"), B("moe.rows"), {"expr": {"mul": ["tokens", k]}}, err]},
            {"op": "moe_gather", "label": l + "gather", "args": [B("xn"), B("moe.perm"), B("moe.x"), {"expr": {"mul": ["tokens", k]}}]},
            {"op": "moe_fc1", "label": l + "fc1", "args": [B("moe.x"), B(f"w.l{i}.w1"), B("moe.act"), B("moe.tiles"), B("moe.tile_count"),
                                                           {"expr": {"mul": ["tokens", k]}}, err]},
            {"op": "moe_fc2", "label": l + "fc2", "args": [B("moe.act"), B(f"w.l{i}.w2"), B("moe.y"), B("moe.tiles"), B("moe.tile_count"),
                                                           {"expr": {"mul": ["tokens", k]}}, err]},
            {"op": "moe_combine", "label": l + "combine", "args": [B("moe.y"), B("moe.perm"), B("moe.w"), B("x")]},
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
    doc["modules"] = C.modules_for(list(modules) + (["gemm_mx"] if mx else []))
    return C.ensure_modules(doc)


def mx_checkpoint(cfg: MoeConfig, weights: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
    """A bf16 checkpoint -> the block-scaled one a `mx_experts` manifest binds: every layer's expert weights quantised to
    MXFP4 (gate/up rows interleaved in groups of 64, nibbles packed, scale atoms per expert), everything else kept."""
    from ..ops import moe as M

    out = {k: v for k, v in weights.items() if ".mlp.experts." not in k}
    for i in range(cfg.layers):
        p = f"model.layers.{i}.mlp.experts."
        w1 = torch.stack([torch.cat([weights[p + f"{e}.gate_proj.weight"], weights[p + f"{e}.up_proj.weight"]], 0) for e in range(cfg.experts)])
        w2 = torch.stack([weights[p + f"{e}.down_proj.weight"] for e in range(cfg.experts)])
        q1, s1, q2, s2 = M.prepare_expert_weights_mx(w1, w2)
        out[p + "w1_mxfp4"], out[p + "w1_scales"], out[p + "w2_mxfp4"], out[p + "w2_scales"] = q1, s1, q2, s2
    return out


class MoeOracle(dense.DenseOracle):
    """The dense oracle with the routed MLP (fp32)."""

    def mlp(self, i: int, xn: torch.Tensor) -> torch.Tensor:
        cfg, w, p = self.cfg, self.w, f"model.layers.{i}.mlp."
        logits = xn.float() @ w[p + "gate.weight"].float().t()
        s = torch.softmax(logits, -1) if cfg.scoring == "softmax" else torch.sigmoid(logits)
        wt, ids = torch.topk(s, cfg.top_k, dim=-1)
        wt = wt / wt.sum(-1, keepdim=True) * cfg.routed_scale
        out = torch.zeros_like(xn, dtype=torch.float32)
        for e in range(cfg.experts):
            tok, j = torch.nonzero(ids == e, as_tuple=True)
            if tok.numel() == 0:
                continue
            x = xn[tok].float()
            a = F.silu(x @ w[p + f"experts.{e}.gate_proj.weight"].float().t()) * (x @ w[p + f"experts.{e}.up_proj.weight"].float().t())
            out.index_add_(0, tok, (a @ w[p + f"experts.{e}.down_proj.weight"].float().t()) * wt[tok, j][:, None])
        return out.to(self.dtype)


# ---- CPU statements ------------------------------------------------------------------------------------
def _register_cpu() -> None:
    from .. import cpu
    from ..ops import moe as M

    def route(g, logits, bias, ids, wts, tokens, experts, k, mode, renorm, scale, ld):
        t = tokens
        i, w = M.route_reference(logits[: t * ld].view(t, ld)[:, :experts], k, bias if isinstance(bias, torch.Tensor) else None,
                                 "softmax" if mode == 1 else "sigmoid", bool(renorm), scale)
        ids[: t * k] = i.reshape(-1)
        wts[: t * k] = w.reshape(-1).float()

    def plan(g, ids, perm, offsets, tiles, tile_count, rows_out, entries, e_lo, e_hi, bm, max_tiles, err, rank, per_rank):
        e_lo, e_hi = e_lo + rank * per_rank, e_hi + rank * per_rank
        flat = ids[:entries]
        at, nt = 0, 0
        tl = tiles.view(-1, 4)
        for e in range(e_lo, e_hi):
            mine = torch.nonzero(flat == e).flatten()
            offsets[e - e_lo] = at
            perm[mine] = torch.arange(at, at + mine.numel(), dtype=perm.dtype)
            for m0 in range(0, mine.numel(), bm):
                tl[nt] = torch.tensor([e - e_lo, at + m0, min(bm, mine.numel() - m0), 0], dtype=tl.dtype)
                nt += 1
            at += mine.numel()
        offsets[e_hi - e_lo] = at
        perm[:entries][(flat < e_lo) | (flat >= e_hi)] = -1
        tile_count[0], rows_out[0] = nt, at

    def gather(g, x, perm, xp, entries, k, hidden):
        for i in range(entries):
            r = int(perm[i])
            if r >= 0:
                xp[r * hidden:(r + 1) * hidden] = x[(i // k) * hidden:(i // k + 1) * hidden]

    def gemm(epi):
        def run(g, a, w, c, tiles, tile_count, M_, N, K, ldc, err):
            A = a._row_stride if hasattr(a, "_row_stride") else K
            tl = tiles.view(-1, 4)
            wv = w.view(torch.bfloat16) if w.dtype != torch.bfloat16 else w
            for t in range(int(tile_count[0])):
                e, r0, nr, _ = (int(v) for v in tl[t])
                rows = cpu._f(a[r0 * K:(r0 + nr) * K].view(nr, K))
                We = cpu._f(wv[e * N * K:(e + 1) * N * K].view(N, K))
                acc = rows @ We.t()
                if epi == "swiglu":
                    acc = F.silu(acc[:, : N // 2]) * acc[:, N // 2:]
                c[r0 * ldc:(r0 + nr) * ldc] = acc.to(torch.bfloat16).reshape(-1)
        return run

    def combine(g, y, perm, wts, shared, out, tokens, k, hidden, accumulate):
        for t in range(g[0]):
            acc = cpu._f(out[t * hidden:(t + 1) * hidden]).clone() if accumulate else torch.zeros(hidden)
            for j in range(k):
                r = int(perm[t * k + j])
                if r >= 0:
                    acc += float(wts[t * k + j]) * cpu._f(y[r * hidden:(r + 1) * hidden])
            out[t * hidden:(t + 1) * hidden] = acc.to(out.dtype)

    def plan_aligned(g, ids, perm, offsets, tiles, tile_count, rows_out, entries, e_lo, e_hi, bm, max_tiles, err, rank, per_rank):
        e_lo, e_hi = e_lo + rank * per_rank, e_hi + rank * per_rank
        flat = ids[:entries]
        at, nt = 0, 0
        tl = tiles.view(-1, 4)
        for e in range(e_lo, e_hi):
            mine = torch.nonzero(flat == e).flatten()
            if mine.numel():
                at = -(-at // bm) * bm
            offsets[e - e_lo] = at
            perm[mine] = torch.arange(at, at + mine.numel(), dtype=perm.dtype)
            for m0 in range(0, mine.numel(), bm):
                tl[nt] = torch.tensor([e - e_lo, at + m0, min(bm, mine.numel() - m0), 0], dtype=tl.dtype)
                nt += 1
            at += mine.numel()
        offsets[e_hi - e_lo] = at
        perm[:entries][(flat < e_lo) | (flat >= e_hi)] = -1
        tile_count[0], rows_out[0] = nt, at

    def gather_q(g, x, perm, q, sf, entries, k, hidden):
        from ..ops import gemm_mx as G

        rows_bound = q.numel() // hidden
        sfm = G.atoms_to_sf(sf, rows_bound, hidden).clone()
        qv = q.view(rows_bound, hidden)
        for i in range(entries):
            r = int(perm[i])
            if r >= 0:
                qq, ss = G.quantize_mxfp8_torch(cpu._f(x[(i // k) * hidden:(i // k + 1) * hidden]).view(1, hidden))
                qv[r] = qq[0]
                sfm[r] = ss[0]
        sf.copy_(G.sf_to_atoms(sfm)[: sf.numel()])

    def gemm_mx(swiglu):
        def run(g, a, w, sfa, sfw, c, M_, N, K, ldc, err, tiles, tile_count, sfw_expert_bytes, sf_out):
            from ..ops import gemm_mx as G

            tl = tiles.view(-1, 4)
            A = G.dequant_mxfp8(a[: M_ * K].view(M_, K), G.atoms_to_sf(sfa[: G.atom_bytes(M_, K)], M_, K))
            out_sf = G.atoms_to_sf(sf_out, M_, N // 2).clone() if swiglu else None
            for t in range(int(tile_count[0])):
                e, r0, nr, _ = (int(v) for v in tl[t])
                We = G.dequant_mxfp4(w[e * N * K // 2:(e + 1) * N * K // 2].view(N, K // 2),
                                     G.atoms_to_sf(sfw[e * sfw_expert_bytes:(e + 1) * sfw_expert_bytes], N, K))
                acc = A[r0:r0 + nr] @ We.t()
                if swiglu:       # W rows: groups of 128 = 64 gate rows + the matching 64 up rows
                    acc = acc.view(nr, N // 128, 2, 64)
                    act = (F.silu(acc[:, :, 0]) * acc[:, :, 1]).reshape(nr, N // 2)
                    qq, ss = G.quantize_mxfp8_torch(act)
                    c.view(-1, ldc)[r0:r0 + nr] = qq
                    out_sf[r0:r0 + nr] = ss
                else:
                    c.view(-1, ldc)[r0:r0 + nr] = acc.to(torch.bfloat16)
            if swiglu:
                sf_out.copy_(G.sf_to_atoms(out_sf)[: sf_out.numel()])
        return run

    cpu.register("kern_moe_route_f32", route)
    cpu.register("kern_moe_plan", plan)
    cpu.register("kern_moe_plan_aligned", plan_aligned)
    cpu.register("kern_moe_gather_quant_mxfp8", gather_q)
    for bn in (256, 128):
        cpu.register(f"kern_moe_gemm_mxfp8_mxfp4_n{bn}", gemm_mx(False))
        cpu.register(f"kern_moe_gemm_mxfp8_mxfp4_swiglu_mxfp8_n{bn}", gemm_mx(True))
    cpu.register("kern_moe_gather_bf16", gather)
    cpu.register("kern_moe_combine_bf16", combine)
    for bn in (256, 128, 64):
        cpu.register(f"kern_moe_gemm_bf16_n{bn}", gemm("store"))
        cpu.register(f"kern_moe_gemm_bf16_swiglu_n{bn}", gemm("swiglu"))


_register_cpu()
