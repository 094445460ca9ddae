"""Hybrid decoder: Gated DeltaNet (linear attention) layers with every ``full_every``-th layer a gated
full-attention layer (QK-norm with ``w + 1``, partial RoPE, sigmoid output gate) — the Qwen3-Next family.

Manifest generator, synthetic checkpoint and PyTorch fp32 oracle. Each GDN layer owns a per-sequence
state (``bytes_per_seq``: conv window + recurrent matrix), each attention layer a paged KV state; the call
brings a page table for the second and a line table for the first.
Reference shape: tools/toy/gen.py:131-220 (stateful manifest), tools/kernels-src/gdn_decode.cu.

Checkpoint naming. Attention layers follow Hugging Face (``self_attn.q_proj`` holds per head
``[q_h ; gate_h]`` rows — the fused weight picks them apart with row-range binds). GDN layers use one tensor
per projection (``linear_attn.{q,k,v,z,b,a}_proj.weight``) rather than Hugging Face's group-interleaved
``in_proj_qkvz``; a converter only needs to de-interleave rows.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F

from ..ops import gdn as G
from . import common as C

I32_MAX = C.I32_MAX


@dataclass
class HybridConfig:
    name: str = "hybrid"
    vocab: int = 151936
    hidden: int = 5120
    layers: int = 64
    full_every: int = 4           # layer i is full attention when (i + 1) % full_every == 0
    heads: int = 24
    kv_heads: int = 4
    head_dim: int = 256
    rot_dim: int = 64
    gdn_k_heads: int = 16
    gdn_v_heads: int = 48
    gdn_dim: int = 128            # key and value head dim of the linear-attention layers
    conv_width: int = 4
    intermediate: int = 17408
    eps: float = 1e-6
    rope_theta: float = 1e7
    page_size: int = 64
    max_tokens: int = 8192
    max_seqs: int = 256
    max_context: int = 8192

    def is_full(self, i: int) -> bool:
        return (i + 1) % self.full_every == 0

    @property
    def table_width(self) -> int:
        return -(-self.max_context // self.page_size)

    @property
    def q_dim(self) -> int:
        return self.heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.kv_heads * self.head_dim

    @property
    def qkvg_dim(self) -> int:
        return 2 * self.q_dim + 2 * self.kv_dim

    @property
    def conv_dim(self) -> int:
        return 2 * self.gdn_k_heads * self.gdn_dim + self.gdn_v_heads * self.gdn_dim

    @property
    def gdn_v_dim(self) -> int:
        return self.gdn_v_heads * self.gdn_dim

    @property
    def gdn_in_dim(self) -> int:
        return self.conv_dim + self.gdn_v_dim + 2 * self.gdn_v_heads

    @property
    def kv_bytes_per_token(self) -> int:
        return 2 * self.kv_dim * 2


TOY_HYBRID = HybridConfig(name="toy-hybrid", vocab=256, hidden=64, layers=4, full_every=4, heads=4, kv_heads=2,
                          head_dim=16, rot_dim=8, gdn_k_heads=2, gdn_v_heads=4, gdn_dim=32, intermediate=128,
                          rope_theta=10000.0, page_size=16, max_tokens=64, max_seqs=4, max_context=64)
TINY_HYBRID = HybridConfig(name="tiny-hybrid", vocab=512, hidden=256, layers=4, full_every=2, heads=4, kv_heads=2,
                           head_dim=64, rot_dim=32, gdn_k_heads=2, gdn_v_heads=4, gdn_dim=64, intermediate=512,
                           rope_theta=10000.0, page_size=16, max_tokens=256, max_seqs=8, max_context=256)
# GDN heads of 128, the size whose prefill runs through the chunked (WY) kernels
TINY_HYBRID_K128 = HybridConfig(name="tiny-hybrid-k128", vocab=512, hidden=256, layers=2, full_every=2, heads=4, kv_heads=2,
                                head_dim=64, rot_dim=32, gdn_k_heads=2, gdn_v_heads=4, gdn_dim=128, intermediate=512,
                                rope_theta=10000.0, page_size=16, max_tokens=256, max_seqs=8, max_context=256)
HYBRID_27B = HybridConfig(name="hybrid-27b")


def weight_names(cfg: HybridConfig) -> dict[str, tuple[tuple[int, ...], str]]:
    """Checkpoint tensor name -> (shape, dtype)."""
    h, out = cfg.hidden, {}
    bf, f32 = "bf16", "f32"
    out["model.embed_tokens.weight"] = ((cfg.vocab, h), bf)
    kd, vd, hv = cfg.gdn_k_heads * cfg.gdn_dim, cfg.gdn_v_dim, cfg.gdn_v_heads
    for i in range(cfg.layers):
        p = f"model.layers.{i}."
        out[p + "input_layernorm.weight"] = ((h,), bf)
        if cfg.is_full(i):
            out[p + "self_attn.q_proj.weight"] = ((2 * cfg.q_dim, h), bf)
            out[p + "self_attn.k_proj.weight"] = ((cfg.kv_dim, h), bf)
            out[p + "self_attn.v_proj.weight"] = ((cfg.kv_dim, h), bf)
            out[p + "self_attn.o_proj.weight"] = ((h, cfg.q_dim), bf)
            out[p + "self_attn.q_norm.weight"] = ((cfg.head_dim,), bf)
            out[p + "self_attn.k_norm.weight"] = ((cfg.head_dim,), bf)
        else:
            for n, rows in (("q", kd), ("k", kd), ("v", vd), ("z", vd), ("b", hv), ("a", hv)):
                out[p + f"linear_attn.{n}_proj.weight"] = ((rows, h), bf)
            out[p + "linear_attn.conv1d.weight"] = ((cfg.conv_dim, cfg.conv_width), bf)
            out[p + "linear_attn.A_log"] = ((hv,), f32)
            out[p + "linear_attn.dt_bias"] = ((hv,), f32)
            out[p + "linear_attn.norm.weight"] = ((cfg.gdn_dim,), bf)
            out[p + "linear_attn.out_proj.weight"] = ((h, vd), bf)
        out[p + "post_attention_layernorm.weight"] = ((h,), bf)
        out[p + "mlp.gate_proj.weight"] = ((cfg.intermediate, h), bf)
        out[p + "mlp.up_proj.weight"] = ((cfg.intermediate, h), bf)
        out[p + "mlp.down_proj.weight"] = ((h, cfg.intermediate), bf)
    out["model.norm.weight"] = ((h,), bf)
    out["lm_head.weight"] = ((cfg.vocab, h), bf)
    return out


def _random(name, shape, dtype, g, device, std):
    if name.endswith("layernorm.weight") or name == "model.norm.weight" or name.endswith("_norm.weight"):
        t = 0.1 * torch.randn(shape, generator=g, device=device)         # applied as (1 + w)
    elif name.endswith("linear_attn.norm.weight"):
        t = 1.0 + 0.1 * torch.randn(shape, generator=g, device=device)
    elif name.endswith("A_log"):
        t = torch.log(torch.empty(shape, device=device).uniform_(1.0, 8.0, generator=g))
    elif name.endswith("dt_bias"):
        t = torch.randn(shape, generator=g, device=device)
    elif name.endswith("conv1d.weight"):
        t = 0.3 * torch.randn(shape, generator=g, device=device)
    else:
        t = std * torch.randn(shape, generator=g, device=device)
    return t.to(torch.bfloat16 if dtype == "bf16" else torch.float32)


def random_weights(cfg: HybridConfig, seed: int = 0, device: str = "cpu", std: float = 0.02) -> dict[str, torch.Tensor]:
    g = torch.Generator(device=device).manual_seed(seed)
    return {n: _random(n, s, dt, g, device, std) for n, (s, dt) in weight_names(cfg).items()}


def load_random_weights(rt, cfg: HybridConfig, seed: int = 0, std: float = 0.02) -> None:
    """Fill the runtime's weights with the synthetic checkpoint, tensor by tensor on the runtime's device."""
    shapes = weight_names(cfg)
    order = {n: i for i, n in enumerate(shapes)}

    def provider(name: str) -> torch.Tensor:
        dev = rt.tensor(next(iter(rt.doc["buffers"]))).device
        g = torch.Generator(device=dev).manual_seed(seed * 1000003 + order[name])
        return _random(name, shapes[name][0], shapes[name][1], g, dev, std)

    rt.load_tensors(provider)


def build_manifest(cfg: HybridConfig) -> dict:
    h, d, hq, hk = cfg.hidden, cfg.head_dim, cfg.heads, cfg.kv_heads
    T, S, W = cfg.max_tokens, cfg.max_seqs, cfg.table_width
    inter, gd, ghk, ghv = cfg.intermediate, cfg.gdn_dim, cfg.gdn_k_heads, cfg.gdn_v_heads
    assert cfg.gdn_in_dim % 8 == 0 and ghv % ghk == 0 and gd in (32, 64, 128) and cfg.rot_dim % 2 == 0
    lb, s_off = C.gdn_line_bytes(ghk, ghv, gd, gd, cfg.conv_width)
    fulls = [i for i in range(cfg.layers) if cfg.is_full(i)]
    gdns = [i for i in range(cfg.layers) if not cfg.is_full(i)]
    assert fulls and gdns
    kv0, st0 = f"kv.l{fulls[0]}", f"gdn.l{gdns[0]}"
    bufs, ops, states = {}, {}, {}
    bufs["token_ids"] = {"dtype": "i64", "shape": ["tokens"], "kind": "input", "fill": "token",
                         "domain": {"min": 0, "max": cfg.vocab - 1}}
    bufs["positions"] = {"dtype": "i64", "shape": ["tokens"], "kind": "input", "fill": "position",
                         "domain": {"min": 0, "max": cfg.max_context - 1}}
    bufs["slot_mapping"] = {"dtype": "i64", "shape": ["tokens"], "kind": "input", "fill": "slot", "domain": {"index_into": kv0}}
    bufs["seq_lens"] = {"dtype": "i32", "shape": ["seqs"], "kind": "input", "fill": "seq_len"}
    bufs["cu_seqlens"] = {"dtype": "i32", "shape": [S + 1], "kind": "input", "fill": "cu_seqlens"}
    bufs["block_table"] = {"dtype": "i32", "shape": ["seqs", W], "kind": "input",
                           "domain": {"index_into": kv0, "stride": cfg.page_size}}
    bufs["lines"] = {"dtype": "i32", "shape": [1, "seqs"], "kind": "input", "domain": {"index_into": st0}}
    bufs["next_token"] = {"dtype": "i64", "shape": ["seqs"], "kind": "output", "fill": "tokens"}
    bufs["error"] = {"dtype": "i32", "shape": [1], "kind": "output", "fill": "error"}
    for name, width in (("x", h), ("xn", h), ("qkvg", cfg.qkvg_dim), ("attn", cfg.q_dim), ("act", inter),
                        ("gin", cfg.gdn_in_dim), ("gconv", cfg.conv_dim), ("gout", cfg.gdn_v_dim)):
        bufs[name] = {"dtype": "bf16", "shape": ["tokens", width], "kind": "workspace"}
    bufs["last"] = {"dtype": "bf16", "shape": ["seqs", h], "kind": "workspace"}
    bufs["last_n"] = {"dtype": "bf16", "shape": ["seqs", h], "kind": "workspace"}
    bufs["logits"] = {"dtype": "bf16", "shape": ["seqs", cfg.vocab], "kind": "workspace"}
    bufs["work"] = {"dtype": "i32", "shape": [2 * (-(-T // max(1, 64 // (hq // hk))) + S)], "kind": "workspace"}
    bufs["work_count"] = {"dtype": "i32", "shape": [1], "kind": "workspace"}
    bufs["work_d"] = {"dtype": "i32", "shape": [2 * S], "kind": "workspace"}
    bufs["work_d_count"] = {"dtype": "i32", "shape": [1], "kind": "workspace"}
    bufs["rope_cos"] = {"dtype": "f32", "shape": [cfg.max_context, cfg.rot_dim // 2], "kind": "carry"}
    bufs["rope_sin"] = {"dtype": "f32", "shape": [cfg.max_context, cfg.rot_dim // 2], "kind": "carry"}

    def weight(name, shape, bind, dtype="bf16"):
        bufs[name] = {"dtype": dtype, "shape": list(shape), "kind": "weight", "bind": bind}

    T_ = lambda n: {"tensor": n}
    weight("w.embed", (cfg.vocab, h), [T_("model.embed_tokens.weight")])
    weight("w.norm", (h,), [T_("model.norm.weight")])
    weight("w.head", (cfg.vocab, h), [T_("lm_head.weight")])
    for i in range(cfg.layers):
        p = f"model.layers.{i}."
        weight(f"w.l{i}.ln1", (h,), [T_(p + "input_layernorm.weight")])
        if cfg.is_full(i):
            states[f"kv.l{i}"] = {"bytes_per_token": cfg.kv_bytes_per_token}
            qp = p + "self_attn.q_proj.weight"
            q_rows = [{"tensor": qp, "rows": [2 * hh * d, 2 * hh * d + d]} for hh in range(hq)]
            g_rows = [{"tensor": qp, "rows": [2 * hh * d + d, 2 * hh * d + 2 * d]} for hh in range(hq)]
            weight(f"w.l{i}.qkvg", (cfg.qkvg_dim, h), q_rows + [T_(p + "self_attn.k_proj.weight"),
                                                                  T_(p + "self_attn.v_proj.weight")] + g_rows)
            weight(f"w.l{i}.o", (h, cfg.q_dim), [T_(p + "self_attn.o_proj.weight")])
            weight(f"w.l{i}.qn", (d,), [T_(p + "self_attn.q_norm.weight")])
            weight(f"w.l{i}.kn", (d,), [T_(p + "self_attn.k_norm.weight")])
        else:
            states[f"gdn.l{i}"] = {"bytes_per_seq": lb}
            weight(f"w.l{i}.gin", (cfg.gdn_in_dim, h), [T_(p + f"linear_attn.{n}_proj.weight") for n in "qkvzba"])
            weight(f"w.l{i}.conv", (cfg.conv_dim, cfg.conv_width), [T_(p + "linear_attn.conv1d.weight")])
            weight(f"w.l{i}.alog", (ghv,), [T_(p + "linear_attn.A_log")], "f32")
            weight(f"w.l{i}.dtb", (ghv,), [T_(p + "linear_attn.dt_bias")], "f32")
            weight(f"w.l{i}.gnorm", (gd,), [T_(p + "linear_attn.norm.weight")])
            weight(f"w.l{i}.gout", (h, cfg.gdn_v_dim), [T_(p + "linear_attn.out_proj.weight")])
        weight(f"w.l{i}.ln2", (h,), [T_(p + "post_attention_layernorm.weight")])
        weight(f"w.l{i}.gu", (2 * inter, h), [T_(p + "mlp.gate_proj.weight"), T_(p + "mlp.up_proj.weight")])
        weight(f"w.l{i}.down", (h, inter), [T_(p + "mlp.down_proj.weight")])

    ops["embed"] = C.embedding_op(h, cfg.vocab)
    ops["norm"] = C.rms_norm_op(h, cfg.eps, plus_one=True)
    ops["norm_last"] = C.rms_norm_op(h, cfg.eps, plus_one=True, rows_var="seqs")
    ops["qkvg_proj"] = C.gemm_op(cfg.qkvg_dim, h, rows_max=T)
    ops["o_proj"] = C.gemm_op(h, cfg.q_dim, epilogue="acc", rows_max=T)
    ops["gate_up"] = C.gemm_op(2 * inter, h, epilogue="swiglu", rows_max=T)
    ops["down_proj"] = C.gemm_op(h, inter, epilogue="acc", rows_max=T)
    ops["lm_head"] = C.gemm_op(cfg.vocab, h, rows_var="seqs", rows_max=S)
    ops["rope_append"] = C.rope_append_op(hq, hk, d, cfg.rot_dim, cfg.page_size, cfg.max_context, cfg.eps, True,
                                          norm_plus_one=True, row_stride=cfg.qkvg_dim)
    ops["attn_plan"] = C.attn_plan_op(hq, hk, S)
    ops["attn_prefill"] = C.attn_prefill_op(hq, hk, d, cfg.page_size, W, cfg.qkvg_dim)
    ops["attn_decode"] = C.attn_decode_op(hq, hk, d, cfg.page_size, W, cfg.qkvg_dim, S)
    ops["attn_gate"] = C.sigmoid_mul_op(cfg.q_dim, cfg.q_dim, cfg.qkvg_dim)
    ops["gdn_in"] = C.gemm_op(cfg.gdn_in_dim, h, rows_max=T)
    ops["gdn_out"] = C.gemm_op(h, cfg.gdn_v_dim, epilogue="acc", rows_max=T)
    for ragged, sfx in ((True, "_p"), (False, "_d")):
        ops["gdn_conv" + sfx] = C.gdn_conv_op(cfg.conv_dim, cfg.conv_width, cfg.gdn_in_dim, lb, ragged)
        ops["gdn_rule" + sfx] = C.gdn_rule_op(ghk, ghv, gd, cfg.gdn_in_dim, lb, s_off, cfg.eps, ragged)
    ops["last_row"] = C.last_row_op(h * 2)
    ops["rope_table"] = C.rope_table_op(cfg.max_context, cfg.rot_dim, cfg.rope_theta)
    ops["pick"] = C.argmax_op(cfg.vocab)

    B = lambda n, off=0: ({"buf": n, "offset": off} if off else {"buf": n})
    err = B("error")

    def mlp(i, lbl):
        return [
            {"op": "norm", "label": lbl + "ln2", "args": [B("x"), B(f"w.l{i}.ln2"), B("xn")]},
            {"op": "gate_up", "label": lbl + "gate_up", "args": [B("xn"), B(f"w.l{i}.gu"), B("act"), {"var": "tokens"}, err]},
            {"op": "down_proj", "label": lbl + "down", "args": [B("act"), B(f"w.l{i}.down"), B("x"), {"var": "tokens"}, err]},
        ]

    def full_layer(i: int, prefill: bool) -> list[dict]:
        kv, lbl = {"state": f"kv.l{i}"}, f"l{i}."
        calls = [
            {"op": "norm", "label": lbl + "ln1", "args": [B("x"), B(f"w.l{i}.ln1"), B("xn")]},
            {"op": "qkvg_proj", "label": lbl + "qkvg", "args": [B("xn"), B(f"w.l{i}.qkvg"), B("qkvg"), {"var": "tokens"}, err]},
            {"op": "rope_append", "label": lbl + "rope",
             "args": [B("qkvg"), kv, B("positions"), B("slot_mapping"), B("rope_cos"), B("rope_sin"), B(f"w.l{i}.qn"),
                      B(f"w.l{i}.kn"), err]},
        ]
        if prefill:
            calls.append({"op": "attn_prefill", "label": lbl + "attn",
                          "args": [B("qkvg"), kv, B("attn"), B("block_table"), B("seq_lens"), B("cu_seqlens"), B("work"),
                                   B("work_count"), err, B("work_d"), B("work_d_count")]})
        else:
            calls.append({"op": "attn_decode", "label": lbl + "attn",
                          "args": [B("qkvg"), kv, B("attn"), B("block_table"), B("seq_lens"), err]})
        calls += [
            {"op": "attn_gate", "label": lbl + "gate", "args": [B("attn"), B("qkvg", (cfg.q_dim + 2 * cfg.kv_dim) * 2), B("attn")]},
            {"op": "o_proj", "label": lbl + "o", "args": [B("attn"), B(f"w.l{i}.o"), B("x"), {"var": "tokens"}, err]},
        ]
        return calls + mlp(i, lbl)

    def gdn_layer(i: int, prefill: bool) -> list[dict]:
        st, lbl, sfx = {"state": f"gdn.l{i}"}, f"l{i}.", "_p" if prefill else "_d"
        cu = [B("cu_seqlens")] if prefill else []
        calls = [
            {"op": "norm", "label": lbl + "ln1", "args": [B("x"), B(f"w.l{i}.ln1"), B("xn")]},
            {"op": "gdn_in", "label": lbl + "gdn_in", "args": [B("xn"), B(f"w.l{i}.gin"), B("gin"), {"var": "tokens"}, err]},
            {"op": "gdn_conv" + sfx, "label": lbl + "conv", "args": [B("gin"), B("gconv"), st, B("lines"), *cu, B(f"w.l{i}.conv"), {"var": "seqs"}, {"var": "tokens"}]},
            {"op": "gdn_rule" + sfx, "label": lbl + "rule",
             "args": [B("gconv"), B("gin", cfg.conv_dim * 2), B("gout"), st, B("lines"), *cu, B(f"w.l{i}.alog"),
                      B(f"w.l{i}.dtb"), B(f"w.l{i}.gnorm"), *([{"var": "seqs"}] if prefill else [])]},
            {"op": "gdn_out", "label": lbl + "gdn_out", "args": [B("gout"), B(f"w.l{i}.gout"), B("x"), {"var": "tokens"}, err]},
        ]
        return calls + mlp(i, lbl)

    def head(src: str) -> list[dict]:
        return [
            {"op": "norm_last", "label": "final_norm", "args": [B(src), B("w.norm"), B("last_n")]},
            {"op": "lm_head", "label": "lm_head", "args": [B("last_n"), B("w.head"), B("logits"), {"var": "seqs"}, err]},
            {"op": "pick", "label": "argmax", "args": [B("logits"), B("next_token")]},
        ]

    prefill = [{"op": "embed", "label": "embed", "args": [B("token_ids"), B("w.embed"), B("x"), err]}]
    # the attention work lists are planned right before the first attention layer, so a pipeline stage made only of
    # linear-attention layers ahead of it neither receives nor forwards them
    plan = {"op": "attn_plan", "label": f"l{fulls[0]}.plan",
            "args": [B("cu_seqlens"), B("work"), B("work_count"), {"var": "seqs"}, {"expr": C.attn_plan_items(hq, hk)},
                     B("work_d"), B("work_d_count")]}
    decode = [{"op": "embed", "label": "embed", "args": [B("token_ids"), B("w.embed"), B("x"), err]}]
    for i in range(cfg.layers):
        layer = full_layer if cfg.is_full(i) else gdn_layer
        if i == fulls[0]:
            prefill.append(plan)
        prefill += layer(i, True)
        decode += layer(i, False)
    prefill += [{"op": "last_row", "label": "last_row", "args": [B("x"), B("last"), B("cu_seqlens")]}] + head("last")
    decode += head("x")
    mods = ["norm_embed", "gemm_bf16", "attn_prep", "attn_paged", "misc", "sampling", "gdn"]
    if gd == 128:
        mods.append("gdn_chunk")      # prefill rows of 128-wide heads run the chunked (WY) kernels
    return {
        "schema_version": 7, "model": cfg.name,
        "vars": {"tokens": {"max": T, "axis": "rows"}, "seqs": {"max": S, "axis": "groups"}},
        "states": states, "buffers": bufs, "modules": C.modules_for(mods), "ops": ops,
        "programs": {
            "load": {"once": True, "calls": [{"op": "rope_table", "args": [B("rope_cos"), B("rope_sin")]}]},
            "prefill": {"batch": {"groups": S, "rows": "tokens"}, "calls": prefill},
            "decode": {"batch": {"groups": S, "rows": 1}, "graph": True, "calls": decode},
        },
    }


# ---- PyTorch fp32 oracle ---------------------------------------------------------------------------
class HybridOracle:
    """Plain PyTorch statement of the hybrid decoder over the same checkpoint tensors.

    ``forward(tokens, cache)``: one sequence; ``cache`` is a per-layer list — ``[k, v]`` for attention
    layers, ``[conv window, S]`` for GDN layers — grown / updated in place. Returns ``[len(tokens), vocab]``."""

    def __init__(self, cfg: HybridConfig, weights: dict[str, torch.Tensor], device="cpu"):
        self.cfg, self.device = cfg, device
        self.w = {k: v.to(device=device, dtype=torch.float32) for k, v in weights.items()}

    class Cache(list):
        length = 0

    def new_cache(self):
        return self.Cache([None, None] for _ in range(self.cfg.layers))

    def _norm(self, x, w, plus_one=True):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + self.cfg.eps) * (w + (1.0 if plus_one else 0.0))

    def _rope(self, x, pos):
        rot = self.cfg.rot_dim
        half = rot // 2
        inv = self.cfg.rope_theta ** (-torch.arange(0, half, dtype=torch.float64, device=x.device) * 2.0 / rot)
        ang = pos.double()[:, None] * inv[None]
        cos, sin = ang.cos().float()[:, None], ang.sin().float()[:, None]
        a, b = x[..., :half], x[..., half:rot]
        return torch.cat([a * cos - b * sin, b * cos + a * sin, x[..., rot:]], -1)

    def _attention(self, i, xn, pos, cache):
        cfg, w, p = self.cfg, self.w, f"model.layers.{i}."
        n, d = xn.shape[0], cfg.head_dim
        qg = (xn @ w[p + "self_attn.q_proj.weight"].t()).view(n, cfg.heads, 2 * d)
        q, gate = qg[..., :d], qg[..., d:].reshape(n, cfg.q_dim)
        k = (xn @ w[p + "self_attn.k_proj.weight"].t()).view(n, cfg.kv_heads, d)
        v = (xn @ w[p + "self_attn.v_proj.weight"].t()).view(n, cfg.kv_heads, d)
        q = self._rope(self._norm(q, w[p + "self_attn.q_norm.weight"]), pos)
        k = self._rope(self._norm(k, w[p + "self_attn.k_norm.weight"]), pos)
        if cache[0] is not None:
            k, v = torch.cat([cache[0], k], 0), torch.cat([cache[1], v], 0)
        cache[0], cache[1] = k, v
        g = cfg.heads // cfg.kv_heads
        s = torch.einsum("rhd,lhd->hrl", q, k.repeat_interleave(g, 1)) / math.sqrt(d)
        mask = torch.arange(k.shape[0], device=xn.device)[None, :] <= pos[:, None]
        s = s.masked_fill(~mask[None], float("-inf"))
        o = torch.einsum("hrl,lhd->rhd", torch.softmax(s, -1), v.repeat_interleave(g, 1)).reshape(n, cfg.q_dim)
        return (o * torch.sigmoid(gate)) @ w[p + "self_attn.o_proj.weight"].t()

    def _gdn(self, i, xn, cache):
        cfg, w, p = self.cfg, self.w, f"model.layers.{i}.linear_attn."
        n, gd, hk, hv = xn.shape[0], cfg.gdn_dim, cfg.gdn_k_heads, cfg.gdn_v_heads
        proj = {c: xn @ w[p + f"{c}_proj.weight"].t() for c in "qkvzba"}
        if cache[0] is None:
            cache[0] = torch.zeros(cfg.conv_width - 1, cfg.conv_dim, device=xn.device)
            cache[1] = torch.zeros(hv, gd, gd, device=xn.device)
        y, cache[0] = G.conv_ref(torch.cat([proj["q"], proj["k"], proj["v"]], -1), cache[0], w[p + "conv1d.weight"])
        q = y[:, :hk * gd].view(n, hk, gd)
        k = y[:, hk * gd:2 * hk * gd].view(n, hk, gd)
        v = y[:, 2 * hk * gd:].view(n, hv, gd)
        o, cache[1] = G.rule_ref(q, k, v, proj["z"].view(n, hv, gd), proj["b"], proj["a"], cache[1], w[p + "A_log"],
                                 w[p + "dt_bias"], w[p + "norm.weight"], cfg.eps)
        return o.reshape(n, hv * gd) @ w[p + "out_proj.weight"].t()

    @torch.no_grad()
    def forward(self, tokens, cache) -> torch.Tensor:
        cfg, w = self.cfg, self.w
        ids = torch.as_tensor(tokens, dtype=torch.long, device=self.device)
        n = ids.numel()
        past = cache.length
        pos = torch.arange(past, past + n, device=self.device)
        x = w["model.embed_tokens.weight"][ids]
        for i in range(cfg.layers):
            p = f"model.layers.{i}."
            xn = self._norm(x, w[p + "input_layernorm.weight"])
            x = x + (self._attention(i, xn, pos, cache[i]) if cfg.is_full(i) else self._gdn(i, xn, cache[i]))
            xn = self._norm(x, w[p + "post_attention_layernorm.weight"])
            act = F.silu(xn @ w[p + "mlp.gate_proj.weight"].t()) * (xn @ w[p + "mlp.up_proj.weight"].t())
            x = x + act @ w[p + "mlp.down_proj.weight"].t()
        cache.length = past + n
        return self._norm(x, w["model.norm.weight"]) @ w["lm_head.weight"].t()
