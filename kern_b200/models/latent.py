"""Latent-attention hybrid decoder: Kimi-Delta-Attention layers (the delta rule with a decay per key channel) with
every ``full_every``-th layer a multi-head latent attention layer (one shared 576-wide latent row per token: 512
compressed + 64 rotary columns), and an MLP that is dense or routed experts — the Kimi-Linear / K3 class of models.

Manifest generator, synthetic checkpoint and PyTorch fp32 oracle. A KDA layer owns a per-sequence state (conv window +
recurrent matrix), a latent layer a paged state of 1152 bytes per token.

Latent attention runs in the absorbed form for prefill and decode alike: the per-head up-projections of keys and
values are folded into the query and output projections when the checkpoint is loaded (`absorb`), so a layer is
``q_a -> norm -> q_abs (heads x 576) -> rotate/append -> attention over latent rows -> o_abs``. Prefill rows run the
decode kernel with one attention row per token (its sequence's page-table row, its own causal reach). The folded
weights are 4x the size of the factors they replace (heads x 512 x q_lora against heads x 128 x q_lora); the oracle
works from the un-folded checkpoint tensors, so a test of one against the other also tests the folding.
Reference: docs/roadmap.md:13-35 (K3 decode: KDA recurrent step, absorbed MLA decode), docs/serve.md:484 (tiers).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F

from ..ops import gdn as G
from . import common as C
from . import moe as M

DQK, DV, NOPE, ROPE = C.MLA_DQK, C.MLA_DV, 128, 64


@dataclass
class LatentConfig:
    name: str = "latent"
    vocab: int = 163840
    hidden: int = 2304
    layers: int = 27
    full_every: int = 4           # layer i is latent attention when (i + 1) % full_every == 0
    heads: int = 32
    q_lora: int = 1536
    kda_k_heads: int = 32
    kda_v_heads: int = 32
    kda_dim: int = 128
    conv_width: int = 4
    intermediate: int = 9216
    experts: int = 0              # 0: dense MLP; else routed experts of `moe_intermediate`
    top_k: int = 8
    moe_intermediate: int = 1024
    scoring: str = "sigmoid"
    routed_scale: float = 1.0
    eps: float = 1e-6
    rope_theta: float = 1e4
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
    def conv_dim(self) -> int:
        return 2 * self.kda_k_heads * self.kda_dim + self.kda_v_heads * self.kda_dim

    @property
    def kda_v_dim(self) -> int:
        return self.kda_v_heads * self.kda_dim

    @property
    def kda_in_dim(self) -> int:          # q | k | v | z | b | per-key gates
        return self.conv_dim + 2 * self.kda_v_dim + self.kda_v_heads

    @property
    def qa_dim(self) -> int:              # q_a | compressed kv | rotary key
        return self.q_lora + DQK


TINY_LATENT = LatentConfig(name="tiny-latent", vocab=512, hidden=256, layers=4, full_every=2, heads=4, q_lora=64,
                           kda_k_heads=2, kda_v_heads=8, kda_dim=64, intermediate=512, page_size=16, max_tokens=256,
                           max_seqs=8, max_context=256)
# KDA heads of 128, the size whose prefill runs through the chunked (WY) kernels
TINY_LATENT_K128 = LatentConfig(name="tiny-latent-k128", vocab=512, hidden=256, layers=2, full_every=2, heads=4, q_lora=64,
                                kda_k_heads=2, kda_v_heads=8, kda_dim=128, intermediate=512, page_size=16, max_tokens=256,
                                max_seqs=8, max_context=256)
TINY_LATENT_MOE = LatentConfig(name="tiny-latent-moe", vocab=512, hidden=256, layers=2, full_every=2, heads=4, q_lora=64,
                               kda_k_heads=2, kda_v_heads=8, kda_dim=64, intermediate=512, experts=16, top_k=4,
                               moe_intermediate=128, page_size=16, max_tokens=256, max_seqs=8, max_context=256)
# the 48B-A3B shape class: 27 layers, every fourth latent attention, 256 experts of 1024, 8 per token
LATENT_48B = LatentConfig(name="latent-48b-a3b", experts=256)


def weight_names(cfg: LatentConfig) -> dict[str, tuple[tuple[int, ...], str]]:
    """Checkpoint tensor name -> (shape, dtype): the un-folded tensors."""
    h, out, bf, f32 = cfg.hidden, {}, "bf16", "f32"
    kd, vd, hv, H = cfg.kda_k_heads * cfg.kda_dim, cfg.kda_v_dim, cfg.kda_v_heads, cfg.heads
    out["model.embed_tokens.weight"] = ((cfg.vocab, h), bf)
    for i in range(cfg.layers):
        p = f"model.layers.{i}."
        out[p + "input_layernorm.weight"] = ((h,), bf)
        if cfg.is_full(i):
            out[p + "self_attn.q_a_proj.weight"] = ((cfg.q_lora, h), bf)
            out[p + "self_attn.q_a_layernorm.weight"] = ((cfg.q_lora,), bf)
            out[p + "self_attn.q_b_proj.weight"] = ((H * (NOPE + ROPE), cfg.q_lora), bf)
            out[p + "self_attn.kv_a_proj_with_mqa.weight"] = ((DQK, h), bf)
            out[p + "self_attn.kv_a_layernorm.weight"] = ((DV,), bf)
            out[p + "self_attn.kv_b_proj.weight"] = ((H * 2 * NOPE, DV), bf)
            out[p + "self_attn.o_proj.weight"] = ((h, H * NOPE), bf)
        else:
            for n, rows in (("q", kd), ("k", kd), ("v", vd), ("z", vd), ("b", hv), ("g", vd)):
                out[p + f"linear_attn.{n}_proj.weight"] = ((rows, h), bf)
            out[p + "linear_attn.conv1d.weight"] = ((cfg.conv_dim, cfg.conv_width), bf)
            out[p + "linear_attn.A_log"] = ((hv,), f32)
            out[p + "linear_attn.dt_bias"] = ((vd,), f32)
            out[p + "linear_attn.norm.weight"] = ((cfg.kda_dim,), bf)
            out[p + "linear_attn.out_proj.weight"] = ((h, vd), bf)
        out[p + "post_attention_layernorm.weight"] = ((h,), bf)
        if cfg.experts:
            I = cfg.moe_intermediate
            out[p + "mlp.gate.weight"] = ((cfg.experts, h), bf)
            for e in range(cfg.experts):
                out[p + f"mlp.experts.{e}.gate_proj.weight"] = ((I, h), bf)
                out[p + f"mlp.experts.{e}.up_proj.weight"] = ((I, h), bf)
                out[p + f"mlp.experts.{e}.down_proj.weight"] = ((h, I), bf)
        else:
            out[p + "mlp.gate_proj.weight"] = ((cfg.intermediate, h), bf)
            out[p + "mlp.up_proj.weight"] = ((cfg.intermediate, h), bf)
            out[p + "mlp.down_proj.weight"] = ((h, cfg.intermediate), bf)
    out["model.norm.weight"] = ((h,), bf)
    out["lm_head.weight"] = ((cfg.vocab, h), bf)
    return out


def _random(name, shape, dtype, g, device, std):
    if name.endswith("layernorm.weight") or name == "model.norm.weight" or name.endswith("linear_attn.norm.weight"):
        t = 1.0 + 0.1 * torch.randn(shape, generator=g, device=device)
    elif name.endswith("A_log"):
        t = torch.log(torch.empty(shape, device=device).uniform_(0.5, 4.0, generator=g))
    elif name.endswith("dt_bias"):
        t = torch.randn(shape, generator=g, device=device)
    elif name.endswith("conv1d.weight"):
        t = 0.3 * torch.randn(shape, generator=g, device=device)
    elif name.endswith("mlp.gate.weight"):
        t = 10 * std * torch.randn(shape, generator=g, device=device)       # a router with opinions
    else:
        t = std * torch.randn(shape, generator=g, device=device)
    return t.to(torch.bfloat16 if dtype == "bf16" else torch.float32)


def random_weights(cfg: LatentConfig, seed: int = 0, device: str = "cpu", std: float = 0.02) -> dict[str, torch.Tensor]:
    g = torch.Generator(device=device).manual_seed(seed)
    return {n: _random(n, s, dt, g, device, std) for n, (s, dt) in weight_names(cfg).items()}


def absorb(cfg: LatentConfig, q_b: torch.Tensor, kv_b: torch.Tensor, o: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Fold the per-head key / value up-projections into the query and output projections (fp32 products, bf16 out):
    q_abs [heads * 576, q_lora] — per head W_UK^T W_q_nope (512 rows) over W_q_rope (64 rows);
    o_abs [hidden, heads * 512] — per head W_o[:, head] W_UV."""
    H = cfg.heads
    qb = q_b.float().view(H, NOPE + ROPE, -1)
    kvb = kv_b.float().view(H, 2 * NOPE, DV)
    w_uk, w_uv = kvb[:, :NOPE], kvb[:, NOPE:]                                   # [H, 128, 512] each
    q_lat = torch.einsum("hnc,hnr->hcr", w_uk, qb[:, :NOPE])                     # [H, 512, q_lora]
    q_abs = torch.cat([q_lat, qb[:, NOPE:]], 1).reshape(H * DQK, -1)
    o_abs = torch.einsum("dhn,hnc->dhc", o.float().view(-1, H, NOPE), w_uv).reshape(o.shape[0], H * DV)
    return q_abs.to(torch.bfloat16), o_abs.to(torch.bfloat16)


def folded(cfg: LatentConfig, weights: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
    """The checkpoint with `self_attn.q_abs.weight` / `self_attn.o_abs.weight` added for every latent layer."""
    out = dict(weights)
    for i in range(cfg.layers):
        if cfg.is_full(i):
            p = f"model.layers.{i}.self_attn."
            out[p + "q_abs.weight"], out[p + "o_abs.weight"] = absorb(cfg, weights[p + "q_b_proj.weight"],
                                                                     weights[p + "kv_b_proj.weight"], weights[p + "o_proj.weight"])
    return out


def load_random_weights(rt, cfg: LatentConfig, seed: int = 0, std: float = 0.02) -> None:
    """Fill the runtime's weights with the synthetic checkpoint, tensor by tensor on the runtime's device; the folded
    tensors of a latent layer are made from that layer's factors as they are asked for."""
    shapes = weight_names(cfg)
    order = {n: i for i, n in enumerate(shapes)}

    def raw(name: str, dev) -> torch.Tensor:
        g = torch.Generator(device=dev).manual_seed(seed * 1000003 + order[name])
        return _random(name, shapes[name][0], shapes[name][1], g, dev, std)

    def provider(name: str) -> torch.Tensor:
        dev = rt.tensor(next(iter(rt.doc["buffers"]))).device
        if name.endswith(("q_abs.weight", "o_abs.weight")):
            p = name.rsplit(".", 2)[0] + "."
            qa, oa = absorb(cfg, raw(p + "q_b_proj.weight", dev), raw(p + "kv_b_proj.weight", dev), raw(p + "o_proj.weight", dev))
            return qa if name.endswith("q_abs.weight") else oa
        return raw(name, dev)

    rt.load_tensors(provider)


def build_manifest(cfg: LatentConfig) -> dict:
    h, H, ql = cfg.hidden, cfg.heads, cfg.q_lora
    T, S, W = cfg.max_tokens, cfg.max_seqs, cfg.table_width
    inter, gd, ghk, ghv = cfg.intermediate, cfg.kda_dim, cfg.kda_k_heads, cfg.kda_v_heads
    assert gd in (64, 128) and ghv % ghk == 0 and ghv % 8 == 0 and ql % 64 == 0, "gate columns start 16-byte aligned"
    lb, s_off = C.gdn_line_bytes(ghk, ghv, gd, gd, cfg.conv_width)
    fulls = [i for i in range(cfg.layers) if cfg.is_full(i)]
    kdas = [i for i in range(cfg.layers) if not cfg.is_full(i)]
    assert fulls and kdas
    kv0, st0 = f"kv.l{fulls[0]}", f"kda.l{kdas[0]}"
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
    for name, width in (("x", h), ("xn", h), ("qa", cfg.qa_dim), ("qan", ql), ("q", H * DQK), ("attn", H * DV), ("act", inter),
                        ("gin", cfg.kda_in_dim), ("gconv", cfg.conv_dim), ("gout", cfg.kda_v_dim)):
        bufs[name] = {"dtype": "bf16", "shape": ["tokens", width], "kind": "workspace"}
    bufs["row_seq"] = {"dtype": "i32", "shape": ["tokens"], "kind": "workspace"}
    bufs["row_len"] = {"dtype": "i32", "shape": ["tokens"], "kind": "workspace"}
    bufs["last"] = {"dtype": "bf16", "shape": ["seqs", h], "kind": "workspace"}
    bufs["last_n"] = {"dtype": "bf16", "shape": ["seqs", h], "kind": "workspace"}
    bufs["logits"] = {"dtype": "bf16", "shape": ["seqs", cfg.vocab], "kind": "workspace"}
    bufs["rope_cos"] = {"dtype": "f32", "shape": [cfg.max_context, ROPE // 2], "kind": "carry"}
    bufs["rope_sin"] = {"dtype": "f32", "shape": [cfg.max_context, ROPE // 2], "kind": "carry"}

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
            states[f"kv.l{i}"] = {"bytes_per_token": DQK * 2}
            weight(f"w.l{i}.qa", (cfg.qa_dim, h), [T_(p + "self_attn.q_a_proj.weight"), T_(p + "self_attn.kv_a_proj_with_mqa.weight")])
            weight(f"w.l{i}.qn", (ql,), [T_(p + "self_attn.q_a_layernorm.weight")])
            weight(f"w.l{i}.kvn", (DV,), [T_(p + "self_attn.kv_a_layernorm.weight")])
            weight(f"w.l{i}.qabs", (H * DQK, ql), [T_(p + "self_attn.q_abs.weight")])
            weight(f"w.l{i}.oabs", (h, H * DV), [T_(p + "self_attn.o_abs.weight")])
        else:
            states[f"kda.l{i}"] = {"bytes_per_seq": lb}
            weight(f"w.l{i}.gin", (cfg.kda_in_dim, h), [T_(p + f"linear_attn.{n}_proj.weight") for n in "qkvzbg"])
            weight(f"w.l{i}.conv", (cfg.conv_dim, cfg.conv_width), [T_(p + "linear_attn.conv1d.weight")])
            weight(f"w.l{i}.alog", (ghv,), [T_(p + "linear_attn.A_log")], "f32")
            weight(f"w.l{i}.dtb", (cfg.kda_v_dim,), [T_(p + "linear_attn.dt_bias")], "f32")
            weight(f"w.l{i}.gnorm", (gd,), [T_(p + "linear_attn.norm.weight")])
            weight(f"w.l{i}.gout", (h, cfg.kda_v_dim), [T_(p + "linear_attn.out_proj.weight")])
        weight(f"w.l{i}.ln2", (h,), [T_(p + "post_attention_layernorm.weight")])
        weight(f"w.l{i}.gu", (2 * inter, h), [T_(p + "mlp.gate_proj.weight"), T_(p + "mlp.up_proj.weight")])
        weight(f"w.l{i}.down", (h, inter), [T_(p + "mlp.down_proj.weight")])

    ops["embed"] = C.embedding_op(h, cfg.vocab)
    ops["norm"] = C.rms_norm_op(h, cfg.eps)
    ops["norm_last"] = C.rms_norm_op(h, cfg.eps, rows_var="seqs")
    ops["q_norm"] = C.rms_norm_op(ql, cfg.eps, x_stride=cfg.qa_dim)
    ops["qa_proj"] = C.gemm_op(cfg.qa_dim, h, rows_max=T)
    ops["q_abs"] = C.gemm_op(H * DQK, ql, rows_max=T)
    ops["o_abs"] = C.gemm_op(h, H * DV, epilogue="acc", rows_max=T)
    ops["gate_up"] = C.gemm_op(2 * inter, h, epilogue="swiglu", rows_max=T)
    ops["down_proj"] = C.gemm_op(h, inter, epilogue="acc", rows_max=T)
    ops["lm_head"] = C.gemm_op(cfg.vocab, h, rows_var="seqs", rows_max=S)
    ops["mla_rope"] = C.mla_rope_append_op(H, cfg.qa_dim, cfg.eps, cfg.max_context)
    ops["mla_rows"] = C.mla_rows_op()
    ops["mla_attn_p"] = C.mla_attn_op(H, cfg.page_size, W, ragged=True)
    ops["mla_attn_d"] = C.mla_attn_op(H, cfg.page_size, W, ragged=False, seqs_max=S)
    ops["kda_in"] = C.gemm_op(cfg.kda_in_dim, h, rows_max=T)
    ops["kda_out"] = C.gemm_op(h, cfg.kda_v_dim, epilogue="acc", rows_max=T)
    for ragged, sfx in ((True, "_p"), (False, "_d")):
        ops["kda_conv" + sfx] = C.gdn_conv_op(cfg.conv_dim, cfg.conv_width, cfg.kda_in_dim, lb, ragged)
        ops["kda_rule" + sfx] = C.kda_rule_op(ghk, ghv, gd, cfg.kda_in_dim, lb, s_off, cfg.eps, ragged)
    ops["last_row"] = C.last_row_op(h * 2)
    ops["rope_table"] = C.rope_table_op(cfg.max_context, ROPE, cfg.rope_theta)
    ops["pick"] = C.argmax_op(cfg.vocab)

    B = lambda n, off=0: ({"buf": n, "offset": off} if off else {"buf": n})
    err = B("error")

    def mlp(i, lbl):
        return [
            {"op": "norm", "label": lbl + "ln2", "args": [B("x"), B(f"w.l{i}.ln2"), B("xn")]},
            {"op": "gate_up", "label": lbl + "gate_up", "args": [B("xn"), B(f"w.l{i}.gu"), B("act"), {"var": "tokens"}, err]},
            {"op": "down_proj", "label": lbl + "down", "args": [B("act"), B(f"w.l{i}.down"), B("x"), {"var": "tokens"}, err]},
        ]

    def latent_layer(i: int, prefill: bool) -> list[dict]:
        kv, lbl = {"state": f"kv.l{i}"}, f"l{i}."
        calls = [
            {"op": "norm", "label": lbl + "ln1", "args": [B("x"), B(f"w.l{i}.ln1"), B("xn")]},
            {"op": "qa_proj", "label": lbl + "qa", "args": [B("xn"), B(f"w.l{i}.qa"), B("qa"), {"var": "tokens"}, err]},
            {"op": "q_norm", "label": lbl + "qn", "args": [B("qa"), B(f"w.l{i}.qn"), B("qan")]},
            {"op": "q_abs", "label": lbl + "q", "args": [B("qan"), B(f"w.l{i}.qabs"), B("q"), {"var": "tokens"}, err]},
            {"op": "mla_rope", "label": lbl + "rope",
             "args": [B("qa", ql * 2), B("q"), kv, B("positions"), B("slot_mapping"), B("rope_cos"), B("rope_sin"),
                      B(f"w.l{i}.kvn"), err]},
        ]
        if prefill:
            calls.append({"op": "mla_attn_p", "label": lbl + "attn",
                          "args": [B("q"), kv, B("attn"), B("block_table"), B("row_len"), err, B("row_seq")]})
        else:
            calls.append({"op": "mla_attn_d", "label": lbl + "attn",
                          "args": [B("q"), kv, B("attn"), B("block_table"), B("seq_lens"), err]})
        calls.append({"op": "o_abs", "label": lbl + "o", "args": [B("attn"), B(f"w.l{i}.oabs"), B("x"), {"var": "tokens"}, err]})
        return calls + mlp(i, lbl)

    def kda_layer(i: int, prefill: bool) -> list[dict]:
        st, lbl, sfx = {"state": f"kda.l{i}"}, f"l{i}.", "_p" if prefill else "_d"
        cu = [B("cu_seqlens")] if prefill else []
        zba, gk = B("gin", cfg.conv_dim * 2), B("gin", (cfg.conv_dim + cfg.kda_v_dim + ghv) * 2)
        calls = [
            {"op": "norm", "label": lbl + "ln1", "args": [B("x"), B(f"w.l{i}.ln1"), B("xn")]},
            {"op": "kda_in", "label": lbl + "kda_in", "args": [B("xn"), B(f"w.l{i}.gin"), B("gin"), {"var": "tokens"}, err]},
            {"op": "kda_conv" + sfx, "label": lbl + "conv",
             "args": [B("gin"), B("gconv"), st, B("lines"), *cu, B(f"w.l{i}.conv"), {"var": "seqs"}, {"var": "tokens"}]},
            {"op": "kda_rule" + sfx, "label": lbl + "rule",
             "args": [B("gconv"), zba, gk, B("gout"), st, B("lines"), *cu, B(f"w.l{i}.alog"), B(f"w.l{i}.dtb"),
                      B(f"w.l{i}.gnorm"), *([{"var": "seqs"}] if prefill else [])]},
            {"op": "kda_out", "label": lbl + "kda_out", "args": [B("gout"), B(f"w.l{i}.gout"), B("x"), {"var": "tokens"}, err]},
        ]
        return calls + mlp(i, lbl)

    def head(src: str) -> list[dict]:
        return [
            {"op": "norm_last", "label": "final_norm", "args": [B(src), B("w.norm"), B("last_n")]},
            {"op": "lm_head", "label": "lm_head", "args": [B("last_n"), B("w.head"), B("logits"), {"var": "seqs"}, err]},
            {"op": "pick", "label": "argmax", "args": [B("logits"), B("next_token")]},
        ]

    prefill = [{"op": "embed", "label": "embed", "args": [B("token_ids"), B("w.embed"), B("x"), err]}]
    decode = [{"op": "embed", "label": "embed", "args": [B("token_ids"), B("w.embed"), B("x"), err]}]
    rows = {"op": "mla_rows", "label": f"l{fulls[0]}.rows",
            "args": [B("positions"), B("cu_seqlens"), B("row_seq"), B("row_len"), {"var": "seqs"}, {"var": "tokens"}]}
    for i in range(cfg.layers):
        layer = latent_layer if cfg.is_full(i) else kda_layer
        if i == fulls[0]:
            prefill.append(rows)
        prefill += layer(i, True)
        decode += layer(i, False)
    prefill += [{"op": "last_row", "label": "last_row", "args": [B("x"), B("last"), B("cu_seqlens")]}] + head("last")
    decode += head("x")
    mods = ["norm_embed", "gemm_bf16", "attn_prep", "attn_paged", "mla_decode", "misc", "sampling", "gdn"]
    if gd == 128:
        mods.append("gdn_chunk")      # prefill rows of 128-wide heads run the chunked (WY) kernels
    doc = {
        "schema_version": 7, "model": cfg.name,
        "vars": {"tokens": {"max": T, "axis": "rows"}, "seqs": {"max": S, "axis": "groups"}},
        "states": states, "buffers": bufs, "modules": C.modules_for(mods), "ops": ops,
        "programs": {
            "load": {"once": True, "calls": [{"op": "rope_table", "args": [B("rope_cos"), B("rope_sin")]}]},
            "prefill": {"batch": {"groups": S, "rows": "tokens"}, "calls": prefill},
            "decode": {"batch": {"groups": S, "rows": 1}, "graph": True, "calls": decode},
        },
    }
    return M.moeify(doc, cfg, mods + ["moe"]) if cfg.experts else doc


class LatentOracle:
    """Plain PyTorch statement of the decoder over the un-folded checkpoint tensors: latent attention the long way
    (keys and values expanded per head from the cached latent rows), KDA token by token.

    ``forward(tokens, cache)``: one sequence; ``cache`` is a per-layer list — ``[latent rows, None]`` for latent layers,
    ``[conv window, S]`` for KDA layers. Returns ``[len(tokens), vocab]``."""

    def __init__(self, cfg: LatentConfig, weights: dict[str, torch.Tensor], device="cpu"):
        self.cfg, self.device = cfg, device
        self.w = {k: v.to(device=device, dtype=torch.float32) for k, v in weights.items()}

    class Cache(list):
        length = 0

    def new_cache(self):
        return self.Cache([None, None] for _ in range(self.cfg.layers))

    def _norm(self, x, w):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + self.cfg.eps) * w

    def _rope(self, x, pos):
        half = ROPE // 2
        inv = self.cfg.rope_theta ** (-torch.arange(0, half, dtype=torch.float64, device=x.device) * 2.0 / ROPE)
        ang = pos.double()[:, None] * inv[None]
        cos, sin = ang.cos().float(), ang.sin().float()
        while cos.dim() < x.dim():
            cos, sin = cos[:, None], sin[:, None]
        a, b = x[..., :half], x[..., half:]
        return torch.cat([a * cos - b * sin, b * cos + a * sin], -1)

    def _attention(self, i, xn, pos, cache):
        cfg, w, p = self.cfg, self.w, f"model.layers.{i}.self_attn."
        n, H = xn.shape[0], cfg.heads
        qa = self._norm(xn @ w[p + "q_a_proj.weight"].t(), w[p + "q_a_layernorm.weight"])
        q = (qa @ w[p + "q_b_proj.weight"].t()).view(n, H, NOPE + ROPE)
        q = torch.cat([q[..., :NOPE], self._rope(q[..., NOPE:], pos)], -1)
        kv = xn @ w[p + "kv_a_proj_with_mqa.weight"].t()
        lat = torch.cat([self._norm(kv[:, :DV], w[p + "kv_a_layernorm.weight"]), self._rope(kv[:, DV:], pos)], -1)
        if cache[0] is not None:
            lat = torch.cat([cache[0], lat], 0)
        cache[0] = lat
        kvb = (lat[:, :DV] @ w[p + "kv_b_proj.weight"].t()).view(-1, H, 2 * NOPE)
        k = torch.cat([kvb[..., :NOPE], lat[:, None, DV:].expand(-1, H, -1)], -1)
        v = kvb[..., NOPE:]
        s = torch.einsum("rhd,lhd->hrl", q, k) / math.sqrt(NOPE + ROPE)
        mask = torch.arange(k.shape[0], device=xn.device)[None, :] <= pos[:, None]
        s = s.masked_fill(~mask[None], float("-inf"))
        o = torch.einsum("hrl,lhd->rhd", torch.softmax(s, -1), v).reshape(n, H * NOPE)
        return o @ w[p + "o_proj.weight"].t()

    def _kda(self, i, xn, cache):
        cfg, w, p = self.cfg, self.w, f"model.layers.{i}.linear_attn."
        n, gd, hk, hv = xn.shape[0], cfg.kda_dim, cfg.kda_k_heads, cfg.kda_v_heads
        proj = {c: xn @ w[p + f"{c}_proj.weight"].t() for c in "qkvzbg"}
        if cache[0] is None:
            cache[0] = torch.zeros(cfg.conv_width - 1, cfg.conv_dim, device=xn.device)
            cache[1] = torch.zeros(hv, gd, gd, device=xn.device)
        y, cache[0] = G.conv_ref(torch.cat([proj["q"], proj["k"], proj["v"]], -1), cache[0], w[p + "conv1d.weight"])
        q = y[:, :hk * gd].view(n, hk, gd)
        k = y[:, hk * gd:2 * hk * gd].view(n, hk, gd)
        v = y[:, 2 * hk * gd:].view(n, hv, gd)
        o, cache[1] = G.kda_rule_ref(q, k, v, proj["z"].view(n, hv, gd), proj["b"], proj["g"].view(n, hv, gd), cache[1],
                                     w[p + "A_log"], w[p + "dt_bias"].view(hv, gd), w[p + "norm.weight"], cfg.eps)
        return o.reshape(n, hv * gd) @ w[p + "out_proj.weight"].t()

    def mlp(self, i, xn):
        cfg, w, p = self.cfg, self.w, f"model.layers.{i}.mlp."
        if not cfg.experts:
            return (F.silu(xn @ w[p + "gate_proj.weight"].t()) * (xn @ w[p + "up_proj.weight"].t())) @ w[p + "down_proj.weight"].t()
        logits = xn @ w[p + "gate.weight"].t()
        s = torch.softmax(logits, -1) if cfg.scoring == "softmax" else torch.sigmoid(logits)
        wt, ids = torch.topk(s, cfg.top_k, dim=-1)
        wt = wt / wt.sum(-1, keepdim=True) * cfg.routed_scale
        out = torch.zeros_like(xn)
        for e in range(cfg.experts):
            tok, j = torch.nonzero(ids == e, as_tuple=True)
            if tok.numel():
                x = xn[tok]
                a = F.silu(x @ w[p + f"experts.{e}.gate_proj.weight"].t()) * (x @ w[p + f"experts.{e}.up_proj.weight"].t())
                out.index_add_(0, tok, (a @ w[p + f"experts.{e}.down_proj.weight"].t()) * wt[tok, j][:, None])
        return out

    @torch.no_grad()
    def forward(self, tokens, cache) -> torch.Tensor:
        cfg, w = self.cfg, self.w
        ids = torch.as_tensor(tokens, dtype=torch.long, device=self.device)
        n, past = ids.numel(), cache.length
        pos = torch.arange(past, past + n, device=self.device)
        x = w["model.embed_tokens.weight"][ids]
        for i in range(cfg.layers):
            p = f"model.layers.{i}."
            xn = self._norm(x, w[p + "input_layernorm.weight"])
            x = x + (self._attention(i, xn, pos, cache[i]) if cfg.is_full(i) else self._kda(i, xn, cache[i]))
            x = x + self.mlp(i, self._norm(x, w[p + "post_attention_layernorm.weight"]))
        cache.length = past + n
        return self._norm(x, w["model.norm.weight"]) @ w["lm_head.weight"].t()
