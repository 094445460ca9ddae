"""Tensor-parallel variant of the dense GQA decoder: one manifest, loaded by every rank of group `tp`.

Attention is split by heads (each rank holds heads / tp query heads and kv_heads / tp KV heads and their
slice of the paged KV cache), the MLP by intermediate columns; the output projections produce partial
sums that the fused peer all-reduce + residual + RMSNorm kernel turns into the next layer's input on
every rank (no NCCL on the path). Weights bind by rank-selected row / column ranges of the same
checkpoint tensors (`bind` with `{group, ranges}`: crates/kern-manifest/src/types.rs:481-541).
The batch is replicated: every rank of the group is fed the same rows.

`sp=True` gives the ragged `prefill` program the sequence-parallel layout (reference: docs/multi-gpu.md:495-528 does it
with NCCL reduce-scatter / all-gather between library GEMMs): attention still runs on all rows by heads, but the
residual stream and the norms live on the rows a rank owns (32-row sub-blocks dealt round-robin). The o / down
projections end in the scatter epilogue (GEMM + reduce-scatter in one kernel: partial rows go from TMEM straight into
the owner's staging slot), `kern_sp_reduce_norm` adds, norms and leaves the owner's rows in `sp.g`, and the QKV /
gate-up GEMMs pull the other owners' rows while their own tiles run (all-gather + GEMM in one kernel). The fixed-shape
`decode` program keeps the replicated layout and the flagless one-shot all-reduce: a handful of rows is latency-bound.
"""
from __future__ import annotations

from . import common as C
from .dense import DenseConfig


def build_manifest_tp(cfg: DenseConfig, fused: bool = True, lamport: bool = True, sp: bool = False, sp_push: bool = True) -> dict:
    """`fused`: the o/down projections push their partial rows to the reducing rank from the GEMM epilogue
    (GEMM + reduce-scatter in one kernel); off, they store the partial and the all-reduce kernel pushes it.
    `lamport`: decode-sized calls use the flagless one-shot all-reduce."""
    n = cfg.tp
    assert n >= 2 and cfg.heads % n == 0 and cfg.kv_heads % n == 0 and cfg.intermediate % (16 * n) == 0
    h, d = cfg.hidden, cfg.head_dim
    hq, hk = cfg.heads // n, cfg.kv_heads // n          # per rank
    inter = cfg.intermediate // n
    qd, kd = hq * d, hk * d
    qkv_dim = qd + 2 * kd
    T, S, W = cfg.max_tokens, cfg.max_seqs, cfg.table_width
    bufs, ops, states = {}, {}, {}
    bufs["token_ids"] = {"dtype": "i64", "shape": ["tokens"], "kind": "input", "fill": "token", "domain": {"min": 0, "max": cfg.vocab - 1}}
    bufs["positions"] = {"dtype": "i64", "shape": ["tokens"], "kind": "input", "fill": "position", "domain": {"min": 0, "max": cfg.max_context - 1}}
    bufs["slot_mapping"] = {"dtype": "i64", "shape": ["tokens"], "kind": "input", "fill": "slot", "domain": {"index_into": "kv.l0"}}
    bufs["seq_lens"] = {"dtype": "i32", "shape": ["seqs"], "kind": "input", "fill": "seq_len"}
    bufs["cu_seqlens"] = {"dtype": "i32", "shape": [S + 1], "kind": "input", "fill": "cu_seqlens"}
    bufs["block_table"] = {"dtype": "i32", "shape": ["seqs", W], "kind": "input", "domain": {"index_into": "kv.l0", "stride": cfg.page_size}}
    bufs["next_token"] = {"dtype": "i64", "shape": ["seqs"], "kind": "output", "fill": "tokens"}
    bufs["error"] = {"dtype": "i32", "shape": [1], "kind": "output", "fill": "error"}
    bufs["x"] = {"dtype": "bf16", "shape": ["tokens", h], "kind": "workspace", "export": True}
    bufs["x_peers"] = {"dtype": "u64", "shape": [n], "kind": "peer", "of": "x", "group": "tp"}
    for name, width in (("xn", h), ("qkv", qkv_dim), ("attn", qd), ("act", inter), ("part", h)):
        bufs[name] = {"dtype": "bf16", "shape": ["tokens", width], "kind": "workspace"}
    bufs["last"] = {"dtype": "bf16", "shape": ["seqs", h], "kind": "workspace"}
    bufs["logits"] = {"dtype": "bf16", "shape": ["seqs", cfg.vocab], "kind": "workspace"}
    bufs["work"] = {"dtype": "i32", "shape": [2 * (-(-T // max(1, 64 // (hq // hk))) + S)], "kind": "workspace"}
    bufs["work_count"] = {"dtype": "i32", "shape": [1], "kind": "workspace"}
    bufs["work_d"] = {"dtype": "i32", "shape": [2 * S], "kind": "workspace"}
    bufs["work_d_count"] = {"dtype": "i32", "shape": [1], "kind": "workspace"}
    bufs["rope_cos"] = {"dtype": "f32", "shape": [cfg.max_context, d // 2], "kind": "carry"}
    bufs["rope_sin"] = {"dtype": "f32", "shape": [cfg.max_context, d // 2], "kind": "carry"}
    bufs.update(C.tp_buffers(h, n, T, lamport=lamport))
    if sp:
        bufs.update(C.sp_buffers(h, n, T))

    def ranked(width: int) -> dict:
        return {"group": "tp", "ranges": [[r * width, (r + 1) * width] for r in range(n)]}

    def weight(name, shape, bind):
        bufs[name] = {"dtype": "bf16", "shape": list(shape), "kind": "weight", "bind": bind}

    weight("w.embed", (cfg.vocab, h), [{"tensor": "model.embed_tokens.weight"}])
    weight("w.norm", (h,), [{"tensor": "model.norm.weight"}])
    weight("w.head", (cfg.vocab, h), [{"tensor": "model.embed_tokens.weight" if cfg.tie_embeddings else "lm_head.weight"}])
    for i in range(cfg.layers):
        p = f"model.layers.{i}."
        states[f"kv.l{i}"] = {"bytes_per_token": 2 * kd * 2}
        weight(f"w.l{i}.ln1", (h,), [{"tensor": p + "input_layernorm.weight"}])
        weight(f"w.l{i}.qkv", (qkv_dim, h), [{"tensor": p + "self_attn.q_proj.weight", "rows": ranked(qd)},
                                              {"tensor": p + "self_attn.k_proj.weight", "rows": ranked(kd)},
                                              {"tensor": p + "self_attn.v_proj.weight", "rows": ranked(kd)}])
        weight(f"w.l{i}.o", (h, qd), [{"tensor": p + "self_attn.o_proj.weight", "cols": ranked(qd)}])
        weight(f"w.l{i}.ln2", (h,), [{"tensor": p + "post_attention_layernorm.weight"}])
        weight(f"w.l{i}.gu", (2 * inter, h), [{"tensor": p + "mlp.gate_proj.weight", "rows": ranked(inter)},
                                               {"tensor": p + "mlp.up_proj.weight", "rows": ranked(inter)}])
        weight(f"w.l{i}.down", (h, inter), [{"tensor": p + "mlp.down_proj.weight", "cols": ranked(inter)}])
        if cfg.qk_norm:
            weight(f"w.l{i}.qn", (d,), [{"tensor": p + "self_attn.q_norm.weight"}])
            weight(f"w.l{i}.kn", (d,), [{"tensor": p + "self_attn.k_norm.weight"}])

    ops["embed"] = C.embedding_op(h, cfg.vocab)
    ops["norm"] = C.rms_norm_op(h, cfg.eps)
    ops["qkv_proj"] = C.gemm_op(qkv_dim, h, rows_max=T)
    # partial sums: pushed to the reducing rank by the GEMM epilogue, finished by the fused all-reduce
    ops["o_proj"] = C.tp_gemm_reduce_op(h, qd, n, T) if fused else C.gemm_op(h, qd, rows_max=T)
    ops["gate_up"] = C.gemm_op(2 * inter, h, epilogue="swiglu", rows_max=T)
    ops["down_proj"] = C.tp_gemm_reduce_op(h, inter, n, T) if fused else C.gemm_op(h, inter, rows_max=T)
    ops["lm_head"] = C.gemm_op(cfg.vocab, h, rows_var="seqs", rows_max=S)
    ops["rope_append"] = C.rope_append_op(hq, hk, d, d, cfg.page_size, cfg.max_context, cfg.eps, cfg.qk_norm)
    ops["attn_plan"] = C.attn_plan_op(hq, hk, S, d)
    ops["attn_prefill"] = C.attn_prefill_op(hq, hk, d, cfg.page_size, W, qkv_dim)
    ops["attn_decode"] = C.attn_decode_op(hq, hk, d, cfg.page_size, W, qkv_dim, S)
    ops["last_row"] = C.last_row_op(h * 2)
    ops["rope_table"] = C.rope_table_op(cfg.max_context, d, cfg.rope_theta)
    ops["pick"] = C.argmax_op(cfg.vocab)
    if lamport:
        ops["lamport_init"] = C.tp_lamport_init_op(h, n)
    ops["allreduce_norm"] = C.tp_allreduce_norm_op(h, cfg.eps, n, T, fused_gemm=fused, lamport=lamport)
    if sp:
        ops["sp_o_proj"] = C.sp_gemm_scatter_op(h, qd, n, T)
        ops["sp_down_proj"] = C.sp_gemm_scatter_op(h, inter, n, T)
        ops["sp_reduce_norm"] = C.sp_reduce_norm_op(h, cfg.eps, n, T, push=sp_push)
        ops["sp_qkv_proj"] = C.sp_ag_gemm_op(qkv_dim, h, n, T, pushed=sp_push)
        ops["sp_gate_up"] = C.sp_ag_gemm_op(2 * inter, h, n, T, epilogue="swiglu", pushed=sp_push)
        ops["sp_last_rows"] = C.sp_last_rows_op(h, n)
        ops.pop("last_row")

    B = lambda name, off=0: ({"buf": name, "offset": off} if off else {"buf": name})
    err = B("error")
    sp_ready = B("sp.flags", C.SP_FLAG_STRIDE * 4)      # row 1 of the flags: "this rank's rows are final"

    def ar(label: str, w: str) -> dict:
        return {"op": "allreduce_norm", "label": label,
                "args": [B("part"), B("x"), B("x_peers"), B("xn"), B(w), B("tp.comm"), B("tp.comm_peers"), B("tp.flags"),
                         B("tp.flags_peers"), B("tp.epochs"), err, {"var": "tokens"}] +
                        ([B("tp.lamport"), B("tp.lamport_peers"), B("tp.lamport_epochs")] if lamport else [])}

    push = [B("tp.comm_peers"), B("tp.epochs")] if fused else []

    def sp_layer(i: int) -> list[dict]:
        """One layer of the sequence-parallel prefill program; `sp.g` holds the layer's normed input (all rows in layer
        0, where every rank normed them itself; the owners' rows afterwards)."""
        kv = {"state": f"kv.l{i}"}
        lbl = f"l{i}."
        rope_args = [B("qkv"), kv, B("positions"), B("slot_mapping"), B("rope_cos"), B("rope_sin")]
        if cfg.qk_norm:
            rope_args += [B(f"w.l{i}.qn"), B(f"w.l{i}.kn")]
        ag_tail = [B("sp.blocks"), B("sp.cta_epochs"), sp_ready, B("sp.state"), err, {"var": "tokens"}]

        def reduce(label: str, w: str) -> dict:
            return {"op": "sp_reduce_norm", "label": label,
                    "args": [B("x"), B("sp.g"), B(w), B("sp.comm"), B("sp.flags"), B("sp.flags_peers"), B("sp.state"), err,
                             {"var": "tokens"}, B("sp.g_peers")]}

        qkv = ({"op": "qkv_proj", "label": lbl + "qkv", "args": [B("sp.g"), B(f"w.l{i}.qkv"), B("qkv"), {"var": "tokens"}, err]}
               if i == 0 else
               {"op": "sp_qkv_proj", "label": lbl + "qkv", "args": [B("sp.g"), B("sp.g_peers"), B(f"w.l{i}.qkv"), B("qkv"), *ag_tail]})
        nxt = f"w.l{i + 1}.ln1" if i + 1 < cfg.layers else "w.norm"
        return [
            qkv,
            {"op": "rope_append", "label": lbl + "rope", "args": rope_args + [err]},
            {"op": "attn_prefill", "label": lbl + "attn",
             "args": [B("qkv"), kv, B("attn"), B("block_table"), B("seq_lens"), B("cu_seqlens"), B("work"),
                      B("work_count"), err, B("work_d"), B("work_d_count")]},
            {"op": "sp_o_proj", "label": lbl + "o",
             "args": [B("attn"), B(f"w.l{i}.o"), B("sp.comm_peers"), B("sp.state"), {"var": "tokens"}, err]},
            reduce(lbl + "rs_attn", f"w.l{i}.ln2"),
            {"op": "sp_gate_up", "label": lbl + "gate_up", "args": [B("sp.g"), B("sp.g_peers"), B(f"w.l{i}.gu"), B("act"), *ag_tail]},
            {"op": "sp_down_proj", "label": lbl + "down",
             "args": [B("act"), B(f"w.l{i}.down"), B("sp.comm_peers"), B("sp.state"), {"var": "tokens"}, err]},
            reduce(lbl + "rs_mlp", nxt),       # leaves the next layer's normed input (or the final norm) on its owners
        ]

    def layer(i: int, prefill: bool) -> list[dict]:
        kv = {"state": f"kv.l{i}"}
        lbl = f"l{i}."
        rope_args = [B("qkv"), kv, B("positions"), B("slot_mapping"), B("rope_cos"), B("rope_sin")]
        if cfg.qk_norm:
            rope_args += [B(f"w.l{i}.qn"), B(f"w.l{i}.kn")]
        calls = [
            {"op": "qkv_proj", "label": lbl + "qkv", "args": [B("xn"), B(f"w.l{i}.qkv"), B("qkv"), {"var": "tokens"}, err]},
            {"op": "rope_append", "label": lbl + "rope", "args": rope_args + [err]},
        ]
        if prefill:
            calls.append({"op": "attn_prefill", "label": lbl + "attn",
                          "args": [B("qkv"), kv, B("attn"), B("block_table"), B("seq_lens"), B("cu_seqlens"), B("work"),
                                   B("work_count"), err, B("work_d"), B("work_d_count")]})
        else:
            calls.append({"op": "attn_decode", "label": lbl + "attn",
                          "args": [B("qkv"), kv, B("attn"), B("block_table"), B("seq_lens"), err]})
        nxt = f"w.l{i + 1}.ln1" if i + 1 < cfg.layers else "w.norm"
        calls += [
            {"op": "o_proj", "label": lbl + "o", "args": [B("attn"), B(f"w.l{i}.o"), B("part"), *push, {"var": "tokens"}, err]},
            ar(lbl + "ar_attn", f"w.l{i}.ln2"),
            {"op": "gate_up", "label": lbl + "gate_up", "args": [B("xn"), B(f"w.l{i}.gu"), B("act"), {"var": "tokens"}, err]},
            {"op": "down_proj", "label": lbl + "down", "args": [B("act"), B(f"w.l{i}.down"), B("part"), *push, {"var": "tokens"}, err]},
            ar(lbl + "ar_mlp", nxt),       # leaves the next layer's normed input (or the final norm) in xn
        ]
        return calls

    def head(src: str) -> list[dict]:
        return [{"op": "lm_head", "label": "lm_head", "args": [B(src), B("w.head"), B("logits"), {"var": "seqs"}, err]},
                {"op": "pick", "label": "argmax", "args": [B("logits"), B("next_token")]}]

    start = [{"op": "embed", "label": "embed", "args": [B("token_ids"), B("w.embed"), B("x"), err]},
             {"op": "norm", "label": "l0.ln1", "args": [B("x"), B("w.l0.ln1"), B("xn")]}]
    prefill = start + [{"op": "attn_plan", "label": "plan",
                        "args": [B("cu_seqlens"), B("work"), B("work_count"), {"var": "seqs"}, {"expr": C.attn_plan_items(hq, hk)},
                                 B("work_d"), B("work_d_count")]}]
    decode = list(start)
    if sp:
        prefill[1] = {"op": "norm", "label": "l0.ln1", "args": [B("x"), B("w.l0.ln1"), B("sp.g")]}
    for i in range(cfg.layers):
        prefill += sp_layer(i) if sp else layer(i, True)
        decode += layer(i, False)
    if sp:
        prefill += [{"op": "sp_last_rows", "label": "last_row",
                     "args": [B("sp.g_peers"), B("last"), B("cu_seqlens"), B("sp.flags"), B("sp.state"), err, {"var": "seqs"}]}]
    else:
        prefill += [{"op": "last_row", "label": "last_row", "args": [B("xn"), B("last"), B("cu_seqlens")]}]
    prefill += head("last")
    decode += head("xn")

    mods = (["norm_embed", "gemm_bf16", "attn_prep", "attn_paged", "misc", "sampling", "tp_allreduce_norm"] +
            (["tp_gemm"] if fused or sp else []) + (["tp_sp", "ag_gemm"] if sp else []))
    return C.ensure_modules({
        "schema_version": 7,
        "model": f"{cfg.name}-tp{n}",
        "vars": {"tokens": {"max": T, "axis": "rows"}, "seqs": {"max": S, "axis": "groups"}},
        "topology": {"groups": {"tp": n}},
        "states": states,
        "buffers": bufs,
        "modules": C.modules_for(mods),
        "ops": ops,
        "programs": {
            "load": {"once": True, "calls": [{"op": "rope_table", "args": [B("rope_cos"), B("rope_sin")]}] +
                     ([{"op": "lamport_init", "args": [B("tp.lamport")]}] if lamport else [])},
            "prefill": {"batch": {"groups": S, "rows": "tokens"}, "calls": prefill},
            "decode": {"batch": {"groups": S, "rows": 1}, "graph": True, "calls": decode},
        },
    })
