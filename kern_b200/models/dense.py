"""Dense GQA decoder (Llama / Qwen3 family): manifest generator, synthetic checkpoint writer and the
PyTorch fp32 oracle of the same architecture.

The generator is the only place that knows the model: which kernels a layer calls, how the
checkpoint's tensors concatenate into fused weights (q|k|v stacked, gate then up stacked for the
SwiGLU epilogue), which tables are derived at load. The engine sees a manifest.
Programs: ``load`` (once: rope tables), ``prefill`` (ragged rows over up to ``seqs`` sequences: prompt
chunks and decode rows mixed, split by ``cu_seqlens``), ``decode`` (one row per sequence, replayed as a
CUDA graph). Reference shape: crates/kern-manifest/tests/fixtures/paged.json, tools/toy/gen.py:40-129.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from . import common as C


@dataclass
class DenseConfig:
    name: str = "dense"
    vocab: int = 151936
    hidden: int = 4096
    layers: int = 36
    heads: int = 32
    kv_heads: int = 8
    head_dim: int = 128
    intermediate: int = 12288
    eps: float = 1e-6
    rope_theta: float = 1e6
    qk_norm: bool = False
    tie_embeddings: bool = False
    page_size: int = 64
    max_tokens: int = 8192        # rows of one call (prefill chunk + decode rows)
    max_seqs: int = 256           # sequences of one call
    max_context: int = 8192       # longest sequence (positions); sizes the page-table row and rope tables
    sampling: bool = False        # sampling fills + sampler instead of greedy argmax
    tp: int = 1                   # tensor-parallel width (see tp.py for the fused variant)

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
    def qkv_dim(self) -> int:
        return self.q_dim + 2 * self.kv_dim

    @property
    def kv_bytes_per_token(self) -> int:
        return 2 * self.kv_dim * 2

    def param_count(self) -> int:
        per = self.hidden * self.qkv_dim + self.q_dim * self.hidden + 3 * self.hidden * self.intermediate + 2 * self.hidden
        head = 0 if self.tie_embeddings else self.vocab * self.hidden
        return self.layers * per + self.vocab * self.hidden + head + self.hidden


TOY = DenseConfig(name="toy", vocab=256, hidden=64, layers=2, heads=4, kv_heads=2, head_dim=16, intermediate=128,
                  eps=1e-6, rope_theta=10000.0, page_size=16, max_tokens=64, max_seqs=4, max_context=64)
# the smallest shape every GPU kernel accepts (head_dim 64), for fast end-to-end GPU tests
TINY = DenseConfig(name="tiny", vocab=512, hidden=256, layers=2, heads=4, kv_heads=2, head_dim=64, intermediate=512,
                   rope_theta=10000.0, page_size=16, max_tokens=256, max_seqs=8, max_context=256)
DENSE_8B = DenseConfig(name="dense-8b")


def weight_names(cfg: DenseConfig) -> dict[str, tuple[int, ...]]:
    """Hugging Face tensor names and shapes of the checkpoint."""
    h, out = cfg.hidden, {}
    out["model.embed_tokens.weight"] = (cfg.vocab, h)
    for i in range(cfg.layers):
        p = f"model.layers.{i}."
        out[p + "input_layernorm.weight"] = (h,)
        out[p + "self_attn.q_proj.weight"] = (cfg.q_dim, h)
        out[p + "self_attn.k_proj.weight"] = (cfg.kv_dim, h)
        out[p + "self_attn.v_proj.weight"] = (cfg.kv_dim, h)
        out[p + "self_attn.o_proj.weight"] = (h, cfg.q_dim)
        if cfg.qk_norm:
            out[p + "self_attn.q_norm.weight"] = (cfg.head_dim,)
            out[p + "self_attn.k_norm.weight"] = (cfg.head_dim,)
        out[p + "post_attention_layernorm.weight"] = (h,)
        out[p + "mlp.gate_proj.weight"] = (cfg.intermediate, h)
        out[p + "mlp.up_proj.weight"] = (cfg.intermediate, h)
        out[p + "mlp.down_proj.weight"] = (h, cfg.intermediate)
    out["model.norm.weight"] = (h,)
    if not cfg.tie_embeddings:
        out["lm_head.weight"] = (cfg.vocab, h)
    return out


def random_weights(cfg: DenseConfig, seed: int = 0, device: str = "cpu", std: float = 0.02) -> dict[str, torch.Tensor]:
    """bf16 N(0, std) projections, norm weights near 1; the synthetic checkpoint of the benchmarks."""
    g = torch.Generator(device=device).manual_seed(seed)
    out = {}
    for name, shape in weight_names(cfg).items():
        if name.endswith("norm.weight"):
            t = 1.0 + 0.1 * torch.randn(shape, generator=g, device=device)
        else:
            t = std * torch.randn(shape, generator=g, device=device)
        out[name] = t.to(torch.bfloat16)
    return out


def build_manifest(cfg: DenseConfig, hosted: bool = False) -> dict:
    """`hosted`: the manifest a host engine (vLLM / SGLang style) drives: KV states are the host's tensors, `prefill` /
    `decode` end at `hidden` (final-norm rows), and a `head` program turns the rows copied into `head_in` into `logits`."""
    h, d, hq, hk = cfg.hidden, cfg.head_dim, cfg.heads, cfg.kv_heads
    T, S, W = cfg.max_tokens, cfg.max_seqs, cfg.table_width
    inter = cfg.intermediate
    assert inter % 16 == 0 and h % 8 == 0
    bufs, ops, states = {}, {}, {}
    bufs["token_ids"] = {"dtype": "i64", "shape": ["tokens"], "kind": "input", "fill": "token",
                         "domain": {"min": 0, "max": cfg.vocab - 1}}
    bufs["positions"] = {"dtype": "i64", "shape": ["tokens"], "kind": "input", "fill": "position",
                         "domain": {"min": 0, "max": cfg.max_context - 1}}
    bufs["slot_mapping"] = {"dtype": "i64", "shape": ["tokens"], "kind": "input", "fill": "slot", "domain": {"index_into": "kv.l0"}}
    bufs["seq_lens"] = {"dtype": "i32", "shape": ["seqs"], "kind": "input", "fill": "seq_len"}
    bufs["cu_seqlens"] = {"dtype": "i32", "shape": [S + 1], "kind": "input", "fill": "cu_seqlens"}
    bufs["block_table"] = {"dtype": "i32", "shape": ["seqs", W], "kind": "input",
                           "domain": {"index_into": "kv.l0", "stride": cfg.page_size}}
    bufs["next_token"] = {"dtype": "i64", "shape": ["seqs"], "kind": "output", "fill": "tokens"}
    bufs["error"] = {"dtype": "i32", "shape": [1], "kind": "output", "fill": "error"}
    for name, shape in (("x", [h]), ("xn", [h]), ("qkv", [cfg.qkv_dim]), ("attn", [cfg.q_dim]), ("act", [inter])):
        bufs[name] = {"dtype": "bf16", "shape": ["tokens", *shape], "kind": "workspace"}
    bufs["last"] = {"dtype": "bf16", "shape": ["seqs", h], "kind": "workspace"}
    bufs["last_n"] = {"dtype": "bf16", "shape": ["seqs", h], "kind": "workspace"}
    bufs["logits"] = {"dtype": "bf16", "shape": ["seqs", cfg.vocab], "kind": "workspace"}
    bufs["work"] = {"dtype": "i32", "shape": [2 * (-(-T // max(1, 64 // (hq // hk))) + S)], "kind": "workspace"}
    bufs["work_count"] = {"dtype": "i32", "shape": [1], "kind": "workspace"}
    bufs["work_d"] = {"dtype": "i32", "shape": [2 * S], "kind": "workspace"}
    bufs["work_d_count"] = {"dtype": "i32", "shape": [1], "kind": "workspace"}
    bufs["rope_cos"] = {"dtype": "f32", "shape": [cfg.max_context, d // 2], "kind": "carry"}
    bufs["rope_sin"] = {"dtype": "f32", "shape": [cfg.max_context, d // 2], "kind": "carry"}
    if cfg.sampling:
        for name, dt, fill in (("temperature", "f32", "temperature"), ("top_k", "i32", "top_k"), ("top_p", "f32", "top_p"),
                               ("min_p", "f32", "min_p"), ("seed", "i64", "seed")):
            bufs[name] = {"dtype": dt, "shape": ["seqs"], "kind": "input", "fill": fill}

    def weight(name, shape, bind):
        bufs[name] = {"dtype": "bf16", "shape": list(shape), "kind": "weight", "bind": bind}

    weight("w.embed", (cfg.vocab, h), [{"tensor": "model.embed_tokens.weight"}])
    weight("w.norm", (h,), [{"tensor": "model.norm.weight"}])
    weight("w.head", (cfg.vocab, h), [{"tensor": "model.embed_tokens.weight" if cfg.tie_embeddings else "lm_head.weight"}])
    for i in range(cfg.layers):
        p = f"model.layers.{i}."
        states[f"kv.l{i}"] = {"bytes_per_token": cfg.kv_bytes_per_token}
        weight(f"w.l{i}.ln1", (h,), [{"tensor": p + "input_layernorm.weight"}])
        weight(f"w.l{i}.qkv", (cfg.qkv_dim, h), [{"tensor": p + "self_attn.q_proj.weight"}, {"tensor": p + "self_attn.k_proj.weight"},
                                                   {"tensor": p + "self_attn.v_proj.weight"}])
        weight(f"w.l{i}.o", (h, cfg.q_dim), [{"tensor": p + "self_attn.o_proj.weight"}])
        weight(f"w.l{i}.ln2", (h,), [{"tensor": p + "post_attention_layernorm.weight"}])
        weight(f"w.l{i}.gu", (2 * inter, h), [{"tensor": p + "mlp.gate_proj.weight"}, {"tensor": p + "mlp.up_proj.weight"}])
        weight(f"w.l{i}.down", (h, inter), [{"tensor": p + "mlp.down_proj.weight"}])
        if cfg.qk_norm:
            weight(f"w.l{i}.qn", (d,), [{"tensor": p + "self_attn.q_norm.weight"}])
            weight(f"w.l{i}.kn", (d,), [{"tensor": p + "self_attn.k_norm.weight"}])

    ops["embed"] = C.embedding_op(h, cfg.vocab)
    ops["norm"] = C.rms_norm_op(h, cfg.eps)
    ops["norm_last"] = C.rms_norm_op(h, cfg.eps, rows_var="seqs")
    ops["qkv_proj"] = C.gemm_op(cfg.qkv_dim, h, rows_max=T)
    ops["o_proj"] = C.gemm_op(h, cfg.q_dim, epilogue="acc", rows_max=T)
    ops["gate_up"] = C.gemm_op(2 * inter, h, epilogue="swiglu", rows_max=T)
    ops["down_proj"] = C.gemm_op(h, inter, epilogue="acc", rows_max=T)
    ops["lm_head"] = C.gemm_op(cfg.vocab, h, rows_var="seqs", rows_max=S)
    ops["rope_append"] = C.rope_append_op(hq, hk, d, d, cfg.page_size, cfg.max_context, cfg.eps, cfg.qk_norm)
    ops["attn_plan"] = C.attn_plan_op(hq, hk, S, d)
    ops["attn_prefill"] = C.attn_prefill_op(hq, hk, d, cfg.page_size, W, cfg.qkv_dim)
    ops["attn_decode"] = C.attn_decode_op(hq, hk, d, cfg.page_size, W, cfg.qkv_dim, S)
    ops["last_row"] = C.last_row_op(h * 2)
    ops["rope_table"] = C.rope_table_op(cfg.max_context, d, cfg.rope_theta)
    ops["pick"] = C.sample_op(cfg.vocab) if cfg.sampling else C.argmax_op(cfg.vocab)

    B = lambda n, off=0: ({"buf": n, "offset": off} if off else {"buf": n})
    err = B("error")

    def layer(i: int, prefill: bool) -> list[dict]:
        kv = {"state": f"kv.l{i}"}
        lbl = f"l{i}."
        rope_args = [B("qkv"), kv, B("positions"), B("slot_mapping"), B("rope_cos"), B("rope_sin")]
        if cfg.qk_norm:
            rope_args += [B(f"w.l{i}.qn"), B(f"w.l{i}.kn")]
        calls = [
            {"op": "norm", "label": lbl + "ln1", "args": [B("x"), B(f"w.l{i}.ln1"), B("xn")]},
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
        calls += [
            {"op": "o_proj", "label": lbl + "o", "args": [B("attn"), B(f"w.l{i}.o"), B("x"), {"var": "tokens"}, err]},
            {"op": "norm", "label": lbl + "ln2", "args": [B("x"), B(f"w.l{i}.ln2"), B("xn")]},
            {"op": "gate_up", "label": lbl + "gate_up", "args": [B("xn"), B(f"w.l{i}.gu"), B("act"), {"var": "tokens"}, err]},
            {"op": "down_proj", "label": lbl + "down", "args": [B("act"), B(f"w.l{i}.down"), B("x"), {"var": "tokens"}, err]},
        ]
        return calls

    def pick_call() -> dict:
        if cfg.sampling:
            return {"op": "pick", "label": "sample", "args": [B("logits"), B("next_token"), B("temperature"), B("top_k"),
                                                               B("top_p"), B("min_p"), B("seed"), B("seq_lens")]}
        return {"op": "pick", "label": "argmax", "args": [B("logits"), B("next_token")]}

    def head(src: str) -> list[dict]:
        return [
            {"op": "norm_last", "label": "final_norm", "args": [B(src), B("w.norm"), B("last_n")]},
            {"op": "lm_head", "label": "lm_head", "args": [B("last_n"), B("w.head"), B("logits"), {"var": "seqs"}, err]},
            pick_call(),
        ]

    prefill = [{"op": "embed", "label": "embed", "args": [B("token_ids"), B("w.embed"), B("x"), err]},
               {"op": "attn_plan", "label": "plan", "args": [B("cu_seqlens"), B("work"), B("work_count"), {"var": "seqs"},
                                                              {"expr": C.attn_plan_items(hq, hk)}, B("work_d"),
                                                              B("work_d_count")]}]
    decode = [{"op": "embed", "label": "embed", "args": [B("token_ids"), B("w.embed"), B("x"), err]}]
    for i in range(cfg.layers):
        prefill += layer(i, True)
        decode += layer(i, False)
    programs = {"load": {"once": True, "calls": [{"op": "rope_table", "args": [B("rope_cos"), B("rope_sin")]}]}}
    if hosted:
        from ..hosted import kv_shape

        shape, strides = kv_shape(hk, cfg.page_size, d)
        for name in states:
            states[name] = {"host": {"dtype": "bf16", "shape": shape, "strides": strides}}   # sized by the host
        for name in ("last", "last_n", "next_token"):
            bufs.pop(name)
        bufs["hidden"] = {"dtype": "bf16", "shape": ["tokens", h], "kind": "output"}
        bufs["head_in"] = {"dtype": "bf16", "shape": ["tokens", h], "kind": "input"}
        bufs["logits"] = {"dtype": "bf16", "shape": ["tokens", cfg.vocab], "kind": "output"}
        ops.pop("norm_last"); ops.pop("last_row"); ops.pop("pick")
        ops["lm_head"] = C.gemm_op(cfg.vocab, h, rows_max=T)
        final = [{"op": "norm", "label": "final_norm", "args": [B("x"), B("w.norm"), B("hidden")]}]
        programs.update({
            "prefill": {"batch": {"groups": S, "rows": "tokens"}, "calls": prefill + final},
            "decode": {"batch": {"groups": S, "rows": 1}, "graph": True, "calls": decode + final},
            "head": {"calls": [{"op": "lm_head", "label": "lm_head",
                                "args": [B("head_in"), B("w.head"), B("logits"), {"var": "tokens"}, err]}]}})
    else:
        prefill += [{"op": "last_row", "label": "last_row", "args": [B("x"), B("last"), B("cu_seqlens")]}] + head("last")
        decode += head("x")
        programs.update({"prefill": {"batch": {"groups": S, "rows": "tokens"}, "calls": prefill},
                         "decode": {"batch": {"groups": S, "rows": 1}, "graph": True, "calls": decode}})

    mods = ["norm_embed", "gemm_bf16", "attn_prep", "attn_paged"] + ([] if hosted else ["misc", "sampling"])
    return C.ensure_modules({
        "schema_version": 7,
        "model": cfg.name,
        "vars": {"tokens": {"max": T, "axis": "rows"}, "seqs": {"max": S, "axis": "groups"}},
        "states": states,
        "buffers": bufs,
        "modules": C.modules_for(mods),
        "ops": ops,
        "programs": programs,
    })


def load_random_weights(rt, cfg: DenseConfig, seed: int = 0, std: float = 0.02) -> None:
    """Fill a runtime's weight buffers with the synthetic checkpoint, generated tensor by tensor on the
    runtime's own device (no file, no host copy): the benchmark's random-init weights."""
    shapes = weight_names(cfg)
    order = {n: i for i, n in enumerate(shapes)}

    def provider(name: str) -> torch.Tensor:
        dev = rt.tensor(next(iter(rt.doc["buffers"]))).device
        g = torch.Generator(device=dev).manual_seed(seed * 1000003 + order[name])
        if name.endswith("norm.weight"):
            t = 1.0 + 0.1 * torch.randn(shapes[name], generator=g, device=dev)
        else:
            t = std * torch.randn(shapes[name], generator=g, device=dev)
        return t.to(torch.bfloat16)

    rt.load_tensors(provider)


# ---- PyTorch fp32 oracle ---------------------------------------------------------------------------
class DenseOracle:
    """Plain PyTorch statement of the decoder over the same checkpoint tensors (fp32 math by default).

    ``forward(tokens, cache)`` runs a list of token ids for one sequence after ``cache`` (a per-layer list
    of (k, v) tensors, grown in place) and returns logits ``[len(tokens), vocab]``."""

    def __init__(self, cfg: DenseConfig, weights: dict[str, torch.Tensor], dtype=torch.float32, device="cpu"):
        self.cfg, self.dtype, self.device = cfg, dtype, device
        self.w = {k: v.to(device=device, dtype=dtype) for k, v in weights.items()}

    def new_cache(self):
        return [[None, None] for _ in range(self.cfg.layers)]

    def _norm(self, x, w):
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.cfg.eps) * w.float()).to(self.dtype)

    def _rope(self, x, pos):
        d = self.cfg.head_dim
        half = d // 2
        inv = self.cfg.rope_theta ** (-torch.arange(0, half, dtype=torch.float64, device=x.device) * 2.0 / d)
        ang = pos.double()[:, None] * inv[None]
        cos, sin = ang.cos().float()[:, None], ang.sin().float()[:, None]
        xf = x.float()
        a, b = xf[..., :half], xf[..., half:]
        return torch.cat([a * cos - b * sin, b * cos + a * sin], -1).to(self.dtype)

    def mlp(self, i: int, xn: torch.Tensor) -> torch.Tensor:
        w, p = self.w, f"model.layers.{i}."
        act = torch.nn.functional.silu((xn @ w[p + "mlp.gate_proj.weight"].t()).float()) * (xn @ w[p + "mlp.up_proj.weight"].t()).float()
        return act.to(self.dtype) @ w[p + "mlp.down_proj.weight"].t()

    @torch.no_grad()
    def forward(self, tokens, cache) -> torch.Tensor:
        cfg, w = self.cfg, self.w
        ids = torch.as_tensor(tokens, dtype=torch.long, device=self.device)
        n = ids.numel()
        past = 0 if cache[0][0] is None else cache[0][0].shape[0]
        pos = torch.arange(past, past + n, device=self.device)
        x = w["model.embed_tokens.weight"][ids]
        g = cfg.heads // cfg.kv_heads
        for i in range(cfg.layers):
            p = f"model.layers.{i}."
            xn = self._norm(x, w[p + "input_layernorm.weight"])
            q = (xn @ w[p + "self_attn.q_proj.weight"].t()).view(n, cfg.heads, cfg.head_dim)
            k = (xn @ w[p + "self_attn.k_proj.weight"].t()).view(n, cfg.kv_heads, cfg.head_dim)
            v = (xn @ w[p + "self_attn.v_proj.weight"].t()).view(n, cfg.kv_heads, cfg.head_dim)
            if cfg.qk_norm:
                q = self._norm(q, w[p + "self_attn.q_norm.weight"])
                k = self._norm(k, w[p + "self_attn.k_norm.weight"])
            q, k = self._rope(q, pos), self._rope(k, pos)
            if cache[i][0] is not None:
                k = torch.cat([cache[i][0], k], 0)
                v = torch.cat([cache[i][1], v], 0)
            cache[i][0], cache[i][1] = k, v
            kk, vv = k.repeat_interleave(g, 1).float(), v.repeat_interleave(g, 1).float()
            s = torch.einsum("rhd,lhd->hrl", q.float(), kk) / math.sqrt(cfg.head_dim)
            mask = torch.arange(k.shape[0], device=self.device)[None, :] <= pos[:, None]
            s = s.masked_fill(~mask[None], float("-inf"))
            o = torch.einsum("hrl,lhd->rhd", torch.softmax(s, -1), vv).reshape(n, cfg.q_dim).to(self.dtype)
            x = x + o @ w[p + "self_attn.o_proj.weight"].t()
            xn = self._norm(x, w[p + "post_attention_layernorm.weight"])
            x = x + self.mlp(i, xn)
        xn = self._norm(x, w["model.norm.weight"])
        head = w["model.embed_tokens.weight"] if cfg.tie_embeddings else w["lm_head.weight"]
        return (xn @ head.t()).float()

    def generate(self, prompt, steps: int):
        cache = self.new_cache()
        logits = self.forward(prompt, cache)
        out = [int(logits[-1].argmax())]
        for _ in range(steps - 1):
            logits = self.forward([out[-1]], cache)
            out.append(int(logits[-1].argmax()))
        return out
