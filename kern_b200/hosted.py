"""Running inside another serving engine (vLLM- or SGLang-style hosts): the host owns the KV cache, the scheduler
and the sampler; this side owns the forward pass.

The hosted-manifest contract:
  * every paged / per-sequence state is declared `host` (dtype, shape with a free leading page count, strides): the
    host allocates it, `bind(host_tensors)` checks each tensor against the declaration and wires its address in;
  * inputs the host fills before every call: token_ids, positions, slot_mapping, seq_lens, cu_seqlens, block_table
    (+ line tables by their domain);
  * programs `prefill` / `decode` leave `hidden` (last-layer rows); `head` turns the rows named by `head_in` into
    `logits`;
  * `forward(...)` enqueues the program on the host's current stream after the host's own work
    (`Runtime.enqueue_after`): no synchronisation on this side.
`to_hosted(doc)` derives such a manifest from a self-hosted one by marking its states `host`.
Reference counterpart: crates/kern-py/python/kern/host.py:18-52, kern_vllm/model.py:1-42 (the contract),
kern_sglang/model.py:1-52.
"""
from __future__ import annotations

import copy

import numpy as np
import torch

_TORCH = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32, "u8": torch.uint8, "i32": torch.int32,
          "i64": torch.int64}
_NAME = {v: k for k, v in _TORCH.items()}


def kv_shape(kv_heads: int, page_size: int, head_dim: int) -> tuple[list[int], list[int]]:
    """(shape, strides in elements) of one layer's paged KV as the attention kernels read it:
    [pages, 2 (k|v), kv_heads, page_size, head_dim], contiguous; the page count is the host's choice (0 = free)."""
    shape = [0, 2, kv_heads, page_size, head_dim]
    strides = [2 * kv_heads * page_size * head_dim, kv_heads * page_size * head_dim, page_size * head_dim, head_dim, 1]
    return shape, strides


def to_hosted(doc: dict, layouts: dict[str, tuple[str, list[int], list[int]]]) -> dict:
    """Mark the named states as host-owned. `layouts`: state -> (dtype, shape, strides in elements)."""
    out = copy.deepcopy(doc)
    for name, (dtype, shape, strides) in layouts.items():
        st = out["states"][name]
        st["host"] = {"dtype": dtype, "shape": list(shape), "strides": list(strides)}
    return out


def region_of(t: torch.Tensor) -> tuple[int, str, list[int], list[int]]:
    """A host tensor as `bind_host` wants it: (address, dtype, shape, strides in elements)."""
    return (t.data_ptr(), _NAME[t.dtype], list(t.shape), list(t.stride()))


class HostedModel:
    """The forward pass of a hosted manifest, driven by a host engine's tensors."""

    def __init__(self, rt):
        self.rt = rt
        self.doc = rt.doc
        self.bound = False
        self.inputs = {n for n, b in self.doc["buffers"].items() if b["kind"] == "input"}

    def bind(self, states: dict[str, torch.Tensor]) -> None:
        """Once the host has allocated its caches: one tensor per host state."""
        if hasattr(self.rt, "bind_host_tensors"):          # host-memory executor: shares the tensors themselves
            self.rt.bind_host_tensors(states)
        else:
            self.rt.bind_host({name: region_of(t) for name, t in states.items()})
        self.bound = True

    def stage(self, **columns) -> None:
        """Copy the host's metadata tensors into the manifest's inputs (device-to-device when both are on the GPU)."""
        for name, t in columns.items():
            if name not in self.inputs or t is None:
                continue
            dst = self.rt.tensor(name).view(-1)
            src = t.reshape(-1)
            if src.device.type == "cpu" and dst.device.type != "cpu":
                self.rt.write(name, src.contiguous())
            else:
                dst[: src.numel()].copy_(src.to(dst.dtype), non_blocking=True)

    def forward(self, program: str, tokens: int, seqs: int, stream: int | None = None, **columns) -> torch.Tensor:
        """Stage the inputs, enqueue the program behind the host's stream, return the `hidden` rows (a view)."""
        if not self.bound and getattr(self.rt, "awaits_host", False):
            raise RuntimeError("host states are not bound yet")
        self.stage(**columns)
        vars_ = {}
        for v, decl in self.doc["vars"].items():
            vars_[v] = tokens if decl.get("axis") == "rows" else seqs
        if stream is not None and hasattr(self.rt, "enqueue_after"):
            self.rt.enqueue_after(program, vars_, stream)
        else:
            self.rt.issue(program, vars_)
        out = "hidden" if "hidden" in self.doc["buffers"] else "x"
        return self.rt.tensor(out)[:tokens]

    def logits(self, rows: int, stream: int | None = None) -> torch.Tensor:
        vars_ = {v: rows for v in self.doc["vars"]}
        if "head" in self.doc["programs"]:
            if stream is not None and hasattr(self.rt, "enqueue_after"):
                self.rt.enqueue_after("head", vars_, stream)
            else:
                self.rt.issue("head", vars_)
        return self.rt.tensor("logits")[:rows]
