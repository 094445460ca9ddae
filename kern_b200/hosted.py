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


def plan_runs(cu_seqlens: list[int], rows_max: int, seqs_max: int, decode_rows: int = 1) -> list[dict]:
    """Cut a host batch into runs the manifest's programs take. `cu_seqlens`: the batch's cumulative new rows per
    sequence (length seqs + 1). A run is a range of whole sequences whose rows fit `rows_max` and whose count fits
    `seqs_max`; maximal stretches of sequences with exactly `decode_rows` new rows each become `decode` runs (a
    fixed-shape program that replays from a CUDA graph), everything else `prefill` runs (ragged). A host that orders
    decode rows first and prompt chunks after them (vLLM's batch order) thus gets one graph replay plus one ragged call.
    A single sequence with more rows than `rows_max` cannot be cut here (its chunks would need the earlier chunk's cache
    length): the host must chunk it, and this raises.
    Reference: crates/kern-py/python/kern_vllm/model.py:179-260 (runs of a batch)."""
    n = len(cu_seqlens) - 1
    rows = [cu_seqlens[i + 1] - cu_seqlens[i] for i in range(n)]
    for i, r in enumerate(rows):
        if r > rows_max:
            raise ValueError(f"sequence {i} brings {r} rows, above the manifest's {rows_max}: the host must chunk it")
        if r < 0:
            raise ValueError("cu_seqlens must not decrease")
    runs: list[dict] = []
    i = 0
    while i < n:
        if rows[i] == 0:                     # a sequence with nothing to do in this call
            i += 1
            continue
        kind = "decode" if rows[i] == decode_rows else "prefill"
        j, tot = i, 0
        while j < n and j - i < seqs_max and tot + rows[j] <= rows_max and rows[j] > 0 and \
                (rows[j] == decode_rows) == (kind == "decode"):
            tot += rows[j]
            j += 1
        runs.append({"program": kind, "seqs": (i, j), "rows": (cu_seqlens[i], cu_seqlens[j])})
        i = j
    return runs


def fresh_slots(positions, cu_seqlens, state_slots) -> list[int]:
    """State slots (per-sequence recurrent / conv state held by the host) that start a sequence in this call: the first
    new row of the sequence is position 0. The host hands out slots without clearing them; the forward pass of a
    recurrent layer reads its slot before it writes it, so these must be zeroed before the call.
    Reference: crates/kern-py/python/kern_vllm/model.py:262-300."""
    out = []
    for s in range(len(cu_seqlens) - 1):
        lo, hi = int(cu_seqlens[s]), int(cu_seqlens[s + 1])
        if hi > lo and int(positions[lo]) == 0 and int(state_slots[s]) >= 0:
            out.append(int(state_slots[s]))
    return out


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

    def limits(self) -> tuple[int, int]:
        """(rows_max, seqs_max) of the manifest's programs."""
        rows = [d["max"] for d in self.doc["vars"].values() if d.get("axis") == "rows"]
        seqs = [d["max"] for d in self.doc["vars"].values() if d.get("axis") != "rows"]
        return (min(rows) if rows else 1 << 30, min(seqs) if seqs else 1 << 30)

    def zero_fresh_states(self, states: dict[str, torch.Tensor], positions, cu_seqlens, state_slots) -> list[int]:
        """Zero the per-sequence state slots of the sequences that start in this call (every host-owned state declared
        `bytes_per_seq`); returns the slots."""
        slots = fresh_slots(positions.tolist() if hasattr(positions, "tolist") else positions,
                            cu_seqlens.tolist() if hasattr(cu_seqlens, "tolist") else cu_seqlens,
                            state_slots.tolist() if hasattr(state_slots, "tolist") else state_slots)
        if slots:
            for name, t in states.items():
                if self.doc["states"].get(name, {}).get("bytes_per_seq"):
                    t[torch.as_tensor(slots, device=t.device)] = 0
        return slots

    def forward_batch(self, cu_seqlens, stream: int | None = None, *, token_ids, positions, slot_mapping, seq_lens,
                      block_table, **more) -> torch.Tensor:
        """A whole host batch, cut into runs (`plan_runs`) when it exceeds what one program call takes or mixes decode
        rows with prompt chunks: every run is staged with its own slices (cu_seqlens rebased to the run) and enqueued in
        order; returns the `hidden` rows of the whole batch in the host's row order."""
        cu = [int(x) for x in (cu_seqlens.tolist() if hasattr(cu_seqlens, "tolist") else cu_seqlens)]
        rows_max, seqs_max = self.limits()
        runs = plan_runs(cu, rows_max, seqs_max)
        total = cu[-1]
        if len(runs) == 1 and runs[0]["rows"] == (0, total) and runs[0]["seqs"] == (0, len(cu) - 1):
            return self.forward(runs[0]["program"], total, len(cu) - 1, stream, token_ids=token_ids, positions=positions,
                                slot_mapping=slot_mapping, seq_lens=seq_lens, cu_seqlens=torch.as_tensor(cu, dtype=torch.int32),
                                block_table=block_table, **more)
        outs = []
        for run in runs:
            (s0, s1), (r0, r1) = run["seqs"], run["rows"]
            local_cu = torch.as_tensor([c - r0 for c in cu[s0:s1 + 1]], dtype=torch.int32)
            extra = {k: (v[s0:s1] if v is not None and hasattr(v, "shape") and v.shape[0] == len(cu) - 1 else v) for k, v in more.items()}
            h = self.forward(run["program"], r1 - r0, s1 - s0, stream, token_ids=token_ids[r0:r1], positions=positions[r0:r1],
                             slot_mapping=slot_mapping[r0:r1], seq_lens=seq_lens[s0:s1], cu_seqlens=local_cu,
                             block_table=block_table[s0:s1], **extra)
            outs.append(h.clone())          # the next run overwrites the program's output buffer
        return torch.cat(outs, 0) if outs else self.rt.tensor("hidden" if "hidden" in self.doc["buffers"] else "x")[:0]

    def logits(self, rows: int, stream: int | None = None) -> torch.Tensor:
        vars_ = {v: rows for v in self.doc["vars"]}
        if "head" in self.doc["programs"]:
            if stream is not None and hasattr(self.rt, "enqueue_after"):
                self.rt.enqueue_after("head", vars_, stream)
            else:
                self.rt.issue("head", vars_)
        return self.rt.tensor("logits")[:rows]
