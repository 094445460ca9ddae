"""``KernForCausalLM``: the vLLM model class over a hosted kern_b200 manifest.

vLLM calls ``forward(input_ids, positions)`` inside its own forward context (which carries the attention metadata
and the KV-cache tensors it allocated through `KernAttentionBackend`) and ``compute_logits(hidden)``. On the first
call the KV tensors of every layer are bound to the manifest's host states ``kv.l<i>``; the batch is cut into
runs (`kern_b200.hosted.plan_runs`): stretches of one-row sequences run `decode`, the rest `prefill`, and a batch above
the manifest's bounds is cut at sequence boundaries; per-sequence state slots of sequences that start in the call are zeroed.
Under tensor parallelism every rank runs its shard's manifest and the logits are all-gathered by vLLM.
Reference counterpart: crates/kern-py/python/kern_vllm/model.py:179-374.
"""
from __future__ import annotations

import json
import os
from pathlib import Path

import torch
from torch import nn

from kern_b200.hosted import HostedModel
from kern_b200.runtime import Runtime


class KernForCausalLM(nn.Module):
    def __init__(self, *, vllm_config, prefix: str = ""):
        super().__init__()
        cfg = vllm_config.model_config.hf_config
        self.manifest_path = Path(getattr(cfg, "kern_manifest", os.environ.get("KERN_MANIFEST", "")))
        if not self.manifest_path.is_file():
            raise FileNotFoundError("set `kern_manifest` in the model's config.json (or KERN_MANIFEST) to the hosted manifest")
        self.weights_path = getattr(cfg, "kern_weights", os.environ.get("KERN_WEIGHTS"))
        self.doc = json.loads(self.manifest_path.read_text())
        self.model: HostedModel | None = None
        self.kv_states = sorted((n for n, s in self.doc["states"].items() if s.get("host")), key=lambda n: (len(n), n))
        self._anchor = nn.Parameter(torch.zeros(1), requires_grad=False)      # vLLM moves the module; this marks the device
        self._host_states: dict[str, torch.Tensor] = {}

    def load_weights(self, weights) -> set[str]:
        """vLLM's loader offers (name, tensor) pairs; the runtime reads the checkpoint itself (bind rules need whole files)."""
        gpu = self._anchor.device.index or 0
        rt = Runtime(self.doc, weights=self.weights_path, gpu=gpu, stream=torch.cuda.current_stream(gpu).cuda_stream)
        rt.once()
        self.model = HostedModel(rt)
        return {n for n, _ in weights}

    def _bind(self, kv_caches: list[torch.Tensor]) -> None:
        self._host_states = {name: kv for name, kv in zip(self.kv_states, kv_caches)}
        self.model.bind(self._host_states)

    def forward(self, input_ids: torch.Tensor, positions: torch.Tensor, intermediate_tensors=None, inputs_embeds=None):
        from vllm.forward_context import get_forward_context

        ctx = get_forward_context()
        md = ctx.attn_metadata
        if isinstance(md, dict):
            md = next(iter(md.values()))
        if not self.model.bound:
            self._bind([layer.kv_cache[ctx.virtual_engine] for layer in ctx.no_compile_layers.values() if hasattr(layer, "kv_cache")])
        stream = torch.cuda.current_stream().cuda_stream
        cu = md.query_start_loc
        # the host's per-sequence state slots (recurrent / conv state of hybrid models): a sequence that starts in this
        # call gets a slot the host has not cleared
        state_slots = getattr(md, "state_indices_tensor", None)
        if state_slots is not None and self._host_states:
            self.model.zero_fresh_states(self._host_states, positions, cu, state_slots)
        # decode rows and prompt chunks of one vLLM batch run as a graph-replayed `decode` call plus a ragged `prefill`
        # call; a batch above the manifest's bounds is cut at sequence boundaries
        more = {"state_slots": state_slots} if state_slots is not None else {}
        return self.model.forward_batch(cu, stream, token_ids=input_ids, positions=positions, slot_mapping=md.slot_mapping,
                                        seq_lens=md.seq_lens, block_table=md.block_table_tensor, **more)

    def compute_logits(self, hidden_states: torch.Tensor, sampling_metadata=None) -> torch.Tensor:
        rows = hidden_states.shape[0]
        head_in = self.model.rt.tensor("head_in") if "head_in" in self.doc["buffers"] else None
        if head_in is not None:
            head_in[:rows].copy_(hidden_states)
        return self.model.logits(rows, torch.cuda.current_stream().cuda_stream).float()
