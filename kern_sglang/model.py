"""``KernForCausalLM`` for SGLang: ``forward(input_ids, positions, forward_batch)`` stages SGLang's batch metadata
into the manifest's inputs, binds the pool's per-layer KV buffers (and the conv / recurrent state pools of hybrid
models) to the manifest's host states on first use, and enqueues `prefill` (extend) or `decode` on SGLang's stream.
SGLang's pools are token-granular (page size 1 unless configured): the manifest it is given must have been generated
with the pool's page size.
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
    def __init__(self, config, quant_config=None, prefix: str = ""):
        super().__init__()
        path = Path(getattr(config, "kern_manifest", os.environ.get("KERN_MANIFEST", "")))
        if not path.is_file():
            raise FileNotFoundError("set `kern_manifest` in the model's config.json (or KERN_MANIFEST) to the hosted manifest")
        self.doc = json.loads(path.read_text())
        self.weights_path = getattr(config, "kern_weights", os.environ.get("KERN_WEIGHTS"))
        self.model: HostedModel | None = None
        self.host_states = sorted((n for n, s in self.doc["states"].items() if s.get("host")), key=lambda n: (len(n), n))

    def load_weights(self, weights) -> None:
        gpu = torch.cuda.current_device()
        rt = Runtime(self.doc, weights=self.weights_path, gpu=gpu, stream=torch.cuda.current_stream(gpu).cuda_stream)
        rt.once()
        self.model = HostedModel(rt)
        for _ in weights:
            pass

    def _bind(self, forward_batch) -> None:
        pool = forward_batch.token_to_kv_pool
        states = {}
        for name in self.host_states:
            kind, layer = name.split(".l")
            i = int(layer)
            if kind == "kv":
                states[name] = pool.get_kv_buffer(i) if hasattr(pool, "get_kv_buffer") else pool.kv_buffer[i]
            else:                               # conv / recurrent state pools of hybrid models
                states[name] = forward_batch.req_to_token_pool.get_state_buffer(kind, i)
        self._host_states = states
        self.model.bind(states)

    def forward(self, input_ids: torch.Tensor, positions: torch.Tensor, forward_batch, **kw):
        if not self.model.bound:
            self._bind(forward_batch)
        tokens, seqs = input_ids.numel(), int(forward_batch.batch_size)
        decode = forward_batch.forward_mode.is_decode()
        rows = torch.ones(seqs, dtype=torch.int32) if decode else forward_batch.extend_seq_lens.int().cpu()
        cu = torch.nn.functional.pad(torch.cumsum(rows, 0), (1, 0)).int()
        # state pools of hybrid models are indexed by the request's pool index: a request that starts here gets a slot
        # SGLang has not cleared
        if any(self.doc["states"][n].get("bytes_per_seq") for n in self.host_states):
            self.model.zero_fresh_states(self._host_states, positions, cu, forward_batch.req_pool_indices)
        # a batch above the manifest's bounds is cut at request boundaries (`kern_b200.hosted.plan_runs`)
        hidden = self.model.forward_batch(cu, torch.cuda.current_stream().cuda_stream, token_ids=input_ids, positions=positions,
                                          slot_mapping=forward_batch.out_cache_loc, seq_lens=forward_batch.seq_lens,
                                          block_table=forward_batch.req_to_token_pool.req_to_token[forward_batch.req_pool_indices])
        return self.model.logits(hidden.shape[0] if decode else seqs, torch.cuda.current_stream().cuda_stream)


EntryClass = KernForCausalLM
