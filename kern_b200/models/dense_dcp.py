"""The dense decoder as a member of a decode context-parallel group: weights and the batch are replicated, the KV of
every sequence is dealt over the members by position (position p on member p % w at local index p / w), and the decode
attention is partial attention over the member's own pages + an all-gather of the partials + one merge.

The manifest is the one-GPU decoder with its `decode` program kept, `prefill` dropped (a context-parallel group only
decodes: the context arrives dealt from a prefill tier, `ops/attention.deal_rows`), and `attn_decode` replaced. The
host fills positions and whole sequence lengths as always; the slot of a new token is its local slot on the owning
member and -1 elsewhere (nothing appended).
Reference: docs/pool.md:199-211 (`shard: by position`), crates/kern-pool/src/deal.rs:26 (Interleave).
"""
from __future__ import annotations

from . import common as C
from . import dense


def build_manifest_dcp(cfg: dense.DenseConfig, world: int, splits: int = 4, group: str = "dcp") -> dict:
    doc = dense.build_manifest(cfg)
    hq, hk, d = cfg.heads, cfg.kv_heads, cfg.head_dim
    doc["model"] = f"{doc['model']}-dcp{world}"
    doc["topology"] = {"groups": {group: world}}
    doc["programs"].pop("prefill")
    for name in ("attn_prefill", "attn_plan", "last_row"):
        doc["ops"].pop(name, None)
    for name in ("work", "work_count", "work_d", "work_d_count", "cu_seqlens", "last"):
        doc["buffers"].pop(name, None)
    launched = {l.get("module") for op in doc["ops"].values() for l in op["impl"]["launches"]}
    for name in [m for m in doc["modules"] if m not in launched]:
        doc["modules"].pop(name)          # modules only the dropped ops used
    for st in doc["states"].values():
        st["shard"] = {"by": "position", "group": group}
    doc["ops"]["attn_decode"] = C.attn_decode_dcp_op(hq, hk, d, cfg.page_size, cfg.table_width, cfg.qkv_dim, world, group, splits)
    extra = [{"expr": {"mul": ["seqs", hq * splits * d]}}, {"expr": {"mul": ["seqs", hq * splits * 2]}},
             {"expr": {"mul": ["seqs", hq]}}, {"var": "seqs"}]
    for call in doc["programs"]["decode"]["calls"]:
        if call["op"] == "attn_decode":
            call["args"] = call["args"] + extra
    return doc


def dealt_slot(position: int, pages: list[int], page_size: int, rank: int, world: int) -> int:
    """The KV slot of `position` on member `rank` (its pages hold its local positions), or -1 on the other members."""
    if position % world != rank:
        return -1
    li = position // world
    return pages[li // page_size] * page_size + li % page_size


def dealer(cfg: dense.DenseConfig):
    """How a prefill tier hands a prompt to a decode group of this family: the KV pages are [k|v][kv_head][page][d], not
    token-contiguous, so the rows are dealt by `kern_deal_rows_bf16` reading the prefill runtime's pool and writing every
    member's mapped pool (plain stores into peer memory), one launch per layer and member. -> f(rt, mirrors, src_pages,
    seats, length) for `serve/pd_serve.py`."""
    import torch

    from ..ops import attention as A
    from ..runtime import _CudaView

    def run(rt, mirrors, src_pages: list[int], seats: list[dict], length: int) -> None:
        dev = torch.device(f"cuda:{rt.gpu}")
        W = cfg.table_width
        world = len(seats)
        src_table = torch.zeros(1, W, dtype=torch.int32, device=dev)
        src_table[0, : len(src_pages)] = torch.tensor(src_pages, dtype=torch.int32)
        lens = torch.tensor([length], dtype=torch.int32, device=dev)
        rt.synchronize()                              # the prompt's rows are in this tier's pool
        with torch.cuda.device(dev):
            for m, seat in enumerate(seats):
                dst_table = torch.zeros(1, W, dtype=torch.int32, device=dev)
                dst_table[0, : len(seat["pages"])] = torch.tensor(seat["pages"], dtype=torch.int32)
                for i in range(cfg.layers):
                    name = f"kv.l{i}"
                    dst = torch.as_tensor(_CudaView(mirrors.mapped[m][name], (mirrors.sizes[m][name],), "|u1"), device=dev)
                    A.deal_rows(rt.tensor(name), dst, src_table, dst_table, lens, cfg.kv_heads, cfg.head_dim, cfg.page_size, m, world)
            torch.cuda.synchronize(dev)               # every member's share has landed before Start leaves

    return run
