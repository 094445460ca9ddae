"""Decode context parallelism, the parts that need no GPU: the member manifest verifies and projects its by-position
shards, and the host's dealing of a new token's slot agrees with the pool library's `deal`."""
import json

from kern_b200.models import dense, dense_dcp
from kern_b200.runtime import verify


def test_member_manifest_verifies_and_projects_shards():
    doc = dense_dcp.build_manifest_dcp(dense.TINY, 4)
    m, diags = verify(doc)
    assert m is not None, diags
    p = json.loads(m.protocol(sampled=False))
    assert p["shards"], p.keys()
    assert "prefill" not in doc["programs"]
    entries = [l["entry"] for l in doc["ops"]["attn_decode"]["impl"]["launches"]]
    assert entries == ["kern_dcp_prepare", "kern_attn_decode_paged_d64", "extern:nccl_allgather_f32", "extern:nccl_allgather_f32",
                       "kern_attn_merge_ranks"]
    from kern_b200 import schema
    assert schema.validate(doc) == []


def test_dealt_slot_follows_position_modulo_world():
    page = 16
    pages = [7, 9, 4]
    for world in (2, 4):
        for rank in range(world):
            owned = [p for p in range(90) if dense_dcp.dealt_slot(p, pages, page, rank, world) >= 0]
            assert owned == [p for p in range(90) if p % world == rank]
            for p in owned:
                li = p // world
                assert dense_dcp.dealt_slot(p, pages, page, rank, world) == pages[li // page] * page + li % page


def test_dense_decoder_as_a_two_rank_decode_group_over_gloo():
    """Two CPU ranks: each prefills on a whole-context runtime, deals its KV rows into its member pool, and the group
    decodes through partial attention + all-gather + merge; logits equal the whole-context decoder's."""
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29657", "-m", "kern_b200.parallel.dcp_check", "--cpu"]
    p = subprocess.run(cmd, cwd=root, env=dict(os.environ, PYTHONPATH=root), capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, (p.stdout[-2000:], p.stderr[-2000:])
    line = next(json.loads(l) for l in p.stdout.splitlines() if l.startswith("{"))
    assert line["ok"] and line["world"] == 2 and line["tokens_agree"] == line["of"], line


def test_ranks_stage_a_by_position_group():
    """The serving host's staging for a decode group that deals positions over its members: every member leases its own
    share of a sequence, its item carries its own page table, and a new token's slot is its dealt slot on the owner and
    -1 on the others."""
    from types import SimpleNamespace

    import pytest

    from kern_b200.serve.ranks import Ranks

    world = 4
    doc = dense_dcp.build_manifest_dcp(dense.TINY, world)
    m, _ = verify(doc)
    proto = json.loads(m.protocol(sampled=False))
    page = dense.TINY.page_size
    ranks = Ranks(proto, page, [64] * world, [8] * world, tp=world, by_position=True)
    lease = ranks.lease(0, 70)                                  # 70 positions: members hold 18, 18, 17, 17
    assert [l.capacity >= n for l, n in zip(lease.members, (18, 18, 17, 17))] == [True] * 4
    assert [len(l.pages) for l in lease.members] == [2, 2, 2, 2]
    seq = SimpleNamespace(lease=lease, length=37, sampling=None)
    from kern_b200.fills import Sampling
    seq.sampling = Sampling()
    staged = ranks.stage(0, [(seq, [5])])
    slot_name = next(f["name"] for f in proto["fills"] if f["fill"] == "slot")
    for member in range(world):
        item = ranks.item_for(staged, member)
        slot = item["rows"][slot_name][1][0]
        if 37 % world == member:
            assert slot == dense_dcp.dealt_slot(37, list(lease.members[member].pages), page, member, world) >= 0
        else:
            assert slot == -1
    with pytest.raises(NotImplementedError):
        ranks.checkpoint(lease, 32)
