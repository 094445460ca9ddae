"""Rank groups: who is who, and the handshake that maps every member's exported memory into the others.

One process per GPU. The handles of a rank's exported buffers travel over whatever channel the host
already has — here a `torch.distributed` process group (gloo or nccl object collectives) — and
`Runtime.connect` maps them and fills the manifest's `peer` buffers with the mapped addresses.
Rank numbering follows the reference: world rank q is member q % t of `tp` group q // t, and member q of
every other group (crates/kern-serve/src/executor.rs:86-111; crates/kern-py/python/kern/group.py:20-51).
"""
from __future__ import annotations

import torch.distributed as dist


def topology(groups: dict[str, int], rank: int, world: int) -> dict[str, tuple[int, int]]:
    """This rank's (index, size) in every group of a manifest's topology."""
    out = {}
    t = groups.get("tp", 1)
    for name, size in groups.items():
        if name == "tp":
            out[name] = (rank % size, size)
        elif size == world:
            out[name] = (rank, size)
        elif size * t == world:
            out[name] = (rank // t, size)     # one member per tp group
        else:
            raise ValueError(f"group `{name}` of {size} does not tile a world of {world} with tp={t}")
    return out


def members_of(groups: dict[str, int], group: str, rank: int, world: int) -> list[int]:
    """World ranks of the instance of `group` that `rank` belongs to, in member order."""
    t = groups.get("tp", 1)
    size = groups[group]
    if group == "tp":
        base = rank // size * size
        return [base + i for i in range(size)]
    if size == world:
        return list(range(world))
    return [i * t + rank % t for i in range(size)]


def connect(rt, pg=None) -> None:
    """Exchange offers over the process group and map every group's peers."""
    groups = rt.doc.get("topology", {}).get("groups", {})
    if not groups:
        return
    if not dist.is_initialized():
        # one process: every group has one member, whose peer tables hold its own addresses (a kernel that walks
        # the table must not find a null pointer there)
        for g in groups:
            rt.connect(g, [rt.offer()])
        return
    rank, world = dist.get_rank(pg), dist.get_world_size(pg)
    offers = [None] * world
    dist.all_gather_object(offers, rt.offer(), group=pg)
    for g in groups:
        rt.connect(g, [offers[r] for r in members_of(groups, g, rank, world)])


def start(rt, pg=None) -> None:
    """connect, run the `once` programs, and line everyone up before the first step."""
    connect(rt, pg)
    rt.once()
    rt.synchronize()
    if dist.is_initialized():
        dist.barrier(group=pg)
