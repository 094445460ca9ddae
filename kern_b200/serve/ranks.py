"""Head-side accounting of every rank's pool, and the staging of one lockstep call for a rank group.

The head owns no GPU. It keeps one :class:`Pool` per rank (same geometry as that rank reported in its Hello), so a
lease, checkpoint or restore is a decision made here and sent to the ranks as acts (zero a slot, copy pages).
A sequence holds a :class:`GroupLease`: a lease on every member rank of its ``tp`` group, taken all-or-nothing. A call is
staged as one ``Item`` per member (same fills, that member's own page and line tables) and fanned out.
Reference counterpart: crates/kern-serve/src/ranks.rs:111-149 (Groups), :153-193 (Act/Order/Answer),
:199-275 (Row/Snapshot), :470-547 (lease/checkpoint/retire), :633-745 (stage), :781-850 (Staged),
:855-936 (Layout).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

from .. import _native, fills


class Groups:
    """World rank q is member q % t of tp group q // t."""

    def __init__(self, world: int, tp: int = 1):
        if world % tp:
            raise ValueError(f"a world of {world} does not tile into tp groups of {tp}")
        self.world, self.tp, self.count = world, tp, world // tp

    def members(self, g: int) -> list[int]:
        return list(range(g * self.tp, (g + 1) * self.tp))

    def group_of(self, q: int) -> int:
        return q // self.tp


class GroupLease:
    """One sequence's lease on every member rank of its group; reads like a single lease (the members' pools see
    the same operations in the same order, so their page and slot ids agree, which `lease` checks)."""

    def __init__(self, group: int, members: list):
        self.group, self.members = group, members

    pages = property(lambda self: self.members[0].pages)
    slot = property(lambda self: self.members[0].slot)
    capacity = property(lambda self: self.members[0].capacity)
    shared_pages = property(lambda self: self.members[0].shared_pages)

    def slots_of(self, a: int, b: int):
        return self.members[0].slots_of(a, b)

    def slot_of(self, pos: int) -> int:
        return self.members[0].slot_of(pos)

    def release(self) -> None:
        for m in self.members:
            m.release()


class GroupKept:
    """A frozen prefix held on every member (a prefix-cache entry or a checkpoint)."""

    def __init__(self, group: int, members: list):
        self.group, self.members = group, members

    len = property(lambda self: self.members[0].len)
    has_slot = property(lambda self: self.members[0].has_slot)
    pages = property(lambda self: self.members[0].pages)

    def page_ids(self):
        return self.members[0].page_ids()


class Layout:
    """Row split of one call over t ranks (sequence-parallel regions of a TP layer): contiguous blocks, as even as
    whole rows allow; a rank sees its own block first, then the others in rank order. ``blocks`` are the prefix
    sums of the block lengths in that rank's order, which is what the ``blocks`` fill carries."""

    def __init__(self, total: int, t: int):
        base, extra = divmod(total, t)
        self.lens = [base + (1 if i < extra else 0) for i in range(t)]
        self.starts = [sum(self.lens[:i]) for i in range(t)]
        self.total, self.t = total, t

    def order(self, member: int) -> list[int]:
        """Source row of every row of `member`'s view."""
        ranks = [member] + [r for r in range(self.t) if r != member]
        return [self.starts[r] + i for r in ranks for i in range(self.lens[r])]

    def blocks(self, member: int) -> list[int]:
        ranks = [member] + [r for r in range(self.t) if r != member]
        out, at = [0], 0
        for r in ranks:
            at += self.lens[r]
            out.append(at)
        return out


@dataclass
class Staged:
    group: int
    call: fills.Call
    seqs: list
    new: list[list[int]]

    def emitted(self, answers: list[dict]) -> list[list[int]]:
        """Tokens per real sequence; every member must have emitted the same ones."""
        first = answers[0]
        for a in answers[1:]:
            if a["tokens"] != first["tokens"] or a.get("counts") != first.get("counts"):
                raise RuntimeError(f"members of group {self.group} disagree on the emitted tokens")
        toks, counts = first["tokens"], first.get("counts") or []
        out = []
        for i in range(self.call.real):
            n = int(counts[i]) if counts else 1
            out.append([int(x) for x in toks[i][:n]])
        return out

    def commit(self) -> None:
        for sq, new in zip(self.seqs, self.new):
            sq.length += len(new)
            sq.tokens.extend(new)


class Ranks:
    """`by_position`: the groups are decode context-parallel groups (a member manifest of `models/dense_dcp.py`): the
    batch is replicated like a tensor-parallel group's, but member m of w holds positions p = m (mod w) at local position
    p // w, so its lease covers its own share of the tokens, its page table is its own, and a new token's slot is its
    dealt slot on the owner and -1 (skipped by the append kernel) on the others. Prefix checkpoints are whole-sequence
    objects and are not taken for such groups (a request's context arrives by a dealt push from a prefill tier).
    Reference: crates/kern-serve/src/ranks.rs:313-369 (replicated groups)."""

    def __init__(self, protocol: dict, unit: int, pages: list[int], slots: list[int], tp: int = 1, by_position: bool = False):
        self.p, self.unit = protocol, unit
        self.by_position = by_position
        self.groups = Groups(len(pages), tp)
        row_pages = min((t["width"] * t["stride"] // unit for t in protocol["page_tables"]), default=0)
        # every member of a group gets the group's smallest geometry: identical pools fed identical operations
        # hand out identical page and slot ids, which is what lets one table row serve the whole group
        gmin = lambda v, q: min(v[r] for r in self.groups.members(self.groups.group_of(q)))
        self.pools = [_native.Pool(unit, gmin(pages, q), gmin(slots, q), row_pages) for q in range(len(pages))]
        self.acts: list[list[dict]] = [[] for _ in pages]      # queued for each rank's next order

    # ---- memory decisions (all-or-nothing over the members) ----
    def _each(self, g: int, fn):
        done = []
        try:
            for m, q in enumerate(self.groups.members(g)):
                done.append(fn(m, q))
        except _native.Denied:
            for d in done:
                lease = d[0] if isinstance(d, tuple) else d
                if hasattr(lease, "release"):
                    lease.release()
            raise
        return done

    def queue_copies(self, g: int, copies: dict) -> None:
        for q, c in zip(self.groups.members(g), copies.get("members", [])):
            if c["pages"] or c["slot"] is not None:
                self.acts[q].append({"copy": {"pages": [list(x) for x in c["pages"]],
                                              "slot": list(c["slot"]) if c["slot"] is not None else None}})

    def queue_zero(self, g: int, slot: int) -> None:
        for q in self.groups.members(g):
            self.acts[q].append({"zero": slot})

    @staticmethod
    def _copies(per_member: list[dict]) -> dict:
        """The members' copy lists in one dict shaped like a single pool's (`slot` tells a restored state apart
        from a fresh one), with the per-member lists under `members`."""
        return {"pages": per_member[0]["pages"], "slot": per_member[0]["slot"], "members": per_member}

    def lease(self, g: int, tokens: int) -> GroupLease:
        if self.by_position:
            w = self.groups.tp
            # member m's share of the first `tokens` positions: tokens // w, one more for the first tokens % w members
            return GroupLease(g, self._each(g, lambda m, q: self.pools[q].lease(max(1, tokens // w + (1 if m < tokens % w else 0)))))
        leases = self._each(g, lambda m, q: self.pools[q].lease(tokens))
        if any(l.slot != leases[0].slot or l.pages != leases[0].pages for l in leases[1:]):
            raise RuntimeError(f"group {g}: member pools have diverged")
        return GroupLease(g, leases)

    def _whole_sequences_only(self, what: str) -> None:
        if self.by_position:
            raise NotImplementedError(f"{what}: a group that deals positions over its members keeps no whole-sequence prefixes")

    def checkpoint(self, lease: GroupLease, n: int):
        self._whole_sequences_only("checkpoint")
        got = [self.pools[q].checkpoint(l, n) for q, l in zip(self.groups.members(lease.group), lease.members)]
        return GroupKept(lease.group, [c for c, _ in got]), self._copies([cp for _, cp in got])

    def restore(self, kept: GroupKept, n: int, tokens: int):
        self._whole_sequences_only("restore")
        got = self._each(kept.group, lambda m, q: self.pools[q].restore(kept.members[m], n, tokens))
        return GroupLease(kept.group, [l for l, _ in got]), self._copies([cp for _, cp in got])

    def fork(self, lease: GroupLease, n: int, tokens: int):
        self._whole_sequences_only("fork")
        got = self._each(lease.group, lambda m, q: self.pools[q].fork(lease.members[m], n, tokens))
        return GroupLease(lease.group, [l for l, _ in got]), self._copies([cp for _, cp in got])

    def retire(self, lease: GroupLease, n: int) -> GroupKept:
        return GroupKept(lease.group, [self.pools[q].retire(l, n)
                                       for q, l in zip(self.groups.members(lease.group), lease.members)])

    # ---- one call ----
    def _entries(self, batch, member: int) -> list[fills.Entry]:
        out = []
        w = self.groups.tp
        for sq, new in batch:
            l = sq.lease.members[member]
            if self.by_position:
                # position p lives on member p % w at local position p // w; the other members skip the row
                slots = [l.slot_of(p // w) if p % w == member else -1 for p in range(sq.length, sq.length + len(new))]
            else:
                slots = l.slots_of(sq.length, sq.length + len(new))
            out.append(fills.Entry(length=sq.length, new=new, pages=l.pages, slot=l.slot, slots=slots, sampling=sq.sampling))
        return out

    def stage(self, g: int, batch: list, pad: int = 0, round: bool = False) -> Staged:
        """`batch`: [(sequence, new tokens)] where a sequence carries `.lease` (a GroupLease), `.length`, `.sampling`."""
        call = fills.build(self.p, self.unit, self._entries(batch, 0), pad, round=round)
        return Staged(group=g, call=call, seqs=[sq for sq, _ in batch], new=[new for _, new in batch])

    def item_for(self, staged: Staged, member: int, read: bool = True) -> dict:
        """The member's own view of the call: same fills, its own leases' tables and slots."""
        call = staged.call
        cols = call.columns
        fw_round = call.forward["count"] is not None and call.forward["rows"] not in (1, "var")
        if member > 0:
            cols = fills.build(self.p, self.unit, self._entries(list(zip(staged.seqs, staged.new)), member),
                               call.groups - call.real, round=fw_round).columns
        fw = call.forward
        return {"program": call.program, "vars": call.vars, "groups": call.groups, "emits": fw["emits"], "count": fw["count"],
                "read": read, "rows": {n: [dt, v.tolist()] for n, (dt, v) in cols.items()}}

    def orders(self, staged: list[Staged], read: bool = True) -> list[dict | None]:
        """One order per world rank: its queued acts plus (if its group runs) its item. Ranks with neither get None."""
        out: list[dict | None] = [None] * self.groups.world
        for st in staged:
            for m, q in enumerate(self.groups.members(st.group)):
                out[q] = {"acts": self.acts[q], "item": self.item_for(st, m, read)}
                self.acts[q] = []
        for q in range(self.groups.world):
            if out[q] is None and self.acts[q]:
                out[q] = {"acts": self.acts[q]}
                self.acts[q] = []
        return out


class GroupPool:
    """One group's pools behind the single-pool interface the scheduler speaks."""

    def __init__(self, ranks: Ranks, g: int):
        self.ranks, self.g = ranks, g
        self._first = ranks.pools[ranks.groups.members(g)[0]]

    unit = property(lambda self: self._first.unit)
    total_pages = property(lambda self: self._first.total_pages)
    free_pages = property(lambda self: min(self.ranks.pools[q].free_pages for q in self.ranks.groups.members(self.g)))
    free_slots = property(lambda self: min(self.ranks.pools[q].free_slots for q in self.ranks.groups.members(self.g)))

    def pages_for(self, tokens: int) -> int:
        return self._first.pages_for(tokens)

    def room(self, pages: int, slot: bool) -> bool:
        return all(self.ranks.pools[q].room(pages, slot) for q in self.ranks.groups.members(self.g))

    def lease(self, tokens: int):
        return self.ranks.lease(self.g, tokens)

    def checkpoint(self, lease, n):
        return self.ranks.checkpoint(lease, n)

    def restore(self, kept, n, tokens):
        return self.ranks.restore(kept, n, tokens)

    def fork(self, lease, n, tokens):
        return self.ranks.fork(lease, n, tokens)

    def retire(self, lease, n):
        return self.ranks.retire(lease, n)


class GroupEngine:
    """The engine interface (open / close / step, `.pool`, `.rt.run_copies/zero_slot`) over one rank group behind
    executors: the same scheduler drives one local GPU or a tensor-parallel group of rank processes."""

    class _Acts:
        def __init__(self, ranks, g):
            self.ranks, self.g = ranks, g

        def run_copies(self, copies: dict) -> None:
            self.ranks.queue_copies(self.g, copies)

        def zero_slot(self, slot: int) -> None:
            self.ranks.queue_zero(self.g, slot)

    def __init__(self, executors, protocol: dict, unit: int, tp: int = 1, group: int = 0, ranks: Ranks | None = None,
                 by_position: bool = False):
        self.ex, self.p, self.unit, self.g = executors, protocol, unit, group
        self.ranks = ranks or Ranks(protocol, unit, executors.pages, executors.slots, tp, by_position=by_position)
        self.pool = GroupPool(self.ranks, group)
        self.rt = self._Acts(self.ranks, group)
        self.rows_max, self.groups_max = protocol["rows"]["max"], protocol["groups"]["max"]
        self.forwards, self.page_tables = protocol["forwards"], protocol["page_tables"]
        self.steps = 0

    def open(self, tokens_capacity: int, sampling=None):
        from ..engine import Sequence

        lease = self.pool.lease(tokens_capacity)
        if lease.slot >= 0:
            self.rt.zero_slot(lease.slot)
        return Sequence(lease=lease, sampling=sampling or fills.Sampling())

    def close(self, seq) -> None:
        seq.lease.release()

    def step(self, batch, eager: bool = False, read: bool = True, timed: bool = False, pad: int = 0, round: bool = False):
        if not batch or sum(len(t) for _, t in batch) == 0:
            return []
        staged = self.ranks.stage(self.g, batch, pad, round)
        answers = self.ex.run(self.ranks.orders([staged], read))
        staged.commit()
        self.steps += 1
        if not read or staged.call.forward["emits"] is None:
            return None
        return staged.emitted([answers[q] for q in self.ranks.groups.members(self.g)])
