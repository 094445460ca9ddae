"""Spec-round glue, device-side comparison and the gate kernels against their host statements."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_spec_splice_rows_accept(cuda):
    from kern_b200.ops import spec
    from kern_b200.ops.launcher import Kernels

    torch.manual_seed(0)
    seqs, block, dstride, page = 5, 6, 7, 16
    anchor = torch.randint(0, 1000, (seqs,), device=cuda)
    drafts = torch.randint(0, 1000, (seqs, dstride), device=cuda)
    ids = torch.zeros(seqs * block, dtype=torch.int64, device=cuda)
    spec.splice(anchor, None, ids, block, mask=77)
    assert ids.view(seqs, block)[:, 0].tolist() == anchor.tolist() and bool((ids.view(seqs, block)[:, 1:] == 77).all())
    spec.splice(anchor, drafts, ids, block, dstride)
    assert torch.equal(ids.view(seqs, block)[:, 1:], drafts[:, :block - 1])
    table = torch.randperm(40, device=cuda)[: seqs * 4].view(seqs, 4).int()
    base = torch.tensor([0, 15, 30, -1, 58], device=cuda)
    pos, slots, lens = spec.rows(base, table, block, page)
    torch.cuda.synchronize()
    Kernels.get(cuda).check_error()
    for i, b in enumerate(base.tolist()):
        for j in range(block):
            p = b + j
            want = -1 if b < 0 else int(table[i, p // page]) * page + p % page
            assert int(slots[i * block + j]) == want and int(pos[i * block + j]) == (0 if b < 0 else p)
        assert int(lens[i]) == (0 if b < 0 else b + block)
    verify = ids.clone().view(seqs, block)
    verify[:, :block - 1] = drafts[:, :block - 1]       # row j predicts what follows draft j
    verify[1, 2] += 1                                   # sequence 1 misses at draft 2
    verify[3, 0] += 1                                   # sequence 3 misses at once
    line_in = torch.zeros(2, 8, block, dtype=torch.int32, device=cuda)
    line_in[:, :seqs, 0] = torch.arange(1, seqs + 1, device=cuda).int()
    count, emitted, adv = spec.accept(drafts, verify.flatten(), block, dstride, line_in, 8)
    rc, re = spec.accept_reference(drafts, verify.flatten(), block, dstride)
    assert count.cpu().tolist() == rc.tolist() == [6, 3, 6, 1, 6]
    assert torch.equal(emitted.cpu(), re)
    for i in range(seqs):
        a = int(count[i]) - 1
        assert adv[0, i].tolist() == [i + 1 if e == a else 0 for e in range(block)]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_cmp_reduce_and_changed_blocks(cuda, dtype):
    from kern_b200.ops import compare

    torch.manual_seed(1)
    a = torch.randn(100_003, device=cuda).to(dtype)
    b = a.clone()
    assert compare.cmp_reduce(a, b).equal
    b[5] = -a[5] if float(a[5]) != 0 else 1.0
    b[77] = float("nan")
    a[900], b[900] = 0.0, -0.0
    a[901], b[901] = float("nan"), float("nan")
    b[50_000] = a[50_000] + a[50_000].abs() * 0.5 + 1
    got, ref = compare.cmp_reduce(a, b), compare.cmp_reference(a, b)
    assert (got.n_diff, got.signed_zero, got.nan_only_one_side, got.measured) == (ref.n_diff, ref.signed_zero, ref.nan_only_one_side, ref.measured) == (3, 1, 1, 2)
    assert abs(got.max_abs - ref.max_abs) <= 1e-6 * max(1.0, ref.max_abs) and got.max_ulp > 0
    pre = torch.zeros(1000 * 64 + 13, dtype=torch.uint8, device=cuda)
    post = pre.clone()
    post[64 * 3 + 1] = 1
    post[64 * 999 + 63] = 9
    post[64 * 1000 + 12] = 2
    ch = compare.changed_blocks(pre, post)
    assert ch.nonzero().flatten().tolist() == [3, 999, 1000]


def test_logit_rows(cuda):
    from kern_b200.ops import compare

    torch.manual_seed(2)
    a = torch.randn(7, 5000, device=cuda).to(torch.bfloat16)
    b = (a.float() + 0.05 * torch.randn(7, 5000, device=cuda)).to(torch.bfloat16)
    ia, ib, margin, kl = compare.logit_rows(a, b)
    assert ia.tolist() == a.float().argmax(-1).tolist() and ib.tolist() == b.float().argmax(-1).tolist()
    top2 = a.float().topk(2, -1).values
    torch.testing.assert_close(margin, top2[:, 0] - top2[:, 1], rtol=1e-5, atol=1e-6)
    la, lb = torch.log_softmax(a.float(), -1), torch.log_softmax(b.float(), -1)
    torch.testing.assert_close(kl, (la.exp() * (la - lb)).sum(-1), rtol=2e-2, atol=1e-5)


def test_hold_times_out_with_an_error_status_and_mark_publishes(cuda):
    """A wait that nothing satisfies gives up after its limit and reports; the context stays usable."""
    import struct

    from kern_b200.ops.launcher import Kernels, i32, i64, ptr

    k = Kernels.get(cuda)
    counter = torch.zeros(1, dtype=torch.int64, device=cuda)
    err = torch.zeros(1, dtype=torch.int32, device=cuda)
    u64 = lambda v: struct.pack("<Q", v)
    k.launch("signals", "kern_hold", (1,), (32,), [ptr(counter), u64(3), i64(2_000_000), ptr(err), i32(41)])   # 2 ms limit
    torch.cuda.synchronize()
    assert int(err) == 41
    err.zero_()
    for _ in range(3):
        k.launch("signals", "kern_arrive", (1,), (32,), [ptr(counter)])
    k.launch("signals", "kern_hold", (1,), (32,), [ptr(counter), u64(3), i64(2_000_000), ptr(err), i32(41)])
    k.launch("signals", "kern_mark", (1,), (32,), [ptr(counter), u64(99)])
    torch.cuda.synchronize()
    assert int(err) == 0 and int(counter) == 99
    out = torch.zeros(4, device=cuda)
    tot = torch.zeros(1, device=cuda)
    for i in range(3):
        k.launch("signals", "kern_lanes_step", (1,), (32,), [ptr(out), i32(i), struct.pack("<f", float(i + 1)), i64(100_000)])
    k.launch("signals", "kern_lanes_join", (1,), (32,), [ptr(out), ptr(tot), i32(3)])
    torch.cuda.synchronize()
    assert float(tot) == 6.0
