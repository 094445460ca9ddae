"""The hosted-manifest contract with a fake host engine: the host owns the KV tensors and the batch metadata, this
side runs prefill / decode / head; logits must match the oracle. Also the adapters' static pieces."""
import pytest
import torch

from kern_b200 import hosted
from kern_b200.cpu import CpuRuntime
from kern_b200.models import dense


def test_fake_host_prefill_decode_head():
    cfg = dense.TOY
    w = dense.random_weights(cfg, seed=6, std=0.08)
    doc = dense.build_manifest(cfg, hosted=True)
    rt = CpuRuntime(doc, weights=w)
    rt.once()
    model = hosted.HostedModel(rt)
    assert rt.awaits_host
    pages = 12
    kv = {f"kv.l{i}": torch.zeros(pages, 2, cfg.kv_heads, cfg.page_size, cfg.head_dim, dtype=torch.bfloat16) for i in range(cfg.layers)}
    with pytest.raises(ValueError):
        model.bind({"kv.l0": kv["kv.l0"]})                       # a layer is missing
    with pytest.raises(ValueError):
        model.bind({**kv, "kv.l1": torch.zeros(pages, 2, cfg.kv_heads, cfg.page_size + 1, cfg.head_dim, dtype=torch.bfloat16)})
    model.bind(kv)
    assert not rt.awaits_host
    oracle = dense.DenseOracle(cfg, w)
    # the host's view of two sequences: its own page assignment
    table = torch.tensor([[3, 7, 0, 0], [5, 1, 9, 0]], dtype=torch.int32)
    prompts = [torch.randint(1, cfg.vocab, (n,), generator=torch.Generator().manual_seed(n)).tolist() for n in (9, 21)]
    caches = [oracle.new_cache() for _ in prompts]
    lens = [0, 0]

    def call(new):
        rows = sum(len(t) for t in new)
        tok = torch.tensor([t for ts in new for t in ts])
        pos = torch.tensor([lens[i] + j for i, ts in enumerate(new) for j in range(len(ts))])
        slot = torch.tensor([int(table[i, p // cfg.page_size]) * cfg.page_size + p % cfg.page_size
                             for i, ts in enumerate(new) for p in range(lens[i], lens[i] + len(ts))])
        for i, ts in enumerate(new):
            lens[i] += len(ts)
        cu = torch.tensor([0] + [sum(len(t) for t in new[:i + 1]) for i in range(len(new))], dtype=torch.int32)
        program = "decode" if all(len(t) == 1 for t in new) else "prefill"
        hidden = model.forward(program, rows, len(new), None, token_ids=tok, positions=pos, slot_mapping=slot,
                               seq_lens=torch.tensor(lens, dtype=torch.int32), cu_seqlens=cu, block_table=table)
        last = hidden[(cu[1:] - 1).long()]                        # the host picks the rows it wants logits for
        rt.tensor("head_in")[: len(new)] = last
        return model.logits(len(new)).float()

    got = call(prompts)
    nxt = []
    for i, p in enumerate(prompts):
        ref = oracle.forward(p, caches[i])[-1]
        assert float((got[i] - ref).abs().max()) < 0.08
        nxt.append(int(ref.argmax()))
    for _ in range(3):
        got = call([[t] for t in nxt])
        for i in range(2):
            ref = oracle.forward([nxt[i]], caches[i])[-1]
            assert float((got[i] - ref).abs().max()) < 0.1
            nxt[i] = int(ref.argmax())
    assert float(kv["kv.l0"][3].abs().sum()) > 0 and float(kv["kv.l0"][2].abs().sum()) == 0     # written into the host's pages


def test_backend_declares_the_kernels_layout():
    pytest.importorskip("torch")
    from kern_vllm.backend import KERNEL_BLOCK, KernAttentionBackend

    assert KernAttentionBackend.get_kv_cache_shape(10, KERNEL_BLOCK, 8, 128) == (10, 2, 8, 64, 128)
    with pytest.raises(ValueError):
        KernAttentionBackend.get_kv_cache_shape(10, 16, 8, 128)
    shape, strides = hosted.kv_shape(8, 64, 128)
    assert shape[1:] == [2, 8, 64, 128] and strides == list(torch.empty(1, 2, 8, 64, 128).stride())


def test_plan_runs_cuts_a_host_batch():
    """Decode rows first and prompt chunks after them become one fixed-shape run and one ragged run; a batch above the
    manifest's bounds is cut at sequence boundaries; a sequence above the row bound is the host's to chunk."""
    cu = [0, 1, 2, 3, 10, 30]                                     # three decode rows, two prompt chunks
    runs = hosted.plan_runs(cu, rows_max=64, seqs_max=8)
    assert runs == [{"program": "decode", "seqs": (0, 3), "rows": (0, 3)}, {"program": "prefill", "seqs": (3, 5), "rows": (3, 30)}]
    runs = hosted.plan_runs(cu, rows_max=20, seqs_max=2)
    assert [(r["program"], r["seqs"]) for r in runs] == [("decode", (0, 2)), ("decode", (2, 3)), ("prefill", (3, 4)), ("prefill", (4, 5))]
    assert hosted.plan_runs([0, 5, 5, 9], 64, 8) == [{"program": "prefill", "seqs": (0, 1), "rows": (0, 5)},
                                                     {"program": "prefill", "seqs": (2, 3), "rows": (5, 9)}]
    with pytest.raises(ValueError):
        hosted.plan_runs([0, 100], rows_max=64, seqs_max=8)
    assert hosted.fresh_slots([0, 1, 2, 17, 0], [0, 3, 4, 5], [4, 2, 6]) == [4, 6]
    assert hosted.fresh_slots([0, 1], [0, 2], [-1]) == []


def test_a_mixed_host_batch_runs_as_decode_then_prefill_and_matches():
    """`forward_batch` on a batch that mixes decode rows with a new prompt (the order vLLM uses) and exceeds the
    sequence bound of one call: the runs' hidden rows, concatenated, give the same logits as the oracle."""
    import dataclasses

    cfg = dataclasses.replace(dense.TOY, max_seqs=2)              # two sequences per call: three need two runs
    w = dense.random_weights(cfg, seed=6, std=0.08)
    rt = CpuRuntime(dense.build_manifest(cfg, hosted=True), weights=w)
    rt.once()
    model = hosted.HostedModel(rt)
    kv = {f"kv.l{i}": torch.zeros(16, 2, cfg.kv_heads, cfg.page_size, cfg.head_dim, dtype=torch.bfloat16) for i in range(cfg.layers)}
    model.bind(kv)
    assert model.limits() == (cfg.max_tokens, 2)
    oracle = dense.DenseOracle(cfg, w)
    table = torch.tensor([[3, 7, 0, 0], [5, 1, 9, 0], [2, 4, 0, 0]], dtype=torch.int32)
    gen = torch.Generator().manual_seed(4)
    prompts = [torch.randint(1, cfg.vocab, (n,), generator=gen).tolist() for n in (9, 12, 14)]
    caches = [oracle.new_cache() for _ in prompts]
    lens = [0, 0, 0]

    def call(new, which):
        tok = torch.tensor([t for ts in new for t in ts])
        pos = torch.tensor([lens[i] + j for i, ts in zip(which, new) for j in range(len(ts))])
        slot = torch.tensor([int(table[i, p // cfg.page_size]) * cfg.page_size + p % cfg.page_size
                             for i, ts in zip(which, new) for p in range(lens[i], lens[i] + len(ts))])
        for i, ts in zip(which, new):
            lens[i] += len(ts)
        cu = [0]
        for ts in new:
            cu.append(cu[-1] + len(ts))
        hidden = model.forward_batch(cu, None, token_ids=tok, positions=pos, slot_mapping=slot,
                                     seq_lens=torch.tensor([lens[i] for i in which], dtype=torch.int32), block_table=table[which])
        last = hidden[[c - 1 for c in cu[1:]]]
        out = []
        for r in range(0, len(new), 2):                              # the head takes as many rows as a call has sequences
            n = min(2, len(new) - r)
            rt.tensor("head_in")[:n] = last[r:r + n]
            out.append(model.logits(n).float().clone())
        return torch.cat(out)

    got = call(prompts[:2], [0, 1])                                  # two prompts first
    nxt = [int(oracle.forward(p, caches[i])[-1].argmax()) for i, p in enumerate(prompts[:2])]
    # now: two decode rows and a new prompt in one host batch (three sequences: above the bound of one call)
    got = call([[nxt[0]], [nxt[1]], prompts[2]], [0, 1, 2])
    refs = [oracle.forward([nxt[0]], caches[0])[-1], oracle.forward([nxt[1]], caches[1])[-1], oracle.forward(prompts[2], caches[2])[-1]]
    for g, r in zip(got, refs):
        assert float((g - r).abs().max()) < 0.1
