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
