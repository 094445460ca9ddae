"""Pieces of the A/B harness that need no engine: the delta store of span images."""
def test_delta_images_rebuild_every_image_and_keep_less_than_whole_copies():
    """A buffer's first image is kept whole, later ones as the 64-byte blocks that changed; any key rebuilds exactly, in
    recording order (one delta per ask) or out of it (from the first image again)."""
    import torch

    from kern_b200.testing.abtest import DeltaImages

    g = torch.Generator().manual_seed(0)
    imgs = [torch.randint(0, 256, (1000,), generator=g, dtype=torch.uint8)]
    for k in range(5):
        nxt = imgs[-1].clone()
        nxt[64 * k:64 * k + 10] += 1                 # one block changes
        nxt[999] = k                                 # and the odd tail past the last whole block
        imgs.append(nxt)
    d = DeltaImages()
    for k, im in enumerate(imgs):
        d.put(("step", k), "x", im)
    d.put(("step", 0), "y", imgs[3])                 # another buffer has its own chain
    for k in (0, 1, 2, 3, 4, 5, 2, 0, 5):            # in order, then back and forth
        assert torch.equal(d.get(("step", k), "x"), imgs[k]), k
    assert torch.equal(d.get(("step", 0), "y"), imgs[3]) and d.has(("step", 4), "x") and not d.has(("step", 9), "x")
    assert d.full_bytes == 7 * 1000 and d.kept_bytes < 2 * 1000 + 5 * (64 + 40 + 4) + 200
    got = d.get(("step", 1), "x")
    got[:] = 0                                       # what `get` returns is the caller's to change
    assert torch.equal(d.get(("step", 1), "x"), imgs[1])
