"""Block-scaled tcgen05 GEMMs (MXFP8 x MXFP8, MXFP8 x MXFP4) against a plain PyTorch fp32 statement over the dequantised
operands; the device quantiser against the same arithmetic in PyTorch; the scale-factor atom layout round trip."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_scale_atom_layout_round_trip():
    from kern_b200.ops import gemm_mx as G

    sf = torch.randint(100, 140, (300, 24), dtype=torch.uint8)
    atoms = G.sf_to_atoms(sf)
    assert atoms.numel() == G.atom_bytes(300, 24 * 32)
    assert torch.equal(G.atoms_to_sf(atoms, 300, 24 * 32), sf)
    # spot check of the documented offsets
    r, kb = 171, 13
    off = ((r // 128) * 6 + kb // 4) * 512 + (r % 32) * 16 + ((r // 32) % 4) * 4 + kb % 4
    assert int(atoms[off]) == int(sf[r, kb])


def _rand_operands(m, n, k, fp4, seed, cuda):
    from kern_b200.ops import gemm_mx as G

    g = torch.Generator(device="cpu").manual_seed(seed)
    a = torch.randn(m, k, generator=g) * torch.exp2(torch.randint(-3, 4, (m, k // 32), generator=g).float()).repeat_interleave(32, 1)
    w = torch.randn(n, k, generator=g) * torch.exp2(torch.randint(-3, 4, (n, k // 32), generator=g).float()).repeat_interleave(32, 1)
    aq, asf = G.quantize_mxfp8_torch(a)
    if fp4:
        wq, wsf = G.quantize_mxfp4_torch(w)
        wd = G.dequant_mxfp4(wq, wsf)
    else:
        wq, wsf = G.quantize_mxfp8_torch(w)
        wd = G.dequant_mxfp8(wq, wsf)
    want = G.dequant_mxfp8(aq, asf) @ wd.t()
    return aq.to(cuda), G.sf_to_atoms(asf).to(cuda), wq.to(cuda), G.sf_to_atoms(wsf).to(cuda), want


@pytest.mark.parametrize("fp4", [False, True])
@pytest.mark.parametrize("m,n,k,bn", [(128, 128, 128, 128), (128, 128, 512, 128), (300, 384, 1024, 128), (1000, 512, 2048, 256),
                                      (64, 7168, 2048, 128)])
def test_block_scaled_gemm_matches_fp32(cuda, fp4, m, n, k, bn):
    from kern_b200.ops import gemm_mx as G
    from kern_b200.ops.launcher import Kernels

    aq, asf, wq, wsf, want = _rand_operands(m, n, k, fp4, 7 + m + n, cuda)
    got = G.gemm_mx(aq, asf, wq, wsf, fp4, bn=bn)
    torch.cuda.synchronize()
    Kernels.get(cuda).check_error()
    err = (got.float().cpu() - want).abs().max().item()
    scale = want.abs().max().item()
    assert err <= 1e-2 * scale + 1e-3, (err, scale)


def test_device_quantiser_matches_torch(cuda):
    from kern_b200.ops import gemm_mx as G

    torch.manual_seed(3)
    x = (torch.randn(200, 512, device=cuda) * torch.exp2(torch.randint(-6, 7, (200, 16), device=cuda).float()).repeat_interleave(32, 1))
    x[5, 64:96] = 0                                     # an all-zero block keeps scale 1
    x = x.to(torch.bfloat16)
    q, atoms = G.quantize_mxfp8(x)
    torch.cuda.synchronize()
    q_ref, sf_ref = G.quantize_mxfp8_torch(x.cpu())
    sf = G.atoms_to_sf(atoms.cpu(), 200, 512)
    assert torch.equal(sf, sf_ref)
    assert torch.equal(q.cpu(), q_ref)
    back = G.dequant_mxfp8(q.cpu(), sf)
    rel = ((back - x.float().cpu()).abs() / (x.float().cpu().abs().amax(-1, keepdim=True) + 1e-9)).max().item()
    assert rel < 0.07


@pytest.mark.parametrize("t,h,inter,e,k,bn", [(64, 512, 256, 8, 2, 128), (300, 1024, 512, 16, 4, 256), (33, 2048, 768 + 256, 16, 3, 256)])
def test_routed_layer_mxfp4_experts(cuda, t, h, inter, e, k, bn):
    """Route -> aligned plan -> gather + quantise -> FC1 (SwiGLU, MXFP8 out) -> FC2 -> combine, against the fp32 statement
    with the same quantisation points."""
    from kern_b200.ops import moe
    from kern_b200.ops.launcher import Kernels

    torch.manual_seed(t + e)
    x = (torch.randn(t, h, device=cuda) * 0.5).to(torch.bfloat16)
    wr = (torch.randn(e, h, device=cuda) * 0.2).to(torch.bfloat16)
    w1 = (torch.randn(e, 2 * inter, h, device=cuda) * 0.05).to(torch.bfloat16)
    w2 = (torch.randn(e, h, inter, device=cuda) * 0.05).to(torch.bfloat16)
    w1q, sf1, w2q, sf2 = moe.prepare_expert_weights_mx(w1, w2)
    got = moe.moe_layer_mx(x, wr, w1q, sf1, w2q, sf2, k, scale=1.5, bn=bn)
    torch.cuda.synchronize()
    Kernels.get(cuda).check_error()
    ref = moe.moe_reference_mx(x, wr, w1, w2, k, scale=1.5)
    err = (got.float() - ref).abs().max().item()
    assert err <= 0.03 * ref.abs().max().item() + 2e-3, (err, ref.abs().max().item())
