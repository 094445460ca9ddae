"""tcgen05 bf16 GEMM against the PyTorch fp32 statement of the same op."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rand(m, n, device, scale=1.0):
    return (torch.randn(m, n, device=device, dtype=torch.float32) * scale).to(torch.bfloat16)


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (128, 256, 512), (256, 512, 1024), (1, 256, 128),
                                   (77, 384, 320), (300, 1000, 448), (2048, 4096, 4096)])
@pytest.mark.parametrize("bn", [None, 32, 64, 128, 256])
def test_gemm_store(cuda, m, n, k, bn):
    from kern_b200.ops.gemm import gemm, gemm_reference
    from kern_b200.ops.launcher import Kernels

    torch.manual_seed(m * 7 + n * 3 + k)
    a, w = _rand(m, k, cuda), _rand(n, k, cuda, 0.1)
    out = gemm(a, w, bn=bn)
    torch.cuda.synchronize()
    Kernels.get(cuda).check_error()
    ref = gemm_reference(a, w)
    torch.testing.assert_close(out.float(), ref.float(), rtol=2e-2, atol=2e-2 * (k ** 0.5) * 0.1)


@pytest.mark.parametrize("epilogue", ["f32", "acc", "swiglu"])
@pytest.mark.parametrize("m,n,k", [(64, 512, 256), (257, 1024, 768)])
def test_gemm_epilogues(cuda, epilogue, m, n, k):
    from kern_b200.ops.gemm import gemm, gemm_reference
    from kern_b200.ops.launcher import Kernels

    torch.manual_seed(1)
    a, w = _rand(m, k, cuda), _rand(n, k, cuda, 0.1)
    if epilogue == "acc":
        c = _rand(m, n, cuda)
        ref = gemm_reference(a, w, "acc", c.clone())
        out = gemm(a, w, out=c, epilogue="acc")
    else:
        out = gemm(a, w, epilogue=epilogue)
        ref = gemm_reference(a, w, epilogue)
    torch.cuda.synchronize()
    Kernels.get(cuda).check_error()
    torch.testing.assert_close(out.float(), ref.float(), rtol=2e-2, atol=3e-2)


def test_gemm_partial_rows_and_strided_a(cuda):
    from kern_b200.ops.gemm import gemm, gemm_reference

    torch.manual_seed(2)
    big = _rand(512, 1024, cuda)
    a = big[:, 256:768]  # row stride 1024, 512 columns
    w = _rand(384, 512, cuda, 0.1)
    out = torch.zeros(512, 384, device=cuda, dtype=torch.bfloat16)
    gemm(a, w, out=out, m=100)
    torch.cuda.synchronize()
    ref = gemm_reference(a[:100], w)
    torch.testing.assert_close(out[:100].float(), ref.float(), rtol=2e-2, atol=3e-2)
    assert float(out[100:].abs().max()) == 0.0


@pytest.mark.parametrize("m,n,k", [(128, 256, 128), (77, 384, 512), (300, 1024, 1024), (2048, 4096, 4096)])
def test_gemm_fp8_e4m3(cuda, m, n, k):
    """kind::f8f6f4 GEMM against fp32 math on the same quantised operands, and the quantiser against torch's cast."""
    from kern_b200.ops import gemm_fp8 as F8
    from kern_b200.ops.launcher import Kernels

    torch.manual_seed(m + n)
    a = (torch.randn(m, k, device=cuda) * 2).to(torch.bfloat16)
    w = (torch.randn(n, k, device=cuda) * 0.5).to(torch.bfloat16)
    aq, sa = F8.quantize(a)
    wq, sw = F8.quantize(w)
    torch.cuda.synchronize()
    assert abs(float(sa) - float(a.float().abs().max()) / 448) < 1e-6
    ref_q = (a.float() / sa).to(torch.float8_e4m3fn).view(torch.uint8)
    assert (aq != ref_q).float().mean() < 1e-3          # identical but for ties in rounding
    out = F8.gemm_fp8(aq, wq, sa, sw)
    torch.cuda.synchronize()
    Kernels.get(cuda).check_error()
    ref = F8.dequant(aq, sa) @ F8.dequant(wq, sw).t()
    torch.testing.assert_close(out.float(), ref, rtol=1.6e-2, atol=1e-2 * float(ref.abs().max()))
    res = torch.randn(m, n, device=cuda).to(torch.bfloat16)
    out2 = F8.gemm_fp8(aq, wq, sa, sw, residual=res, out=torch.empty_like(res))
    torch.testing.assert_close(out2.float(), ref + res.float(), rtol=1.6e-2, atol=1e-2 * float(ref.abs().max()))


@pytest.mark.parametrize("epilogue", ["store", "f32", "acc", "swiglu"])
@pytest.mark.parametrize("m,n,k", [(1, 256, 128), (2, 1000, 448), (3, 4096, 4096), (4, 776, 1024)])
def test_gemv_small_rows(cuda, epilogue, m, n, k):
    """A handful of rows take the weight-streaming kernel; same results as the fp32 statement."""
    from kern_b200.ops.gemm import GEMV_ROWS, gemm, gemm_reference
    from kern_b200.ops.launcher import Kernels

    assert m <= GEMV_ROWS
    if epilogue == "swiglu" and n % 16:
        n = n // 16 * 16
    torch.manual_seed(m * 7 + n)
    a = torch.randn(m + 3, k + 64, device=cuda).to(torch.bfloat16)[:m, :k]          # a strided view: lda != k
    w = (torch.randn(n, k, device=cuda) * k ** -0.5).to(torch.bfloat16)
    res = torch.randn(m, n, device=cuda).to(torch.bfloat16) if epilogue == "acc" else None
    out = res.clone() if res is not None else None
    got = gemm(a, w, out=out, epilogue=epilogue)
    torch.cuda.synchronize()
    Kernels.get(cuda).check_error()
    ref = gemm_reference(a, w, epilogue, res)
    torch.testing.assert_close(got.float(), ref.float(), rtol=1.6e-2, atol=1.6e-2)


@pytest.mark.parametrize("epilogue", ["store", "acc", "swiglu"])
@pytest.mark.parametrize("m,n,k", [(256, 256, 64), (300, 512, 320), (1000, 1024, 1024), (2049, 4096, 2048)])
def test_gemm_256_row_tiles(cuda, epilogue, m, n, k):
    """The 256-row tile (two MMAs per K step sharing one B tile, both accumulators in TMEM) against the fp32 statement."""
    from kern_b200.ops.gemm import gemm, gemm_reference
    from kern_b200.ops.launcher import Kernels

    torch.manual_seed(m + n + k)
    a = torch.randn(m, k, device=cuda).to(torch.bfloat16)
    w = (torch.randn(n, k, device=cuda) * k ** -0.5).to(torch.bfloat16)
    res = torch.randn(m, n, device=cuda).to(torch.bfloat16) if epilogue == "acc" else None
    out = res.clone() if res is not None else None
    got = gemm(a, w, out=out, epilogue=epilogue, bn=256, bm=256)
    torch.cuda.synchronize()
    Kernels.get(cuda).check_error()
    torch.testing.assert_close(got.float(), gemm_reference(a, w, epilogue, res).float(), rtol=1.6e-2, atol=1.6e-2)


def test_extern_gemm_builtins_gpu(cuda):
    """The GEMM built-ins a package may name (`extern:cublaslt_*`) on a GPU: served by the runtime's own tcgen05
    kernels (bf16 and e4m3 with device scales)."""
    from kern_b200.runtime import Runtime
    from kern_b200.testing.extern_gemm import check, manifest

    rt = Runtime(manifest(512, 384, 512))
    for m in (1, 200, 512):
        check(rt, "cuda", m, 384, 512)
    rt.check_error()
