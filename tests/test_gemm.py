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
