"""The runtime's GEMM built-ins (`extern:cublaslt_*`, `extern:cublas_*`) through the host-memory executor."""


def test_extern_gemm_builtins_cpu():
    from kern_b200.cpu import CpuRuntime
    from kern_b200.testing.extern_gemm import check, manifest

    check(CpuRuntime(manifest(64, 96, 128)), "cpu", 37, 96, 128)
