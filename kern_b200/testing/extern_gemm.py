"""A manifest whose ops are the runtime's GEMM built-ins (`extern:cublaslt_bf16_tn[_acc]`, `extern:cublas_bf16_tn_f32`,
`extern:cublaslt_fp8_tn[_f32]`, `extern:cublaslt_mxfp8_tn`) — the vocabulary a package written against the reference's runtime names; here the
runtime's own tcgen05 kernels serve it. Used by the tests and as an example of the arg forms.
Reference: crates/kern-runtime/src/compile.rs:174-183 (arg forms), cublas.rs:78 / :329 / :387."""
from __future__ import annotations


def manifest(m_max: int, n: int, k: int) -> dict:
    from ..ops.gemm_mx import atom_bytes

    buf = lambda dt, shape, kind="workspace": {"dtype": dt, "shape": shape, "kind": kind}
    B = lambda name: {"buf": name}
    g6 = ["in buffer<bf16>", "in buffer<bf16>", "out buffer<bf16>", "i32", "i32", "i32"]
    ext = lambda entry: {"launches": [{"entry": entry}]}
    return {
        "schema_version": 7, "model": "extern-gemm", "vars": {"m": {"max": m_max}}, "states": {}, "modules": {},
        "buffers": {"a": buf("bf16", [m_max, k], "input"), "w": buf("bf16", [n, k], "input"),
                    "c": buf("bf16", [m_max, n], "output"), "acc": buf("bf16", [m_max, n], "output"),
                    "c32": buf("f32", [m_max, n], "output"),
                    "a8": buf("u8", [m_max, k], "input"), "w8": buf("u8", [n, k], "input"),
                    "sa": buf("f32", [1], "input"), "sw": buf("f32", [1], "input"),
                    "c8": buf("bf16", [m_max, n], "output"), "c8f": buf("f32", [m_max, n], "output"),
                    "sfa": buf("u8", [atom_bytes(m_max, k)], "input"), "sfw": buf("u8", [atom_bytes(n, k)], "input"),
                    "cmx": buf("bf16", [m_max, n], "output")},
        "ops": {
            "mm": {"params": g6, "impl": ext("extern:cublaslt_bf16_tn")},
            "mm_acc": {"params": ["in buffer<bf16>", "in buffer<bf16>", "inout buffer<bf16>", "i32", "i32", "i32"],
                       "impl": ext("extern:cublaslt_bf16_tn_acc")},
            "mm_f32": {"params": ["in buffer<bf16>", "in buffer<bf16>", "out buffer<f32>", "i32", "i32", "i32"],
                       "impl": ext("extern:cublas_bf16_tn_f32")},
            "mm8": {"params": ["in buffer<u8>", "in buffer<u8>", "out buffer<bf16>", "in buffer<f32>", "in buffer<f32>",
                               "i32", "i32", "i32"], "impl": ext("extern:cublaslt_fp8_tn")},
            "mm8_f32": {"params": ["in buffer<u8>", "in buffer<u8>", "out buffer<f32>", "in buffer<f32>", "in buffer<f32>",
                                   "i32", "i32", "i32"], "impl": ext("extern:cublaslt_fp8_tn_f32")},
            "mmx": {"params": ["in buffer<u8>", "in buffer<u8>", "out buffer<bf16>", "in buffer<u8>", "in buffer<u8>",
                               "i32", "i32", "i32"], "impl": ext("extern:cublaslt_mxfp8_tn")},
        },
        "programs": {"step": {"calls": [
            {"op": "mm", "args": [B("a"), B("w"), B("c"), {"var": "m"}, {"i32": n}, {"i32": k}]},
            {"op": "mm", "args": [B("a"), B("w"), B("acc"), {"var": "m"}, {"i32": n}, {"i32": k}]},
            {"op": "mm_acc", "args": [B("a"), B("w"), B("acc"), {"var": "m"}, {"i32": n}, {"i32": k}]},     # acc = 2 a w^T
            {"op": "mm_f32", "args": [B("a"), B("w"), B("c32"), {"var": "m"}, {"i32": n}, {"i32": k}]},
            {"op": "mm8", "args": [B("a8"), B("w8"), B("c8"), B("sa"), B("sw"), {"var": "m"}, {"i32": n}, {"i32": k}]},
            {"op": "mm8_f32", "args": [B("a8"), B("w8"), B("c8f"), B("sa"), B("sw"), {"var": "m"}, {"i32": n}, {"i32": k}]},
            {"op": "mmx", "args": [B("a8"), B("w8"), B("cmx"), B("sfa"), B("sfw"), {"var": "m"}, {"i32": n}, {"i32": k}]},
        ]}}}


def check(rt, device: str, m: int, n: int, k: int) -> None:
    """Run the five built-ins on random operands and compare with PyTorch fp32."""
    import torch

    torch.manual_seed(5)
    a = (torch.randn(m, k, device=device) * 0.5).to(torch.bfloat16)
    w = (torch.randn(n, k, device=device) * 0.5).to(torch.bfloat16)
    a8 = (torch.randn(m, k, device=device)).to(torch.float8_e4m3fn)
    w8 = (torch.randn(n, k, device=device)).to(torch.float8_e4m3fn)
    sa, sw = torch.tensor([0.5], device=device), torch.tensor([0.25], device=device)
    from ..ops import gemm_mx as G

    sfa = torch.randint(124, 131, (m, k // 32), dtype=torch.uint8, device=device)
    sfw = torch.randint(124, 131, (n, k // 32), dtype=torch.uint8, device=device)
    for name, t in (("a", a), ("w", w), ("a8", a8.view(torch.uint8)), ("w8", w8.view(torch.uint8)), ("sa", sa), ("sw", sw),
                    ("sfa", G.sf_to_atoms(sfa)), ("sfw", G.sf_to_atoms(sfw))):
        rt.tensor(name).view(-1)[: t.numel()] = t.reshape(-1)
    rt.run("step", {"m": m})
    rt.synchronize() if hasattr(rt, "synchronize") else None
    ref = a.float() @ w.float().t()
    ref8 = (a8.float() * 0.5) @ (w8.float() * 0.25).t()
    get = lambda name: rt.tensor(name).view(-1)[: m * n].view(m, n).float()
    torch.testing.assert_close(get("c"), ref, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(get("acc"), 2 * ref, rtol=3e-2, atol=3e-2)
    torch.testing.assert_close(get("c32"), ref, rtol=1e-3, atol=1e-3)
    torch.testing.assert_close(get("c8"), ref8, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(get("c8f"), ref8, rtol=1e-3, atol=1e-3)
    refx = G.dequant_mxfp8(a8.view(torch.uint8), sfa) @ G.dequant_mxfp8(w8.view(torch.uint8), sfw).t()
    torch.testing.assert_close(get("cmx"), refx, rtol=2e-2, atol=2e-2 * float(refx.abs().max()))
