"""Gated DeltaNet kernels (causal conv + SiLU, gated delta rule) against the PyTorch fp32 statement:
ragged prefill chunks, then decode rows continuing from the stored state, with a padding (null-line) row."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def bf(x):
    return x.to(torch.bfloat16)


@pytest.mark.parametrize("hk,hv,d", [(2, 4, 32), (2, 6, 64), (4, 12, 128)])
def test_gdn_prefill_then_decode(cuda, hk, hv, d):
    from kern_b200.ops import gdn
    from kern_b200.ops.launcher import Kernels

    torch.manual_seed(hk * 100 + d)
    width, dk, dv = 4, d, d
    conv_dim = 2 * hk * dk + hv * dv
    zba_dim = hv * dv + 2 * hv
    x_stride = conv_dim + zba_dim
    lb, s_off = gdn.line_bytes(hk, hv, dk, dv, width)
    lens = [13, 1, 40]
    seqs = len(lens)
    lines_n = 6
    state = torch.zeros(lines_n, lb, dtype=torch.uint8, device=cuda)
    lines = torch.tensor([3, 1, 5], dtype=torch.int32, device=cuda)
    w = bf(torch.randn(conv_dim, width, device=cuda) * 0.5)
    bias = bf(torch.randn(conv_dim, device=cuda) * 0.1)
    A_log = torch.randn(hv, device=cuda) * 0.5
    dt_bias = torch.randn(hv, device=cuda) * 0.5
    norm_w = bf(1 + 0.1 * torch.randn(dv, device=cuda))

    ref_win = [torch.zeros(width - 1, conv_dim, device=cuda) for _ in lens]
    ref_S = [torch.zeros(hv, dv, dk, device=cuda) for _ in lens]

    def run(rows_per_seq, decode, fused=False):
        T = sum(rows_per_seq)
        x = bf(torch.randn(T, x_stride, device=cuda))
        cu = torch.tensor([0] + list(torch.tensor(rows_per_seq).cumsum(0)), dtype=torch.int32, device=cuda)
        y = torch.empty(T, conv_dim, dtype=torch.bfloat16, device=cuda)
        out = torch.empty(T, hv * dv, dtype=torch.bfloat16, device=cuda)
        cu_arg = None if decode else cu
        gdn.conv(x, y, state, lines, cu_arg, w, bias, seqs, conv_dim, width, lb)
        zba = x[:, conv_dim:]
        if fused:
            gdn.step(y, zba, out, state, lines, A_log, dt_bias, norm_w, seqs, hk, hv, dk, dv,
                     0, hv * dv, hv * dv + hv, lb, s_off)
        else:
            gdn.rule(y, zba, out, state, lines, cu_arg, A_log, dt_bias, norm_w, seqs, hk, hv, dk, dv,
                     0, hv * dv, hv * dv + hv, lb, s_off)
        torch.cuda.synchronize()
        Kernels.get(cuda).check_error()
        for s, n in enumerate(rows_per_seq):
            r0 = int(cu[s])
            xs = x[r0:r0 + n].float()
            yr, ref_win[s] = gdn.conv_ref(xs[:, :conv_dim], ref_win[s], w, bias)
            torch.testing.assert_close(y[r0:r0 + n].float(), yr, rtol=2e-2, atol=2e-2)
            yb = y[r0:r0 + n].float()          # the rule kernel reads the bf16 conv output
            q = yb[:, :hk * dk].view(n, hk, dk)
            k = yb[:, hk * dk:2 * hk * dk].view(n, hk, dk)
            v = yb[:, 2 * hk * dk:].view(n, hv, dv)
            z = xs[:, conv_dim:conv_dim + hv * dv].view(n, hv, dv)
            b = xs[:, conv_dim + hv * dv:conv_dim + hv * dv + hv]
            a = xs[:, conv_dim + hv * dv + hv:]
            o, ref_S[s] = gdn.rule_ref(q, k, v, z, b, a, ref_S[s], A_log, dt_bias, norm_w)
            torch.testing.assert_close(out[r0:r0 + n].float().view(n, hv, dv), o, rtol=3e-2, atol=3e-2)
            ln = int(lines[s])
            S_dev = state[ln, s_off:].view(torch.float32).view(hv, dv, dk)
            torch.testing.assert_close(S_dev, ref_S[s], rtol=1e-3, atol=1e-3)
            win_dev = state[ln, :(width - 1) * conv_dim * 2].view(torch.bfloat16).view(width - 1, conv_dim)
            torch.testing.assert_close(win_dev.float(), bf(ref_win[s]).float(), rtol=0, atol=0)

    run(lens, decode=False)
    for i in range(4):
        run([1, 1, 1], decode=True, fused=i % 2 == 0)      # the fused step and the two-launch form continue each other
    # untouched lines (0 = null, 2, 4) stayed zero
    for ln in (0, 2, 4):
        assert int(state[ln].count_nonzero()) == 0


def test_gdn_null_line_is_read_as_zero_and_never_written(cuda):
    from kern_b200.ops import gdn

    hk, hv, d, width = 2, 4, 64, 4
    conv_dim = 2 * hk * d + hv * d
    lb, s_off = gdn.line_bytes(hk, hv, d, d, width)
    state = torch.full((2, lb), 0x3c, dtype=torch.uint8, device=cuda)      # garbage in the null line
    lines = torch.zeros(2, dtype=torch.int32, device=cuda)
    x = bf(torch.randn(2, conv_dim + hv * d + 2 * hv, device=cuda))
    y = torch.empty(2, conv_dim, dtype=torch.bfloat16, device=cuda)
    out = torch.empty(2, hv * d, dtype=torch.bfloat16, device=cuda)
    w = bf(torch.randn(conv_dim, width, device=cuda))
    gdn.conv(x, y, state, lines, None, w, None, 2, conv_dim, width, lb)
    gdn.rule(y, x[:, conv_dim:], out, state, lines, None, torch.zeros(hv, device=cuda), torch.zeros(hv, device=cuda),
             bf(torch.ones(d, device=cuda)), 2, hk, hv, d, d, 0, hv * d, hv * d + hv, lb, s_off)
    out2 = torch.empty_like(out)
    gdn.step(y, x[:, conv_dim:], out2, state, lines, torch.zeros(hv, device=cuda), torch.zeros(hv, device=cuda),
             bf(torch.ones(d, device=cuda)), 2, hk, hv, d, d, 0, hv * d, hv * d + hv, lb, s_off)
    torch.cuda.synchronize()
    assert bool((state == 0x3c).all())
    torch.testing.assert_close(out2.float(), out.float(), rtol=2e-2, atol=2e-2)
    yr, _ = gdn.conv_ref(x[:1, :conv_dim].float(), torch.zeros(width - 1, conv_dim, device=cuda), w)
    torch.testing.assert_close(y[:1].float(), yr, rtol=2e-2, atol=2e-2)
    assert bool(torch.isfinite(out.float()).all())


def test_gdn_chunked_prefill_matches_the_statement(cuda):
    """The chunked (WY) prefill path against the sequential fp32 statement: ragged lengths around the 64-token chunk,
    a non-zero incoming state, then the sequential kernel continues from the state the chunked one left."""
    from kern_b200.ops import gdn
    from kern_b200.ops.launcher import Kernels

    torch.manual_seed(7)
    hk, hv, d, width = 2, 6, 128, 4
    conv_dim = 2 * hk * d + hv * d
    x_stride = conv_dim + hv * d + 2 * hv
    lb, s_off = gdn.line_bytes(hk, hv, d, d, width)
    lens = [200, 64, 1, 65]
    seqs = len(lens)
    state = torch.zeros(seqs + 2, lb, dtype=torch.uint8, device=cuda)
    lines = torch.tensor([2, 4, 1, 5], dtype=torch.int32, device=cuda)
    S0 = [torch.randn(hv, d, d, device=cuda) * 0.2 for _ in lens]
    for s, ln in enumerate(lines.tolist()):
        state[ln, s_off:].view(torch.float32).view(hv, d, d).copy_(S0[s])
    A_log = torch.randn(hv, device=cuda) * 0.5
    dt_bias = torch.randn(hv, device=cuda) * 0.5
    norm_w = bf(1 + 0.1 * torch.randn(d, device=cuda))
    T = sum(lens)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=cuda)
    x = bf(torch.randn(T, x_stride, device=cuda))
    y = x[:, :conv_dim].contiguous()            # the rule reads post-conv rows; any bf16 rows serve here
    out = torch.empty(T, hv * d, dtype=torch.bfloat16, device=cuda)
    gdn.rule_chunked(y, x[:, conv_dim:], out, state, lines, cu, A_log, dt_bias, norm_w, seqs, hk, hv, d, d,
                     0, hv * d, hv * d + hv, lb, s_off)
    torch.cuda.synchronize()
    Kernels.get(cuda).check_error()
    for s, n in enumerate(lens):
        r0 = int(cu[s])
        yb, xs = y[r0:r0 + n].float(), x[r0:r0 + n].float()
        q = yb[:, :hk * d].view(n, hk, d)
        k = yb[:, hk * d:2 * hk * d].view(n, hk, d)
        v = yb[:, 2 * hk * d:].view(n, hv, d)
        z = xs[:, conv_dim:conv_dim + hv * d].view(n, hv, d)
        b = xs[:, conv_dim + hv * d:conv_dim + hv * d + hv]
        a = xs[:, conv_dim + hv * d + hv:]
        o, S1 = gdn.rule_ref(q, k, v, z, b, a, S0[s], A_log, dt_bias, norm_w)
        torch.testing.assert_close(out[r0:r0 + n].float().view(n, hv, d), o, rtol=3e-2, atol=3e-2)
        S_dev = state[int(lines[s]), s_off:].view(torch.float32).view(hv, d, d)
        # tf32 products (10-bit mantissa operands, f32 accumulation) against the all-f32 statement
        torch.testing.assert_close(S_dev, S1, rtol=5e-3, atol=5e-3)
    assert int(state[0].count_nonzero()) == 0 and int(state[3].count_nonzero()) == 0


@pytest.mark.parametrize("d", [64, 128])
def test_kda_decode_step_per_key_decay(cuda, d):
    """The fused decode step with a decay per key channel against its fp32 statement, three steps in a row from a
    non-zero state, one padding (null-line) row."""
    from kern_b200.ops import gdn
    from kern_b200.ops.launcher import Kernels

    torch.manual_seed(3 + d)
    hk, hv, width = 2, 6, 4
    conv_dim = 2 * hk * d + hv * d
    zb = hv * d + hv
    lb, s_off = gdn.line_bytes(hk, hv, d, d, width)
    seqs = 3
    state = torch.zeros(5, lb, dtype=torch.uint8, device=cuda)
    lines = torch.tensor([2, 0, 4], dtype=torch.int32, device=cuda)
    S = [torch.randn(hv, d, d, device=cuda) * 0.2 if ln > 0 else torch.zeros(hv, d, d, device=cuda) for ln in lines.tolist()]
    for i, ln in enumerate(lines.tolist()):
        if ln > 0:
            state[ln, s_off:].view(torch.float32).view(hv, d, d).copy_(S[i])
    A_log = torch.randn(hv, device=cuda) * 0.5
    dt_bias = torch.randn(hv * d, device=cuda) * 0.5
    norm_w = bf(1 + 0.1 * torch.randn(d, device=cuda))
    # ragged rows first (the token-by-token kernel), then single-row steps continue from the state it left
    lens = [37, 5, 1]
    T = sum(lens)
    cu = torch.tensor([0, 37, 42, 43], dtype=torch.int32, device=cuda)
    y = bf(torch.randn(T, conv_dim, device=cuda))
    zba = bf(torch.randn(T, zb, device=cuda))
    gk = bf(torch.randn(T, hv * d, device=cuda))
    out = torch.empty(T, hv * d, dtype=torch.bfloat16, device=cuda)
    gdn.kda_rule(y, zba, gk, out, state, lines, cu, A_log, dt_bias, norm_w, seqs, hk, hv, d, d, 0, hv * d, lb, s_off)
    torch.cuda.synchronize()
    Kernels.get(cuda).check_error()
    for i, n in enumerate(lens):
        r0 = int(cu[i])
        yf = y[r0:r0 + n].float()
        q, k, v = yf[:, :hk * d].view(n, hk, d), yf[:, hk * d:2 * hk * d].view(n, hk, d), yf[:, 2 * hk * d:].view(n, hv, d)
        z = zba[r0:r0 + n, :hv * d].float().view(n, hv, d)
        b = zba[r0:r0 + n, hv * d:hv * d + hv].float()
        o, S1 = gdn.kda_rule_ref(q, k, v, z, b, gk[r0:r0 + n].float().view(n, hv, d), S[i], A_log, dt_bias.view(hv, d), norm_w)
        torch.testing.assert_close(out[r0:r0 + n].float().view(n, hv, d), o, rtol=3e-2, atol=3e-2)
        if int(lines[i]) > 0:
            S[i] = S1
            torch.testing.assert_close(state[int(lines[i]), s_off:].view(torch.float32).view(hv, d, d), S1, rtol=1e-3, atol=1e-3)
    for _ in range(3):
        y = bf(torch.randn(seqs, conv_dim, device=cuda))
        zba = bf(torch.randn(seqs, zb, device=cuda))
        gk = bf(torch.randn(seqs, hv * d, device=cuda))
        out = torch.empty(seqs, hv * d, dtype=torch.bfloat16, device=cuda)
        gdn.kda_step(y, zba, gk, out, state, lines, A_log, dt_bias, norm_w, seqs, hk, hv, d, d, 0, hv * d, lb, s_off)
        torch.cuda.synchronize()
        Kernels.get(cuda).check_error()
        for i in range(seqs):
            yf = y[i:i + 1].float()
            q, k, v = yf[:, :hk * d].view(1, hk, d), yf[:, hk * d:2 * hk * d].view(1, hk, d), yf[:, 2 * hk * d:].view(1, hv, d)
            z = zba[i:i + 1, :hv * d].float().view(1, hv, d)
            b = zba[i:i + 1, hv * d:hv * d + hv].float()
            o, S1 = gdn.kda_rule_ref(q, k, v, z, b, gk[i:i + 1].float().view(1, hv, d), S[i], A_log, dt_bias.view(hv, d), norm_w)
            torch.testing.assert_close(out[i:i + 1].float().view(1, hv, d), o, rtol=3e-2, atol=3e-2)
            if int(lines[i]) > 0:
                S[i] = S1
                torch.testing.assert_close(state[int(lines[i]), s_off:].view(torch.float32).view(hv, d, d), S1, rtol=1e-3, atol=1e-3)
    assert int(state[0].count_nonzero()) == 0


def test_kda_chunked_prefill_matches_the_statement(cuda):
    """The chunked (WY) form of the per-key-decay rule against its token-by-token fp32 statement: sequences of several
    chunks with ragged tails, a null-line row, strong and weak decays, from non-zero states."""
    from kern_b200.ops import gdn
    from kern_b200.ops.launcher import Kernels

    torch.manual_seed(11)
    hk, hv, d, width = 2, 6, 128, 4
    conv_dim = 2 * hk * d + hv * d
    zb = hv * d + hv + 2                      # z | b | pad: the gate rows start 16-byte aligned
    lb, s_off = gdn.line_bytes(hk, hv, d, d, width)
    lens = [150, 64, 5, 70]
    seqs, T = len(lens), sum(lens)
    state = torch.zeros(6, lb, dtype=torch.uint8, device=cuda)
    lines = torch.tensor([2, 4, 0, 5], dtype=torch.int32, device=cuda)
    S = [torch.randn(hv, d, d, device=cuda) * 0.2 if ln > 0 else torch.zeros(hv, d, d, device=cuda) for ln in lines.tolist()]
    for i, ln in enumerate(lines.tolist()):
        if ln > 0:
            state[ln, s_off:].view(torch.float32).view(hv, d, d).copy_(S[i])
    A_log = torch.log(torch.empty(hv, device=cuda).uniform_(0.05, 4.0))      # from almost no decay to e^-12 per token
    dt_bias = torch.randn(hv * d, device=cuda)
    norm_w = bf(1 + 0.1 * torch.randn(d, device=cuda))
    cu = torch.tensor([0] + torch.tensor(lens).cumsum(0).tolist(), dtype=torch.int32, device=cuda)
    y = bf(torch.randn(T, conv_dim, device=cuda))
    row = bf(torch.randn(T, zb + hv * d, device=cuda))
    zba, gk = row[:, :zb], row[:, zb:]
    out = torch.empty(T, hv * d, dtype=torch.bfloat16, device=cuda)
    gdn.kda_rule_chunked(y, zba, gk, out, state, lines, cu, A_log, dt_bias, norm_w, seqs, hk, hv, d, d, 0, hv * d, lb, s_off)
    torch.cuda.synchronize()
    Kernels.get(cuda).check_error()
    for i, n in enumerate(lens):
        r0 = int(cu[i])
        yf = y[r0:r0 + n].float()
        q, k, v = yf[:, :hk * d].view(n, hk, d), yf[:, hk * d:2 * hk * d].view(n, hk, d), yf[:, 2 * hk * d:].view(n, hv, d)
        z = zba[r0:r0 + n, :hv * d].float().view(n, hv, d)
        b = zba[r0:r0 + n, hv * d:hv * d + hv].float()
        o, S1 = gdn.kda_rule_ref(q, k, v, z, b, gk[r0:r0 + n].float().view(n, hv, d), S[i], A_log, dt_bias.view(hv, d), norm_w)
        torch.testing.assert_close(out[r0:r0 + n].float().view(n, hv, d), o, rtol=3e-2, atol=3e-2)
        if int(lines[i]) > 0:
            # tf32 products against the all-f32 statement
            torch.testing.assert_close(state[int(lines[i]), s_off:].view(torch.float32).view(hv, d, d), S1, rtol=5e-3, atol=5e-3)
    assert int(state[0].count_nonzero()) == 0 and int(state[3].count_nonzero()) == 0
