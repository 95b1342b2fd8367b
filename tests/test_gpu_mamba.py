"""Mamba kernels (depthwise conv + SiLU, segmented selective scan) vs the fp32 oracle."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("K", [4, 3])
def test_conv1d_silu_fwd_bwd(K):
    from summa_b200 import ops
    from summa_b200.ops import reference
    torch.manual_seed(0)
    B, T, C = 2, 300, 264
    xz = torch.randn(B, T, 2 * C, device="cuda").to(torch.bfloat16).requires_grad_()
    w = (torch.randn(C, 1, K, device="cuda") * 0.5).requires_grad_()
    b = (torch.randn(C, device="cuda") * 0.1).requires_grad_()
    x = xz[..., :C]
    y = ops.conv1d_silu(x, w, b)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr = xz.detach().float().requires_grad_(); wr = w.detach().clone().requires_grad_(); br = b.detach().clone().requires_grad_()
    yr = torch.nn.functional.silu(reference.depthwise_conv1d(xr[..., :C], wr, br))
    yr.backward(dy.float())
    torch.testing.assert_close(y.float(), yr, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(xz.grad.float(), xr.grad, rtol=3e-2, atol=3e-2)
    torch.testing.assert_close(w.grad, wr.grad, rtol=3e-2, atol=0.5)
    torch.testing.assert_close(b.grad, br.grad, rtol=3e-2, atol=0.5)


def test_conv1d_with_state_matches_full():
    from summa_b200 import ops
    torch.manual_seed(1)
    B, T, C, K = 2, 64, 128, 4
    x = torch.randn(B, T, C, device="cuda").to(torch.bfloat16)
    w = torch.randn(C, 1, K, device="cuda") * 0.5
    b = torch.randn(C, device="cuda") * 0.1
    full = ops.conv1d_silu(x, w, b)
    state = x[:, 29:32].transpose(1, 2).contiguous()          # inputs t = 29..31
    part = ops.conv1d_silu(x[:, 32:].contiguous(), w, b, state)
    torch.testing.assert_close(part.float(), full[:, 32:].float(), rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("N,C,T", [(16, 128, 37), (128, 48, 100), (64, 64, 65), (16, 80, 257)])
def test_selective_scan_fwd_bwd(N, C, T):
    from summa_b200 import ops
    from summa_b200.ops import native, reference
    torch.manual_seed(0)
    B = 2
    u = torch.randn(B, T, C, device="cuda").to(torch.bfloat16).requires_grad_()
    delta = (torch.randn(B, T, C, device="cuda") - 1.0).to(torch.bfloat16).requires_grad_()
    a_log = (torch.rand(C, N, device="cuda") * 1.5).requires_grad_()
    proj = torch.randn(B, T, 8 + 2 * N, device="cuda").to(torch.bfloat16).requires_grad_()
    D = torch.randn(C, device="cuda").requires_grad_()
    A = -torch.exp(a_log)
    y, _ = ops.selective_scan(u, delta, A, proj[..., 8:8 + N], proj[..., 8 + N:], D)
    dy = torch.randn_like(y)
    y.backward(dy)
    torch.cuda.synchronize()
    assert native.read_error_flag() == 0
    ur = u.detach().float().requires_grad_(); dr = delta.detach().float().requires_grad_()
    alr = a_log.detach().clone().requires_grad_(); pr = proj.detach().float().requires_grad_()
    Dr = D.detach().clone().requires_grad_()
    yr, _ = reference.selective_scan(ur, dr, -torch.exp(alr), pr[..., 8:8 + N], pr[..., 8 + N:], Dr)
    yr.backward(dy.float())

    def close(a, b, name, tol=0.04):
        err = (a.float() - b).abs().max().item()
        ref = b.abs().max().item()
        assert err <= tol * ref + 1e-2, (name, err, ref)
    close(y, yr, "y")
    close(u.grad, ur.grad, "du")
    close(delta.grad, dr.grad, "ddelta")
    close(proj.grad, pr.grad, "dBC")
    close(a_log.grad, alr.grad, "dA")
    close(D.grad, Dr.grad, "dD")


def test_scan_state_carry_matches_full():
    from summa_b200 import ops
    torch.manual_seed(2)
    B, T, C, N = 1, 96, 64, 16
    u = torch.randn(B, T, C, device="cuda").to(torch.bfloat16)
    delta = (torch.randn(B, T, C, device="cuda") - 1.0).to(torch.bfloat16)
    A = -torch.exp(torch.rand(C, N, device="cuda"))
    Bm = torch.randn(B, T, N, device="cuda").to(torch.bfloat16)
    Cm = torch.randn(B, T, N, device="cuda").to(torch.bfloat16)
    D = torch.randn(C, device="cuda")
    with torch.no_grad():
        full, hf = ops.selective_scan(u, delta, A, Bm, Cm, D, None, True)
        y1, h1 = ops.selective_scan(u[:, :50].contiguous(), delta[:, :50].contiguous(), A, Bm[:, :50].contiguous(),
                                    Cm[:, :50].contiguous(), D, None, True)
        outs = [y1]
        h = h1
        for t in range(50, T):
            yt, h = ops.selective_scan(u[:, t:t + 1].contiguous(), delta[:, t:t + 1].contiguous(), A,
                                       Bm[:, t:t + 1].contiguous(), Cm[:, t:t + 1].contiguous(), D, h, True)
            outs.append(yt)
    inc = torch.cat(outs, 1)
    torch.testing.assert_close(inc.float(), full.float(), rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(h, hf, rtol=1e-3, atol=1e-3)
