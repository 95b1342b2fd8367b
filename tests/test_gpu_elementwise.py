"""Fused elementwise kernels against fp32 PyTorch references."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("H", [1024, 1536, 4096, 72])
def test_rmsnorm_fwd_bwd(H):
    from summa_b200 import ops
    from summa_b200.ops import reference
    torch.manual_seed(0)
    x = torch.randn(3, 37, H, device="cuda").to(torch.bfloat16).requires_grad_()
    g = (1 + 0.1 * torch.randn(H, device="cuda")).requires_grad_()
    y = ops.rmsnorm(x, g, 1e-5)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr = x.detach().float().requires_grad_()
    gr = g.detach().clone().requires_grad_()
    yr = reference.rmsnorm(xr, gr, 1e-5)
    yr.backward(dy.float())
    torch.testing.assert_close(y.float(), yr, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(x.grad.float(), xr.grad, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(g.grad, gr.grad, rtol=2e-2, atol=5e-2)


def test_add_rmsnorm():
    from summa_b200 import ops
    from summa_b200.ops import reference
    torch.manual_seed(1)
    H = 1024
    x = torch.randn(2, 65, H, device="cuda").to(torch.bfloat16).requires_grad_()
    r = torch.randn(2, 65, H, device="cuda").to(torch.bfloat16).requires_grad_()
    g = torch.ones(H, device="cuda").requires_grad_()
    y, s = ops.add_rmsnorm(x, r, g, 1e-5)
    dy, ds = torch.randn_like(y), torch.randn_like(s)
    (y.float() * dy.float()).sum().add((s.float() * ds.float()).sum()).backward()
    xr = x.detach().float().requires_grad_(); rr = r.detach().float().requires_grad_()
    sr = xr + rr
    yr = reference.rmsnorm(sr, g.detach(), 1e-5)
    ((yr * dy.float()).sum() + (sr * ds.float()).sum()).backward()
    torch.testing.assert_close(s.float(), sr, rtol=1e-2, atol=2e-2)
    torch.testing.assert_close(y.float(), yr, rtol=2e-2, atol=3e-2)
    torch.testing.assert_close(x.grad.float(), xr.grad, rtol=3e-2, atol=5e-2)
    torch.testing.assert_close(r.grad.float(), rr.grad, rtol=3e-2, atol=5e-2)


def test_swiglu_and_mul_silu():
    from summa_b200 import ops
    from summa_b200.ops import reference
    torch.manual_seed(2)
    x = torch.randn(5, 33, 2 * 2816, device="cuda").to(torch.bfloat16).requires_grad_()
    y = ops.gated_act(x, "swiglu")
    dy = torch.randn_like(y)
    y.backward(dy)
    xr = x.detach().float().requires_grad_()
    yr = reference.gated_act(xr, "swiglu")
    yr.backward(dy.float())
    torch.testing.assert_close(y.float(), yr, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(x.grad.float(), xr.grad, rtol=2e-2, atol=2e-2)
    xz = torch.randn(4, 19, 2 * 512, device="cuda").to(torch.bfloat16).requires_grad_()
    a, z = xz[..., :512], xz[..., 512:]
    o = ops.mul_silu(a, z)
    do = torch.randn_like(o)
    o.backward(do)
    xzr = xz.detach().float().requires_grad_()
    (xzr[..., :512] * torch.nn.functional.silu(xzr[..., 512:])).backward(do.float())
    torch.testing.assert_close(xz.grad.float(), xzr.grad, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("norm", [False, True])
def test_qk_norm_rope(D, norm):
    from summa_b200 import ops
    from summa_b200.ops import reference
    torch.manual_seed(3)
    B, S, Hq, Hkv = 2, 50, 4, 2
    q = torch.randn(B, S, Hq, D, device="cuda").to(torch.bfloat16).requires_grad_()
    k = torch.randn(B, S, Hkv, D, device="cuda").to(torch.bfloat16).requires_grad_()
    qg = (1 + 0.1 * torch.randn(D, device="cuda")).requires_grad_() if norm else None
    kg = (1 + 0.1 * torch.randn(D, device="cuda")).requires_grad_() if norm else None
    cos, sin = reference.rope_table(128, D, 10000.0, None, "cuda")
    qo, ko = ops.qk_norm_rope(q, k, qg, kg, 1e-5, cos, sin, 7)
    dq, dk = torch.randn_like(qo), torch.randn_like(ko)
    ((qo.float() * dq.float()).sum() + (ko.float() * dk.float()).sum()).backward()
    qr = q.detach().float().requires_grad_(); kr = k.detach().float().requires_grad_()
    qgr = qg.detach().clone().requires_grad_() if norm else None
    kgr = kg.detach().clone().requires_grad_() if norm else None
    qro, kro = reference.qk_norm_rope(qr, kr, qgr, kgr, 1e-5, cos, sin, 7)
    ((qro * dq.float()).sum() + (kro * dk.float()).sum()).backward()
    torch.testing.assert_close(qo.float(), qro, rtol=2e-2, atol=3e-2)
    torch.testing.assert_close(ko.float(), kro, rtol=2e-2, atol=3e-2)
    torch.testing.assert_close(q.grad.float(), qr.grad, rtol=3e-2, atol=5e-2)
    torch.testing.assert_close(k.grad.float(), kr.grad, rtol=3e-2, atol=5e-2)
    if norm:
        torch.testing.assert_close(qg.grad, qgr.grad, rtol=3e-2, atol=2e-1)
        torch.testing.assert_close(kg.grad, kgr.grad, rtol=3e-2, atol=2e-1)


@pytest.mark.parametrize("name", ["gelu", "gelu_tanh", "relu", "silu"])
@pytest.mark.parametrize("gated", [False, True])
def test_activation_family_fwd_bwd(name, gated):
    """GELU (erf and tanh forms), ReLU and SiLU, plain and gated ([gate | value] -> act(gate) * value), forward
    and backward against the fp32 oracle."""
    from summa_b200 import ops
    from summa_b200.ops import reference
    torch.manual_seed(0)
    rows, I = 300, 256
    x = (torch.randn(rows, (2 if gated else 1) * I, device="cuda") * 1.5).to(torch.bfloat16).requires_grad_()
    w = torch.randn(rows, I, device="cuda")
    y = ops.gated_act(x, name) if gated else ops.activation(name, x)
    (y.float() * w).sum().backward()
    xr = x.detach().float().requires_grad_()
    yr = reference.gated_act(xr, name) if gated else reference.activation(name, xr)
    (yr * w).sum().backward()
    assert y.dtype == torch.bfloat16
    torch.testing.assert_close(y.float(), yr, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(x.grad.float(), xr.grad, rtol=3e-2, atol=3e-2)


@pytest.mark.parametrize("H,bias", [(1024, True), (1536, False), (200, True)])
def test_layernorm_fwd_bwd(H, bias):
    from summa_b200 import ops
    from summa_b200.ops import reference
    torch.manual_seed(1)
    rows = 777
    x = (torch.randn(rows, H, device="cuda") * 2 + 0.5).to(torch.bfloat16).requires_grad_()
    gamma = (1 + 0.1 * torch.randn(H, device="cuda")).requires_grad_()
    beta = (0.1 * torch.randn(H, device="cuda")).requires_grad_() if bias else None
    w = torch.randn(rows, H, device="cuda")
    y = ops.layernorm(x, gamma, beta if bias else torch.zeros(H, device="cuda"), 1e-5)
    (y.float() * w).sum().backward()
    xr = x.detach().float().requires_grad_()
    gr = gamma.detach().clone().requires_grad_()
    br = beta.detach().clone().requires_grad_() if bias else torch.zeros(H, device="cuda")
    yr = reference.layernorm(xr, gr, br, 1e-5)
    (yr * w).sum().backward()
    torch.testing.assert_close(y.float(), yr, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(x.grad.float(), xr.grad, rtol=4e-2, atol=4e-2)
    torch.testing.assert_close(gamma.grad, gr.grad, rtol=3e-2, atol=3e-2 * max(1.0, gr.grad.abs().max().item()))
    if bias:
        torch.testing.assert_close(beta.grad, br.grad, rtol=3e-2, atol=3e-2 * max(1.0, br.grad.abs().max().item()))
