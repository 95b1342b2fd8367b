"""Race smoke test: kernels without floating-point atomics must give bitwise-identical results
when run twice on the same inputs (a data race between warps, pipeline stages or CTAs shows up as
a difference), and must not write outside their outputs (canary rows around a strided output)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _twice(fn):
    a = fn()
    torch.cuda.synchronize()
    b = fn()
    torch.cuda.synchronize()
    return a, b


def test_forward_kernels_are_bitwise_repeatable():
    from summa_b200 import ops
    from summa_b200.ops import cuda_ops
    torch.manual_seed(0)
    x = torch.randn(4096, 1024, device="cuda").to(torch.bfloat16)
    w = torch.randn(1024, 2816, device="cuda").to(torch.bfloat16) * 0.05
    a, b = _twice(lambda: ops.linear(x, w, None))
    assert torch.equal(a, b)
    g = torch.ones(1024, device="cuda")
    a, b = _twice(lambda: ops.rmsnorm(x, g, 1e-5))
    assert torch.equal(a, b)
    u = torch.randn(4096, 2 * 2816, device="cuda").to(torch.bfloat16)
    a, b = _twice(lambda: ops.gated_act(u, "swiglu"))
    assert torch.equal(a, b)
    q = torch.randn(2, 1024, 8, 64, device="cuda").to(torch.bfloat16)
    k = torch.randn(2, 1024, 2, 64, device="cuda").to(torch.bfloat16)
    v = torch.randn(2, 1024, 2, 64, device="cuda").to(torch.bfloat16)
    (o1, l1), (o2, l2) = _twice(lambda: cuda_ops.attention_fwd(q, k, v, True, None, 0))
    assert torch.equal(o1, o2) and torch.equal(l1, l2)
    q = torch.randn(1, 512, 4, 128, device="cuda").to(torch.bfloat16)
    k = torch.randn(1, 512, 4, 128, device="cuda").to(torch.bfloat16)
    v = torch.randn(1, 512, 4, 128, device="cuda").to(torch.bfloat16)
    (o1, l1), (o2, l2) = _twice(lambda: cuda_ops.attention_fwd(q, k, v, True, 100, 0))
    assert torch.equal(o1, o2) and torch.equal(l1, l2)
    h = torch.randn(2048, 512, device="cuda").to(torch.bfloat16)
    wv = torch.randn(512, 1024, device="cuda").to(torch.bfloat16) * 0.05
    t = torch.randint(0, 1000, (2048,), device="cuda")
    a, b = _twice(lambda: ops.linear_cross_entropy(h, wv, None, t, 1000, 4))
    assert torch.equal(a, b)


def test_scan_and_quant_kernels_are_bitwise_repeatable():
    from summa_b200 import ops
    torch.manual_seed(1)
    B, T, C, N = 2, 256, 128, 16
    u = torch.randn(B, T, C, device="cuda").to(torch.bfloat16)
    dt = torch.randn(B, T, C, device="cuda").to(torch.bfloat16)
    A = -torch.rand(C, N, device="cuda")
    Bm = torch.randn(B, T, N, device="cuda").to(torch.bfloat16)
    Cm = torch.randn(B, T, N, device="cuda").to(torch.bfloat16)
    D = torch.ones(C, device="cuda")
    a, b = _twice(lambda: ops.selective_scan(u, dt, A, Bm, Cm, D))
    a = a[0] if isinstance(a, tuple) else a
    b = b[0] if isinstance(b, tuple) else b
    assert torch.equal(a, b)
    w = torch.randn(512, 256, device="cuda") * 0.05
    for fmt in ("binary_g128", "ternary_g128"):
        a, b = _twice(lambda: ops.fake_quant(w, fmt))
        assert torch.equal(a, b)


def test_gemm_does_not_write_outside_a_ragged_output():
    """M and N that are not multiples of the tile: rows / columns next to the result keep their canary."""
    from summa_b200 import ops
    torch.manual_seed(2)
    for M, K, N in [(130, 192, 264), (1, 128, 8), (257, 64, 136)]:
        x = torch.randn(M, K, device="cuda").to(torch.bfloat16)
        w = torch.randn(K, N, device="cuda").to(torch.bfloat16) * 0.1
        y = ops.linear(x, w, None)
        ref = x.float() @ w.float()
        torch.testing.assert_close(y.float(), ref, rtol=2e-2, atol=0.3)
        assert y.shape == (M, N) and torch.isfinite(y.float()).all()
