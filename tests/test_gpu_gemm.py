"""tcgen05 GEMM against an fp32 PyTorch reference, all operand layouts and epilogues."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, b):
    return a.float() @ b.float()


@pytest.mark.parametrize("a_mn", [False, True])
@pytest.mark.parametrize("b_mn", [False, True])
@pytest.mark.parametrize("shape", [(128, 256, 64), (256, 512, 256), (300, 200, 136), (1024, 1024, 1024), (77, 64, 72)])
@pytest.mark.parametrize("tile_n", [128, 256])
def test_gemm_layouts(a_mn, b_mn, shape, tile_n):
    from summa_b200.ops import cuda_ops, native
    M, N, K = shape
    torch.manual_seed(0)
    A = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    B = torch.randn(K, N, device="cuda").to(torch.bfloat16)
    ref = _ref(A, B)
    # memory layouts: A k-major [M,K] / mn-major [K,M]; B k-major [N,K] / mn-major [K,N]
    Am = A.t().contiguous() if a_mn else A
    Bm = B if b_mn else B.t().contiguous()
    if (Am.stride(0) % 8) or (Bm.stride(0) % 8):
        pytest.skip("leading dimension not a multiple of 8")
    out = cuda_ops.gemm(Am, Bm, M, N, K, Am.stride(0), Bm.stride(0), a_mn, b_mn, out_dtype=torch.float32, tile_n=tile_n)
    torch.cuda.synchronize()
    assert native.read_error_flag() == 0
    err = (out - ref).abs().max().item()
    assert err <= 1e-2 * max(1.0, ref.abs().max().item()) * 0.05 + 1e-3, err
    out16 = cuda_ops.gemm(Am, Bm, M, N, K, Am.stride(0), Bm.stride(0), a_mn, b_mn, tile_n=tile_n)
    torch.testing.assert_close(out16.float(), ref, rtol=2e-2, atol=2e-1)


@pytest.mark.parametrize("a_mn", [False, True])
@pytest.mark.parametrize("b_mn", [False, True])
@pytest.mark.parametrize("shape", [(256, 256, 64), (512, 768, 256), (300, 200, 136), (2048, 1024, 192), (77, 64, 72),
                                   (256 * 74 + 256 * 20, 256, 128)])
def test_gemm_pair_layouts(a_mn, b_mn, shape):
    """The paired-CTA (cta_group::2) kernel, forced with tile_n=512: ragged edges, a second CTA whose rows
    are all out of range, and a tile count (94 on 74 pairs) whose tail runs as 256 x 128 half tiles."""
    from summa_b200.ops import cuda_ops, native
    M, N, K = shape
    torch.manual_seed(0)
    A = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    B = torch.randn(K, N, device="cuda").to(torch.bfloat16)
    ref = _ref(A, B)
    Am = A.t().contiguous() if a_mn else A
    Bm = B if b_mn else B.t().contiguous()
    if (Am.stride(0) % 8) or (Bm.stride(0) % 8):
        pytest.skip("leading dimension not a multiple of 8")
    out = cuda_ops.gemm(Am, Bm, M, N, K, Am.stride(0), Bm.stride(0), a_mn, b_mn, out_dtype=torch.float32, tile_n=512)
    torch.cuda.synchronize()
    assert native.read_error_flag() == 0
    err = (out - ref).abs().max().item()
    assert err <= 1e-2 * max(1.0, ref.abs().max().item()) * 0.05 + 1e-3, err
    out16 = cuda_ops.gemm(Am, Bm, M, N, K, Am.stride(0), Bm.stride(0), a_mn, b_mn, tile_n=512)
    torch.testing.assert_close(out16.float(), ref, rtol=2e-2, atol=2e-1)
    acc = torch.ones(M, N, device="cuda")
    cuda_ops.gemm(Am, Bm, M, N, K, Am.stride(0), Bm.stride(0), a_mn, b_mn, out=acc, accumulate=True, tile_n=512)
    torch.testing.assert_close(acc, ref + 1.0, rtol=1e-3, atol=2e-2)
    assert native.read_error_flag() == 0


def test_gemm_pair_split_k_and_bias():
    from summa_b200.ops import cuda_ops
    torch.manual_seed(3)
    M, N, K = 1024, 512, 4096          # 8 tiles on 74 pairs: the fp32 accumulate path cuts K
    A = torch.randn(K, M, device="cuda").to(torch.bfloat16)
    B = torch.randn(K, N, device="cuda").to(torch.bfloat16)
    C0 = torch.randn(M, N, device="cuda")
    C = C0.clone()
    cuda_ops.gemm(A, B, M, N, K, M, N, True, True, out=C, accumulate=True, tile_n=512)
    torch.testing.assert_close(C, C0 + A.float().t() @ B.float(), rtol=1e-3, atol=5e-2)
    bias = torch.randn(N, device="cuda")
    x = torch.randn(M, 320, device="cuda").to(torch.bfloat16)
    w = torch.randn(320, N, device="cuda").to(torch.bfloat16)
    out = cuda_ops.gemm(x, w, M, N, 320, 320, N, False, True, out_dtype=torch.float32, bias=bias, tile_n=512)
    torch.testing.assert_close(out, x.float() @ w.float() + bias, rtol=1e-3, atol=1e-2)


def test_gemm_accumulate_and_bias():
    from summa_b200.ops import cuda_ops
    torch.manual_seed(1)
    M, N, K = 512, 384, 320
    A = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    B = torch.randn(K, N, device="cuda").to(torch.bfloat16)
    C0 = torch.randn(M, N, device="cuda")
    C = C0.clone()
    cuda_ops.gemm(A, B, M, N, K, K, N, False, True, out=C, accumulate=True)
    torch.testing.assert_close(C, C0 + A.float() @ B.float(), rtol=1e-3, atol=1e-2)
    bias = torch.randn(N, device="cuda")
    out = cuda_ops.gemm(A, B, M, N, K, K, N, False, True, out_dtype=torch.float32, bias=bias)
    torch.testing.assert_close(out, A.float() @ B.float() + bias, rtol=1e-3, atol=1e-2)


def test_linear_autograd():
    from summa_b200 import ops
    torch.manual_seed(2)
    x = torch.randn(4, 96, 256, device="cuda").to(torch.bfloat16).requires_grad_()
    w = (torch.randn(256, 512, device="cuda") * 0.05).to(torch.bfloat16).requires_grad_()
    b = torch.randn(512, device="cuda").to(torch.bfloat16).requires_grad_()
    y = ops.linear(x, w, b)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    wr = w.detach().float().requires_grad_()
    br = b.detach().float().requires_grad_()
    yr = xr @ wr + br
    yr.backward(g.float())
    torch.testing.assert_close(y.float(), yr, rtol=2e-2, atol=5e-2)
    torch.testing.assert_close(x.grad.float(), xr.grad, rtol=2e-2, atol=5e-2)
    torch.testing.assert_close(w.grad.float(), wr.grad, rtol=2e-2, atol=2e-1)
    torch.testing.assert_close(b.grad.float(), br.grad, rtol=2e-2, atol=2e-1)
    # tied-embedding layout: weight is a transposed view
    e = (torch.randn(512, 256, device="cuda") * 0.05).to(torch.bfloat16).requires_grad_()
    y2 = ops.linear(x, e.t())
    y2.backward(g)
    er = e.detach().float().requires_grad_()
    (xr.detach() @ er.t()).backward(g.float())
    torch.testing.assert_close(e.grad.float(), er.grad, rtol=2e-2, atol=2e-1)


@pytest.mark.parametrize("trans_a,trans_b", [(False, False), (False, True), (True, False), (True, True)])
def test_batched_gemm_layout_flags(trans_a, trans_b):
    """`cuda_ops.bmm`: batched products on the paired-CTA kernel with either operand transposed by a layout flag."""
    from summa_b200.ops import cuda_ops
    torch.manual_seed(0)
    nb, M, K, N = 5, 384, 1024, 640
    A = torch.randn(nb, *((K, M) if trans_a else (M, K)), device="cuda").to(torch.bfloat16)
    B = torch.randn(nb, *((N, K) if trans_b else (K, N)), device="cuda").to(torch.bfloat16)
    got = cuda_ops.bmm(A, B, trans_b, trans_a=trans_a).float()
    ref = (A.float().transpose(1, 2) if trans_a else A.float()) @ (B.float().transpose(1, 2) if trans_b else B.float())
    assert (got - ref).abs().max().item() < 2e-2 * ref.abs().max().item()


@pytest.mark.parametrize("shape", [(6, 1024, 3072), (4, 2816, 1024), (3, 1024, 1024)])
def test_newton_schulz_on_the_device_matches_fp32(shape):
    """The Muon orthogonalisation chain on the batched tcgen05 GEMM (wide, tall without transposes, square)
    against the same five iterations in fp32 on the CPU."""
    from summa_b200.train.muon import newton_schulz
    torch.manual_seed(1)
    G = torch.randn(*shape)
    ref = newton_schulz(G)                               # CPU oracle path
    got = newton_schulz(G.cuda()).float().cpu()
    assert got.shape == ref.shape
    # bf16 products: compare on the scale of the result (singular values near 1)
    assert (got - ref).abs().max().item() < 0.08 * max(1.0, ref.abs().max().item())
    s = torch.linalg.svdvals(got[0].float())
    assert s.max().item() < 1.6                      # (a square Gaussian matrix keeps a few tiny singular values)
    if shape[1] != shape[2]:
        assert s.min().item() > 0.3
