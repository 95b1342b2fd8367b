"""tcgen05 flash attention against the fp32 PyTorch reference."""
import pytest
import torch

pytestmark = pytest.mark.gpu

CASES = [
    # B, Sq, Sk, Hq, Hkv, D, causal, window, q_offset
    (2, 256, 256, 4, 4, 64, True, None, 0),
    (1, 512, 512, 4, 2, 128, True, None, 0),
    (2, 300, 300, 2, 1, 64, True, None, 0),
    (1, 384, 384, 2, 2, 64, False, None, 0),
    (1, 640, 640, 2, 2, 64, True, 100, 0),
    (1, 100, 356, 2, 2, 128, True, None, 256),
    (1, 37, 37, 2, 2, 64, True, None, 0),
    (1, 1024, 1024, 2, 2, 128, False, 200, 0),
]


@pytest.mark.parametrize("case", CASES)
def test_attention_forward(case):
    from summa_b200.ops import cuda_ops, native, reference
    B, Sq, Sk, Hq, Hkv, D, causal, window, off = case
    torch.manual_seed(0)
    q = torch.randn(B, Sq, Hq, D, device="cuda").to(torch.bfloat16)
    k = torch.randn(B, Sk, Hkv, D, device="cuda").to(torch.bfloat16)
    v = torch.randn(B, Sk, Hkv, D, device="cuda").to(torch.bfloat16)
    o, lse = cuda_ops.attention_fwd(q, k, v, causal, window, off)
    torch.cuda.synchronize()
    assert native.read_error_flag() == 0
    ro, rlse = reference.attention(q, k, v, causal, window, None, off, return_lse=True)
    torch.testing.assert_close(o.float(), ro.float(), rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(lse, rlse, rtol=1e-2, atol=2e-2)


def test_attention_forward_packed_qkv_views():
    """q/k/v as strided views into one packed activation (no copies)."""
    from summa_b200.ops import cuda_ops, reference
    torch.manual_seed(1)
    B, S, Hq, Hkv, D = 2, 512, 8, 2, 64
    qkv = torch.randn(B, S, (Hq + 2 * Hkv) * D, device="cuda").to(torch.bfloat16)
    q = qkv[..., :Hq * D].unflatten(-1, (Hq, D))
    k = qkv[..., Hq * D:(Hq + Hkv) * D].unflatten(-1, (Hkv, D))
    v = qkv[..., (Hq + Hkv) * D:].unflatten(-1, (Hkv, D))
    o, _ = cuda_ops.attention_fwd(q, k, v, True, None, 0)
    ro = reference.attention(q, k, v, True, None)
    torch.testing.assert_close(o.float(), ro.float(), rtol=2e-2, atol=2e-2)


BWD_CASES = [
    (2, 256, 4, 4, 64, True, None),
    (1, 512, 4, 2, 128, True, None),
    (2, 300, 2, 1, 64, True, None),
    (1, 384, 2, 2, 64, False, None),
    (1, 640, 2, 2, 128, True, 100),
    (1, 77, 2, 2, 64, True, None),
]


@pytest.mark.parametrize("case", BWD_CASES)
def test_attention_backward(case):
    from summa_b200 import ops
    from summa_b200.ops import native, reference
    B, S, Hq, Hkv, D, causal, window = case
    torch.manual_seed(0)
    q = torch.randn(B, S, Hq, D, device="cuda").to(torch.bfloat16).requires_grad_()
    k = torch.randn(B, S, Hkv, D, device="cuda").to(torch.bfloat16).requires_grad_()
    v = torch.randn(B, S, Hkv, D, device="cuda").to(torch.bfloat16).requires_grad_()
    o = ops.attention(q, k, v, causal=causal, window=window)
    do = torch.randn_like(o)
    o.backward(do)
    torch.cuda.synchronize()
    assert native.read_error_flag() == 0
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    ro = reference.attention(qr, kr, vr, causal, window)
    ro.backward(do.float())
    torch.testing.assert_close(o.float(), ro, rtol=2e-2, atol=2e-2)
    for name, a, b in (("dq", q.grad, qr.grad), ("dk", k.grad, kr.grad), ("dv", v.grad, vr.grad)):
        err = (a.float() - b).abs().max().item()
        ref = b.abs().max().item()
        assert err <= 0.03 * ref + 0.03, (name, err, ref)


def test_packed_attention_matches_split():
    from summa_b200.ops import cuda_ops, reference
    torch.manual_seed(2)
    B, S, Hq, Hkv, D = 2, 384, 4, 2, 64
    qkv = torch.randn(B, S, (Hq + 2 * Hkv) * D, device="cuda").to(torch.bfloat16).requires_grad_()
    o = cuda_ops.packed_attention(qkv, Hq, Hkv, D, True, None)
    do = torch.randn_like(o)
    o.backward(do)
    ref = qkv.detach().float().requires_grad_()
    q, k, v = cuda_ops._split_packed(ref, Hq, Hkv, D)
    ro = reference.attention(q, k, v, True, None)
    ro.backward(do.float())
    torch.testing.assert_close(o.float(), ro, rtol=2e-2, atol=2e-2)
    err = (qkv.grad.float() - ref.grad).abs().max().item()
    assert err <= 0.03 * ref.grad.abs().max().item() + 0.03, err


@pytest.mark.parametrize("B,Hq,Hkv,Sk", [(1, 32, 8, 300), (4, 8, 8, 1), (3, 16, 2, 2049), (64, 4, 1, 2304), (2, 8, 1, 128)])
def test_decode_attention_split_kv(B, Hq, Hkv, Sk):
    """Split-KV decode kernel against an fp32 reference over a strided cache view."""
    from summa_b200.ops import cuda_ops, native
    torch.manual_seed(Sk)
    D, cap = 128, Sk + 37
    q = torch.randn(B, 1, Hq, D, device="cuda").bfloat16()
    kc = torch.randn(B, cap, Hkv, D, device="cuda").bfloat16()
    vc = torch.randn(B, cap, Hkv, D, device="cuda").bfloat16()
    o = cuda_ops.decode_attention(q, kc[:, :Sk], vc[:, :Sk], True, None, Sk - 1)
    G = Hq // Hkv
    kf = kc[:, :Sk].float().repeat_interleave(G, dim=2)
    vf = vc[:, :Sk].float().repeat_interleave(G, dim=2)
    s = torch.einsum("bqhd,bkhd->bhqk", q.float(), kf) / D ** 0.5
    ref = torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s, dim=-1), vf)
    torch.testing.assert_close(o.float(), ref, rtol=2e-2, atol=2e-2)
    assert native.read_error_flag() == 0
