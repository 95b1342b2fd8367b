"""MoE routing plan, grouped expert GEMM and the fused expert MLP vs the masked-dense oracle."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("T,E,k", [(300, 8, 2), (1000, 64, 4), (77, 15, 2)])
def test_route_plan_is_stable_and_padded(T, E, k):
    from summa_b200.ops import cuda_ops, reference
    torch.manual_seed(0)
    logits = torch.randn(T, E, device="cuda")
    plan = cuda_ops.RoutePlan(logits, k)
    torch.cuda.synchronize()
    ridx, _ = reference.moe_route(logits, k)
    assert torch.equal(plan.idx.long(), ridx)
    counts = torch.bincount(ridx.reshape(-1), minlength=E)
    assert torch.equal(plan.counts.long(), counts)
    meta = plan.meta.cpu().tolist()
    off = 0
    flat = ridx.reshape(-1).cpu()
    dest = plan.dest.cpu()
    rr = plan.row_route.cpu()
    for e in range(E):
        assert meta[e] == off and off % 128 == 0
        routes = (flat == e).nonzero().flatten()
        assert torch.equal(dest[routes], torch.arange(off, off + len(routes), dtype=torch.int32))   # stable order
        assert torch.equal(rr[off:off + len(routes)].long(), routes)
        pad_end = off + (len(routes) + 127) // 128 * 128
        assert (rr[off + len(routes):pad_end] == -1).all()
        te = plan.tile_expert.cpu()[off // 128:pad_end // 128]
        assert (te == e).all()
        off = pad_end
    assert meta[E] == off and meta[E + 1] == off // 128


def test_router_logits_kernel():
    from summa_b200 import ops
    torch.manual_seed(1)
    x = torch.randn(333, 512, device="cuda").to(torch.bfloat16)
    w = torch.randn(512, 64, device="cuda") * 0.05
    a = ops.router_logits(x, w)
    torch.testing.assert_close(a, x.float() @ w, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("T,H,I,E,k", [(500, 256, 128, 8, 2), (2048, 512, 256, 64, 4)])
def test_moe_experts_fwd_bwd(T, H, I, E, k):
    from summa_b200 import ops
    from summa_b200.ops import native, reference
    torch.manual_seed(0)
    x = torch.randn(T, H, device="cuda").to(torch.bfloat16).requires_grad_()
    rw = (torch.randn(H, E, device="cuda") * 0.1).requires_grad_()
    wi = (torch.randn(E, H, 2 * I, device="cuda") * 0.05).to(torch.bfloat16).requires_grad_()
    wd = (torch.randn(E, I, H, device="cuda") * 0.05).to(torch.bfloat16).requires_grad_()
    logits = ops.router_logits(x, rw)
    idx, gates = ops.moe_route(logits, k)
    out = ops.moe_experts(x, idx, gates, wi, wd, None, None, "swiglu", True)
    do = torch.randn_like(out)
    out.backward(do)
    torch.cuda.synchronize()
    assert native.read_error_flag() == 0
    xr = x.detach().float().requires_grad_(); rwr = rw.detach().clone().requires_grad_()
    wir = wi.detach().float().requires_grad_(); wdr = wd.detach().float().requires_grad_()
    lr = xr @ rwr
    gr = torch.softmax(torch.gather(lr, 1, idx), dim=-1)
    ro = reference.moe_experts_dense(xr, idx, gr, wir, wdr, None, None, "swiglu", True)
    ro.backward(do.float())

    def close(a, b, name, tol=0.05):
        err = (a.float() - b).abs().max().item()
        ref = b.abs().max().item()
        assert err <= tol * ref + 2e-2, (name, err, ref)
    close(out, ro, "out")
    close(x.grad, xr.grad, "dx")
    close(wi.grad, wir.grad, "dwi")
    close(wd.grad, wdr.grad, "dwd")
    close(rw.grad, rwr.grad, "drouter", 0.08)


def test_moe_model_trains():
    from summa_b200 import mal
    from summa_b200.models import Transformer
    from summa_b200.train.engine import FlatTrainEngine, OptimConfig, train_step
    src = """
    attention a { num_heads: 4 bias: false }
    ffn f { hidden_dim: 128 activation: swiglu bias: false moe { experts: 8 top_k: 2 load_balance_loss_weight: 0.01 router_z_loss_weight: 0.001 } }
    block b { attention: a ffn: f norm: rmsnorm { eps: 1e-5 } }
    model m { vocab_size: 1000 max_seq_len: 512 hidden_size: 256 num_layers: 2 block: b }
    """
    cfg = mal.parse_mal(src)
    torch.manual_seed(0)
    m = Transformer(cfg, init_std=0.02).to("cuda")
    m.stream_dtype = torch.bfloat16
    eng = FlatTrainEngine(m, OptimConfig(lr=1e-3))
    tok = torch.randint(0, 1000, (4, 257), device="cuda")
    losses = [float(train_step(m, eng, tok[:, :-1], tok[:, 1:])[0]) for _ in range(8)]
    assert losses[-1] < losses[0] - 0.3, losses


@pytest.mark.parametrize("T,E,k,lb,z", [(300, 8, 2, 0.01, 0.001), (4096, 64, 4, 0.02, 0.0), (77, 15, 2, 0.0, 0.01), (1000, 256, 8, 0.01, 0.001)])
def test_router_aux_loss_kernels_match_the_fp32_reference(T, E, k, lb, z):
    """Load-balance + z loss of the router logits: value and gradient of the native kernels against the plain
    PyTorch formula, with the counts taken from the device routing plan; two calls give the same bits."""
    from summa_b200 import ops
    from summa_b200.ops import native, reference
    torch.manual_seed(T + E)
    logits = (torch.randn(T, E, device="cuda") * 2.0).requires_grad_(True)
    idx, _ = ops.moe_route(logits.detach(), k)
    assert getattr(idx, "_sb_plan", None) is not None
    launches = []
    orig = native.call
    native.call = lambda name, *a: (launches.append(name), orig(name, *a))[1]
    try:
        aux = ops.moe_aux_loss(logits, idx, E, lb, z)
        (aux * 3.0).backward()
    finally:
        native.call = orig
    assert launches == ["sb_moe_aux_fwd", "sb_moe_aux_bwd"]
    ref_logits = logits.detach().clone().requires_grad_(True)
    ref = reference.moe_aux_loss(ref_logits, idx, E, lb, z)
    (ref * 3.0).backward()
    torch.testing.assert_close(aux, ref, rtol=1e-5, atol=1e-7)
    torch.testing.assert_close(logits.grad, ref_logits.grad, rtol=1e-4, atol=1e-9)
    again = ops.moe_aux_loss(logits.detach(), idx, E, lb, z)
    assert torch.equal(again, aux.detach())                                # fixed summation order
    # an index tensor without a plan (e.g. produced elsewhere) takes its counts from a histogram
    plain = idx.clone()
    torch.testing.assert_close(ops.moe_aux_loss(logits.detach(), plain, E, lb, z), ref.detach(), rtol=1e-5, atol=1e-7)
    assert native.read_error_flag() == 0
