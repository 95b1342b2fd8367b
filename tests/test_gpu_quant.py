"""int4 g128 kernels (GEMV, dequant), argmax, and the quantised model path."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,K,N", [(1, 512, 768), (8, 4096, 768), (64, 1792, 4096), (3, 256, 132), (17, 4096, 3584),
                                   (33, 1024, 1040), (64, 14336, 512)])
def test_int4_gemv_and_dequant(M, K, N):
    from summa_b200 import ops
    from summa_b200.ops import reference
    torch.manual_seed(0)
    w = torch.randn(K, N) * 0.05
    packed, scales = reference.quantize_int4_g128(w)
    packed, scales = packed.cuda(), scales.cuda()
    x = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    # the device paths expand each weight to bf16 (q * scale rounded once), like the prefill GEMM
    wq = reference.dequantize_int4_g128(packed.cpu(), scales.cpu()).bfloat16().float()
    ref = x.float().cpu() @ wq
    tol = dict(rtol=2e-2, atol=2e-2 * max(1.0, ref.abs().max().item() / 8))
    y = ops.int4_gemv(x, packed, scales)                                      # CUDA-core weight-streaming kernel
    torch.testing.assert_close(y.float().cpu(), ref, **tol)
    res = torch.randn(M, N, device="cuda").to(torch.bfloat16)
    y2 = ops.int4_gemv(x, packed, scales, res, reference.repack_int4_k8(packed))   # tcgen05 kernel + fused residual
    torch.testing.assert_close(y2.float().cpu(), ref + res.float().cpu(), **tol)
    d = ops.int4_dequant(packed, scales)
    torch.testing.assert_close(d.float().cpu(), reference.dequantize_int4_g128(packed.cpu(), scales.cpu()),
                               rtol=1e-2, atol=1e-3)


@pytest.mark.parametrize("M,K,N", [(65, 256, 384), (128, 1024, 1028), (300, 4096, 512), (1024, 2048, 2560), (257, 512, 132),
                                   (300, 512, 24576)])
def test_int4_prefill_matmul_expands_the_weight_inside_the_gemm(M, K, N, monkeypatch):
    """More than 64 rows: the fused dequant-GEMM (row tiles of 128 or 256, weight tiles expanded on their way into
    tensor memory) against the fp32 product with the dequantised weight, with and without the fused residual, on
    row counts that leave a partial last tile and column counts that leave a partial 128-column tile."""
    from summa_b200 import ops
    from summa_b200.models.quantized import QuantLinear
    from summa_b200.ops import reference
    torch.manual_seed(0)
    w = torch.randn(K, N) * 0.05
    packed, scales = reference.quantize_int4_g128(w)
    packed, scales = packed.cuda(), scales.cuda()
    k8 = reference.repack_int4_k8(packed)
    x = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    wq = reference.dequantize_int4_g128(packed.cpu(), scales.cpu()).bfloat16().float()
    ref = x.float().cpu() @ wq
    tol = dict(rtol=2e-2, atol=2e-2 * max(1.0, ref.abs().max().item() / 8))
    assert ops.int4_prefill_usable(x, k8, K, N)
    y = ops.int4_matmul(x, k8, scales)
    torch.testing.assert_close(y.float().cpu(), ref, **tol)
    res = torch.randn(M, N, device="cuda").to(torch.bfloat16)
    y2 = ops.int4_matmul(x, k8, scales, res)
    torch.testing.assert_close(y2.float().cpu(), ref + res.float().cpu(), **tol)
    # the layer takes that path for prefill-sized inputs and agrees with the older expand-then-GEMM form
    layer = QuantLinear(packed, scales)
    from summa_b200.models import quantized
    from summa_b200.ops import native
    monkeypatch.setattr(quantized, "PREFILL_FUSED_MAX_ROWS", 4096)      # the layer's default keeps it to <= 512 rows
    launches = []
    orig = native.call
    native.call = lambda name, *a: (launches.append(name), orig(name, *a))[1]
    try:
        got = layer(x.view(1, M, K), residual=res.view(1, M, N))
    finally:
        native.call = orig
    assert launches == ["sb_w4a16_gemm"], launches
    torch.testing.assert_close(got.view(M, N).float().cpu(), ref + res.float().cpu(), **tol)
    if N % 8 == 0:                                        # the plain GEMM's own shape rule
        old = ops.linear(x, ops.int4_dequant(packed, scales), None) + res
        torch.testing.assert_close(got.view(M, N).float(), old.float(), rtol=2e-2, atol=tol["atol"])
    assert native.read_error_flag() == 0


def test_argmax_rows():
    from summa_b200 import ops
    torch.manual_seed(1)
    for dt in (torch.float32, torch.bfloat16):
        x = torch.randn(7, 32001, device="cuda").to(dt)
        assert torch.equal(ops.argmax(x), x.float().argmax(dim=-1))


def test_quantized_model_generation_matches_dequantized():
    from summa_b200 import mal
    from summa_b200.models import Transformer
    from summa_b200.models.generate import SamplingConfig, TextGenerator
    from summa_b200.models.quantized import QuantLinear, quantize_model_int4
    src = """
    attention a { num_heads: 4 num_kv_heads: 2 bias: false }
    ffn f { hidden_dim: 512 activation: swiglu bias: false }
    block b { attention: a ffn: f norm: rmsnorm { eps: 1e-5 } }
    model m { vocab_size: 1000 max_seq_len: 512 hidden_size: 256 num_layers: 2 block: b }
    """
    cfg = mal.parse_mal(src)
    torch.manual_seed(0)
    m = Transformer(cfg, init_std=0.05).to("cuda").prepare_inference(torch.bfloat16)
    n = quantize_model_int4(m)
    assert n == 8
    # oracle: same model with the dequantised weights as ordinary bf16 linears
    ref = Transformer(cfg, init_std=0.05).to("cuda").prepare_inference(torch.bfloat16)
    ref.load_state_dict({k: v for k, v in m.state_dict().items() if "packed" not in k and "scales" not in k},
                        strict=False)
    for (name, q) in [(n_, mod) for n_, mod in m.named_modules() if isinstance(mod, QuantLinear)]:
        tgt = ref.get_submodule(name)
        tgt.weight.data.copy_(q.dequantized())
    prompt = torch.randint(0, 1000, (100,)).tolist()
    with torch.no_grad():
        a = m(torch.tensor([prompt], device="cuda"))            # prefill path (dequant + GEMM)
        b = ref(torch.tensor([prompt], device="cuda"))
    torch.testing.assert_close(a.float(), b.float(), rtol=5e-2, atol=5e-2)
    out = TextGenerator(m, None, eos_id=None).generate_ids(prompt, SamplingConfig(max_new_tokens=8))
    assert len(out) == 8


def test_device_sampler_matches_host_rules():
    from summa_b200 import ops
    torch.manual_seed(4)
    V = 5003
    logits = torch.randn(3, V, device="cuda")
    seen = [[1, 5, 7, 7, 4999], [int(logits[1].argmax())], []]
    bm = ops.seen_bitmap(seen, V, "cuda")
    # greedy with penalty == host rule
    got = ops.sample_rows(logits, bm.clone(), None, penalty=1.7, temperature=0.0, top_k=0).cpu()
    for r in range(3):
        lf = logits[r].float().cpu().clone()
        ids = torch.tensor(sorted(set(seen[r])), dtype=torch.long)
        if len(ids):
            v = lf[ids]
            lf[ids] = torch.where(v > 0, v / 1.7, v * 1.7)
        assert int(got[r]) == int(lf.argmax())
    # the pick is recorded in the bit map
    bm2 = bm.clone()
    tok = ops.sample_rows(logits, bm2, None, penalty=1.0, temperature=0.0, top_k=0)
    t0 = int(tok[2]); assert (int(bm2[2, t0 // 32]) >> (t0 % 32)) & 1
    # top-k sampling follows softmax over the k best (frequency test), full sampling stays in the support
    row = torch.tensor([[2.0, 1.0, 0.5, 0.0, -1.0, -4.0, -9.0, -9.0]], device="cuda").repeat(4000, 1)
    u = torch.rand(4000, device="cuda", generator=torch.Generator(device="cuda").manual_seed(1))
    picks = ops.sample_rows(row, None, u, temperature=0.8, top_k=3).cpu()
    assert set(picks.tolist()) <= {0, 1, 2}
    want = torch.softmax(torch.tensor([2.0, 1.0, 0.5]) / 0.8, dim=0)
    freq = torch.bincount(picks, minlength=3).float() / 4000
    assert (freq - want).abs().max().item() < 0.03
    full = ops.sample_rows(row, None, u, temperature=1.0, top_k=0).cpu()
    wantf = torch.softmax(row[0].cpu(), dim=0)
    freqf = torch.bincount(full, minlength=8).float() / 4000
    assert (freqf - wantf).abs().max().item() < 0.03


@pytest.mark.parametrize("fmt", ["binary_g128", "ternary_g128"])
@pytest.mark.parametrize("shape", [(512, 256), (300, 77), (4096, 1024)])
def test_fake_quant_kernel_matches_reference(fmt, shape):
    """One-warp-per-group fake-quant kernel (bitonic sort + prefix scan for the ternary support)
    against the sort / cumsum formulation in PyTorch fp32."""
    from summa_b200 import ops
    from summa_b200.ops import reference
    torch.manual_seed(0)
    w = (torch.randn(*shape) * 0.05).cuda()
    w.requires_grad_(True)
    q = ops.fake_quant(w, fmt)
    ref = reference.fake_quant_values(w.detach().cpu(), fmt)
    got = q.detach().float().cpu()
    if fmt == "binary_g128":
        torch.testing.assert_close(got, ref, rtol=1e-5, atol=1e-7)
    else:
        # fp32 summation order differs (warp scan vs sequential): near-ties may pick the neighbouring prefix
        assert torch.isclose(got, ref, rtol=1e-4, atol=1e-7).float().mean() > 0.99
        wc = w.detach().cpu()
        e_got, e_ref = (got - wc).pow(2).sum(), (ref - wc).pow(2).sum()
        assert abs(e_got - e_ref) < 1e-4 * e_ref
    (q * 2.0).sum().backward()
    torch.testing.assert_close(w.grad, torch.full_like(w, 2.0))           # straight-through
    wb = w.detach().to(torch.bfloat16)
    qb = ops.fake_quant(wb, fmt)
    refb = reference.fake_quant_values(wb.cpu().float(), fmt).to(torch.bfloat16)
    assert torch.isclose(qb.float().cpu(), refb.float(), rtol=1e-2, atol=1e-6).float().mean() > 0.99


@pytest.mark.parametrize("fmt", ["binary_g128", "ternary_g128"])
@pytest.mark.parametrize("M,K,N", [(1, 512, 256), (4, 1024, 1024), (7, 333, 128), (16, 2048, 4096)])
def test_hquant_gemv_and_dequant(fmt, M, K, N):
    from summa_b200 import ops
    from summa_b200.train import quantization as Q
    torch.manual_seed(1)
    w = torch.randn(K, N) * 0.05
    pt = Q.quantize_tensor(w, fmt)
    dec = pt.decode()                                                       # host oracle
    codes = torch.from_numpy(pt.codes).cuda()
    scales = torch.from_numpy(pt.scales.view("float16")).cuda()
    d32 = ops.hquant_dequant(codes, scales, K * N, fmt, torch.float32).view(K, N)
    torch.testing.assert_close(d32.cpu(), dec, rtol=0, atol=0)
    d16 = ops.hquant_dequant(codes, scales, K * N, fmt, torch.bfloat16).view(K, N)
    torch.testing.assert_close(d16.float().cpu(), dec.bfloat16().float(), rtol=0, atol=0)
    x = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    res = torch.randn(M, N, device="cuda").to(torch.bfloat16)
    ref = x.float().cpu() @ dec
    y = ops.hquant_gemv(x, codes, scales, N, fmt)
    tol = dict(rtol=2e-2, atol=2e-2 * max(1.0, ref.abs().max().item() / 8))
    torch.testing.assert_close(y.float().cpu(), ref, **tol)
    y2 = ops.hquant_gemv(x, codes, scales, N, fmt, res)
    torch.testing.assert_close(y2.float().cpu(), ref + res.float().cpu(), **tol)


@pytest.mark.parametrize("M,K,N", [(1, 4096, 6144), (1, 4096, 1536), (2, 1024, 4096), (4, 14336, 4096), (3, 512, 36),
                                   (1, 4096, 28672), (1, 256, 132), (8, 4096, 4096), (7, 1024, 52), (5, 384, 24)])
def test_w4_small_batch_gemv_one_launch(M, K, N):
    """Batch 1..4 decode GEMV over the repacked weights (one launch, residual fused) against the
    dequantised fp32 product."""
    from summa_b200 import ops
    from summa_b200.ops import native, reference
    torch.manual_seed(M + K + N)
    w = torch.randn(K, N) * 0.05
    packed, scales = reference.quantize_int4_g128(w)
    packed, scales = packed.cuda(), scales.cuda()
    k8 = reference.repack_int4_k8(packed)
    x = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    res = torch.randn(M, N, device="cuda").to(torch.bfloat16)
    wq = reference.dequantize_int4_g128(packed.cpu(), scales.cpu())
    ref = x.float().cpu() @ wq
    tol = dict(rtol=2e-2, atol=2e-2 * max(1.0, ref.abs().max().item() / 8))
    launches = []
    orig = native.call
    native.call = lambda name, *a: (launches.append(name), orig(name, *a))[1]
    import summa_b200.ops.cuda_ops as co
    co.N.call = native.call
    try:
        y = ops.int4_gemv(x, packed, scales, None, k8)
        y2 = ops.int4_gemv(x, packed, scales, res, k8)
    finally:
        native.call = orig
        co.N.call = orig
    assert launches == (["sb_w4_gemv_cluster"] * 2 if M <= 4 else ["sb_w4a16_gemm"] * 2)
    torch.testing.assert_close(y.float().cpu(), ref, **tol)
    torch.testing.assert_close(y2.float().cpu(), ref + res.float().cpu(), **tol)
    # the mma-fragment form of the same product (1..8 rows), with and without the fused RMSNorm
    native.register("sb_w4_gemv_mma", [native.P] * 5 + [native.I, native.I, native.I, native.L, native.P, native.F, native.P])
    gamma = (1.0 + 0.1 * torch.randn(K)).cuda()
    y5 = torch.empty_like(y)
    native.call("sb_w4_gemv_mma", x.data_ptr(), k8.data_ptr(), scales.data_ptr(), res.data_ptr(), y5.data_ptr(),
                M, N, K, K, None, 0.0, native.stream())
    torch.testing.assert_close(y5.float().cpu(), ref + res.float().cpu(), **tol)
    refn = ops.rmsnorm(x, gamma, 1e-5).float().cpu() @ wq
    native.call("sb_w4_gemv_mma", x.data_ptr(), k8.data_ptr(), scales.data_ptr(), res.data_ptr(), y5.data_ptr(),
                M, N, K, K, gamma.data_ptr(), 1e-5, native.stream())
    torch.testing.assert_close(y5.float().cpu(), refn + res.float().cpu(), rtol=2e-2,
                               atol=2e-2 * max(1.0, refn.abs().max().item() / 8))
    if M > 4:
        return
    # the persistent streaming form (fp16 magic numbers, asynchronous weight ring), with and without the fused norm
    native.register("sb_w4_gemv_stream", [native.P] * 5 + [native.I, native.I, native.I, native.L, native.P, native.F,
                                                           native.I, native.P])
    y6 = torch.empty_like(y)
    native.call("sb_w4_gemv_stream", x.data_ptr(), k8.data_ptr(), scales.data_ptr(), res.data_ptr(), y6.data_ptr(),
                M, N, K, K, None, 0.0, 0, native.stream())
    torch.testing.assert_close(y6.float().cpu(), ref + res.float().cpu(), **tol)
    native.call("sb_w4_gemv_stream", x.data_ptr(), k8.data_ptr(), scales.data_ptr(), res.data_ptr(), y6.data_ptr(),
                M, N, K, K, gamma.data_ptr(), 1e-5, 0, native.stream())
    torch.testing.assert_close(y6.float().cpu(), refn + res.float().cpu(), rtol=2e-2,
                               atol=2e-2 * max(1.0, refn.abs().max().item() / 8))
    if N % 8 == 0:
        # gated: silu(g) * v for W = [gate | value]
        yg = torch.empty(M, N // 2, device="cuda", dtype=torch.bfloat16)
        native.call("sb_w4_gemv_stream", x.data_ptr(), k8.data_ptr(), scales.data_ptr(), None, yg.data_ptr(),
                    M, N, K, K, None, 0.0, 1, native.stream())
        gv = ref.to(torch.bfloat16).float()
        refg = torch.nn.functional.silu(gv[:, :N // 2]) * gv[:, N // 2:]
        torch.testing.assert_close(yg.float().cpu(), refg, rtol=3e-2, atol=3e-2 * max(1.0, refg.abs().max().item() / 8))
    # the single-CTA-per-column-block form of the same kernel
    y3 = torch.empty_like(y)
    native.call("sb_w4_gemv_small", x.data_ptr(), k8.data_ptr(), scales.data_ptr(), res.data_ptr(), y3.data_ptr(),
                M, N, K, K, native.stream())
    torch.testing.assert_close(y3.float().cpu(), ref + res.float().cpu(), **tol)
    # RMSNorm fused into the staging of x
    gamma = (1.0 + 0.1 * torch.randn(K)).cuda()
    xn = ops.rmsnorm(x, gamma, 1e-5)
    refn = xn.float().cpu() @ wq
    y4 = ops.int4_gemv(x, packed, scales, res, k8, norm=(gamma, 1e-5))
    toln = dict(rtol=2e-2, atol=2e-2 * max(1.0, refn.abs().max().item() / 8))
    torch.testing.assert_close(y4.float().cpu(), refn + res.float().cpu(), **toln)
    assert native.read_error_flag() == 0


@pytest.mark.parametrize("M,K,I", [(1, 4096, 14336), (2, 1024, 512), (4, 512, 36), (1, 4096, 3584)])
def test_w4_gated_in_projection_with_norm_and_swiglu(M, K, I):
    """rmsnorm -> [gate | value] projection -> silu(gate) * value in one launch against the separate ops."""
    from summa_b200 import ops
    from summa_b200.models.layers import Linear
    from summa_b200.models.quantized import QuantLinear, in_proj_swiglu
    from summa_b200.ops import native
    torch.manual_seed(K + I)
    lin = Linear(K, 2 * I, bias=False)
    with torch.no_grad():
        lin.weight.copy_(torch.randn(K, 2 * I) * 0.05)
    q = QuantLinear.from_linear(lin.cuda())
    x = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    gamma = (1.0 + 0.1 * torch.randn(K)).cuda()
    got = in_proj_swiglu(q, x, norm=(gamma, 1e-5))
    u = ops.rmsnorm(x, gamma, 1e-5).float() @ q.dequantized().float()
    u = u.to(torch.bfloat16).float()
    ref = torch.nn.functional.silu(u[:, :I]) * u[:, I:]
    assert got.shape == (M, I)
    torch.testing.assert_close(got.float(), ref, rtol=3e-2, atol=3e-2 * max(1.0, ref.abs().max().item() / 8))
    assert native.read_error_flag() == 0


@pytest.mark.parametrize("M,Hq,Hkv,D,K", [(1, 32, 8, 128, 4096), (3, 8, 2, 128, 1024), (2, 4, 4, 64, 512)])
def test_w4_qkv_projection_with_rope_and_cache_append(M, Hq, Hkv, D, K):
    """RMSNorm -> qkv GEMV -> RoPE -> KV append in one launch against projection + the separate
    RoPE / append kernel."""
    import ctypes
    from summa_b200 import ops
    from summa_b200.ops import cuda_ops, native, reference
    torch.manual_seed(Hq + D + K)
    N = (Hq + 2 * Hkv) * D
    w = torch.randn(K, N) * 0.05
    packed, scales = reference.quantize_int4_g128(w)
    packed, scales = packed.cuda(), scales.cuda()
    k8 = reference.repack_int4_k8(packed)
    x = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    gamma = (1.0 + 0.1 * torch.randn(K)).cuda()
    cap, pos_v = 16, 5
    ang = torch.rand(cap, D // 2, device="cuda") * 6.28
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    pos = torch.tensor([pos_v], dtype=torch.int32, device="cuda")
    kc1 = torch.zeros(M, cap, Hkv, D, device="cuda", dtype=torch.bfloat16); vc1 = torch.zeros_like(kc1)
    kc2 = torch.zeros_like(kc1); vc2 = torch.zeros_like(kc1)
    # separate kernels
    qkv1 = ops.int4_gemv(x, packed, scales, None, k8, norm=(gamma, 1e-5))
    cs = (ctypes.c_long * 3)(kc1.stride(0), kc1.stride(1), kc1.stride(2))
    native.register("sb_decode_rope_append", [native.P] * 6 + [native.I] * 4 + [native.L, native.P, native.I, native.P])
    native.call("sb_decode_rope_append", qkv1.data_ptr(), cos.data_ptr(), sin.data_ptr(), kc1.data_ptr(), vc1.data_ptr(),
                pos.data_ptr(), M, Hq, Hkv, D, qkv1.stride(0), cs, cap, native.stream())
    # fused
    qkv2 = cuda_ops.int4_gemv_rope_append(x, k8, scales, (gamma, 1e-5), cos, sin, kc2, vc2, pos, Hq, Hkv, D, cap)
    torch.cuda.synchronize()
    tol = dict(rtol=2e-2, atol=2e-2 * max(1.0, qkv1.float().abs().max().item() / 8))
    torch.testing.assert_close(qkv2[:, :Hq * D].float(), qkv1[:, :Hq * D].float(), **tol)
    torch.testing.assert_close(kc2.float(), kc1.float(), **tol)
    torch.testing.assert_close(vc2.float(), vc1.float(), **tol)
    assert float(kc2[:, pos_v].abs().sum()) > 0 and float(kc2[:, pos_v + 1].abs().sum()) == 0
    assert native.read_error_flag() == 0


@pytest.mark.parametrize("fmt", ["binary_g128", "ternary_g128", "int4_g128"])
def test_archive_model_runs_on_the_device_kernels(tmp_path, fmt):
    """A quantised archive loaded into a CUDA model: prefill-sized and decode-sized inputs go through the
    dequant + tensor-core GEMM and the code-streaming GEMV paths and agree with the decoded dense model."""
    from summa_b200 import mal
    from summa_b200.models import Transformer
    from summa_b200.models.quantized import HQuantLinear, QuantLinear, load_archive
    from summa_b200.train import quantization as Q
    cfg = mal.parse_mal("""attention a { num_heads: 2 } ffn f { hidden_dim: 256 }
      block b { attention: a ffn: f norm: rmsnorm { eps: 1e-5 } }
      model t { vocab_size: 300 max_seq_len: 128 hidden_size: 128 num_layers: 2 block: b }""")
    torch.manual_seed(0)
    src = Transformer(cfg, init_std=0.05)
    Q.export_archive(src, fmt, str(tmp_path / "a"))
    dst = Transformer(cfg, init_std=0.05)
    info = load_archive(dst, str(tmp_path / "a"))
    assert info["kernel_layers"] > 0
    dst = dst.cuda().eval().prepare_inference(torch.bfloat16)
    assert any(isinstance(m, (HQuantLinear, QuantLinear)) for m in dst.modules())
    ref = Transformer(cfg, init_std=0.05)
    packed = Q.quantize_model(src, fmt)
    with torch.no_grad():
        for n, p in ref.named_parameters():
            p.copy_(packed[n].decode() if n in packed else dict(src.named_parameters())[n])
    ref = ref.cuda().eval().prepare_inference(torch.bfloat16)
    for shape in ((1, 1), (2, 3), (2, 96)):                   # decode-sized rows and a prefill-sized batch
        tok = torch.randint(0, 300, shape, device="cuda")
        with torch.no_grad():
            a, b = dst(tok).float(), ref(tok).float()
        assert (a - b).abs().max().item() < 0.05 * max(1.0, b.abs().max().item()), (fmt, shape)
