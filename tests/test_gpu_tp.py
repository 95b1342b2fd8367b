"""One-shot peer-memory all-reduce and tensor-parallel inference on 2 GPUs vs NCCL and vs
the unsharded model. Skipped when fewer than 2 GPUs are visible."""
import os
import subprocess
import sys
import textwrap

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent("""
    import os, sys, torch, torch.distributed as dist
    sys.path.insert(0, %r)
    from summa_b200 import mal
    from summa_b200.models import Transformer
    from summa_b200.ops import native
    from summa_b200.parallel.tp import TensorParallelGroup, shard_model, prefill_sequence_parallel
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()
    tp = TensorParallelGroup(dist.group.WORLD, dev, mode="fused", max_tokens=1024, hidden=1024)
    # 1) the kernel against NCCL, many sizes and back-to-back epochs
    for it, n in enumerate([8, 4096, 1000 * 8, 64 * 16384, 2048, 8 * 4096, 4096]):
        g = torch.Generator().manual_seed(100 * it + rank)
        x = torch.randn(n, generator=g).to(dev).to(torch.bfloat16)
        ref = x.float().clone()
        dist.all_reduce(ref)
        y = tp.all_reduce(x.clone())
        err = (y.float() - ref).abs().max().item()
        assert err < 0.05 * world, (n, err)
        r = torch.randn(n, generator=g).to(dev).to(torch.bfloat16)        # residual fused into the reduction
        y = tp.all_reduce(x.clone(), residual=r)
        err = (y.float() - ref - r.float()).abs().max().item()
        assert err < 0.05 * world + 0.05, (n, err)
    assert native.read_error_flag() == 0
    if rank == 0:
        print("MULTIMEM_ACTIVE", int(bool(tp.stage_mc)))
    # 1b) row-parallel quantised projection with the all-reduce in its epilogue (one kernel per rank)
    from summa_b200.models.layers import Linear
    from summa_b200.models.quantized import QuantLinear
    for it, (Mr, Kl) in enumerate([(1, 512), (3, 1024), (1, 512), (4, 256), (2, 512)]):
        torch.manual_seed(500 + 10 * it + rank)
        lin = Linear(Kl, 1024, bias=False)
        with torch.no_grad():
            lin.weight.copy_(torch.randn(Kl, 1024) * 0.05)
        q = QuantLinear.from_linear(lin.to(dev))
        xr = torch.randn(Mr, Kl, device=dev).to(torch.bfloat16)
        torch.manual_seed(900 + it)
        res = torch.randn(Mr, 1024).to(dev).to(torch.bfloat16)          # replicated residual
        ref = xr.float() @ q.dequantized().float()
        dist.all_reduce(ref)
        ref = ref + res.float()
        y = tp.gemv_allreduce(xr, q, res)
        assert y is not None
        err = (y.float() - ref).abs().max().item()
        assert err < 0.03 * max(1.0, ref.abs().max().item()), ("gemv_allreduce", it, err)
        chk = y.float().sum().reshape(1).clone(); chk2 = chk.clone()
        dist.all_reduce(chk2, op=dist.ReduceOp.MAX)
        assert chk2.item() == chk.item(), "ranks hold different sums"
    assert native.read_error_flag() == 0
    # 2) sharded model vs unsharded
    cfg = mal.get_builtin_model("llama_350m"); cfg.num_layers = 2
    torch.manual_seed(3)
    full = Transformer(cfg, init_std=0.02).to(dev).prepare_inference(torch.bfloat16)
    torch.manual_seed(3)
    sh = Transformer(cfg, init_std=0.02).to(dev).prepare_inference(torch.bfloat16)
    shard_model(sh, tp)
    tok = torch.randint(0, cfg.vocab_size, (2, 64), generator=torch.Generator().manual_seed(9)).to(dev)
    with torch.no_grad():
        a = full(tok).float(); b = sh(tok).float()
        assert (a - b).abs().max().item() < 0.08, (a - b).abs().max().item()
        st = sh.make_state(2, 128)
        last = sh.forward_with_state(tok[:, :60], st)[:, -1]
        for t in range(60, 64):
            last = sh.forward_with_state(tok[:, t:t + 1], st)[:, -1]
        assert (last.float() - a[:, -1]).abs().max().item() < 0.08
    # 3) fused all-gather -> GEMM and GEMM -> reduce-scatter against NCCL + matmul
    for it, (M, K, N) in enumerate([(512, 1024, 768), (1024, 1024, 2816), (256, 1024, 136)]):
        g = torch.Generator().manual_seed(7 + it)
        xfull = (torch.randn(M, K, generator=g) * 0.5).to(dev).to(torch.bfloat16)     # same on every rank
        w = (torch.randn(K, N, generator=torch.Generator().manual_seed(50 + it + 10 * rank)) * 0.05).to(dev).to(torch.bfloat16)
        bias = torch.randn(N, generator=g).to(dev).to(torch.bfloat16)
        rows = M // world
        for rep in range(3):
            tp.own_rows(it & 1, M, K).copy_(xfull[rank * rows:(rank + 1) * rows])
            c = tp.ag_gemm(it & 1, M, K, w, bias)
            ref = xfull.float() @ w.float() + bias.float()
            err = (c.float() - ref).abs().max().item()
            assert err < 0.05 * max(1.0, ref.abs().max().item()), ("ag_gemm", M, K, N, rep, err)
        # reduce-scatter: every rank multiplies its own K-shard
        a = (torch.randn(M, K, generator=torch.Generator().manual_seed(90 + it + 10 * rank)) * 0.5).to(dev).to(torch.bfloat16)
        N2 = min(N, 1024)                      # the inbox slots are sized for hidden-wide outputs
        w2 = w[:, :N2].contiguous()
        res = torch.randn(rows, N2, generator=g).to(dev).to(torch.bfloat16)
        for rep in range(3):
            out = tp.gemm_rs(a, w2, res)
            part = (a.float() @ w2.float()).to(torch.bfloat16).float()
            dist.all_reduce(part)
            ref = part[rank * rows:(rank + 1) * rows] + res.float()
            err = (out.float() - ref).abs().max().item()
            assert err < 0.05 * max(1.0, ref.abs().max().item()), ("gemm_rs", M, K, N, rep, err)
    torch.cuda.synchronize()
    assert native.read_error_flag() == 0
    # 4) sequence-parallel prefill (fused kernels) vs the unsharded model, then decode on
    with torch.no_grad():
        tok2 = torch.randint(0, cfg.vocab_size, (2, 256), generator=torch.Generator().manual_seed(19)).to(dev)
        ref_logits = full(tok2)[:, -1].float()
        st2 = sh.make_state(2, 512)
        lg = prefill_sequence_parallel(sh, tp, tok2, st2).float()
        assert (lg - ref_logits).abs().max().item() < 0.1, (lg - ref_logits).abs().max().item()
        nxt = lg.argmax(-1, keepdim=True)
        a1 = sh.forward_next_logits_with_state(nxt, st2).float()
        b1 = full(torch.cat([tok2, nxt], dim=1))[:, -1].float()
        assert (a1 - b1).abs().max().item() < 0.1, (a1 - b1).abs().max().item()
    torch.cuda.synchronize()
    assert native.read_error_flag() == 0
    # 5) tensor-parallel TRAINING: column-parallel -> SiLU -> row-parallel (sequence parallel in between), forward
    #    and backward through the fused kernels against the unsharded computation
    from summa_b200.parallel.tp import column_parallel_linear, row_parallel_linear
    H, I, M = 1024, 2048, 1024
    gen = torch.Generator().manual_seed(123)
    W1 = (torch.randn(H, I, generator=gen) * 0.03).to(dev).to(torch.bfloat16)
    W2 = (torch.randn(I, H, generator=gen) * 0.03).to(dev).to(torch.bfloat16)
    xf = (torch.randn(M, H, generator=gen) * 0.5).to(dev).to(torch.bfloat16)
    wgt = torch.randn(M, H, generator=gen).to(dev)
    rows, s_ = M // world, I // world
    for rep in range(2):
        w1s = W1[:, rank * s_:(rank + 1) * s_].contiguous().requires_grad_()
        w2s = W2[rank * s_:(rank + 1) * s_].contiguous().requires_grad_()
        x_own = xf[rank * rows:(rank + 1) * rows].clone().requires_grad_()
        h = column_parallel_linear(x_own, w1s, tp, 0)
        a = torch.nn.functional.silu(h.float()).to(torch.bfloat16)
        y_own = row_parallel_linear(a, w2s, tp, None, 1)
        (y_own.float() * wgt[rank * rows:(rank + 1) * rows]).sum().backward()
        xr = xf.float().requires_grad_(); w1r = W1.float().requires_grad_(); w2r = W2.float().requires_grad_()
        hr = (xr @ w1r).to(torch.bfloat16).float()
        yr = torch.nn.functional.silu(hr).to(torch.bfloat16).float() @ w2r
        (yr * wgt).sum().backward()
        def close(got, want, what):
            err = (got.float() - want.float()).abs().max().item()
            tol = 0.05 * max(1.0, want.float().abs().max().item())
            assert err < tol, ("tp-train", what, rep, err, tol)
        close(y_own, yr[rank * rows:(rank + 1) * rows], "y")
        close(w2s.grad, w2r.grad[rank * s_:(rank + 1) * s_], "dW2")
        close(w1s.grad, w1r.grad[:, rank * s_:(rank + 1) * s_], "dW1")
        close(x_own.grad, xr.grad[rank * rows:(rank + 1) * rows], "dx")
    torch.cuda.synchronize()
    assert native.read_error_flag() == 0
    if rank == 0:
        print("TP_OK")
    dist.barrier()
    dist.destroy_process_group()
""") % ROOT


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("multimem", ["0", "1"])
def test_tp_allreduce_and_sharded_model(tmp_path, multimem):
    """multimem=1: the all-reduce runs as `multimem.ld_reduce` on the multicast address of the
    symmetric staging buffer (when the allocation has one; otherwise the peer-store kernel runs)."""
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", NCCL_NVLS_ENABLE="0", SUMMA_TP_MULTIMEM=multimem,
               SUMMA_TP_FUSED_GEMV="1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29557", str(script)],
                       capture_output=True, text=True, env=env, timeout=900)
    if r.returncode != 0 or "TP_OK" not in r.stdout:
        print(r.stdout[-3000:])
        print(r.stderr[-6000:])
    assert r.returncode == 0 and "TP_OK" in r.stdout
    print([l for l in r.stdout.splitlines() if "MULTIMEM_ACTIVE" in l])
