"""Fused expert-parallel dispatch / return kernels on 2 GPUs: forward output and gradients of a
sharded MoE layer against the unsharded layer, and against the all_to_all form."""
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
    from summa_b200.models.layers import SparseMoe
    from summa_b200.ops import native
    from summa_b200.parallel.ep import ExpertParallelGroup, shard_experts
    local_rank = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()
    src = '''
    attention a { num_heads: 4 bias: false }
    ffn f { hidden_dim: 128 activation: swiglu bias: false moe { experts: 8 top_k: 2 load_balance_loss_weight: 0.01 } }
    block b { attention: a ffn: f norm: rmsnorm { eps: 1e-5 } }
    model m { vocab_size: 50 max_seq_len: 32 hidden_size: 256 num_layers: 1 block: b }
    '''
    cfg = mal.parse_mal(src)
    ffn = cfg.block_for_layer(0).ffn
    T, H = 300, 256
    def make():
        torch.manual_seed(3)
        m = SparseMoe(ffn, H, init_std=0.05).to(dev)
        m.moe.experts.in_weight.data = m.moe.experts.in_weight.data.bfloat16()
        m.moe.experts.down_weight.data = m.moe.experts.down_weight.data.bfloat16()
        return m
    full, fused, coll = make(), make(), make()
    ep_f = ExpertParallelGroup(dist.group.WORLD, dev, 8, H, max_tokens=T, top_k=2, mode="fused")
    ep_c = ExpertParallelGroup(dist.group.WORLD, dev, 8, H, max_tokens=T, top_k=2, mode="collective")
    for m, ep in ((fused, ep_f), (coll, ep_c)):
        holder = torch.nn.Module(); holder.m = m
        shard_experts(holder, ep)
    xs = [(torch.randn(T, H, generator=torch.Generator().manual_seed(20 + r)) * 0.5).to(dev).bfloat16() for r in range(world)]
    for rep in range(3):                       # several rounds: epochs and buffer reuse
        outs = {}
        for name, m in (("fused", fused), ("coll", coll)):
            m.zero_grad()
            x = xs[rank].clone().requires_grad_()
            out, aux = m(x)
            (out.float().square().sum() + aux).backward()
            outs[name] = (out.float(), x.grad.float(), m.moe.experts.in_weight.grad.float(), m.moe.experts.down_weight.grad.float())
        full.zero_grad()
        for r in range(world):
            xr = xs[r].clone().requires_grad_()
            o, a = full(xr)
            (o.float().square().sum() + a).backward()
            if r == rank:
                ref_out, ref_dx = o.float(), xr.grad.float()
        lo, hi = rank * 4, rank * 4 + 4
        ref = (ref_out, ref_dx, full.moe.experts.in_weight.grad.float()[lo:hi], full.moe.experts.down_weight.grad.float()[lo:hi])
        for name in ("fused", "coll"):
            for got, want, what in zip(outs[name], ref, ("out", "dx", "d_in_w", "d_down_w")):
                err = (got - want).abs().max().item()
                tol = 0.05 * max(1.0, want.abs().max().item())
                assert err < tol, (name, what, rep, err, tol)
    torch.cuda.synchronize()
    assert native.read_error_flag() == 0
    # an owner buffer that is too small: every sender derives the overflow from the shared count matrix and
    # sends that owner nothing (no store may leave the buffer), the owner exposes no rows, bit 32 is recorded
    ep_s = ExpertParallelGroup(dist.group.WORLD, dev, 8, H, max_tokens=T, top_k=2, mode="fused", capacity_factor=0.05)
    small = make()
    holder = torch.nn.Module(); holder.m = small
    shard_experts(holder, ep_s)
    with torch.no_grad():
        out, _ = small(xs[rank].clone())
    torch.cuda.synchronize()
    assert native.read_error_flag() & 32
    # the context is intact (the arithmetic below runs); `out` holds no routed contribution for the overflowed owner
    y = torch.ones(8, device=dev) * 2
    assert float(y.sum()) == 16.0
    if rank == 0:
        print("EP_OK")
    dist.barrier()
    dist.destroy_process_group()
""") % ROOT


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_ep_fused_matches_unsharded(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29559", str(script)],
                       capture_output=True, text=True, env=env, timeout=900)
    if r.returncode != 0 or "EP_OK" not in r.stdout:
        print(r.stdout[-3000:])
        print(r.stderr[-6000:])
    assert r.returncode == 0 and "EP_OK" in r.stdout
