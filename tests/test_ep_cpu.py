"""Expert parallelism on CPU ranks (gloo, world_size 2, all_to_all form): forward output and
input / router / expert gradients match the unsharded MoE layer."""
import os
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent("""
    import os, sys, torch, torch.distributed as dist
    sys.path.insert(0, %r)
    from summa_b200 import mal
    from summa_b200.models.layers import SparseMoe
    from summa_b200.parallel.ep import ExpertParallelGroup, shard_experts
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    src = '''
    attention a { num_heads: 2 bias: false }
    ffn f { hidden_dim: 24 activation: swiglu bias: false moe { experts: 4 top_k: 2 load_balance_loss_weight: 0.01 } }
    block b { attention: a ffn: f norm: rmsnorm { eps: 1e-5 } }
    model m { vocab_size: 50 max_seq_len: 32 hidden_size: 16 num_layers: 1 block: b }
    '''
    cfg = mal.parse_mal(src)
    ffn = cfg.block_for_layer(0).ffn
    torch.manual_seed(3)
    full = SparseMoe(ffn, 16, init_std=0.2)
    torch.manual_seed(3)
    local = SparseMoe(ffn, 16, init_std=0.2)
    ep = ExpertParallelGroup(dist.group.WORLD, torch.device("cpu"), 4, 16, max_tokens=10, top_k=2)
    holder = torch.nn.Module(); holder.m = local
    shard_experts(holder, ep)
    assert local.moe.experts.in_weight.shape[0] == 2
    # every rank has its own tokens; the oracle runs both ranks' tokens through the full layer
    xs = [torch.randn(10, 16, generator=torch.Generator().manual_seed(20 + r)) for r in range(world)]
    x = xs[rank].clone().requires_grad_()
    out, aux = local(x)
    (out.square().sum() + aux).backward()
    xo = xs[rank].clone().requires_grad_()
    ref, aux_ref = full(xo)
    assert (out - ref).abs().max().item() < 1e-5, (out - ref).abs().max().item()
    # expert gradients need the other rank's tokens too: accumulate the oracle over all ranks' tokens
    full.zero_grad()
    for r in range(world):
        xr = xs[r].clone().requires_grad_()
        o, a = full(xr)
        (o.square().sum() + a).backward()
        if r == rank:
            assert (x.grad - xr.grad).abs().max().item() < 1e-4
    lo, hi = rank * 2, rank * 2 + 2
    assert (local.moe.experts.in_weight.grad - full.moe.experts.in_weight.grad[lo:hi]).abs().max().item() < 1e-4
    assert (local.moe.experts.down_weight.grad - full.moe.experts.down_weight.grad[lo:hi]).abs().max().item() < 1e-4
    if rank == 0:
        print("EP_OK")
    dist.destroy_process_group()
""") % ROOT


def test_ep2_gloo_matches_unsharded(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29549", str(script)],
                       capture_output=True, text=True, env=env, timeout=600)
    if r.returncode != 0 or "EP_OK" not in r.stdout:
        print(r.stdout[-3000:])
        print(r.stderr[-6000:])
    assert r.returncode == 0 and "EP_OK" in r.stdout
