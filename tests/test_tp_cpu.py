"""Tensor-parallel sharding on CPU ranks (gloo, world_size 2): the sharded model's logits
and incremental decode match the unsharded model."""
import os
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent("""
    import os, sys, torch, torch.distributed as dist
    sys.path.insert(0, %r)
    from summa_b200 import mal
    from summa_b200.models import Transformer
    from summa_b200.parallel.tp import TensorParallelGroup, shard_model
    dist.init_process_group("gloo")
    rank = dist.get_rank()
    src = '''
    attention a { num_heads: 4 num_kv_heads: 2 bias: true }
    ffn f { hidden_dim: 96 activation: swiglu bias: true }
    block b { attention: a ffn: f norm: rmsnorm { eps: 1e-5 } }
    model m { vocab_size: 100 max_seq_len: 64 hidden_size: 64 num_layers: 2 block: b }
    '''
    cfg = mal.parse_mal(src)
    torch.manual_seed(5)
    full = Transformer(cfg, init_std=0.05).eval()
    torch.manual_seed(5)
    sharded = Transformer(cfg, init_std=0.05).eval()
    tp = TensorParallelGroup(dist.group.WORLD, torch.device("cpu"))
    shard_model(sharded, tp)
    tok = torch.randint(0, 100, (2, 17), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        a = full(tok); b = sharded(tok)
        assert (a - b).abs().max().item() < 1e-4, (a - b).abs().max().item()
        # incremental decode through the KV cache
        st = sharded.make_state(2, 32)
        outs = [sharded.forward_with_state(tok[:, :9], st)[:, -1]]
        for t in range(9, 17):
            outs.append(sharded.forward_with_state(tok[:, t:t + 1], st)[:, -1])
        assert (outs[-1] - a[:, -1]).abs().max().item() < 1e-4
    if rank == 0:
        print("TP_OK")
    dist.destroy_process_group()
""") % ROOT


def test_tp2_gloo_matches_unsharded(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29547", str(script)],
                       capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0 and "TP_OK" in r.stdout, (r.stdout[-2000:], r.stderr[-4000:])
