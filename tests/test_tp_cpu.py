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


VOCAB_WORKER = textwrap.dedent("""
    import os, sys, torch, torch.distributed as dist
    sys.path.insert(0, %r)
    from summa_b200 import ops
    from summa_b200.parallel.tp import VocabParallelHead, shard_head, vocab_parallel_cross_entropy
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    torch.manual_seed(5)
    T, H, V = 37, 48, 301                               # V is not a multiple of the shard width: padded columns
    hidden = torch.randn(T, H, requires_grad=True)
    weight = (torch.randn(H, V) * 0.2).requires_grad_(True)
    targets = torch.randint(0, V, (T,))
    ref = ops.linear_cross_entropy(hidden, weight, None, targets, V, 4)
    ref.backward()
    h2 = hidden.detach().clone().requires_grad_(True)
    ws = shard_head(weight.detach(), rank, world).requires_grad_(True)
    loss = vocab_parallel_cross_entropy(h2, ws, targets, dist.group.WORLD, V)
    loss.backward()
    torch.testing.assert_close(loss, ref, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(h2.grad, hidden.grad, rtol=1e-4, atol=1e-6)
    per = ws.shape[1]
    lo, hi = rank * per, min((rank + 1) * per, V)
    torch.testing.assert_close(ws.grad[:, :hi - lo], weight.grad[:, lo:hi], rtol=1e-4, atol=1e-6)
    assert float(ws.grad[:, hi - lo:].abs().sum()) == 0.0
    head = VocabParallelHead(ws.detach(), dist.group.WORLD, V)
    torch.testing.assert_close(head(hidden.detach()), hidden.detach() @ weight.detach(), rtol=1e-5, atol=1e-5)
    if rank == 0:
        print("VOCAB_OK")
    dist.destroy_process_group()
""") % ROOT


def test_vocab_parallel_cross_entropy_and_head(tmp_path):
    """Head sharded over the vocabulary on 2 gloo ranks: loss, both gradients and the gathered
    logits equal the unsharded forms (padded columns stay out of the softmax)."""
    script = tmp_path / "worker.py"
    script.write_text(VOCAB_WORKER)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29549", str(script)],
                       capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0 and "VOCAB_OK" in r.stdout, r.stderr[-3000:]
