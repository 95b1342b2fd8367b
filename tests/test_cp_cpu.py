"""Context-parallel attention on 2 gloo ranks: outputs and gradients of the sequence-sharded form
(contiguous and zigzag layouts, causal and full) equal attention over the whole sequence."""
import os
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent("""
    import os, sys, torch, torch.distributed as dist
    sys.path.insert(0, %r)
    from summa_b200 import ops
    from summa_b200.parallel import cp
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    torch.manual_seed(3)
    B, S, Hq, Hkv, D = 2, 48, 4, 2, 16
    q = torch.randn(B, S, Hq, D); k = torch.randn(B, S, Hkv, D); v = torch.randn(B, S, Hkv, D)
    w = torch.randn(B, S, Hq, D)                       # weights of a scalar loss
    for causal in (True, False):
        qf, kf, vf = (t.clone().requires_grad_(True) for t in (q, k, v))
        ref = ops.attention(qf, kf, vf, causal, None, 0)
        (ref * w).sum().backward()
        for zigzag in (False, True):
            if zigzag:
                cut = lambda t: cp.zigzag_split(t, rank, world)
            else:
                cut = lambda t: t[:, rank * (S // world):(rank + 1) * (S // world)]
            ql, kl, vl = (cut(t).clone().requires_grad_(True) for t in (q, k, v))
            out = cp.context_parallel_attention(ql, kl, vl, dist.group.WORLD, causal, zigzag)
            (out * cut(w)).sum().backward()
            torch.testing.assert_close(out, cut(ref.detach()), rtol=1e-4, atol=1e-5)
            torch.testing.assert_close(ql.grad, cut(qf.grad), rtol=1e-4, atol=1e-5)
            torch.testing.assert_close(kl.grad, cut(kf.grad), rtol=1e-4, atol=1e-5)
            torch.testing.assert_close(vl.grad, cut(vf.grad), rtol=1e-4, atol=1e-5)
    pos = cp.zigzag_positions(rank, world, S)
    assert torch.equal(cp.zigzag_split(torch.arange(S)[None], rank, world, dim=1)[0], pos)
    parts = [cp.zigzag_split(q, r, world) for r in range(world)]
    assert torch.equal(cp.zigzag_merge(parts), q)
    if rank == 0:
        print("CP_OK")
    dist.destroy_process_group()
""") % ROOT


def test_context_parallel_attention_matches_full_sequence(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29555", str(script)],
                       capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0 and "CP_OK" in r.stdout, r.stderr[-3000:]
