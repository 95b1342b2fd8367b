"""Pipeline parallelism on CPU ranks (gloo, 2 stages, 1F1B over 4 micro-batches): loss and
gradients match the single-process model."""
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
    from summa_b200.parallel.pp import PipelineStage, split_layers
    dist.init_process_group("gloo")
    rank = dist.get_rank()
    assert [list(r) for r in split_layers(5, 2)] == [[0, 1, 2], [3, 4]]
    cfg = mal.get_builtin_model("bench_tiny"); cfg.num_layers = 4
    torch.manual_seed(11)
    model = Transformer(cfg, init_std=0.05)
    g = torch.Generator().manual_seed(2)
    data = torch.randint(0, cfg.vocab_size, (4, 2, 17), generator=g)          # 4 micro-batches of [2, 16+1]
    stage = PipelineStage(model, dist.group.WORLD, (2, 16, cfg.hidden_size))
    loss = stage.step([d[:, :-1] for d in data], [d[:, 1:] for d in data], n_micro=4)
    # oracle: the whole model on this process, mean over the same micro-batches
    torch.manual_seed(11)
    ref = Transformer(cfg, init_std=0.05)
    tot = 0.0
    for d in data:
        l = ref.forward_loss(d[:, :-1], d[:, 1:]) / 4
        l.backward(); tot += float(l)
    if stage.last:
        assert abs(float(loss) - tot) < 1e-5, (float(loss), tot)
    owned = {id(p) for p in stage.owned_parameters()}
    checked = 0
    for (n, p), (_, q) in zip(model.named_parameters(), ref.named_parameters()):
        if id(p) in owned:
            assert p.grad is not None, n
            assert (p.grad - q.grad).abs().max().item() < 1e-5, n
            checked += 1
        else:
            assert p.grad is None or float(p.grad.abs().sum()) == 0.0, n
    assert checked > 0
    dist.barrier()
    if rank == 0:
        print("PP_OK")
    dist.destroy_process_group()
""") % ROOT


def test_pp2_gloo_matches_single_process(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29551", str(script)],
                       capture_output=True, text=True, env=env, timeout=600)
    if r.returncode != 0 or "PP_OK" not in r.stdout:
        print(r.stdout[-3000:])
        print(r.stderr[-6000:])
    assert r.returncode == 0 and "PP_OK" in r.stdout
