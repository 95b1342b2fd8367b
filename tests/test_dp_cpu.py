"""Data-parallel host logic on CPU ranks (gloo, world_size 2): sharded optimizer state,
gradient reduction and parameter redistribution match single-process training."""
import os
import subprocess
import sys
import textwrap

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent("""
    import os, sys, torch, torch.distributed as dist
    sys.path.insert(0, %r)
    from summa_b200 import mal
    from summa_b200.models import Transformer
    from summa_b200.parallel.dp import DataParallelGroup
    from summa_b200.train.engine import FlatTrainEngine, OptimConfig, train_step
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    cfg = mal.get_builtin_model("bench_tiny")
    torch.manual_seed(7)
    model = Transformer(cfg, init_std=0.02)
    dp = DataParallelGroup(dist.group.WORLD, torch.device("cpu"))
    eng = FlatTrainEngine(model, OptimConfig(lr=1e-3), dp=dp, param_dtype=torch.float32)
    g = torch.Generator().manual_seed(3)
    data = torch.randint(0, 256, (4, 4, 33), generator=g)      # steps x global batch x seq+1
    for step in range(4):
        tok = data[step, rank * 2:(rank + 1) * 2]
        loss, norm = train_step(model, eng, tok[:, :-1], tok[:, 1:])
    if rank == 0:
        torch.save(eng.params_flat.clone(), sys.argv[1])
    dist.destroy_process_group()
""") % ROOT


def test_dp2_gloo_matches_single_process(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    out = tmp_path / "params.pt"
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29541", str(script), str(out)],
                       capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stderr[-3000:]
    dp_params = torch.load(out)

    sys.path.insert(0, ROOT)
    from summa_b200 import mal
    from summa_b200.models import Transformer
    from summa_b200.train.engine import FlatTrainEngine, OptimConfig, train_step
    cfg = mal.get_builtin_model("bench_tiny")
    torch.manual_seed(7)
    model = Transformer(cfg, init_std=0.02)
    eng = FlatTrainEngine(model, OptimConfig(lr=1e-3), param_dtype=torch.float32)
    g = torch.Generator().manual_seed(3)
    data = torch.randint(0, 256, (4, 4, 33), generator=g)
    for step in range(4):
        # DP averages the per-rank mean gradients: the gradient of the global-batch mean
        tok = data[step]
        eng.zero_grad()
        for r_ in range(2):
            t = tok[r_ * 2:(r_ + 1) * 2]
            loss = model.forward_loss(t[:, :-1], t[:, 1:])
            loss.backward()
        eng.step(grad_scale=0.5)
    n = eng.numel
    torch.testing.assert_close(dp_params[:n], eng.params_flat[:n], rtol=1e-4, atol=1e-5)


MUON_WORKER = WORKER.replace('OptimConfig(lr=1e-3), dp=dp, param_dtype=torch.float32)',
                             'OptimConfig(lr=1e-3), dp=dp, param_dtype=torch.float32, muon=True)')


def test_dp2_muon_matches_single_process(tmp_path):
    """Muon under data parallelism: full-matrix updates from the gathered reduced gradients
    equal single-process Muon on the global batch; AdamW stops at the first Muon matrix."""
    assert "muon=True" in MUON_WORKER
    script = tmp_path / "worker.py"
    script.write_text(MUON_WORKER)
    out = tmp_path / "params.pt"
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29543", str(script), str(out)],
                       capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stderr[-3000:]
    dp_params = torch.load(out)

    sys.path.insert(0, ROOT)
    from summa_b200 import mal
    from summa_b200.models import Transformer
    from summa_b200.train.engine import FlatTrainEngine, OptimConfig
    cfg = mal.get_builtin_model("bench_tiny")
    torch.manual_seed(7)
    model = Transformer(cfg, init_std=0.02)
    eng = FlatTrainEngine(model, OptimConfig(lr=1e-3), param_dtype=torch.float32, muon=True)
    assert 0 < eng.adamw_numel < eng.numel
    g = torch.Generator().manual_seed(3)
    data = torch.randint(0, 256, (4, 4, 33), generator=g)
    for step in range(4):
        tok = data[step]
        eng.zero_grad()
        for r_ in range(2):
            t = tok[r_ * 2:(r_ + 1) * 2]
            model.forward_loss(t[:, :-1], t[:, 1:]).backward()
        eng.step(grad_scale=0.5)
    n = eng.numel
    torch.testing.assert_close(dp_params[:n], eng.params_flat[:n], rtol=2e-4, atol=2e-5)
