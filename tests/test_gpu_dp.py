"""Fused reduce-scatter + AdamW + all-gather kernels on 2 GPUs vs the NCCL-collective
path with identical math. Skipped when fewer than 2 GPUs are visible."""
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
    from summa_b200.parallel.dp import DataParallelGroup
    from summa_b200.train.engine import FlatTrainEngine, OptimConfig, train_step
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rank = dist.get_rank()
    results = {}
    for mode in ("fused", "collective"):
        cfg = mal.get_builtin_model("llama_350m"); cfg.num_layers = 2
        torch.manual_seed(11)
        model = Transformer(cfg, init_std=0.02).to(dev)
        model.stream_dtype = torch.bfloat16
        dp = DataParallelGroup(dist.group.WORLD, dev, mode=mode)
        eng = FlatTrainEngine(model, OptimConfig(lr=1e-3), dp=dp, muon=sys.argv[1].startswith("muon"))
        g = torch.Generator().manual_seed(100 + rank)
        losses = []
        ga = 2 if sys.argv[1].endswith("ga2") else 1
        for step in range(4):
            tok = torch.randint(0, cfg.vocab_size, (2 * ga, 257), generator=g).to(dev)
            loss, norm = train_step(model, eng, tok[:, :-1], tok[:, 1:], grad_accum=ga)
            losses.append(float(loss))
        torch.cuda.synchronize()
        results[mode] = (eng.params_flat.float().clone(), losses, float(norm))
        if mode == "fused":
            mm_active = dp.multimem and bool(dp._mc_ptrs.get("grads"))
            # buckets reduced during the backward pass (all of them: one forward pass per micro-batch)
            overlapped = sum(j["launched"] for j in getattr(eng, "_ov_jobs", []))
            assert overlapped == (cfg.num_layers if os.environ.get("SUMMA_DP_OVERLAP") == "1" else 0), overlapped
        assert native.read_error_flag() == 0
    a, b = results["fused"][0], results["collective"][0]
    err = (a - b).abs().max().item()
    # every rank must hold identical parameters after the fused all-gather
    chk = a.sum().reshape(1).clone(); chk2 = chk.clone()
    dist.all_reduce(chk2, op=dist.ReduceOp.MAX)
    assert abs(chk2.item() - chk.item()) < 1e-3, "ranks diverged"
    assert err < 2e-2, err
    assert abs(results["fused"][2] - results["collective"][2]) < 1e-2 * max(1.0, results["collective"][2])
    if rank == 0:
        print("DP_OK", err, results["fused"][1], results["collective"][1], "multimem", mm_active, "overlapped", overlapped)
    dist.destroy_process_group()
""") % ROOT


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("optim", ["adamw", "muon", "adamw-multimem", "adamw-overlap", "adamw-overlap-ga2", "muon-overlap"])
def test_fused_dp_step_matches_collectives(tmp_path, optim):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", NCCL_NVLS_ENABLE="0",
               SUMMA_DP_MULTIMEM="1" if optim.endswith("multimem") else "0",
               SUMMA_DP_OVERLAP="1" if "overlap" in optim else "0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29553", str(script), optim],
                       capture_output=True, text=True, env=env, timeout=900)
    if r.returncode != 0 or "DP_OK" not in r.stdout:
        print(r.stdout[-3000:])
        print(r.stderr[-6000:])
    assert r.returncode == 0 and "DP_OK" in r.stdout
    print([l for l in r.stdout.splitlines() if "DP_OK" in l][0][-40:])
