"""Pipeline and context parallelism on two GPUs over NCCL with the native kernels: the 1F1B pipeline's loss and
stage gradients against the whole model on one device, and sequence-sharded attention (contiguous and zigzag
layouts) against attention over the whole sequence. Skipped when fewer than 2 GPUs are visible."""
import os
import subprocess
import sys
import textwrap

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

PREAMBLE = """
    import os, sys, torch, torch.distributed as dist
    sys.path.insert(0, %r)
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()
""" % ROOT

PP_WORKER = textwrap.dedent(PREAMBLE + """
    from summa_b200 import mal
    from summa_b200.models import Transformer
    from summa_b200.ops import native
    from summa_b200.parallel.pp import PipelineStage
    cfg = mal.get_builtin_model("llama_350m"); cfg.num_layers = 4
    S, MB, NM = 256, 2, 4
    def build():
        torch.manual_seed(11)
        m = Transformer(cfg, init_std=0.02).to(dev).to(torch.bfloat16)
        m.stream_dtype = torch.bfloat16
        return m
    model = build()
    g = torch.Generator().manual_seed(2)
    data = torch.randint(0, cfg.vocab_size, (NM, MB, S + 1), generator=g).to(dev)
    stage = PipelineStage(model, dist.group.WORLD, (MB, S, cfg.hidden_size), dtype=torch.bfloat16)
    loss = stage.step([d[:, :-1] for d in data], [d[:, 1:] for d in data], n_micro=NM)
    ref = build()
    tot = 0.0
    for d in data:
        l = ref.forward_loss(d[:, :-1], d[:, 1:]) / NM
        l.backward(); tot += float(l)
    if stage.last:
        assert abs(float(loss) - tot) < 2e-2 * max(1.0, abs(tot)), (float(loss), tot)
    owned = {id(p) for p in stage.owned_parameters()}
    checked = 0
    for (n, p), (_, q) in zip(model.named_parameters(), ref.named_parameters()):
        if id(p) in owned:
            assert p.grad is not None, n
            a, b = p.grad.float(), q.grad.float()
            err = (a - b).abs().max().item()
            assert err < 5e-2 * max(1e-3, b.abs().max().item()), (n, err, b.abs().max().item())
            checked += 1
    assert checked > 0 and native.read_error_flag() == 0
    dist.barrier()
    if rank == 0:
        print("PP_OK", checked)
    dist.destroy_process_group()
""")

CP_WORKER = textwrap.dedent(PREAMBLE + """
    from summa_b200 import ops
    from summa_b200.ops import native
    from summa_b200.parallel import cp
    torch.manual_seed(3)
    B, S, Hq, Hkv, D = 2, 1024, 8, 2, 64
    q, k, v, w = (torch.randn(B, S, h, D, device=dev).to(torch.bfloat16) for h in (Hq, Hkv, Hkv, Hq))
    for causal in (True, False):
        qf, kf, vf = (t.clone().requires_grad_(True) for t in (q, k, v))
        ref = ops.attention(qf, kf, vf, causal, None, 0)
        (ref.float() * w.float()).sum().backward()
        for zigzag in (False, True):
            if zigzag:
                cut = lambda t: cp.zigzag_split(t, rank, world)
            else:
                cut = lambda t: t[:, rank * (S // world):(rank + 1) * (S // world)]
            ql, kl, vl = (cut(t).contiguous().clone().requires_grad_(True) for t in (q, k, v))
            out = cp.context_parallel_attention(ql, kl, vl, dist.group.WORLD, causal, zigzag)
            (out.float() * cut(w).float()).sum().backward()
            for got, want, what in ((out, cut(ref.detach()), "out"), (ql.grad, cut(qf.grad), "dq"),
                                    (kl.grad, cut(kf.grad), "dk"), (vl.grad, cut(vf.grad), "dv")):
                err = (got.float() - want.float()).abs().max().item()
                tol = 4e-2 * max(1.0, want.float().abs().max().item())
                assert err < tol, (causal, zigzag, what, err, tol)
    assert native.read_error_flag() == 0
    if rank == 0:
        print("CP_OK")
    dist.destroy_process_group()
""")


def _run(tmp_path, source, port, marker):
    script = tmp_path / "worker.py"
    script.write_text(source)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", str(port), str(script)],
                       capture_output=True, text=True, env=env, timeout=900)
    if r.returncode != 0 or marker not in r.stdout:
        print(r.stdout[-3000:])
        print(r.stderr[-6000:])
    assert r.returncode == 0 and marker in r.stdout


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_pipeline_1f1b_on_two_gpus_matches_one_device(tmp_path):
    _run(tmp_path, PP_WORKER, 29561, "PP_OK")


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_context_parallel_attention_on_two_gpus_matches_full_sequence(tmp_path):
    _run(tmp_path, CP_WORKER, 29562, "CP_OK")
