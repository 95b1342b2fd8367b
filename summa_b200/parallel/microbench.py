"""Fused compute + collective kernels against their library forms, device-timed.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \\
        -m summa_b200.parallel.microbench [--tokens 8192] [--hidden 4096] [--ffn 14336] [--iters 20]

Every rank runs the same sequence; each op is warmed up, then timed with CUDA events on the launching
stream around `iters` back-to-back calls, and the MAXIMUM over ranks is reported (rank 0 prints one JSON
line per op). The roofline of a fused op is the slower of its FLOPs at the measured cuBLAS bf16 peak and
the bytes that must cross NVLink at the measured peer-copy bandwidth (770 GB/s per direction per GPU).

  ag_gemm      all-gather(x [M/P, K]) @ W [K, N/P]    fused tcgen05 kernel  vs  NCCL all_gather + GEMM
  gemm_rs      reduce-scatter(x [M, K/P] @ W [K/P, N]) fused kernel          vs  GEMM + NCCL reduce_scatter
  all_reduce   decode-sized activations                one-shot peer kernel  vs  NCCL all_reduce
  ep_moe       one expert-parallel MoE layer (top-2)   peer-memory dispatch / combine around the grouped GEMMs
                                                       vs  all_to_all_single + per-expert matmuls
  dp_step      64 M parameters                         fused reduce-scatter + clip + AdamW + all-gather
                                                       vs  NCCL reduce_scatter + torch AdamW + all_gather

Every op also reports `max_abs_diff` between the two forms, as the maximum over ranks.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

NVLINK_GBS = 770.0


def _peaks():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return float(p.get("bf16_tflops", 1590.0)), "measured"
    except (OSError, ValueError):
        return 1590.0, "fallback"


def _timed(fn, iters: int, warmup: int = 5) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--ffn", type=int, default=14336)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--copiers", type=int, default=0, help="copier CTAs of the all-gather -> GEMM kernel (0 = its default)")
    ap.add_argument("--only", default="", help="comma-separated subset of ag_gemm,gemm_rs,all_reduce,ep_moe,dp_step")
    ap.add_argument("--experts", type=int, default=0, help="ep_moe: experts in total (default 8 per rank)")
    ap.add_argument("--expert-ffn", type=int, default=1024)
    a = ap.parse_args()
    from .. import ops
    from ..ops import native
    from .tp import TensorParallelGroup
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rank, P = dist.get_rank(), dist.get_world_size()
    M, H, F = a.tokens, a.hidden, a.ffn
    if P < 2 or M % (128 * P) or F % P:
        raise SystemExit("needs >= 2 ranks, tokens % (128 * ranks) == 0 and ffn % ranks == 0")
    peak, peak_src = _peaks()
    tp = TensorParallelGroup(dist.group.WORLD, dev, mode="fused", max_tokens=M, hidden=H)
    torch.manual_seed(1 + rank)
    rows = M // P
    out = []

    def rank_max(v: float) -> float:
        """The largest value any rank saw (a numerics check passes only if it passes everywhere)."""
        t = torch.tensor([v], device=dev, dtype=torch.float32)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def report(op, fused_ms, lib_ms, flops, link_bytes, **kw):
        if "max_abs_diff" in kw:
            kw["max_abs_diff"] = round(rank_max(kw["max_abs_diff"]), 4)
        floor_ms = max(flops / (peak * 1e12), link_bytes / (NVLINK_GBS * 1e9)) * 1e3
        out.append(dict(op=op, fused_ms=round(fused_ms, 4), library_ms=round(lib_ms, 4),
                        speedup=round(lib_ms / fused_ms, 3), roofline_ms=round(floor_ms, 4),
                        frac_of_roofline=round(floor_ms / fused_ms, 3), peak=f"{peak:.0f} TFLOP/s ({peak_src}), "
                        f"{NVLINK_GBS:.0f} GB/s per direction", ranks=P, **kw))

    # ---- all-gather -> GEMM (column-parallel in-projection: N = 2 * ffn / P)
    Ncol = 2 * F // P
    w_col = (torch.randn(H, Ncol, device=dev) * 0.02).to(torch.bfloat16)
    x_own = torch.randn(rows, H, device=dev).to(torch.bfloat16)
    x_full = torch.empty(M, H, device=dev, dtype=torch.bfloat16)

    def fused_ag():
        tp.own_rows(0, M, H).copy_(x_own)
        return tp.ag_gemm(0, M, H, w_col, None, copiers=a.copiers)

    def lib_ag():
        dist.all_gather_into_tensor(x_full, x_own)
        return ops.linear(x_full, w_col, None)

    only = set(filter(None, a.only.split(",")))
    if not only or "ag_gemm" in only:
        err = (fused_ag().float() - lib_ag().float()).abs().max().item()
        report("ag_gemm", _timed(fused_ag, a.iters), _timed(lib_ag, a.iters), 2.0 * M * H * Ncol,
               (P - 1) * rows * H * 2.0, M=M, K=H, N=Ncol, max_abs_diff=round(err, 4), copiers=a.copiers)

    # ---- GEMM -> reduce-scatter (row-parallel down-projection: K = ffn / P)
    Krow = F // P
    w_row = (torch.randn(Krow, H, device=dev) * 0.02).to(torch.bfloat16)
    u = torch.randn(M, Krow, device=dev).to(torch.bfloat16)
    res = torch.randn(rows, H, device=dev).to(torch.bfloat16)
    y_rs = torch.empty(rows, H, device=dev, dtype=torch.bfloat16)

    def fused_rs():
        return tp.gemm_rs(u, w_row, res)

    def lib_rs():
        full = ops.linear(u, w_row, None)
        dist.reduce_scatter_tensor(y_rs, full)
        return y_rs + res

    if not only or "gemm_rs" in only:
        err = (fused_rs().float() - lib_rs().float()).abs().max().item()
        report("gemm_rs", _timed(fused_rs, a.iters), _timed(lib_rs, a.iters), 2.0 * M * Krow * H,
               (P - 1) * rows * H * 2.0, M=M, K=Krow, N=H, max_abs_diff=round(err, 4))

    # ---- decode-sized all-reduce
    for n in ((4096, 64 * 4096) if (not only or "all_reduce" in only) else ()):
        v = torch.randn(n, device=dev).to(torch.bfloat16)

        def fused_arr():
            return tp.all_reduce(v)

        def lib_arr():
            w = v.clone()
            dist.all_reduce(w)
            return w

        err = (fused_arr().float() - lib_arr().float()).abs().max().item()
        report(f"all_reduce_{n}", _timed(fused_arr, a.iters * 5), _timed(lib_arr, a.iters * 5), 0.0,
               (P - 1) * n * 2.0, elements=n, max_abs_diff=err)
    # ---- expert-parallel MoE layer: dispatch + grouped GEMMs + combine in peer memory against all_to_all_single
    if not only or "ep_moe" in only:
        from .. import mal
        from ..models.layers import SparseMoe
        from .ep import ExpertParallelGroup, shard_experts
        E = a.experts or 8 * P
        Tl = M // P                                 # tokens per rank
        cfg = mal.parse_mal(f"""attention a {{ num_heads: 4 bias: false }}
            ffn f {{ hidden_dim: {a.expert_ffn} activation: swiglu bias: false moe {{ experts: {E} top_k: 2 }} }}
            block b {{ attention: a ffn: f norm: rmsnorm {{ eps: 1e-5 }} }}
            model m {{ vocab_size: 64 max_seq_len: 32 hidden_size: {H} num_layers: 1 block: b }}""")
        ffn = cfg.block_for_layer(0).ffn
        layers = {}
        for mode in ("fused", "collective"):
            torch.manual_seed(7)                    # the same experts in both forms
            m = SparseMoe(ffn, H, init_std=0.02).to(dev)
            m.moe.experts.in_weight.data = m.moe.experts.in_weight.data.bfloat16()
            m.moe.experts.down_weight.data = m.moe.experts.down_weight.data.bfloat16()
            holder = torch.nn.Module()
            holder.m = m
            shard_experts(holder, ExpertParallelGroup(dist.group.WORLD, dev, E, H, max_tokens=Tl, top_k=2, mode=mode))
            layers[mode] = m
        xe = (torch.randn(Tl, H, device=dev) * 0.5).to(torch.bfloat16)

        def run_moe(mode):
            with torch.no_grad():
                return layers[mode](xe)[0]

        err = (run_moe("fused").float() - run_moe("collective").float()).abs().max().item()
        report("ep_moe_forward", _timed(lambda: run_moe("fused"), a.iters), _timed(lambda: run_moe("collective"), a.iters),
               2.0 * Tl * 2 * 3 * H * a.expert_ffn, 2.0 * Tl * 2 * H * 2.0 * (P - 1) / P, tokens_per_rank=Tl, experts=E,
               expert_ffn=a.expert_ffn, max_abs_diff=err)
        del layers

    # ---- data-parallel optimizer step: reduce-scatter + clip + AdamW + all-gather in peer memory against NCCL
    if not only or "dp_step" in only:
        from ..train.engine import FlatTrainEngine, OptimConfig
        from .dp import DataParallelGroup
        n_el = 64 * 1024 * 1024                     # 64 M parameters: 256 MB of fp32 gradients per rank
        res = {}
        for mode in ("fused", "collective"):
            torch.manual_seed(5)
            lin = torch.nn.Linear(8192, n_el // 8192, bias=False, device=dev)
            eng = FlatTrainEngine(lin, OptimConfig(lr=1e-3), dp=DataParallelGroup(dist.group.WORLD, dev, mode=mode))
            gsrc = torch.randn(n_el, device=dev, generator=torch.Generator(device=dev).manual_seed(50 + rank))

            def one(eng=eng, gsrc=gsrc):
                eng.grads_flat[:n_el].copy_(gsrc)
                return eng.step()

            one()
            ms = _timed(one, max(4, a.iters // 2), warmup=2)
            res[mode] = (ms, eng.params_flat[:n_el].float().clone())
            del eng, lin
        err = (res["fused"][1] - res["collective"][1]).abs().max().item()
        report("dp_step_64m", res["fused"][0], res["collective"][0], 0.0,
               (P - 1) / P * n_el * 4.0 + (P - 1) / P * n_el * 2.0, parameters=n_el, max_abs_diff=err)
    flag = native.read_error_flag()
    if rank == 0:
        for o in out:
            o["device_error_word"] = flag
            print(json.dumps(o))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
