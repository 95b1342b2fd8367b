"""Headline benchmark: training tokens/s of the dense Llama-style ~350M decoder
(24 layers, d_model 1024, 16 heads, SwiGLU 2816, vocab 32000, bf16), seq 2048,
micro-batch 8 per GPU, data-parallel over N GPUs of one node (weak scaling).

    python bench.py --gpus 1 --steps 10 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

Timed region = K full optimizer steps (forward, backward, gradient reduce-scatter,
clip, AdamW, parameter all-gather), device-timed with CUDA events, max over ranks.
Tokens are synthetic Zipf(1.1) draws from a fixed seed and weights are random-init
N(0, 0.02). `--impl reference` reports that the reference (a Rust workspace) cannot
be installed here. `--impl torch` runs the same model on stock PyTorch library ops
(cuBLAS, SDPA, fused AdamW, DDP over NCCL): the same-box baseline. The default line also
carries that comparison (`vs_baseline_torch`) and a short run of the one configuration the
reference published a number for (`secondary`, retriever-100m); `--no-extras` skips both.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CONFIGS = {
    # name: (preset, seq, micro_batch, data, parallelism fmt)
    "llama350m": dict(preset="llama_350m", seq=2048, micro_batch=8, data="zipf"),
    "tiny": dict(preset="bench_tiny", seq=128, micro_batch=8, data="uniform"),
    "hybrid": dict(preset="hybrid_mamba_1536", seq=8192, micro_batch=2, data="uniform"),
    "moe": dict(preset="moe_64e_top4", seq=4096, micro_batch=4, data="zipf"),
    # the reference's published setup: seq 1024, micro-batch 27, 8 accumulated micro-batches per optimizer step
    "retriever100m": dict(preset="retriever_100m", seq=1024, micro_batch=27, data="uniform", grad_accum=8),
}
PUBLISHED_TOK_S = {"retriever100m": 51769.0}   # reference's best published number (A100-40G)


def reference_arm() -> None:
    print(json.dumps({
        "impl": "reference",
        "unavailable": "reference is a Rust/Burn/CubeCL cargo workspace with no Python package at its root; "
                       "pip install of the reference tree fails and neither cargo nor rustc exists in this image",
    }))


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    def __init__(self, index: int):
        self.index = index
        self.rows = []
        self.proc = None

    def start(self):
        q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits", "-i", str(self.index),
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) >= 7:
                self.rows.append(parts)

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        for r in self.rows:
            try:
                sm.append(float(r[0])); mx = float(r[1])
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def make_batches(cfg, vocab, n_batches, seed, pin):
    import torch
    g = torch.Generator().manual_seed(seed)
    B, S = cfg["micro_batch"] * cfg.get("grad_accum", 1), cfg["seq"]
    out = []
    if cfg["data"] == "zipf":
        ranks = torch.arange(1, vocab + 1, dtype=torch.float64)
        probs = ranks.pow(-1.1)
        probs /= probs.sum()
    for _ in range(n_batches):
        if cfg["data"] == "zipf":
            t = torch.multinomial(probs, B * (S + 1), replacement=True, generator=g).view(B, S + 1)
        else:
            t = torch.randint(0, vocab, (B, S + 1), generator=g)
        t = t.to(torch.int64)
        out.append(t.pin_memory() if pin else t)
    return out


def _dist_env():
    return (int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")),
            int(os.environ.get("LOCAL_RANK", "0")))


def _l2_policy(mdef, cfg, use_cuda) -> str:
    if not use_cuda:
        return "host run: no device cache to defeat"
    B, S = cfg["micro_batch"] * cfg.get("grad_accum", 1), cfg["seq"]
    # bf16 residual stream saved per layer plus the token batch: every step streams far more than the 126 MB L2
    act_gb = B * S * mdef.hidden_size * 2 * mdef.num_layers * 4 / 1e9
    return f"inputs larger than L2 (~{act_gb:.1f} GB of saved activations and {mdef.estimated_params() * 2 / 1e9:.2f} GB of weights per step)"


def _timed_region(one_step, W, K, use_cuda, world, dev, launches=None):
    """W untimed steps, then K steps between barrier + synchronize on both sides; CUDA events, max over ranks."""
    import torch
    import torch.distributed as dist

    def sync():
        if use_cuda:
            torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            if use_cuda:
                torch.cuda.synchronize()

    for i in range(W):
        one_step(i)
    sync()
    if launches is not None:
        launches["n"] = 0
    if use_cuda:
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
    t0 = time.perf_counter()
    last = None
    for i in range(K):
        last = one_step(W + i)
    if use_cuda:
        ev1.record()
    sync()
    wall = time.perf_counter() - t0
    ms = max(ev0.elapsed_time(ev1), 0.0) if use_cuda else wall * 1e3
    if world > 1:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms, wall * 1e3, last


def run_ours(config: str, K: int, W: int, use_cuda: bool, sample_clocks: bool, optimizer: str = "adamw") -> dict:
    """This package's kernels and engine on `config`; returns the fields of the JSON line."""
    import torch
    import torch.distributed as dist
    from summa_b200 import mal
    from summa_b200.models import Transformer
    from summa_b200.ops import native
    from summa_b200.train.engine import FlatTrainEngine, OptimConfig, train_step

    cfg = CONFIGS[config]
    world, rank, local = _dist_env()
    dev = torch.device("cuda", local) if use_cuda else torch.device("cpu")
    dp = None
    if world > 1:
        from summa_b200.parallel.dp import DataParallelGroup
        dp = DataParallelGroup(dist.group.WORLD, dev)

    mdef = mal.get_builtin_model(cfg["preset"])
    torch.manual_seed(1234)
    if use_cuda:
        with torch.device(dev):                      # draw the weights on the device (large presets init in seconds)
            model = Transformer(mdef, init_std=0.02)
    else:
        model = Transformer(mdef, init_std=0.02)
    parallelism = f"dp{world}"
    muon = optimizer == "muon"
    if use_cuda:
        model = model.to(dev)
        model.stream_dtype = torch.bfloat16
        moe_cfgs = [b.ffn.moe for b in (mdef.block_for_layer(i) for i in range(mdef.num_layers)) if b.ffn is not None
                    and b.ffn.moe is not None]
        if world > 1 and moe_cfgs:
            # experts sharded over the ranks (expert parallel), everything else data parallel
            from summa_b200.parallel.ep import ExpertParallelGroup, shard_experts
            for prm in model.parameters():
                if prm.dim() >= 2:
                    prm.data = prm.data.to(torch.bfloat16)
            ep = ExpertParallelGroup(dist.group.WORLD, dev, moe_cfgs[0].experts, mdef.hidden_size,
                                     max_tokens=cfg["micro_batch"] * cfg["seq"], top_k=moe_cfgs[0].top_k,
                                     capacity_factor=0.0)    # worst case: Zipf tokens at random init are far from balanced
            shard_experts(model, ep)
            parallelism = f"dp{world}+ep{world}"
        engine = FlatTrainEngine(model, OptimConfig(lr=3e-4), dp=dp, param_dtype=torch.bfloat16, muon=muon)
    else:
        engine = FlatTrainEngine(model, OptimConfig(lr=3e-4), dp=dp, param_dtype=torch.float32, muon=muon)
    model.train()

    batches = make_batches(cfg, mdef.vocab_size, 8, seed=100 + rank, pin=use_cuda)
    GA = cfg.get("grad_accum", 1)
    B, S = cfg["micro_batch"] * GA, cfg["seq"]
    tokens_per_step = B * S * world

    launches = {"n": 0}
    _orig_call = native.call

    def counting_call(name, *a):
        launches["n"] += 1
        return _orig_call(name, *a)
    native.call = counting_call
    import summa_b200.ops.cuda_ops as _co
    _co.N.call = counting_call
    dev_batches = [b.to(dev) for b in batches] if use_cuda else batches

    def step_device(i):
        t = dev_batches[i % len(dev_batches)]
        loss, _ = train_step(model, engine, t[:, :-1], t[:, 1:], grad_accum=GA)
        return loss

    def step_e2e(i):
        t = batches[i % len(batches)].to(dev, non_blocking=True)        # pinned host memory -> device, every step
        loss, _ = train_step(model, engine, t[:, :-1], t[:, 1:], grad_accum=GA)
        return float(loss.item())                                       # device -> host, every step

    sampler = ClockSampler(local)
    if use_cuda and rank == 0 and sample_clocks:
        sampler.start()
    try:
        ms_dev, _, last_loss = _timed_region(step_device, W, K, use_cuda, world, dev, launches)
        n_launch = launches["n"]
        clocks = sampler.stop() if (use_cuda and rank == 0 and sample_clocks) else None
        ms_e2e, wall_e2e, _ = _timed_region(step_e2e, W, K, use_cuda, world, dev)
        if use_cuda:
            ms_e2e = max(ms_e2e, wall_e2e) if world == 1 else ms_e2e     # e2e includes the host-side readback
        err = native.read_error_flag() if use_cuda else 0
    finally:
        native.call = _orig_call
        _co.N.call = _orig_call
    out = {
        "value": tokens_per_step * K / (ms_dev / 1e3), "ms_per_step": ms_dev / K,
        "e2e": {"value": tokens_per_step * K / (ms_e2e / 1e3), "unit": "tokens/s", "ms_per_step": ms_e2e / K,
                "h2d_bytes_per_step": B * (S + 1) * 8, "d2h_bytes_per_step": 4},
        "gpu_launches": n_launch, "final_loss": float(last_loss) if last_loss is not None else None,
        "device_error_word": err, "clocks": clocks,
        "config": {"model": mdef.name, "params": mdef.estimated_params(), "global_batch": B * world, "seq_len": S,
                   "grad_accum": GA, "micro_batch": cfg["micro_batch"], "parallelism": parallelism,
                   "optimizer": ("muon(block matrices)+adamw+clip" if muon else "adamw+clip"),
                   "l2_policy": _l2_policy(mdef, cfg, use_cuda)},
        "data": f"synthetic {cfg['data']} tokens, random-init N(0,0.02) weights",
    }
    del engine, model, dev_batches
    if use_cuda:
        torch.cuda.empty_cache()
    return out


def run_torch(config: str, K: int, W: int) -> dict:
    """The same-box baseline: the same `Transformer` on stock PyTorch library ops (cuBLAS matmuls,
    `scaled_dot_product_attention`, `F.rms_norm`, chunked `F.cross_entropy`), fp32 parameters cast to
    bf16 at each use (what autocast does), `clip_grad_norm_`, `torch.optim.AdamW(fused=True)`, and
    `DistributedDataParallel` (bucketed NCCL all-reduce overlapped with backward) on more than one GPU.
    None of this package's kernels run in this arm."""
    import torch
    import torch.distributed as dist
    from summa_b200 import mal, ops
    from summa_b200.models import Transformer

    cfg = CONFIGS[config]
    world, rank, local = _dist_env()
    dev = torch.device("cuda", local)
    mdef = mal.get_builtin_model(cfg["preset"])
    blocks = [mdef.block_for_layer(i) for i in range(mdef.num_layers)]
    if any(b.ssm is not None or (b.ffn is not None and b.ffn.moe is not None) or b.memory is not None for b in blocks):
        return {"unavailable": "the stock-PyTorch arm covers dense attention models only (no library kernel for the "
                               "selective scan or the grouped expert GEMM at these shapes)"}
    ops.set_backend("library")
    try:
        torch.manual_seed(1234)
        with torch.device(dev):
            model = Transformer(mdef, init_std=0.02)
        model.stream_dtype = torch.bfloat16
        model.train()

        class _Loss(torch.nn.Module):
            def __init__(self, m):
                super().__init__()
                self.m = m

            def forward(self, tokens, targets):
                return self.m.forward_loss(tokens, targets)

        wrapped = _Loss(model)
        if world > 1:
            wrapped = torch.nn.parallel.DistributedDataParallel(wrapped, device_ids=[local], gradient_as_bucket_view=True)
        params = [p for p in model.parameters() if p.requires_grad]
        decay = [p for p in params if p.dim() >= 2]
        rest = [p for p in params if p.dim() < 2]
        opt = torch.optim.AdamW([{"params": decay, "weight_decay": 0.1}, {"params": rest, "weight_decay": 0.1}],
                                lr=3e-4, betas=(0.9, 0.95), eps=1e-8, fused=True)
        batches = make_batches(cfg, mdef.vocab_size, 8, seed=100 + rank, pin=True)
        dev_batches = [b.to(dev) for b in batches]
        GA = cfg.get("grad_accum", 1)
        B, S = cfg["micro_batch"] * GA, cfg["seq"]
        micro = cfg["micro_batch"]

        def step(t):
            opt.zero_grad(set_to_none=True)
            total = None
            for g in range(GA):
                tt = t[g * micro:(g + 1) * micro]
                loss = wrapped(tt[:, :-1], tt[:, 1:])
                (loss / GA).backward()
                total = loss.detach() if total is None else total + loss.detach()
            torch.nn.utils.clip_grad_norm_(params, 1.0)
            opt.step()
            return total / GA

        ms_dev, _, last = _timed_region(lambda i: step(dev_batches[i % 8]), W, K, True, world, dev)
        ms_e2e, wall, _ = _timed_region(lambda i: float(step(batches[i % 8].to(dev, non_blocking=True)).item()),
                                        W, K, True, world, dev)
        if world == 1:
            ms_e2e = max(ms_e2e, wall)
        tokens_per_step = B * S * world
        out = {"value": tokens_per_step * K / (ms_dev / 1e3), "ms_per_step": ms_dev / K,
               "e2e": {"value": tokens_per_step * K / (ms_e2e / 1e3), "unit": "tokens/s", "ms_per_step": ms_e2e / K,
                       "h2d_bytes_per_step": B * (S + 1) * 8, "d2h_bytes_per_step": 4},
               "final_loss": float(last), "parallelism": f"ddp{world}"}
        del opt, wrapped, model, dev_batches
        torch.cuda.empty_cache()
        return out
    finally:
        ops.set_backend("native")


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "torch"],
                    help="ours: this package; torch: the stock-PyTorch + NCCL baseline on the same model; "
                         "reference: the upstream project (cannot be installed here)")
    ap.add_argument("--config", default="llama350m", choices=sorted(CONFIGS))
    ap.add_argument("--optimizer", default="adamw", choices=["adamw", "muon"],
                    help="muon: Newton-Schulz Muon on the block matrices + AdamW on the rest (the reference's recipe)")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the stock-PyTorch comparison and the retriever-100m secondary run of the default line")
    ap.add_argument("--cpu", action="store_true", help="run the plumbing config on CPU (tiny only)")
    args = ap.parse_args()
    world, rank, local = _dist_env()
    if args.impl == "reference":
        if rank == 0:
            reference_arm()
        return

    import torch
    import torch.distributed as dist
    use_cuda = torch.cuda.is_available() and not args.cpu
    if args.gpus != world and world > 1:
        raise SystemExit(f"--gpus {args.gpus} != WORLD_SIZE {world}")
    W = max(args.warmup, 3) if use_cuda else args.warmup
    K = args.steps
    if use_cuda:
        torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl" if use_cuda else "gloo",
                                device_id=torch.device("cuda", local) if use_cuda else None)

    pub = PUBLISHED_TOK_S.get(args.config)
    base = {"metric": "train_tokens_per_second", "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W,
            "higher_is_better": True, "scaling": "weak", "dtype": "bf16" if use_cuda else "fp32"}
    if args.impl == "torch":
        if not use_cuda:
            raise SystemExit("--impl torch needs a GPU")
        r = run_torch(args.config, K, W)
        if rank == 0:
            if "unavailable" in r:
                print(json.dumps({"impl": "torch", "unavailable": r["unavailable"]}))
            else:
                print(json.dumps({**base, "impl": "torch", "value": r["value"], "ms_per_step": r["ms_per_step"],
                                  "vs_baseline": (r["value"] / pub) if pub else None, "e2e": r["e2e"],
                                  "final_loss": r["final_loss"], "gpu_launches": 0,
                                  "config": {"model": CONFIGS[args.config]["preset"], "parallelism": r["parallelism"],
                                             "optimizer": "torch.optim.AdamW(fused)+clip_grad_norm_"}}))
        if world > 1:
            dist.destroy_process_group()
        return

    ours = run_ours(args.config, K, W, use_cuda, sample_clocks=True, optimizer=args.optimizer)
    out = {**base, "value": ours["value"], "ms_per_step": ours["ms_per_step"],
           "vs_baseline": (ours["value"] / pub) if pub else None, "data": ours["data"], "config": ours["config"],
           "clocks": ours["clocks"] or {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}, "e2e": ours["e2e"],
           "gpu_launches": ours["gpu_launches"], "final_loss": ours["final_loss"],
           "device_error_word": ours["device_error_word"]}
    if use_cuda and not args.no_extras and args.config == "llama350m":
        # (1) the same model on stock PyTorch library ops, same box, same steps: the baseline the kernels must beat
        tk = min(K, 10)
        tr = run_torch(args.config, tk, 3)
        if "unavailable" not in tr:
            out["vs_baseline_torch"] = {"value": ours["value"] / tr["value"], "e2e": ours["e2e"]["value"] / tr["e2e"]["value"],
                                        "torch_tokens_per_second": tr["value"], "torch_e2e_tokens_per_second": tr["e2e"]["value"],
                                        "torch_ms_per_step": tr["ms_per_step"], "steps": tk,
                                        "what": "same Transformer on cuBLAS + SDPA + F.rms_norm + fused AdamW (+ DDP/NCCL)"}
        # (2) the one configuration the reference published a number for (A100-40G): retriever-100m hybrid
        sec = run_ours("retriever100m", 2, 3, use_cuda, sample_clocks=False)
        spub = PUBLISHED_TOK_S["retriever100m"] * world
        out["secondary"] = {"config": sec["config"], "value": sec["value"], "unit": "tokens/s",
                            "ms_per_step": sec["ms_per_step"], "e2e_value": sec["e2e"]["value"], "steps": 2, "warmup": 3,
                            "published_tokens_per_second_per_gpu": PUBLISHED_TOK_S["retriever100m"],
                            "vs_published": sec["value"] / spub, "device_error_word": sec["device_error_word"],
                            "published_source": "docs/segmented-selective-scan.md:207-208 (1 x A100-40G, B27)"}
    if rank == 0:
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
