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
be installed here.
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


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="llama350m", choices=sorted(CONFIGS))
    ap.add_argument("--cpu", action="store_true", help="run the plumbing config on CPU (tiny only)")
    args = ap.parse_args()
    if args.impl == "reference":
        if int(os.environ.get("RANK", "0")) == 0:
            reference_arm()
        return

    import torch
    import torch.distributed as dist
    from summa_b200 import mal
    from summa_b200.models import Transformer
    from summa_b200.ops import native
    from summa_b200.train.engine import FlatTrainEngine, OptimConfig, train_step

    cfg = CONFIGS[args.config]
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    use_cuda = torch.cuda.is_available() and not args.cpu
    if args.gpus != world and world > 1:
        raise SystemExit(f"--gpus {args.gpus} != WORLD_SIZE {world}")
    W = max(args.warmup, 3) if use_cuda else args.warmup
    K = args.steps

    dp = None
    if use_cuda:
        torch.cuda.set_device(local)
        dev = torch.device("cuda", local)
    else:
        dev = torch.device("cpu")
    if world > 1:
        dist.init_process_group("nccl" if use_cuda else "gloo", device_id=dev if use_cuda else None)
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
        engine = FlatTrainEngine(model, OptimConfig(lr=3e-4), dp=dp, param_dtype=torch.bfloat16)
    else:
        engine = FlatTrainEngine(model, OptimConfig(lr=3e-4), dp=dp, param_dtype=torch.float32)
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

    def sync():
        if use_cuda:
            torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            if use_cuda:
                torch.cuda.synchronize()

    def one_step(i, e2e):
        host = batches[i % len(batches)]
        if e2e or not use_cuda:
            t = host.to(dev, non_blocking=True)
        else:
            t = dev_batches[i % len(dev_batches)]
        loss, norm = train_step(model, engine, t[:, :-1], t[:, 1:], grad_accum=GA)
        if e2e:
            return float(loss.item())
        return loss

    dev_batches = [b.to(dev) for b in batches] if use_cuda else batches

    def timed(e2e: bool):
        for i in range(W):
            one_step(i, e2e)
        sync()
        launches["n"] = 0
        if use_cuda:
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record()
        t0 = time.perf_counter()
        last = None
        for i in range(K):
            last = one_step(W + i, e2e)
        if use_cuda:
            ev1.record()
        sync()
        wall = time.perf_counter() - t0
        ms = ev0.elapsed_time(ev1) if use_cuda else wall * 1e3
        if e2e and use_cuda:
            ms = max(ms, wall * 1e3 - 0.0)      # e2e includes the host-side readback
        if world > 1:
            t = torch.tensor([ms], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms, last

    sampler = ClockSampler(local)
    if use_cuda and rank == 0:
        sampler.start()
    ms_dev, last_loss = timed(False)
    n_launch = launches["n"]
    clocks = sampler.stop() if (use_cuda and rank == 0) else {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
    ms_e2e, last_e2e = timed(True)
    err = native.read_error_flag() if use_cuda else 0

    if rank == 0:
        value = tokens_per_step * K / (ms_dev / 1e3)
        e2e_val = tokens_per_step * K / (ms_e2e / 1e3)
        pub = PUBLISHED_TOK_S.get(args.config)
        out = {
            "metric": "train_tokens_per_second",
            "value": value, "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms_dev / K, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": (value / pub) if pub else None,
            "dtype": "bf16" if use_cuda else "fp32",
            "data": f"synthetic {cfg['data']} tokens, random-init N(0,0.02) weights",
            "config": {"model": mdef.name, "params": mdef.estimated_params(), "global_batch": B * world,
                       "seq_len": S, "grad_accum": GA, "micro_batch": cfg["micro_batch"],
                       "parallelism": parallelism, "optimizer": "adamw+clip",
                       "l2_policy": "inputs larger than L2 (activations ~15 GB per step)"},
            "clocks": clocks,
            "e2e": {"value": e2e_val, "unit": "tokens/s", "ms_per_step": ms_e2e / K,
                    "h2d_bytes_per_step": B * (S + 1) * 8, "d2h_bytes_per_step": 4},
            "gpu_launches": n_launch,
            "final_loss": float(last_loss) if last_loss is not None else None,
            "device_error_word": err,
        }
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
