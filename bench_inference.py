"""Inference benchmark: 7B-class dense decoder (32 x 4096, 32 query / 8 KV heads, SwiGLU 14336,
vocab 32000), weights random-init then group-quantised to 4 bit (group 128, bf16 scales),
tensor-parallel over N GPUs; prefill of a uniform-random prompt, then greedy decode.

    python bench_inference.py --gpus 1 --batch 1
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port P bench_inference.py --gpus 8 --batch 64

Prints one JSON line: decode tokens/s (whole job, all sequences) and the median time to first
token, both device-timed with CUDA events and taken as the max over ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--prompt", type=int, default=2048)
    ap.add_argument("--decode", type=int, default=256)
    ap.add_argument("--reps", type=int, default=3)
    ap.add_argument("--preset", default="dense_7b_gqa")
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (0 = preset); reported in config")
    ap.add_argument("--no-quant", action="store_true")
    a = ap.parse_args()

    import torch
    import torch.distributed as dist
    from summa_b200 import mal
    from summa_b200.models.engine import InferenceEngine
    from summa_b200.ops import native

    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    group = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        group = dist.group.WORLD
    rank = dist.get_rank() if world > 1 else 0

    cfg = mal.get_builtin_model(a.preset)
    if a.layers:
        cfg.num_layers = a.layers
    cfg.max_seq_len = max(cfg.max_seq_len, a.prompt + a.decode + 8)
    eng = InferenceEngine.build(cfg, dev, tp_group=group, quantize=None if a.no_quant else "int4",
                                max_prefill_tokens=a.batch * a.prompt, quantize_head=not a.no_quant)
    g = torch.Generator().manual_seed(1234)
    prompt = torch.randint(0, cfg.vocab_size, (a.batch, a.prompt), generator=g).to(dev)

    ttft, dec = [], []
    for rep in range(a.reps + 1):                       # first repetition is the warm-up
        eng.reset(a.batch, a.prompt + a.decode + 8)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        e0.record()
        first = eng.prefill(prompt)
        e1.record()
        out = eng.decode(first, a.decode)
        e2.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1), e1.elapsed_time(e2)], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if rep > 0:
            ttft.append(float(t[0]))
            dec.append(float(t[1]))
    ttft.sort(); dec.sort()
    ttft_ms, dec_ms = ttft[len(ttft) // 2], dec[len(dec) // 2]
    if rank == 0:
        print(json.dumps({
            "metric": "decode_tokens_per_second", "value": a.batch * a.decode / dec_ms * 1e3, "unit": "tokens/s",
            "p50_ttft_ms": ttft_ms, "prefill_tokens_per_second": a.batch * a.prompt / ttft_ms * 1e3,
            "ms_per_decode_step": dec_ms / a.decode, "n_gpus": world, "higher_is_better": True, "dtype": "bf16",
            "data": "synthetic uniform tokens, random-init N(0,0.02) weights",
            "config": {"model": a.preset, "layers": cfg.num_layers, "weights": "bf16" if a.no_quant else "int4 g128 bf16 scales",
                       "batch": a.batch, "prompt": a.prompt, "decode": a.decode, "parallelism": f"tp{world}",
                       "kv_cache": "bf16"},
            "sample_tokens": out[0, :8].tolist(), "device_error_word": native.read_error_flag()}))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
