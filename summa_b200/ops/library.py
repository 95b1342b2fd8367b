"""Stock PyTorch library ops for CUDA tensors: the measured baseline, not a product path.

`ops.set_backend("library")` routes the model's hot ops here, so the SAME `Transformer` runs the way a
plain PyTorch program would run it on this GPU: cuBLAS for every matmul, `scaled_dot_product_attention`
(flash / cuDNN kernels, native GQA) for attention, `F.rms_norm`, eager SiLU-gate, and a row-chunked
`F.cross_entropy` over bf16-GEMM logits (the chunking the reference's loss uses,
`summa-llm/src/model/linear_cross_entropy/reference.rs:66-90`). `bench.py --impl torch` times that
model with `torch.optim.AdamW(fused=True)`, `clip_grad_norm_` and NCCL data parallelism and reports
it next to this package's kernels.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def rmsnorm(x, gamma, eps):
    return F.rms_norm(x, (x.shape[-1],), gamma.to(x.dtype), eps)


def attention(q, k, v, causal):
    """q `[B, S, H, D]`, k / v `[B, S, KV, D]` -> `[B, S, H, D]`."""
    o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=causal,
                                       enable_gqa=k.shape[2] != q.shape[2])
    return o.transpose(1, 2)


def swiglu(x):
    gate, value = x.chunk(2, dim=-1)
    return F.silu(gate) * value


def linear_cross_entropy(hidden, weight, bias, targets, vocab_size, chunks=4):
    """Mean cross-entropy of `hidden @ weight (+ bias)` over the logical vocabulary, in row chunks."""
    rows = hidden.shape[0]
    per = (rows + chunks - 1) // chunks
    w = weight.to(hidden.dtype)
    total = hidden.new_zeros((), dtype=torch.float32)
    for s in range(0, rows, per):
        logits = hidden[s:s + per] @ w
        if bias is not None:
            logits = logits + bias.to(logits.dtype)
        total = total + F.cross_entropy(logits[:, :vocab_size].float(), targets[s:s + per], reduction="sum")
    return total / rows
