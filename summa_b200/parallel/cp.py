"""Context parallelism: one long sequence sharded over the ranks of an NVSwitch domain.

Every rank keeps `S / P` positions of the residual stream (norms, projections, FFN and loss touch
only local rows); attention is the one op that needs other ranks' keys and values. They are
all-gathered into LOCAL buffers (NCCL on GPUs, gloo on CPU ranks; an NVSwitch all-gather moves
each K/V byte once per rank) and the local flash-attention kernel runs on local queries against
the gathered keys with its `q_offset` argument, so no attention kernel ever reads a peer's memory.
The backward pass is autograd through the same kernel plus a reduce-scatter of dK / dV.

Causal attention over contiguous shards would give the last rank P times the work of the first;
with `zigzag=True` the sequence is cut into 2P chunks and rank r holds chunks r and 2P-1-r, which
balances the causal work to within one chunk. The reference has no context parallelism and handles
long sequences on one device only (`summa-llm/src/model/fused_attention.rs:264-404`,
`summa-llm/src/model/backend.rs:39-55`).
"""
from __future__ import annotations

from typing import List, Tuple

import torch
import torch.distributed as dist

from .. import ops


def zigzag_chunks(rank: int, world: int) -> Tuple[int, int]:
    return rank, 2 * world - 1 - rank


def zigzag_split(x: torch.Tensor, rank: int, world: int, dim: int = 1) -> torch.Tensor:
    """This rank's two chunks of a full-sequence tensor, concatenated along `dim`."""
    S = x.shape[dim]
    if S % (2 * world):
        raise ValueError(f"sequence length {S} is not a multiple of {2 * world}")
    c = S // (2 * world)
    a, b = zigzag_chunks(rank, world)
    return torch.cat([x.narrow(dim, a * c, c), x.narrow(dim, b * c, c)], dim=dim)


def zigzag_positions(rank: int, world: int, seq_len: int, device=None) -> torch.Tensor:
    """Global positions of this rank's local rows (for RoPE and targets)."""
    c = seq_len // (2 * world)
    a, b = zigzag_chunks(rank, world)
    return torch.cat([torch.arange(a * c, (a + 1) * c, device=device), torch.arange(b * c, (b + 1) * c, device=device)])


def zigzag_merge(parts: List[torch.Tensor], dim: int = 1) -> torch.Tensor:
    """Inverse of `zigzag_split` over the list of every rank's local tensor (rank order)."""
    world = len(parts)
    c = parts[0].shape[dim] // 2
    chunks = [None] * (2 * world)
    for r, p in enumerate(parts):
        a, b = zigzag_chunks(r, world)
        chunks[a], chunks[b] = p.narrow(dim, 0, c), p.narrow(dim, c, c)
    return torch.cat(chunks, dim=dim)


class _GatherSequence(torch.autograd.Function):
    """All-gather along dim 1 into a local buffer; backward = reduce-scatter (sum) of the gradient."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        P = dist.get_world_size(group)
        xc = x.contiguous()
        parts = [torch.empty_like(xc) for _ in range(P)]
        dist.all_gather(parts, xc, group=group)
        return torch.stack(parts)                       # [P, B, S_local, ...]

    @staticmethod
    def backward(ctx, g):
        P, r = dist.get_world_size(ctx.group), dist.get_rank(ctx.group)
        g = g.contiguous()
        if dist.get_backend(ctx.group) == "gloo":       # no reduce_scatter on gloo: all-reduce, keep own slice
            dist.all_reduce(g, group=ctx.group)
            return g[r], None
        out = torch.empty_like(g[0])
        dist.reduce_scatter(out, list(g.unbind(0)), group=ctx.group)
        return out, None


def context_parallel_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, group, causal: bool = True,
                               zigzag: bool = True) -> torch.Tensor:
    """q `[B, S_local, Hq, D]`, k / v `[B, S_local, Hkv, D]` (RoPE already applied with GLOBAL
    positions) -> attention output for the local rows `[B, S_local, Hq, D]`.

    Contiguous layout (`zigzag=False`): rank r holds positions [r*S_local, (r+1)*S_local).
    Zigzag layout: rank r holds chunks r and 2P-1-r of 2P equal chunks (see `zigzag_split`)."""
    P, r = dist.get_world_size(group), dist.get_rank(group)
    S = q.shape[1]
    kg = _GatherSequence.apply(k, group)
    vg = _GatherSequence.apply(v, group)
    if not zigzag:
        kf = torch.cat(list(kg.unbind(0)), dim=1)
        vf = torch.cat(list(vg.unbind(0)), dim=1)
        if causal:                                      # keys after this rank's last query are never visible
            kf, vf = kf[:, :(r + 1) * S], vf[:, :(r + 1) * S]
        return ops.attention(q, kf.contiguous(), vf.contiguous(), causal, None, r * S if causal else 0)
    if S % 2:
        raise ValueError("zigzag layout needs an even local length")
    c = S // 2
    kf = zigzag_merge(list(kg.unbind(0)), dim=1)
    vf = zigzag_merge(list(vg.unbind(0)), dim=1)
    outs = []
    for j, chunk in enumerate(zigzag_chunks(r, P)):
        qj = q[:, j * c:(j + 1) * c].contiguous()
        if causal:
            hi = (chunk + 1) * c
            outs.append(ops.attention(qj, kf[:, :hi].contiguous(), vf[:, :hi].contiguous(), True, None, chunk * c))
        else:
            outs.append(ops.attention(qj, kf.contiguous(), vf.contiguous(), False, None, 0))
    return torch.cat(outs, dim=1)
