"""Tensor parallelism for inference: attention heads and FFN columns are sharded across
the ranks of one NVSwitch domain.

Column-parallel projections (`qkv_proj`, FFN `in_proj`) keep a slice of the output
columns; row-parallel projections (`o_proj`, `down_proj`) keep the matching slice of
input rows and their partial outputs are summed across ranks. The sum runs either through
NCCL (`mode="collective"`, the baseline) or through the one-shot peer-memory all-reduce of
`csrc/tp_comm.cu` (`mode="fused"`): every rank stores its partial rows into all peers'
symmetric buffers and each rank adds the eight slices locally, which for decode-sized
activations is a single sub-10 µs kernel instead of a ring.

The reference has no tensor-parallel path (`summa-llm/src/model/backend.rs:39-55`).
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from ..models.layers import FeedForward, Linear, MultiHeadAttention
from ..ops import native


class TensorParallelGroup:
    def __init__(self, group, device: torch.device, mode: str = "fused", max_elems: int = 64 * 16384):
        self.group = group
        self.device = device
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.mode = mode if device.type == "cuda" else "collective"
        self.epoch = 0
        if self.mode == "fused":
            import torch.distributed._symmetric_memory as symm_mem
            # per rank: `world` inbox slots of max_elems bf16 each, double buffered
            self.max_elems = max_elems
            self.inbox = symm_mem.empty(2 * self.world * max_elems, dtype=torch.bfloat16, device=device)
            h = symm_mem.rendezvous(self.inbox, group.group_name)
            self.inbox.zero_()
            self.inbox_ptrs = (ctypes.c_void_p * self.world)(*[int(p) for p in h.buffer_ptrs])
            self.sig = symm_mem.empty(64, dtype=torch.int32, device=device)
            hs = symm_mem.rendezvous(self.sig, group.group_name)
            self.sig.zero_()
            self.sig_ptrs = (ctypes.c_void_p * self.world)(*[int(p) for p in hs.buffer_ptrs])
            self._keep = (h, hs)
            native.register("sb_tp_allreduce", [native.P, native.P, native.P, native.P, native.L, native.L,
                                                native.I, native.I, ctypes.c_uint, native.P])
            torch.cuda.synchronize()
            dist.barrier(group)

    def all_reduce(self, y: torch.Tensor) -> torch.Tensor:
        """Sum `y` over the group (in place semantics: returns the reduced tensor)."""
        if self.world == 1:
            return y
        if self.mode != "fused" or y.numel() > self.max_elems or y.dtype != torch.bfloat16:
            dist.all_reduce(y, group=self.group)
            return y
        yc = y.contiguous()
        out = torch.empty_like(yc)
        self.epoch += 1
        native.call("sb_tp_allreduce", yc.data_ptr(), out.data_ptr(), self.inbox_ptrs, self.sig_ptrs, yc.numel(),
                    self.max_elems, self.rank, self.world, self.epoch, native.stream())
        return out.view(y.shape)


class RowParallelLinear(nn.Module):
    def __init__(self, inner: nn.Module, tp: TensorParallelGroup):
        super().__init__()
        self.inner = inner
        self.tp = tp

    def forward(self, x):
        return self.tp.all_reduce(self.inner(x))


def _slice_linear(lin: Linear, cols=None, rows=None) -> Linear:
    w = lin.weight.detach()
    if cols is not None:
        w = torch.cat([w[:, a:b] for a, b in cols], dim=1)
    if rows is not None:
        w = w[rows[0]:rows[1]]
    out = Linear(w.shape[0], w.shape[1], bias=False)
    out.weight = nn.Parameter(w.contiguous().clone(), requires_grad=False)
    if lin.bias is not None:
        b = lin.bias.detach()
        if cols is not None:
            b = torch.cat([b[a:b_] for a, b_ in cols])
            out.bias = nn.Parameter(b.clone(), requires_grad=False)
        elif rows is not None:
            # a row-parallel bias is added once: keep it on rank 0's shard only
            out.bias = nn.Parameter(b.clone(), requires_grad=False) if rows[0] == 0 else None
    return out


def shard_model(model, tp: TensorParallelGroup):
    """Shard every attention and dense-FFN block of `model` in place for rank `tp.rank`."""
    P, r = tp.world, tp.rank
    for blk in model.layers:
        a = blk.attention
        if isinstance(a, MultiHeadAttention):
            if a.num_heads % P or a.num_kv_heads % P:
                raise ValueError(f"heads {a.num_heads}/{a.num_kv_heads} not divisible by tensor-parallel size {P}")
            D = a.head_dim
            hq, hkv = a.num_heads // P, a.num_kv_heads // P
            q0, k0, v0 = 0, a.q_dim, a.q_dim + a.kv_dim
            cols = [(q0 + r * hq * D, q0 + (r + 1) * hq * D), (k0 + r * hkv * D, k0 + (r + 1) * hkv * D),
                    (v0 + r * hkv * D, v0 + (r + 1) * hkv * D)]
            a.qkv_proj = _slice_linear(a.qkv_proj, cols=cols)
            a.o_proj = RowParallelLinear(_slice_linear(a.o_proj, rows=(r * hq * D, (r + 1) * hq * D)), tp)
            a.num_heads, a.num_kv_heads = hq, hkv
            a.q_dim, a.kv_dim = hq * D, hkv * D
        ff = blk.feed_forward
        if isinstance(ff, FeedForward):
            I = ff.down_proj.d_in
            if I % P:
                raise ValueError(f"FFN width {I} not divisible by tensor-parallel size {P}")
            s = I // P
            cols = [(r * s, (r + 1) * s)] + ([(I + r * s, I + (r + 1) * s)] if ff.gated else [])
            ff.in_proj = _slice_linear(ff.in_proj, cols=cols)
            ff.down_proj = RowParallelLinear(_slice_linear(ff.down_proj, rows=(r * s, (r + 1) * s)), tp)
    return model
