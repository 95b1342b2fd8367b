"""Expert parallelism: the experts of every MoE layer are sharded over the ranks of one
NVSwitch domain (rank o owns experts [o*E/P, (o+1)*E/P)), tokens stay where they are.

`mode="fused"` (CUDA): routing stays local (top-k, histogram and the expert-sorted, padded
"source layout" of `ops/csrc/moe.cu`); the dispatch kernel gathers each routed token row and
stores it straight into its final row of the owning rank's compact buffer over NVLink, the
owner runs the grouped tcgen05 GEMMs on that buffer, and the return kernel stores every
output row back into the source layout of the rank it came from (`ops/csrc/ep_comm.cu`).
All offsets derive from one P x E count matrix that the ranks publish to each other, so the
host never sees a count and no per-row metadata crosses the link. The backward pass runs the
same two exchanges on the gradients.

`mode="collective"`: the same math through `all_to_all_single` (NCCL on GPUs, gloo on CPU
ranks): the baseline and the oracle for tests. The reference has no expert parallelism
(`summa-llm/src/model/backend.rs:39-55`).
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.distributed as dist

from .. import ops
from ..ops import native


class _OwnerPlan:
    """Grouped-GEMM metadata of the owner's compact layout (device resident)."""

    def __init__(self, El: int, max_rows: int, device):
        self.E, self.max_rows = El, max_rows
        self.meta = torch.zeros(El + 2, device=device, dtype=torch.int32)
        self.tile_expert = torch.zeros(max_rows // 128, device=device, dtype=torch.int32)
        self.counts = torch.zeros(El, device=device, dtype=torch.int32)

    @property
    def num_m_tiles_ptr(self) -> int:
        return self.meta.data_ptr() + 4 * (self.E + 1)


class ExpertParallelGroup:
    def __init__(self, group, device: torch.device, num_experts: int, hidden: int, max_tokens: int, top_k: int,
                 mode: str = "fused", capacity_factor: float = 0.0):
        """`max_tokens`: tokens per rank per MoE call. `capacity_factor`: rows the owner's compact
        buffer can take, as a multiple of the balanced share (0 = worst case, every route of
        every rank lands on one owner)."""
        self.group, self.device = group, device
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if num_experts % self.world:
            raise ValueError(f"{num_experts} experts not divisible by expert-parallel size {self.world}")
        self.E, self.El, self.H, self.k = num_experts, num_experts // self.world, hidden, top_k
        self.mode = mode if device.type == "cuda" else "collective"
        self.epoch = 0
        self.src_rows = -(-(max_tokens * top_k + num_experts * 127) // 128) * 128
        worst = self.world * max_tokens * top_k
        rows = worst if capacity_factor <= 0 else min(worst, int(capacity_factor * max_tokens * top_k))
        self.own_rows = -(-(rows + self.El * 127) // 128) * 128
        if self.mode == "fused":
            import torch.distributed._symmetric_memory as symm_mem
            keep = []

            def sym(numel, dtype):
                t = symm_mem.empty(numel, dtype=dtype, device=device)
                h = symm_mem.rendezvous(t, group.group_name)
                t.zero_()
                keep.append(h)
                return t, (ctypes.c_void_p * self.world)(*[int(p) for p in h.buffer_ptrs])

            self.recv, self.recv_ptrs = sym(self.own_rows * hidden, torch.bfloat16)
            self.ret, self.ret_ptrs = sym(self.src_rows * hidden, torch.bfloat16)
            self.count_mat, self.count_ptrs = sym(self.world * num_experts, torch.int32)
            self.sig, self.sig_ptrs = sym(64, torch.int32)
            self._keep = keep
            P, I, L = native.P, native.I, native.L
            common = [P, P, P, P]
            native.register("sb_ep_counts", common + [P, I, I, I, ctypes.c_uint, P])
            native.register("sb_ep_dispatch", common + [P, L, P, P, P, P, P, I, I, I, I, I, I, ctypes.c_uint, I, P])
            native.register("sb_ep_meta", common + [P, P, P, P, I, I, I, I, I, ctypes.c_uint, P])
            native.register("sb_ep_return", common + [P, P, P, I, I, I, I, I, ctypes.c_uint, P])
            native.register("sb_ep_wait_return", common + [I, I, I, ctypes.c_uint, P])
            torch.cuda.synchronize()
            dist.barrier(group)

    # ------------------------------------------------------------------ fused primitives
    def _common(self):
        return (self.recv_ptrs, self.ret_ptrs, self.count_ptrs, self.sig_ptrs)

    def exchange_to_owner(self, plan, x=None, src_rows=None) -> "tuple[torch.Tensor, _OwnerPlan]":
        """One dispatch round: publish counts, push rows (gathered from `x` `[T, H]` or taken from
        `src_rows` in source layout), wait on the owner side. Returns (compact rows view, owner plan)."""
        self.epoch += 1
        st = native.stream()
        native.call("sb_ep_counts", *self._common(), plan.counts.data_ptr(), self.E, self.rank, self.world, self.epoch, st)
        xp = x.data_ptr() if x is not None else None
        ldx = x.stride(0) if x is not None else 0
        sp = src_rows.data_ptr() if src_rows is not None else None
        native.call("sb_ep_dispatch", *self._common(), xp, ldx, sp, plan.row_route.data_ptr(), plan.meta.data_ptr(),
                    plan.tile_expert.data_ptr(), plan.counts.data_ptr(), plan.max_rows, self.E, self.H, plan.k, self.rank,
                    self.world, self.epoch, self.own_rows, st)
        op = _OwnerPlan(self.El, self.own_rows, self.device)
        native.call("sb_ep_meta", *self._common(), op.meta.data_ptr(), op.tile_expert.data_ptr(), op.counts.data_ptr(),
                    self.recv.data_ptr(), self.E, self.H, self.own_rows // 128, self.rank, self.world, self.epoch, st)
        return self.recv.view(self.own_rows, self.H), op

    def exchange_to_source(self, y: torch.Tensor, op: _OwnerPlan) -> torch.Tensor:
        """One return round: push compact rows `y` back to their sources and wait for this rank's
        own rows. Returns the source-layout view (valid until the next return round)."""
        st = native.stream()
        native.call("sb_ep_return", *self._common(), y.data_ptr(), op.meta.data_ptr(), op.tile_expert.data_ptr(),
                    self.own_rows, self.E, self.H, self.rank, self.world, self.epoch, st)
        native.call("sb_ep_wait_return", *self._common(), self.E, self.rank, self.world, self.epoch, st)
        return self.ret.view(self.src_rows, self.H)

    # ------------------------------------------------------------------ layer entry point
    def forward(self, x, idx, gates, experts, act, gated):
        """Routed expert MLP for local tokens `x` `[T, H]` with LOCAL expert shards in `experts`."""
        if (self.mode == "fused" and x.is_cuda and x.dtype == torch.bfloat16 and gated and act in ("swiglu", "silu")
                and experts.in_bias is None and getattr(idx, "_sb_plan", None) is not None):
            from ..ops import cuda_ops
            return cuda_ops.ep_moe_experts(self, x, gates, experts.in_weight, experts.down_weight, idx._sb_plan)
        return _collective_moe(self, x, idx, gates, experts, act, gated)


def _collective_moe(ep: ExpertParallelGroup, x, idx, gates, experts, act, gated):
    """all_to_all_single form (differentiable through torch.distributed.nn-free manual autograd:
    the exchanges are wrapped in an autograd Function whose backward is the reverse exchange)."""
    T, H = x.shape
    k = idx.shape[1]
    P, El = ep.world, ep.El
    flat_e = idx.reshape(-1)
    order = torch.argsort(flat_e, stable=True)
    token_of = order // k
    counts = torch.bincount(flat_e, minlength=ep.E)
    send_counts = counts.view(P, El).sum(dim=1)
    # exchange the per-expert counts so that owners can split what they receive by expert
    all_counts = torch.empty(P * ep.E, dtype=counts.dtype, device=x.device)
    dist.all_gather_into_tensor(all_counts, counts, group=ep.group)
    all_counts = all_counts.view(P, ep.E)[:, ep.rank * El:(ep.rank + 1) * El]       # [src, local expert]
    recv_counts = all_counts.sum(dim=1)
    send_list, recv_list = send_counts.tolist(), recv_counts.tolist()
    routed = x.index_select(0, token_of)
    recv = _AllToAll.apply(routed, send_list, recv_list, ep.group)
    # received rows are (src, local expert)-ordered; run each expert on its pieces
    pieces = all_counts.reshape(-1).tolist()
    chunks = list(torch.split(recv, pieces, dim=0))
    outs = [None] * len(chunks)
    for el in range(El):
        sel = [s * El + el for s in range(P)]
        seg = torch.cat([chunks[i] for i in sel], dim=0)
        if seg.shape[0]:
            h = seg @ experts.in_weight[el].to(seg.dtype)
            if experts.in_bias is not None:
                h = h + experts.in_bias[el].to(h.dtype)
            h = ops.reference.gated_act(h, act) if gated else ops.reference.activation(act, h.float()).to(h.dtype)
            y = h @ experts.down_weight[el].to(h.dtype)
            if experts.down_bias is not None:
                y = y + experts.down_bias[el].to(y.dtype)
        else:
            y = seg.new_zeros(0, H)
        for i, part in zip(sel, torch.split(y, [pieces[i] for i in sel], dim=0)):
            outs[i] = part
    back = _AllToAll.apply(torch.cat(outs, dim=0), recv_list, send_list, ep.group)
    w = gates.reshape(-1).index_select(0, order).to(back.dtype)
    out = torch.zeros(T, H, dtype=back.dtype, device=x.device)
    return out.index_add(0, token_of, back * w[:, None]).to(x.dtype)


class _AllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, send, recv, group):
        ctx.send, ctx.recv, ctx.group = send, recv, group
        out = x.new_empty(sum(recv), *x.shape[1:])
        dist.all_to_all_single(out, x.contiguous(), output_split_sizes=recv, input_split_sizes=send, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        out = g.new_empty(sum(ctx.send), *g.shape[1:])
        dist.all_to_all_single(out, g.contiguous(), output_split_sizes=ctx.send, input_split_sizes=ctx.recv,
                               group=ctx.group)
        return out, None, None, None


def shard_experts(model, ep: ExpertParallelGroup):
    """Keep only this rank's experts in every MoE layer of `model` and route through `ep`.
    Routers, shared experts and everything else stay replicated (their gradients are reduced
    by data parallelism; expert gradients are local)."""
    from ..models.layers import SparseMoe
    lo, hi = ep.rank * ep.El, (ep.rank + 1) * ep.El
    for mod in model.modules():
        if isinstance(mod, SparseMoe):
            bank = mod.moe.experts
            for name in ("in_weight", "down_weight", "in_bias", "down_bias"):
                p = getattr(bank, name)
                if p is not None:
                    q = torch.nn.Parameter(p.detach()[lo:hi].clone(), requires_grad=p.requires_grad)
                    q._sb_local = True          # never reduced across ranks (see train.engine.FlatTrainEngine)
                    setattr(bank, name, q)
            mod.ep = ep
    return model
