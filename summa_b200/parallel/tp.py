"""Tensor parallelism for inference: attention heads and FFN columns are sharded across
the ranks of one NVSwitch domain.

Column-parallel projections (`qkv_proj`, FFN `in_proj`) keep a slice of the output
columns; row-parallel projections (`o_proj`, `down_proj`) keep the matching slice of
input rows and their partial outputs are summed across ranks. The sum runs either through
NCCL (`mode="collective"`, the baseline) or through the one-shot peer-memory all-reduce of
`csrc/tp_comm.cu` (`mode="fused"`): every rank stores its partial rows into all peers'
symmetric buffers and each rank adds the eight slices locally, which for decode-sized
activations is a single sub-10 µs kernel instead of a ring.

Prefill-sized activations run sequence-parallel (`prefill_sequence_parallel`): each rank
keeps M/P rows of the residual stream, the column-parallel projections run as the fused
all-gather -> GEMM kernel and the row-parallel ones as the fused GEMM -> reduce-scatter kernel
of `csrc/gemm.cu`, so every activation byte crosses NVLink once, overlapped with the tensor-core
tiles, and norms / residual adds touch only M/P rows.

The reference has no tensor-parallel path (`summa-llm/src/model/backend.rs:39-55`).
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from ..models.layers import FeedForward, Linear, MultiHeadAttention
from ..ops import native


class TensorParallelGroup:
    def __init__(self, group, device: torch.device, mode: str = "fused", max_elems: int = 64 * 16384,
                 max_tokens: int = 0, hidden: int = 0):
        """`max_tokens` / `hidden` size the buffers of the sequence-parallel prefill path
        (0 = that path is not used)."""
        self.group = group
        self.device = device
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.mode = mode if device.type == "cuda" else "collective"
        self.epoch = 0
        self.gemm_epoch = 0
        self.max_tokens, self.hidden = 0, 0
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
                                                native.I, native.I, native.P, native.P, native.P])
            # NVLS form of the all-reduce (`multimem.ld_reduce` on the multicast address of a
            # symmetric staging buffer): opt-in, needs a multicast-capable allocation
            self.stage_mc = 0
            if os.environ.get("SUMMA_TP_MULTIMEM", "0") == "1":
                self.stage = symm_mem.empty(2 * max_elems, dtype=torch.bfloat16, device=device)
                hm = symm_mem.rendezvous(self.stage, group.group_name)
                self.stage.zero_()
                self.stage_mc = int(getattr(hm, "multicast_ptr", 0) or 0)
                # its own signal pad: the words of `self.sig` are all taken by the peer-store all-reduce
                # and the fused GEMMs
                self.sig_mm = symm_mem.empty(64, dtype=torch.int32, device=device)
                hsm = symm_mem.rendezvous(self.sig_mm, group.group_name)
                self.sig_mm.zero_()
                self.sig_mm_ptrs = (ctypes.c_void_p * self.world)(*[int(p) for p in hsm.buffer_ptrs])
                self._keep = self._keep + (hm, hsm)
                native.register("sb_tp_allreduce_mm", [native.P, native.P, native.P, native.P, native.P, native.L,
                                                       native.L, native.I, native.I, native.P, native.P, native.P])
            self.epoch_word = torch.zeros(1, dtype=torch.int32, device=device)   # call number, owned by the kernel
            # row-parallel decode projections with the all-reduce in their epilogue (`hquant.cu`): fp32 partials
            # per (parity, source rank, row <= 4, column) and one flag per (32-column block, source rank).
            # Opt-in (SUMMA_TP_FUSED_GEMV=1): correct, but measured slower than projection + one-shot
            # all-reduce on 2 GPUs (349 against 417 decode tokens/s), so the default is the two-kernel form.
            self.ar_hidden = hidden if (hidden > 0 and self.world <= 8 and
                                        os.environ.get("SUMMA_TP_FUSED_GEMV", "0") == "1") else 0
            if self.ar_hidden:
                self.ar_inbox = symm_mem.empty(2 * self.world * 4 * hidden, dtype=torch.float32, device=device)
                hai = symm_mem.rendezvous(self.ar_inbox, group.group_name)
                self.ar_inbox.zero_()
                self.ar_flags = symm_mem.empty(((hidden + 31) // 32) * 8, dtype=torch.int32, device=device)
                haf = symm_mem.rendezvous(self.ar_flags, group.group_name)
                self.ar_flags.zero_()
                self.ar_inbox_ptrs = (ctypes.c_void_p * self.world)(*[int(p) for p in hai.buffer_ptrs])
                self.ar_flag_ptrs = (ctypes.c_void_p * self.world)(*[int(p) for p in haf.buffer_ptrs])
                self.ar_words = torch.zeros(2, dtype=torch.int32, device=device)      # call number, CTA counter
                self._keep = self._keep + (hai, haf)
                native.register("sb_w4_gemv_cluster_allreduce",
                                [native.P] * 5 + [native.I, native.I, native.I, native.L, native.P, native.P, native.P,
                                 native.P, native.L, native.I, native.I, native.P])
            keep = list(self._keep)
            if max_tokens > 0 and self.world > 1:
                if max_tokens % (128 * self.world):
                    raise ValueError(f"max_tokens must be a multiple of {128 * self.world}")
                self.max_tokens, self.hidden = max_tokens, hidden
                # two full-size activation buffers (attention input, FFN input) whose own-row
                # blocks are written in place, and the reduce-scatter inbox (2 parities x P slots)
                self.xbufs, self.xbuf_ptrs, self.xbuf_mc = [], [], []
                for _ in range(2):
                    xb = symm_mem.empty(max_tokens * hidden, dtype=torch.bfloat16, device=device)
                    hx = symm_mem.rendezvous(xb, group.group_name)
                    self.xbufs.append(xb)
                    self.xbuf_ptrs.append((ctypes.c_void_p * self.world)(*[int(p) for p in hx.buffer_ptrs]))
                    self.xbuf_mc.append(int(getattr(hx, "multicast_ptr", 0) or 0))
                    keep.append(hx)
                # all-gather role of the paired-CTA GEMM: per-rank "done" words and one flag per 128-row chunk
                # (symmetric), chunk / exit counters (local); its own call counter
                self.ag_flags = symm_mem.empty(8 + max_tokens // 128, dtype=torch.int32, device=device)
                hf = symm_mem.rendezvous(self.ag_flags, group.group_name)
                self.ag_flags.zero_()
                self.ag_flag_ptrs = (ctypes.c_void_p * self.world)(*[int(p) for p in hf.buffer_ptrs])
                self.ag_counters = torch.zeros(max_tokens // 128 + 1, dtype=torch.int32, device=device)
                self.ag_pair_epoch = 0
                self.ag_multimem = os.environ.get("SUMMA_TP_AG_MULTIMEM", "1") == "1"
                keep.append(hf)
                native.register("sb_tp_ag_gemm_pair", [native.P] * 5 + [native.I, native.P, native.P] + [native.I] * 8 +
                                [ctypes.c_uint, native.P])
                self.slot_capacity = (max_tokens // self.world) * hidden
                self.rs_inbox = symm_mem.empty(2 * self.world * self.slot_capacity, dtype=torch.bfloat16, device=device)
                hr = symm_mem.rendezvous(self.rs_inbox, group.group_name)
                self.rs_inbox_ptrs = (ctypes.c_void_p * self.world)(*[int(p) for p in hr.buffer_ptrs])
                keep.append(hr)
                native.register("sb_tp_ag_gemm", [native.P, native.P, native.P, native.P, native.I, native.P,
                                                  native.I, native.I, native.I, native.I, native.I, native.I,
                                                  native.I, native.I, ctypes.c_uint, native.I, native.P])
                native.register("sb_tp_gemm_rs", [native.P, native.P, native.P, native.P, native.P, native.P,
                                                  native.I, native.I, native.I, native.I, native.I, native.I,
                                                  native.L, native.I, native.I, ctypes.c_uint, native.P])
            self._keep = tuple(keep)
            torch.cuda.synchronize()
            dist.barrier(group)

    # ------------------------------------------------------------------ sequence-parallel pieces
    def own_rows(self, which: int, M: int, K: int) -> torch.Tensor:
        """This rank's `[M/P, K]` row block of activation buffer `which`, to be written in place."""
        rows = M // self.world
        return self.xbufs[which][:M * K].view(M, K)[self.rank * rows:(self.rank + 1) * rows]

    def ag_gemm(self, which: int, M: int, K: int, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
                copiers: int = 0, transposed: bool = False) -> torch.Tensor:
        """gather(buffer `which`)[M, K] @ weight[K, N] (+ bias): fused all-gather -> GEMM. `transposed`: `weight`
        is stored `[N, K]` (the product with its transpose, without a copy)."""
        N = weight.shape[0] if transposed else weight.shape[1]
        b_mn = 0 if transposed else 1
        out = torch.empty(M, N, dtype=torch.bfloat16, device=self.device)
        bptr = bias.data_ptr() if bias is not None else None
        if (copiers == 0 and M % (256 * self.world) == 0 and K % 64 == 0 and N >= 256
                and os.environ.get("SUMMA_TP_AG_PAIR", "1") == "1"):
            # paired-CTA kernel with the gather as a push: every rank stores its rows once (through the switch's
            # multicast where the buffer has one), consumers wait per 128-row chunk; no copier CTAs
            self.ag_pair_epoch += 1
            native.call("sb_tp_ag_gemm_pair", self.xbuf_ptrs[which], (self.xbuf_mc[which] or None) if (self.ag_multimem and self.world > 2) else None,
                        weight.data_ptr(), out.data_ptr(), bptr, 1 if (bias is not None and bias.dtype == torch.bfloat16) else 0,
                        self.ag_flag_ptrs, self.ag_counters.data_ptr(), M, N, K, weight.stride(0), N, b_mn, self.rank,
                        self.world, self.ag_pair_epoch, native.stream())
            return out
        self.gemm_epoch += 1
        native.call("sb_tp_ag_gemm", self.xbuf_ptrs[which], weight.data_ptr(), out.data_ptr(), bptr,
                    1 if (bias is not None and bias.dtype == torch.bfloat16) else 0, self.sig_ptrs, M, N, K,
                    weight.stride(0), N, b_mn, self.rank, self.world, self.gemm_epoch, copiers, native.stream())
        return out

    def gemm_rs(self, a: torch.Tensor, weight: torch.Tensor, residual: Optional[torch.Tensor] = None,
                transposed: bool = False) -> torch.Tensor:
        """reduce_scatter(a[M, K_local] @ weight[K_local, N]) (+ residual[M/P, N]) -> `[M/P, N]`. `transposed`:
        `weight` is stored `[N, K_local]`."""
        M, K = a.shape
        N = weight.shape[0] if transposed else weight.shape[1]
        out = torch.empty(M // self.world, N, dtype=torch.bfloat16, device=self.device)
        self.gemm_epoch += 1
        native.call("sb_tp_gemm_rs", a.data_ptr(), weight.data_ptr(), self.rs_inbox_ptrs, self.sig_ptrs,
                    out.data_ptr(), residual.data_ptr() if residual is not None else None, M, N, K, a.stride(0),
                    weight.stride(0), 0 if transposed else 1, self.slot_capacity, self.rank, self.world, self.gemm_epoch,
                    native.stream())
        return out

    def gemv_allreduce(self, x: torch.Tensor, qlin, residual: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """sum over ranks of `x[M <= 4, K_local] @ dequant(qlin)` (+ residual) in ONE kernel per rank: the
        row-parallel decode projection whose epilogue exchanges the partials over peer memory. Returns None
        when the fused form does not apply (the caller then runs projection + all-reduce)."""
        if (self.mode != "fused" or not getattr(self, "ar_hidden", 0) or qlin.d_out != self.ar_hidden
                or qlin.bias is not None or x.dim() != 2 or x.shape[0] > 4 or x.dtype != torch.bfloat16
                or not x.is_cuda or qlin.d_in % 128 or qlin.d_in > 20480 or x.stride(1) != 1 or x.stride(0) % 8
                or x.data_ptr() % 16):
            return None
        res = None
        if residual is not None:
            res = residual.reshape(-1, qlin.d_out).contiguous()
            if res.dtype != torch.bfloat16:
                return None
        y = torch.empty(x.shape[0], qlin.d_out, dtype=torch.bfloat16, device=x.device)
        native.call("sb_w4_gemv_cluster_allreduce", x.data_ptr(), qlin.packed_k8().data_ptr(), qlin.scales.data_ptr(),
                    res.data_ptr() if res is not None else None, y.data_ptr(), x.shape[0], qlin.d_out, qlin.d_in,
                    x.stride(0), self.ar_inbox_ptrs, self.ar_flag_ptrs, self.ar_words.data_ptr(),
                    self.ar_words[1:].data_ptr(), self.ar_hidden, self.rank, self.world, native.stream())
        return y

    def all_reduce(self, y: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Sum `y` over the group (in place semantics: returns the reduced tensor); `residual` (same
        shape, replicated) is added once to the sum, inside the kernel on the fused path."""
        if self.world == 1:
            return y if residual is None else y + residual
        if self.mode != "fused" or y.numel() > self.max_elems or y.numel() % 8 or y.dtype != torch.bfloat16:
            dist.all_reduce(y, group=self.group)
            return y if residual is None else y + residual
        yc = y.contiguous()
        out = torch.empty_like(yc)
        res = None
        if residual is not None:
            res = residual.contiguous()
            if res.dtype != torch.bfloat16 or res.data_ptr() % 16:
                res = None
        rp = res.data_ptr() if res is not None else None
        if self.stage_mc:
            native.call("sb_tp_allreduce_mm", yc.data_ptr(), out.data_ptr(), self.stage.data_ptr(), self.stage_mc,
                        self.sig_mm_ptrs, yc.numel(), self.max_elems, self.rank, self.world,
                        self.epoch_word.data_ptr(), rp, native.stream())
        else:
            native.call("sb_tp_allreduce", yc.data_ptr(), out.data_ptr(), self.inbox_ptrs, self.sig_ptrs, yc.numel(),
                        self.max_elems, self.rank, self.world, self.epoch_word.data_ptr(), rp, native.stream())
        out = out.view(y.shape)
        return out if (residual is None or res is not None) else out + residual


# ---------------------------------------------------------------------- tensor-parallel TRAINING (sequence parallel)
class _ColumnParallelLinearFn(torch.autograd.Function):
    """y[M, N/P] = gather(x_own[M/P, K]) @ W[K, N/P] on the fused all-gather -> GEMM kernel. Backward uses the
    other fused kernel: dx_own = reduce_scatter(dy @ W^T) (GEMM -> reduce-scatter over the transposed weight,
    no copy), dW = gather(x)^T @ dy on the plain GEMM with the gathered activation that was kept."""

    @staticmethod
    def forward(ctx, x_own, weight, tp, which):
        rows, K = x_own.shape
        M = rows * tp.world
        tp.own_rows(which, M, K).copy_(x_own)
        y = tp.ag_gemm(which, M, K, weight)
        # the gather buffer is reused by the next layer: keep this layer's gathered input for dW
        ctx.save_for_backward(tp.xbufs[which][:M * K].view(M, K).clone(), weight)
        ctx.tp = tp
        return y

    @staticmethod
    def backward(ctx, dy):
        from ..ops import cuda_ops
        xfull, weight = ctx.saved_tensors
        tp = ctx.tp
        M, K = xfull.shape
        Nl = weight.shape[1]
        dyc = dy.contiguous()
        dx_own = tp.gemm_rs(dyc, weight, None, transposed=True) if ctx.needs_input_grad[0] else None
        dw = None
        if ctx.needs_input_grad[1]:
            main = getattr(weight, "main_grad", None)
            if main is not None:
                cuda_ops.gemm(xfull, dyc, K, Nl, M, K, Nl, True, True, out=main, accumulate=True)
            else:
                dw = cuda_ops.gemm(xfull, dyc, K, Nl, M, K, Nl, True, True, out_dtype=torch.float32).to(weight.dtype)
        return dx_own, dw, None, None


class _RowParallelLinearFn(torch.autograd.Function):
    """y_own[M/P, N] = reduce_scatter(x[M, K/P] @ W[K/P, N]) (+ residual_own) on the fused GEMM -> reduce-scatter
    kernel. Backward: dx = gather(dy_own) @ W^T on the fused all-gather -> GEMM kernel, dW = x^T @ gather(dy_own)
    with the gathered gradient that kernel leaves in the symmetric buffer."""

    @staticmethod
    def forward(ctx, x, weight, residual_own, tp, which):
        y = tp.gemm_rs(x.contiguous(), weight, residual_own)
        ctx.save_for_backward(x, weight)
        ctx.tp, ctx.which, ctx.has_res = tp, which, residual_own is not None
        return y

    @staticmethod
    def backward(ctx, dy_own):
        from ..ops import cuda_ops
        x, weight = ctx.saved_tensors
        tp, which = ctx.tp, ctx.which
        M, Kl = x.shape
        Nn = weight.shape[1]
        tp.own_rows(which, M, Nn).copy_(dy_own)
        dx = tp.ag_gemm(which, M, Nn, weight, transposed=True)              # [M, K/P]
        dw = None
        if ctx.needs_input_grad[1]:
            dyfull = tp.xbufs[which][:M * Nn].view(M, Nn)                    # valid until the next fused call on `which`
            xc = x.contiguous()
            main = getattr(weight, "main_grad", None)
            if main is not None:
                cuda_ops.gemm(xc, dyfull, Kl, Nn, M, Kl, Nn, True, True, out=main, accumulate=True)
            else:
                dw = cuda_ops.gemm(xc, dyfull, Kl, Nn, M, Kl, Nn, True, True, out_dtype=torch.float32).to(weight.dtype)
        return (dx if ctx.needs_input_grad[0] else None), dw, (dy_own if ctx.has_res else None), None, None


def column_parallel_linear(x_own: torch.Tensor, weight: torch.Tensor, tp: "TensorParallelGroup", which: int = 0):
    """Differentiable sequence-parallel column-sharded projection: `x_own` `[M/P, K]` (this rank's token rows),
    `weight` `[K, N/P]` (this rank's columns) -> `[M, N/P]`. M % (128 P) == 0, K % 64 == 0, K == tp.hidden."""
    return _ColumnParallelLinearFn.apply(x_own, weight, tp, which)


def row_parallel_linear(x: torch.Tensor, weight: torch.Tensor, tp: "TensorParallelGroup",
                        residual_own: Optional[torch.Tensor] = None, which: int = 1):
    """Differentiable row-sharded projection with the reduce-scatter fused: `x` `[M, K/P]`, `weight` `[K/P, N]`
    -> this rank's token rows `[M/P, N]` (+ `residual_own`). N == tp.hidden."""
    return _RowParallelLinearFn.apply(x, weight, residual_own, tp, which)


class RowParallelLinear(nn.Module):
    """Row-sharded projection; `bias` (full, replicated) is added once after the sum."""

    def __init__(self, inner: nn.Module, tp: TensorParallelGroup, bias: Optional[torch.Tensor] = None):
        super().__init__()
        self.inner = inner
        self.tp = tp
        self.register_buffer("row_bias", bias)

    def forward(self, x, residual=None):
        """`residual`: added to the reduced output (fused into the all-reduce kernel). A quantised inner
        projection with at most 4 rows runs as one kernel: GEMV with the all-reduce in its epilogue."""
        if self.row_bias is None and hasattr(self.inner, "packed_k8"):
            lead = x.shape[:-1]
            y = self.tp.gemv_allreduce(x.reshape(-1, x.shape[-1]), self.inner, residual)
            if y is not None:
                return y.view(*lead, y.shape[-1])
        y = self.tp.all_reduce(self.inner(x), residual)
        return y if self.row_bias is None else y + self.row_bias.to(y.dtype)


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
        # a row-parallel bias is added once, after the sum: RowParallelLinear holds it
    return out


def _full_bias(lin: Linear):
    return lin.bias.detach().clone() if lin.bias is not None else None


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
            a.o_proj = RowParallelLinear(_slice_linear(a.o_proj, rows=(r * hq * D, (r + 1) * hq * D)), tp,
                                         _full_bias(a.o_proj))
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
            ff.down_proj = RowParallelLinear(_slice_linear(ff.down_proj, rows=(r * s, (r + 1) * s)), tp,
                                             _full_bias(ff.down_proj))
    return model


def _can_sequence_parallel(model, tp: TensorParallelGroup, M: int) -> bool:
    if tp.mode != "fused" or tp.world < 2 or tp.max_tokens == 0 or M > tp.max_tokens or M % (128 * tp.world):
        return False
    if tp.hidden != model.cfg.hidden_size or model.cfg.hidden_size % 64:
        return False
    for blk in model.layers:
        if not blk.pre_norm or not blk.residual or blk.memory is not None or blk.ssm is not None:
            return False
        if not isinstance(blk.attention.o_proj, RowParallelLinear) or not isinstance(blk.feed_forward, FeedForward):
            return False
        if not isinstance(blk.feed_forward.down_proj, RowParallelLinear):
            return False
        for lin in (blk.attention.qkv_proj, blk.attention.o_proj.inner, blk.feed_forward.in_proj,
                    blk.feed_forward.down_proj.inner):
            if isinstance(lin, Linear):
                if lin.weight.dtype != torch.bfloat16:
                    return False
            elif not hasattr(lin, "dequantized"):
                return False
    return True


def _bf16_weight(lin) -> torch.Tensor:
    """`[d_in, d_out]` bf16 weight of a plain or group-quantised projection (the latter is
    expanded into a temporary: prefill is compute-bound, the 4-bit form pays off in decode)."""
    return lin.weight if isinstance(lin, Linear) else lin.dequantized()


@torch.no_grad()
def prefill_sequence_parallel(model, tp: TensorParallelGroup, tokens: torch.Tensor, state) -> torch.Tensor:
    """Prefill of a `shard_model`-sharded transformer; returns the last position's logits
    `[B, vocab]` and fills the KV caches in `state`.

    With B*S a multiple of 128 * P the residual stream is kept sequence-parallel (M/P rows per
    rank) and the four projections of a block run as fused all-gather -> GEMM / GEMM -> reduce-
    scatter kernels; otherwise the call falls back to the all-reduce form of the sharded model.
    """
    from .. import ops
    B, S = tokens.shape
    M, H = B * S, model.cfg.hidden_size
    if not _can_sequence_parallel(model, tp, M):
        return model.forward_next_logits_with_state(tokens, state)
    P, r = tp.world, tp.rank
    rows = M // P
    rope = model.rope(tokens.device)
    flat_tok = tokens.reshape(-1)[r * rows:(r + 1) * rows]
    h = model.embed(flat_tok.unsqueeze(0)).reshape(rows, H).to(torch.bfloat16)
    for blk, st in zip(model.layers, state.layers):
        a, ff = blk.attention, blk.feed_forward
        tp.own_rows(0, M, H).copy_(blk.attn_norm(h))
        qkv = tp.ag_gemm(0, M, H, _bf16_weight(a.qkv_proj), a.qkv_proj.bias)
        o = a.attend(qkv.view(B, S, -1), rope, st).reshape(M, a.q_dim)
        res = h if a.o_proj.row_bias is None else h + a.o_proj.row_bias.to(h.dtype)
        h = tp.gemm_rs(o, _bf16_weight(a.o_proj.inner), res)
        tp.own_rows(1, M, H).copy_(blk.ffn_norm(h))
        u = tp.ag_gemm(1, M, H, _bf16_weight(ff.in_proj), ff.in_proj.bias)
        u = ops.gated_act(u, ff.act) if ff.gated else ops.activation(ff.act, u)
        res = h if ff.down_proj.row_bias is None else h + ff.down_proj.row_bias.to(h.dtype)
        h = tp.gemm_rs(u, _bf16_weight(ff.down_proj.inner), res)
    state.pos += S
    # the last position of every sequence lives on whichever rank owns that row
    last = torch.zeros(B, H, dtype=torch.bfloat16, device=h.device)
    for b in range(B):
        row = b * S + S - 1
        if r * rows <= row < (r + 1) * rows:
            last[b] = h[row - r * rows]
    last = tp.all_reduce(last)
    x = model.final_norm(last)
    return model.project_logits(x)


# ---------------------------------------------------------------------------- vocabulary-parallel loss
class _VocabParallelCE(torch.autograd.Function):
    """Mean next-token cross-entropy with the output projection sharded over the vocabulary:
    rank r holds columns [r*V/P, (r+1)*V/P) of the head. Only three scalars per row cross the
    ranks (running max, sum of exponentials, the target's logit), never a logit row."""

    @staticmethod
    def forward(ctx, hidden, weight_shard, targets, group, vocab_size):
        from .. import ops
        P, r = dist.get_world_size(group), dist.get_rank(group)
        Vs = weight_shard.shape[1]
        lo = r * Vs
        valid = max(0, min(Vs, vocab_size - lo))            # logical columns of this shard (padding is masked)
        logits = ops.linear(hidden, weight_shard, None).float()
        if valid < Vs:
            logits[:, valid:] = float("-inf")
        m = logits.max(dim=1).values if valid > 0 else logits.new_full((logits.shape[0],), float("-inf"))
        dist.all_reduce(m, op=dist.ReduceOp.MAX, group=group)
        e = torch.exp(logits - m[:, None])
        packed = torch.stack([e.sum(dim=1), torch.zeros_like(m)])
        mine = (targets >= lo) & (targets < lo + valid)
        idx = (targets - lo).clamp(0, Vs - 1)
        packed[1] = torch.where(mine, logits.gather(1, idx[:, None]).squeeze(1), torch.zeros_like(m))
        dist.all_reduce(packed, group=group)                # one message: [sum exp, target logit]
        lse = m + packed[0].log()
        loss = (lse - packed[1]).mean()
        ctx.save_for_backward(hidden, weight_shard, e / packed[0][:, None], mine, idx)
        ctx.group = group
        return loss

    @staticmethod
    def backward(ctx, g):
        from .. import ops
        hidden, w, prob, mine, idx = ctx.saved_tensors
        T = hidden.shape[0]
        d = prob
        d[mine, idx[mine]] -= 1.0
        d = (d * (g / T)).to(hidden.dtype)
        dh = ops.linear(d, w.t(), None).float()
        dist.all_reduce(dh, group=ctx.group)                # every shard contributes to d(hidden)
        dw = ops.linear(hidden.t(), d, None)
        return dh.to(hidden.dtype), dw.to(w.dtype), None, None, None


def vocab_parallel_cross_entropy(hidden: torch.Tensor, weight_shard: torch.Tensor, targets: torch.Tensor, group,
                                 vocab_size: int) -> torch.Tensor:
    """`hidden [T, H]` (replicated), `weight_shard [H, Vpad / P]` (this rank's head columns),
    `targets [T]`. Equals `ops.linear_cross_entropy` on the unsharded head
    (`summa-llm/src/model/linear_cross_entropy/reference.rs:42-159` is the single-device oracle)."""
    return _VocabParallelCE.apply(hidden, weight_shard, targets, group, vocab_size)


class VocabParallelHead(nn.Module):
    """Inference head sharded over the vocabulary: local logits, then one all-gather of `[B, V/P]`."""

    def __init__(self, weight_shard: torch.Tensor, group, vocab_size: int):
        super().__init__()
        self.register_buffer("weight", weight_shard.contiguous())
        self.group, self.vocab_size = group, vocab_size

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        from .. import ops
        lead = x.shape[:-1]
        local = ops.linear(x.reshape(-1, x.shape[-1]), self.weight, None).contiguous()
        P = dist.get_world_size(self.group)
        parts = [torch.empty_like(local) for _ in range(P)]
        dist.all_gather(parts, local, group=self.group)
        return torch.cat(parts, dim=1)[:, :self.vocab_size].view(*lead, self.vocab_size)


def shard_head(weight: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Columns of rank `rank` of a `[H, V]` head, V zero-padded up to a multiple of 8 * world."""
    H, V = weight.shape
    per = -(-V // (8 * world)) * 8
    out = weight.new_zeros(H, per)
    lo, hi = rank * per, min((rank + 1) * per, V)
    if hi > lo:
        out[:, :hi - lo] = weight[:, lo:hi]
    return out
