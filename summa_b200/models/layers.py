"""Model building blocks: Linear, Norm, attention, Mamba, dense FFN, MoE.

Parameter names and shapes reproduce the reference's checkpoint keys, so a
`weights.safetensors` written by either side loads in the other:
`Linear.weight` is `[d_in, d_out]`, dense FFN `in_proj` is laid out
`[gate | value]`, expert banks are `[E, H, 2I]` / `[E, I, H]`
(`summa-llm/src/model/attention.rs:43-64`, `mamba.rs:28-85`, `ffn.rs:36-40,145-218`).

All math goes through `summa_b200.ops`, which runs the sm_100a kernels for CUDA
tensors and the PyTorch oracles for CPU tensors.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.nn as nn

from .. import ops
from ..mal import BlockDef, FfnDef, ModelDef, NormConfig, SsmDef


class Linear(nn.Module):
    """y = x @ weight (+ bias); weight is `[d_in, d_out]`."""

    def __init__(self, d_in: int, d_out: int, bias: bool = False, init_std: Optional[float] = None):
        super().__init__()
        self.d_in, self.d_out = d_in, d_out
        w = torch.empty(d_in, d_out)
        if init_std is None:
            k = 1.0 / math.sqrt(d_in)
            w.uniform_(-k, k)
        else:
            w.normal_(0.0, init_std)
        self.weight = nn.Parameter(w)
        if bias:
            b = torch.empty(d_out)
            if init_std is None:
                k = 1.0 / math.sqrt(d_in)
                b.uniform_(-k, k)
            else:
                b.zero_()
            self.bias = nn.Parameter(b)
        else:
            self.register_parameter("bias", None)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.linear(x, self.weight, self.bias)


class Norm(nn.Module):
    """RMSNorm / LayerNorm / identity with fp32 statistics (`norm.rs:16-50`)."""

    def __init__(self, cfg: NormConfig, dim: int):
        super().__init__()
        self.kind = cfg.norm_type
        self.eps = cfg.effective_eps()
        if self.kind in ("rmsnorm", "layernorm"):
            self.gamma = nn.Parameter(torch.ones(dim))
        if self.kind == "layernorm":
            self.beta = nn.Parameter(torch.zeros(dim))

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None):
        """With `residual`, returns (norm(x + residual), x + residual)."""
        if residual is not None:
            if self.kind == "rmsnorm":
                return ops.add_rmsnorm(x, residual, self.gamma, self.eps)
            s = x + residual
            return self.forward(s), s
        if self.kind == "rmsnorm":
            return ops.rmsnorm(x, self.gamma, self.eps)
        if self.kind == "layernorm":
            return ops.layernorm(x, self.gamma, self.beta, self.eps)
        return x


@dataclass
class AttentionState:
    k: torch.Tensor            # [B, capacity, KV, D]
    v: torch.Tensor
    length: int = 0


class MultiHeadAttention(nn.Module):
    """Fused-QKV attention with native GQA, optional QK-norm before RoPE."""

    def __init__(self, block: BlockDef, hidden: int, init_std: Optional[float] = None):
        super().__init__()
        a = block.attention
        self.num_heads = block.num_heads()
        self.num_kv_heads = block.num_kv_heads()
        self.head_dim = block.head_dim(hidden)
        self.causal = a.causal
        self.window = a.window_size
        self.dropout = a.dropout
        self.use_rope = a.position_encoding.kind == "rope"
        self.eps = block.norm_eps()
        q_dim = self.num_heads * self.head_dim
        kv_dim = self.num_kv_heads * self.head_dim
        self.q_dim, self.kv_dim = q_dim, kv_dim
        self.qkv_proj = Linear(hidden, q_dim + 2 * kv_dim, a.bias, init_std)
        self.o_proj = Linear(q_dim, hidden, a.bias, init_std)
        if a.qk_norm:
            self.q_norm = Norm(NormConfig("rmsnorm", self.eps), self.head_dim)
            self.k_norm = Norm(NormConfig("rmsnorm", self.eps), self.head_dim)
        else:
            self.q_norm = self.k_norm = None

    def _split(self, qkv: torch.Tensor):
        B, S, _ = qkv.shape
        q = qkv[..., :self.q_dim].unflatten(-1, (self.num_heads, self.head_dim))
        k = qkv[..., self.q_dim:self.q_dim + self.kv_dim].unflatten(-1, (self.num_kv_heads, self.head_dim))
        v = qkv[..., self.q_dim + self.kv_dim:].unflatten(-1, (self.num_kv_heads, self.head_dim))
        return q, k, v

    def forward(self, x: torch.Tensor, rope, state: Optional[AttentionState] = None) -> torch.Tensor:
        return self.o_proj(self.attend(self.qkv_proj(x), rope, state))

    def attend(self, qkv: torch.Tensor, rope, state: Optional[AttentionState] = None) -> torch.Tensor:
        """Attention over a fused `[B, S, q_dim + 2 kv_dim]` projection; returns `[B, S, q_dim]`
        (everything between the two projections, so tensor-parallel runners can supply their own)."""
        B, S, _ = qkv.shape
        offset = state.length if state is not None else 0
        cos, sin = rope if (self.use_rope and rope is not None) else (None, None)
        qg = self.q_norm.gamma if self.q_norm is not None else None
        kg = self.k_norm.gamma if self.k_norm is not None else None
        if (state is None and ops.native_enabled(qkv) and self.head_dim in (64, 128)
                and cos is not None and not (self.dropout > 0.0 and self.training)):
            # packed path: RoPE/QK-norm and attention run straight on the fused activation
            o = ops.packed_qkv_attention(qkv, qg, kg, self.eps, cos, sin, self.num_heads, self.num_kv_heads,
                                         self.head_dim, self.causal, self.window)
            return o.reshape(B, S, self.q_dim)
        q, k, v = ops.packed_qk_rope(qkv, qg, kg, self.eps, cos, sin, self.num_heads, self.num_kv_heads, self.head_dim,
                                     offset)
        if state is None:
            if self.dropout > 0.0 and self.training:
                o = ops.attention_dropout(q, k, v, self.causal, self.window, self.dropout)
            else:
                o = ops.attention(q, k, v, causal=self.causal, window=self.window)
        else:
            end = offset + S
            if end > state.k.shape[1]:
                raise RuntimeError(f"KV cache overflow: {end} > capacity {state.k.shape[1]}")
            ops.kv_append(state.k, state.v, k, v, offset)
            state.length = end
            o = ops.attention(q, state.k[:, :end], state.v[:, :end], causal=self.causal,
                              window=self.window, q_offset=offset)
        return o.reshape(B, S, self.q_dim)

    def make_state(self, batch: int, capacity: int, device, dtype) -> AttentionState:
        shape = (batch, capacity, self.num_kv_heads, self.head_dim)
        return AttentionState(torch.zeros(shape, device=device, dtype=dtype),
                              torch.zeros(shape, device=device, dtype=dtype), 0)


@dataclass
class MambaState:
    conv: torch.Tensor        # [B, d_inner, K-1]
    h: torch.Tensor           # [B, d_inner, N] fp32


class MambaMixer(nn.Module):
    """Mamba-1 mixer (`summa-llm/src/model/mamba.rs:28-211`)."""

    def __init__(self, ssm: SsmDef, model: ModelDef, init_std: Optional[float] = None):
        super().__init__()
        h = model.hidden_size
        self.d_inner = ssm.expand * h
        self.d_state = ssm.state_dim
        self.d_conv = ssm.conv_kernel
        self.dt_rank = model.dt_rank(ssm)
        self.in_proj = Linear(h, 2 * self.d_inner, False, init_std)
        self.conv1d = _DepthwiseConv(self.d_inner, self.d_conv)
        self.x_proj = Linear(self.d_inner, self.dt_rank + 2 * self.d_state, False, init_std)
        self.dt_proj = Linear(self.dt_rank, self.d_inner, True, init_std)
        self.a_log = nn.Parameter(torch.zeros(self.d_inner, self.d_state))
        self.d = nn.Parameter(torch.ones(self.d_inner))
        self.out_proj = Linear(self.d_inner, h, False, init_std)

    def forward(self, x: torch.Tensor, state: Optional[MambaState] = None) -> torch.Tensor:
        B, T, _ = x.shape
        xz = self.in_proj(x)
        xs, z = xz[..., :self.d_inner], xz[..., self.d_inner:]
        conv_state = state.conv if state is not None else None
        if state is not None:
            K1 = self.d_conv - 1
            hist = torch.cat([state.conv.to(xs.dtype), xs.transpose(1, 2)], dim=-1)
            new_conv = hist[..., -K1:].contiguous() if K1 > 0 else state.conv
        xc = ops.conv1d_silu(xs, self.conv1d.weight, self.conv1d.bias, conv_state)
        proj = self.x_proj(xc)
        dt_in = proj[..., :self.dt_rank]
        Bm = proj[..., self.dt_rank:self.dt_rank + self.d_state]
        Cm = proj[..., self.dt_rank + self.d_state:]
        delta = self.dt_proj(dt_in)
        A = -torch.exp(self.a_log.float())
        h0 = state.h if state is not None else None
        y, h_last = ops.selective_scan(xc, delta, A, Bm, Cm, self.d, h0,
                                       need_final_state=state is not None)
        if state is not None:
            state.conv = new_conv
            state.h = h_last
        y = ops.mul_silu(y, z)
        return self.out_proj(y)

    def make_state(self, batch: int, device, dtype) -> MambaState:
        return MambaState(torch.zeros(batch, self.d_inner, self.d_conv - 1, device=device, dtype=dtype),
                          torch.zeros(batch, self.d_inner, self.d_state, device=device, dtype=torch.float32))


class _DepthwiseConv(nn.Module):
    def __init__(self, channels: int, kernel: int):
        super().__init__()
        self.weight = nn.Parameter(torch.randn(channels, 1, kernel) * math.sqrt(1.0 / kernel))
        self.bias = nn.Parameter(torch.zeros(channels))


class FeedForward(nn.Module):
    """Dense FFN: in_proj (h → 2I if gated else I), act(gate)*value, down_proj."""

    def __init__(self, ffn: FfnDef, hidden: int, init_std: Optional[float] = None):
        super().__init__()
        inter = ffn.hidden_dim if ffn.hidden_dim is not None else 4 * hidden
        self.gated = ffn.gate
        self.act = ffn.activation
        self.dropout = ffn.dropout
        self.in_proj = Linear(hidden, 2 * inter if ffn.gate else inter, ffn.bias, init_std)
        self.down_proj = Linear(inter, hidden, ffn.bias, init_std)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        h = self.in_proj(x)
        h = ops.gated_act(h, self.act) if self.gated else ops.activation(self.act, h)
        if self.dropout > 0.0 and self.training:
            h = torch.nn.functional.dropout(h, self.dropout)
        return self.down_proj(h)


class ExpertBank(nn.Module):
    def __init__(self, experts: int, hidden: int, inter: int, gated: bool, bias: bool,
                 init_std: Optional[float] = None):
        super().__init__()
        width = 2 * inter if gated else inter
        k_in, k_dn = 1.0 / math.sqrt(hidden), 1.0 / math.sqrt(inter)
        if init_std is None:
            self.in_weight = nn.Parameter(torch.empty(experts, hidden, width).uniform_(-k_in, k_in))
            self.down_weight = nn.Parameter(torch.empty(experts, inter, hidden).uniform_(-k_dn, k_dn))
        else:
            self.in_weight = nn.Parameter(torch.empty(experts, hidden, width).normal_(0, init_std))
            self.down_weight = nn.Parameter(torch.empty(experts, inter, hidden).normal_(0, init_std))
        if bias:
            self.in_bias = nn.Parameter(torch.zeros(experts, width))
            self.down_bias = nn.Parameter(torch.zeros(experts, hidden))
        else:
            self.register_parameter("in_bias", None)
            self.register_parameter("down_bias", None)


class _Router(nn.Module):
    def __init__(self, hidden: int, experts: int, init_std: Optional[float] = None):
        super().__init__()
        k = 1.0 / math.sqrt(hidden)
        w = torch.empty(hidden, experts)
        self.weight = nn.Parameter(w.uniform_(-k, k) if init_std is None else w.normal_(0, init_std))


class _Moe(nn.Module):
    """Holder so checkpoint keys read `feed_forward.moe.{router,experts,shared_experts}`."""

    def __init__(self, ffn: FfnDef, hidden: int, init_std):
        super().__init__()
        m = ffn.moe
        inter = ffn.hidden_dim if ffn.hidden_dim is not None else 4 * hidden
        self.router = _Router(hidden, m.experts, init_std)
        self.experts = ExpertBank(m.experts, hidden, inter, ffn.gate, ffn.bias, init_std)
        dense = FfnDef(ffn.name, ffn.hidden_dim, ffn.activation, ffn.bias, ffn.dropout, ffn.gate, None)
        self.shared_experts = nn.ModuleList([FeedForward(dense, hidden, init_std)
                                             for _ in range(m.shared_experts)])


class SparseMoe(nn.Module):
    """Dropless token-choice MoE (`summa-llm/src/model/ffn.rs:448-710`).

    Router in fp32; top-k on logits then softmax over the selected logits;
    aux = lb_w * E * sum_e mean(p_e) * frac_e + z_w * mean(logsumexp^2).
    `ep_group` switches the expert computation to the expert-parallel path.
    """

    def __init__(self, ffn: FfnDef, hidden: int, init_std: Optional[float] = None):
        super().__init__()
        self.cfg = ffn.moe
        self.gated = ffn.gate
        self.act = ffn.activation
        self.moe = _Moe(ffn, hidden, init_std)
        self.ep = None      # set by parallel.ep.shard_experts

    def forward(self, x: torch.Tensor, extra_random_expert_seed: Optional[int] = None):
        shape = x.shape
        flat = x.reshape(-1, shape[-1])
        logits = ops.router_logits(flat, self.moe.router.weight)
        idx, gates = ops.moe_route(logits, self.cfg.top_k)
        aux = ops.moe_aux_loss(logits, idx, self.cfg.experts, self.cfg.load_balance_loss_weight,
                               self.cfg.router_z_loss_weight)
        if extra_random_expert_seed is not None:
            idx, gates = _dream_routes(logits, idx, self.cfg.experts, extra_random_expert_seed)
        e = self.moe.experts
        if self.ep is not None:
            out = self.ep.forward(flat, idx, gates, e, self.act, self.gated)
        else:
            out = ops.moe_experts(flat, idx, gates, e.in_weight, e.down_weight, e.in_bias,
                                  e.down_bias, self.act, self.gated)
        for shared in self.moe.shared_experts:
            out = out + shared(flat)
        return out.reshape(shape), aux


def _dream_routes(logits, idx, experts, seed):
    """Dream routing: one extra uniformly random non-selected expert joins the
    softmax of the selected logits (`summa-llm/src/model/ffn.rs:490-514`)."""
    T, k = idx.shape
    g = torch.Generator(device="cpu").manual_seed(int(seed))
    scores = torch.rand(T, experts, generator=g).to(logits.device)
    scores.scatter_(1, idx, -1.0)
    extra = scores.argmax(dim=-1, keepdim=True)
    idx2 = torch.cat([idx, extra], dim=1)
    gates = torch.softmax(torch.gather(logits.float(), 1, idx2), dim=-1)
    return idx2, gates


def build_ffn(ffn: FfnDef, hidden: int, init_std=None) -> nn.Module:
    return SparseMoe(ffn, hidden, init_std) if ffn.moe is not None else FeedForward(ffn, hidden, init_std)
