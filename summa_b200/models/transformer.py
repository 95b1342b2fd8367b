"""`Transformer`: one model implementation for training, generation, retrieval
embedding and tracing (`summa-llm/src/model/transformer.rs:99-1238`,
`block.rs:25-156`).

Layout facts preserved from the reference so checkpoints interchange:
the embedding / head store `padded_vocab_size()` rows with exact-zero padding,
the API speaks the logical vocabulary, the head is absent when weights are tied
(a tied bias lives in `tied_output_bias`), and one RoPE table is shared by every
attention block.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn as nn

from .. import ops
from ..mal import BlockDef, ModelDef
from .layers import (AttentionState, FeedForward, Linear, MambaMixer, MambaState,
                     MultiHeadAttention, Norm, SparseMoe, build_ffn)
from .memory import MemoryChain

EMBEDDING_INIT_STD = 0.02
LOSS_CHUNKS = 4


def validate_config(cfg: ModelDef) -> None:
    """Model-time validation (`transformer.rs:112-316,425-443`)."""
    def pos(name, v):
        if v <= 0:
            raise ValueError(f"{name} must be positive")
    pos("vocab_size", cfg.vocab_size); pos("max_seq_len", cfg.max_seq_len)
    pos("hidden_size", cfg.hidden_size); pos("num_layers", cfg.num_layers)

    def drop(name, v):
        if not (0.0 <= v < 1.0):
            raise ValueError(f"{name} must be in [0, 1)")
    drop("embeddings.dropout", cfg.embeddings.dropout)
    attn_sig = None
    for i in range(cfg.num_layers):
        b = cfg.block_for_layer(i)
        drop("block.dropout", b.dropout)
        if b.memory is not None and b.ffn.moe is not None and False:
            pass
        if b.ssm is not None:
            s = b.ssm
            pos("ssm.state_dim", s.state_dim); pos("ssm.conv_kernel", s.conv_kernel); pos("ssm.expand", s.expand)
            if s.dt_rank is not None:
                pos("ssm.dt_rank", s.dt_rank)
        else:
            h, kv, hd = b.num_heads(), b.num_kv_heads(), b.head_dim(cfg.hidden_size)
            pos("num_heads", h); pos("num_kv_heads", kv); pos("head_dim", hd)
            drop("attention.dropout", b.attention.dropout)
            if h % kv != 0:
                raise ValueError(f"num_heads {h} must be divisible by num_kv_heads {kv}")
            if h * hd != cfg.hidden_size:
                raise ValueError(f"num_heads*head_dim ({h}*{hd}) must equal hidden_size {cfg.hidden_size}")
            pe = b.attention.position_encoding
            if pe.kind not in ("rope", "none"):
                raise ValueError(f"position encoding '{pe.kind}' is not implemented (rope|none)")
            if pe.kind == "rope" and hd % 2 != 0:
                raise ValueError("RoPE needs an even head_dim")
            if pe.kind == "rope":
                sig = (hd, pe.theta, pe.scaling)
                if attn_sig is None:
                    attn_sig = sig
                elif sig != attn_sig:
                    raise ValueError("all attention blocks must share head_dim, rope theta and scaling")
            if b.attention.window_size is not None:
                pos("window_size", b.attention.window_size)
        ffns = [t.ffn for t in b.memory.tiers] if b.memory is not None else [b.ffn]
        for f in ffns:
            drop("ffn.dropout", f.dropout)
            if f.hidden_dim is not None:
                pos("ffn.hidden_dim", f.hidden_dim)
            if f.moe is not None:
                if f.moe.experts < 2:
                    raise ValueError("moe.experts must be >= 2")
                if not (1 <= f.moe.top_k <= f.moe.experts):
                    raise ValueError("moe.top_k must be in [1, experts]")
        if b.memory is not None:
            if not b.memory.tiers:
                raise ValueError("memory needs at least one tier")
            for t in b.memory.tiers:
                if t.reserve_experts.top_k != 1:
                    raise ValueError("reserve_experts.top_k must be 1")
                pos("reserve_experts.capacity", t.reserve_experts.capacity)
                pos("reserve_experts.rank", t.reserve_experts.rank)


class TransformerBlock(nn.Module):
    """One mixer (attention XOR Mamba) + (FFN XOR MemoryChain), pre- or post-norm."""

    def __init__(self, cfg: ModelDef, block: BlockDef, layer: int, init_std: Optional[float] = None):
        super().__init__()
        h = cfg.hidden_size
        self.pre_norm = block.norm_position == "pre"
        self.residual = block.residual
        self.dropout = block.dropout
        self.attn_norm = Norm(block.norm, h)
        self.ffn_norm = Norm(block.norm, h)
        if block.ssm is not None:
            self.ssm = MambaMixer(block.ssm, cfg, init_std)
            self.attention = None
        else:
            self.attention = MultiHeadAttention(block, h, init_std)
            self.ssm = None
        if block.memory is not None:
            self.memory = MemoryChain(block.memory, h, layer, init_std)
            self.feed_forward = None
        else:
            self.feed_forward = build_ffn(block.ffn, h, init_std)
            self.memory = None

    def _drop(self, x):
        if self.dropout > 0.0 and self.training:
            return torch.nn.functional.dropout(x, self.dropout)
        return x

    def _mix(self, x, rope, state):
        if self.ssm is not None:
            return self.ssm(x, state)
        return self.attention(x, rope, state)

    def _res(self, x, y):
        y = self._drop(y)
        return x + y.to(x.dtype) if self.residual else y.to(x.dtype)

    def fusable(self) -> bool:
        """Pre-norm RMSNorm block with plain residuals: its residual adds can ride in the norm kernels."""
        return (self.pre_norm and self.residual and self.memory is None and self.attn_norm.kind == "rmsnorm"
                and self.ffn_norm.kind == "rmsnorm" and not (self.dropout > 0.0 and self.training))

    def forward_deferred(self, x: torch.Tensor, pending: Optional[torch.Tensor], rope, state=None,
                         dream_seed: Optional[int] = None):
        """Same block with the residual adds fused into the following norm (`norm(x + y)` and
        `x + y` come out of one kernel). `pending` is the previous block's branch output that has
        not been added to `x` yet; returns (x, pending, aux) in the same convention."""
        if pending is None:
            n = self.attn_norm(x)
        else:
            n, x = self.attn_norm(pending.to(x.dtype), x)
        mix = self._mix(n, rope, state)
        n, x = self.ffn_norm(mix.to(x.dtype), x)
        aux = None
        if isinstance(self.feed_forward, SparseMoe):
            y, aux = self.feed_forward(n, dream_seed)
        else:
            y = self.feed_forward(n)
        return x, y, aux

    def forward(self, x: torch.Tensor, rope, state=None, dream_seed: Optional[int] = None):
        """Returns (x, aux). `state` is the mixer state (KV cache or Mamba state)."""
        aux = None
        if self.pre_norm:
            x = self._res(x, self._mix(self.attn_norm(x), rope, state))
            if self.memory is not None:
                x, aux = self.memory(x, self.ffn_norm, self._res, dream_seed)
            else:
                n = self.ffn_norm(x)
                if isinstance(self.feed_forward, SparseMoe):
                    y, aux = self.feed_forward(n, dream_seed)
                else:
                    y = self.feed_forward(n)
                x = self._res(x, y)
        else:
            x = self.attn_norm(self._res(x, self._mix(x, rope, state)))
            if self.memory is not None:
                x, aux = self.memory(x, lambda s: s, lambda s, y: self.ffn_norm(self._res(s, y)), dream_seed)
            else:
                if isinstance(self.feed_forward, SparseMoe):
                    y, aux = self.feed_forward(x, dream_seed)
                else:
                    y = self.feed_forward(x)
                x = self.ffn_norm(self._res(x, y))
        return x, aux


@dataclass
class InferenceState:
    layers: list
    pos: int = 0
    capacity: int = 0


class _GradReady(torch.autograd.Function):
    """Identity on the residual stream at the entry of block `index`. Its backward runs after every node of the
    block (the block's first op consumes this tensor), i.e. once the block's weight gradients of this pass
    are enqueued: the training engine uses it to start the reduce-scatter of finished layers while the
    backward pass of the earlier layers is still running."""

    @staticmethod
    def forward(ctx, x, hook, index):
        ctx.hook, ctx.index = hook, index
        hook.on_forward(index)
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        ctx.hook.on_backward(ctx.index)
        return g, None, None


class Transformer(nn.Module):
    def __init__(self, cfg: ModelDef, init_std: Optional[float] = None):
        """`init_std`: when given, every matrix is drawn N(0, init_std) instead of
        the per-layer default initialisers (benchmark configs use 0.02)."""
        super().__init__()
        validate_config(cfg)
        self.cfg = cfg
        h, vpad = cfg.hidden_size, cfg.padded_vocab_size()
        emb = torch.zeros(vpad, h)
        emb[:cfg.vocab_size].normal_(0.0, EMBEDDING_INIT_STD)
        self.embedding = _Embedding(emb)
        self.layers = nn.ModuleList([TransformerBlock(cfg, cfg.block_for_layer(i), i, init_std)
                                     for i in range(cfg.num_layers)])
        self.final_norm = Norm(cfg.output.norm or cfg.block_for_layer(0).norm, h)
        if cfg.embeddings.tie_weights:
            self.lm_head = None
            if cfg.output.bias:
                self.tied_output_bias = nn.Parameter(torch.zeros(vpad))
        else:
            self.lm_head = Linear(h, vpad, cfg.output.bias, init_std)
            with torch.no_grad():
                self.lm_head.weight[:, cfg.vocab_size:] = 0.0
                if self.lm_head.bias is not None:
                    self.lm_head.bias[cfg.vocab_size:] = 0.0
        self._rope = None
        self._rope_key = None
        self._tied_cache = None
        self.stream_dtype: Optional[torch.dtype] = None   # e.g. torch.bfloat16 residual stream

    # ------------------------------------------------------------------ helpers
    def rope(self, device):
        spec = None
        for i in range(self.cfg.num_layers):
            b = self.cfg.block_for_layer(i)
            if b.ssm is None and b.attention.position_encoding.kind == "rope":
                spec = (b.head_dim(self.cfg.hidden_size), b.rope_theta(), b.rope_scaling())
                break
        if spec is None:
            return None
        key = (spec, str(device))
        if self._rope_key != key:
            self._rope = ops.rope_table(self.cfg.max_seq_len, spec[0], spec[1], spec[2], device)
            self._rope_key = key
        return self._rope

    def output_weight(self) -> torch.Tensor:
        """`[H, Vpad]` projection: the head, or the transposed tied embedding."""
        if self.lm_head is not None:
            return self.lm_head.weight
        return self.embedding.weight.t()

    def project_logits(self, x: torch.Tensor) -> torch.Tensor:
        """Hidden states -> logits over the real vocabulary (handles a group-quantised head)."""
        if self.lm_head is not None and not hasattr(self.lm_head, "weight"):
            return self.lm_head(x)[..., :self.cfg.vocab_size]
        return ops.linear(x, self.output_weight(), self.output_bias())[..., :self.cfg.vocab_size]

    def output_bias(self) -> Optional[torch.Tensor]:
        if self.lm_head is not None:
            return self.lm_head.bias
        return getattr(self, "tied_output_bias", None)

    def embed(self, tokens: torch.Tensor) -> torch.Tensor:
        x = ops.embedding(tokens, self.embedding.weight)
        if self.cfg.embeddings.scale is not None:
            x = x * self.cfg.embeddings.scale
        if self.cfg.embeddings.dropout > 0.0 and self.training:
            x = torch.nn.functional.dropout(x, self.cfg.embeddings.dropout)
        if self.stream_dtype is not None:
            x = x.to(self.stream_dtype)
        return x

    # ------------------------------------------------------------------ stateless
    def forward_hidden(self, tokens: torch.Tensor, through_layer: Optional[int] = None,
                       dream_seed: Optional[int] = None, final_norm: bool = True):
        """Hidden states after `through_layer` blocks (all when None) and the summed
        router auxiliary loss."""
        x = self.embed(tokens)
        rope = self.rope(tokens.device)
        aux_total = None
        n = len(self.layers) if through_layer is None else through_layer
        fused = x.is_cuda and self.final_norm.kind == "rmsnorm" and all(self.layers[i].fusable() for i in range(n))
        pending = None
        hook = getattr(self, "grad_ready_hook", None)
        for i in range(n):
            seed = None if dream_seed is None else dream_seed * 1009 + i
            if hook is not None and hook.armed and x.requires_grad:
                x = _GradReady.apply(x, hook, i)
            if fused:
                x, pending, aux = self.layers[i].forward_deferred(x, pending, rope, None, seed)
            else:
                x, aux = self.layers[i](x, rope, None, seed)
            if aux is not None:
                aux_total = aux if aux_total is None else aux_total + aux
        if pending is not None:
            if final_norm:
                x, _ = self.final_norm(pending.to(x.dtype), x)
                return x, aux_total
            x = x + pending.to(x.dtype)
        if final_norm:
            x = self.final_norm(x)
        return x, aux_total

    def forward(self, tokens: torch.Tensor) -> torch.Tensor:
        """Logits `[B, S, vocab_size]` (logical vocabulary)."""
        x, _ = self.forward_hidden(tokens)
        logits = ops.linear(x, self.output_weight(), self.output_bias())
        return logits[..., :self.cfg.vocab_size]

    def forward_loss(self, tokens: torch.Tensor, targets: torch.Tensor, with_router: bool = False,
                     dream_seed: Optional[int] = None):
        """Mean next-token CE over all positions (+ router aux when asked)."""
        x, aux = self.forward_hidden(tokens, dream_seed=dream_seed)
        flat = x.reshape(-1, x.shape[-1])
        loss = ops.linear_cross_entropy(flat, self.output_weight(), self.output_bias(),
                                        targets.reshape(-1), self.cfg.vocab_size, LOSS_CHUNKS)
        if with_router:
            return loss, (aux if aux is not None else loss.new_zeros(()))
        return loss

    def loss_from_hidden(self, hidden: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        """Mean next-token CE from final-normed hidden states (the tail of `forward_loss`; the last
        pipeline stage calls it on the activations it received)."""
        flat = hidden.reshape(-1, hidden.shape[-1])
        return ops.linear_cross_entropy(flat, self.output_weight(), self.output_bias(), targets.reshape(-1),
                                        self.cfg.vocab_size, LOSS_CHUNKS)

    def forward_masked_loss(self, tokens, targets, positions: torch.Tensor, with_router: bool = False,
                            return_logits: bool = False):
        """CE over selected flat positions only (`positions` index B*S)."""
        x, aux = self.forward_hidden(tokens)
        flat = x.reshape(-1, x.shape[-1]).index_select(0, positions)
        tsel = targets.reshape(-1).index_select(0, positions)
        if return_logits:
            loss, logits = ops.reference.linear_cross_entropy(
                flat, self.output_weight(), self.output_bias(), tsel, self.cfg.vocab_size,
                LOSS_CHUNKS, return_logits=True)
        else:
            loss = ops.linear_cross_entropy(flat, self.output_weight(), self.output_bias(), tsel,
                                            self.cfg.vocab_size, LOSS_CHUNKS)
        out = [loss]
        if with_router:
            out.append(aux if aux is not None else loss.new_zeros(()))
        if return_logits:
            out.append(logits)
        return out[0] if len(out) == 1 else tuple(out)

    def forward_loss_and_logits(self, tokens, targets):
        """(loss, logits `[T, vocab]`) for distillation objectives."""
        x, _ = self.forward_hidden(tokens)
        flat = x.reshape(-1, x.shape[-1])
        return ops.reference.linear_cross_entropy(flat, self.output_weight(), self.output_bias(),
                                                  targets.reshape(-1), self.cfg.vocab_size,
                                                  LOSS_CHUNKS, return_logits=True)

    def forward_selected_logits(self, tokens: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        """Logits at selected flat positions, `[P, vocab_size]`."""
        x, _ = self.forward_hidden(tokens)
        flat = x.reshape(-1, x.shape[-1]).index_select(0, positions)
        return ops.linear(flat, self.output_weight(), self.output_bias())[..., :self.cfg.vocab_size]

    def forward_embeddings(self, tokens: torch.Tensor, end_positions: torch.Tensor,
                           layer: Optional[int] = None) -> torch.Tensor:
        """L2-normalised final-norm(hidden at end_positions) from 1-based `layer`
        (all layers when None), in fp32 (`transformer.rs:835-851`)."""
        x, _ = self.forward_hidden(tokens, through_layer=layer)
        B = tokens.shape[0]
        sel = x[torch.arange(B, device=x.device), end_positions].float()
        return sel / sel.norm(dim=-1, keepdim=True).clamp_min(1e-12)

    # ------------------------------------------------------------------ stateful
    def make_state(self, batch: int, capacity: Optional[int] = None, dtype=None) -> InferenceState:
        capacity = capacity or self.cfg.max_seq_len
        p = self.embedding.weight
        dtype = dtype or (self.stream_dtype or p.dtype)
        layers = []
        for blk in self.layers:
            if blk.ssm is not None:
                layers.append(blk.ssm.make_state(batch, p.device, dtype))
            else:
                layers.append(blk.attention.make_state(batch, capacity, p.device, dtype))
        return InferenceState(layers, 0, capacity)

    def forward_hidden_with_state(self, tokens: torch.Tensor, state: InferenceState) -> torch.Tensor:
        x = self.embed(tokens)
        rope = self.rope(tokens.device)
        for blk, st in zip(self.layers, state.layers):
            x, _ = blk(x, rope, st, None)
        state.pos += tokens.shape[1]
        return self.final_norm(x)

    def forward_with_state(self, tokens: torch.Tensor, state: InferenceState) -> torch.Tensor:
        x = self.forward_hidden_with_state(tokens, state)
        return self.project_logits(x)

    def forward_next_logits_with_state(self, tokens: torch.Tensor, state: InferenceState) -> torch.Tensor:
        """Logits of the LAST position only, `[B, vocab_size]`."""
        x = self.forward_hidden_with_state(tokens, state)[:, -1]
        return self.project_logits(x)

    def prepare_inference(self, dtype: torch.dtype = torch.bfloat16) -> "Transformer":
        """Pre-cast matrix weights for inference (norm gains and scan params stay fp32)."""
        self.eval()
        for name, p in self.named_parameters():
            if p.is_floating_point() and p.dim() >= 2 and not name.endswith("a_log"):
                p.data = p.data.to(dtype)
        self.stream_dtype = dtype
        return self

    # ------------------------------------------------------------------ parameter groups
    def muon_parameter_names(self) -> List[str]:
        """2-D matrices inside blocks except routers and memory reserve params
        (`transformer.rs:973-985`)."""
        names = []
        for name, p in self.named_parameters():
            if not name.startswith("layers.") or p.dim() != 2 or not p.requires_grad:
                continue
            if ".router." in name or ".reserve." in name or name.endswith("a_log"):
                continue
            names.append(name)
        return names

    def quant_parameter_names(self, include_embeddings: bool = True, include_head: bool = True) -> List[str]:
        """Every rank >= 2 floating parameter, optionally minus embeddings / head."""
        out = []
        for name, p in self.named_parameters():
            if p.dim() < 2 or not p.is_floating_point() or not p.requires_grad:
                continue
            if not include_embeddings and name.startswith("embedding."):
                continue
            if not include_head and name.startswith("lm_head."):
                continue
            out.append(name)
        return out

    def parameter_accounting(self) -> Tuple[int, int]:
        """(stored trainable parameters, parameters active per token)."""
        stored = sum(p.numel() for p in self.parameters() if p.requires_grad)
        active = stored
        for blk in self.layers:
            ffs = [t.feed_forward for t in blk.memory.tiers] if blk.memory is not None else [blk.feed_forward]
            for ff in ffs:
                if isinstance(ff, SparseMoe):
                    e = ff.moe.experts
                    per = (e.in_weight.numel() + e.down_weight.numel()) // ff.cfg.experts
                    active -= per * (ff.cfg.experts - ff.cfg.top_k)
        return stored, active


class _Embedding(nn.Module):
    def __init__(self, weight: torch.Tensor):
        super().__init__()
        self.weight = nn.Parameter(weight)
