"""Continuum memory: an ordered residual chain of tiers replacing a block's FFN.

Each tier owns an ordinary FFN/MoE plus a fixed-capacity reserve of low-rank
expert slots that start dormant; activating a slot flips a checkpointed flag and
never changes a tensor shape (`summa-llm/src/model/memory.rs:33-113,153-293,
422-584,655-769`).

Checkpoint keys: `memory.tiers.{t}.feed_forward.*`,
`memory.tiers.{t}.reserve.slots.{s}.{router.weight,a,b,active,generation}`.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.nn as nn

from .. import ops
from ..mal import MemoryDef, MemoryTierDef
from .layers import SparseMoe, build_ffn


def _xorshift_fill(rows: int, cols: int, seed: int) -> torch.Tensor:
    """Deterministic pseudo-random values in ±0.02 (xorshift64*)."""
    state = (seed * 0x9E3779B97F4A7C15 + 0xD1B54A32D192ED03) & 0xFFFFFFFFFFFFFFFF or 1
    out = torch.empty(rows * cols, dtype=torch.float32)
    vals = []
    for _ in range(rows * cols):
        state ^= (state >> 12)
        state ^= (state << 25) & 0xFFFFFFFFFFFFFFFF
        state ^= (state >> 27)
        r = (state * 0x2545F4914F6CDD1D) & 0xFFFFFFFFFFFFFFFF
        vals.append(((r >> 40) / float(1 << 24)) * 2.0 - 1.0)
    out.copy_(torch.tensor(vals, dtype=torch.float32))
    return out.view(rows, cols) * 0.02


class _SlotRouter(nn.Module):
    def __init__(self, hidden: int):
        super().__init__()
        self.weight = nn.Parameter(torch.zeros(hidden, 1))


class LowRankExpertSlot(nn.Module):
    def __init__(self, hidden: int, rank: int, seed: int):
        super().__init__()
        self.router = _SlotRouter(hidden)
        self.a = nn.Parameter(_xorshift_fill(hidden, rank, seed))
        self.b = nn.Parameter(torch.zeros(rank, hidden))
        # checkpointed state, not trainable
        self.active = nn.Parameter(torch.zeros(1, dtype=torch.bool), requires_grad=False)
        self.generation = nn.Parameter(torch.zeros(1, dtype=torch.int64), requires_grad=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.linear(ops.linear(x, self.a, None), self.b, None)


class LowRankExpertReserve(nn.Module):
    """Top-1 routing over ACTIVE slots competing with a parameter-free zero lane."""

    def __init__(self, hidden: int, capacity: int, rank: int, top_k: int, seed: int):
        super().__init__()
        if top_k != 1:
            raise ValueError("reserve_experts top_k must be 1")
        self.hidden = hidden
        self.slots = nn.ModuleList([LowRankExpertSlot(hidden, rank, seed * 1000 + s) for s in range(capacity)])

    def active_slots(self) -> List[int]:
        return [i for i, s in enumerate(self.slots) if bool(s.active.item())]

    def activate(self, slot: int) -> None:
        with torch.no_grad():
            self.slots[slot].active.fill_(True)
            self.slots[slot].generation.add_(1)

    def deactivate(self, slot: int) -> None:
        """Reclaims a slot: dormant again, generation raised (stale optimizer state cannot alias the next use), and
        its product zeroed so that it wakes up as the identity the next time (`b` = 0, router = 0)."""
        with torch.no_grad():
            s = self.slots[slot]
            s.active.fill_(False)
            s.generation.add_(1)
            s.b.zero_()
            s.router.weight.zero_()

    def slot_states(self) -> List[tuple]:
        """(active, generation) of every slot, read back from the device (sleep boundaries only)."""
        return [(bool(s.active.item()), int(s.generation.item())) for s in self.slots]

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """Top-1 over the ACTIVE slots against a zero lane, evaluated with a fixed router width: every slot's logit
        is computed, dormant ones are masked to -inf on the device, and every slot's low-rank product is weighted by
        (selected and active) x gate. Nothing is read back to the host, so the forward neither synchronises the
        stream nor changes shape when a slot wakes up (`summa-llm/src/model/memory.rs:295-320`: fixed router width,
        zero fallback lanes); the price is capacity x two rank-r GEMMs over all tokens, small beside the tier's FFN."""
        flat = x.reshape(-1, self.hidden)
        n = len(self.slots)
        W = torch.cat([s.router.weight for s in self.slots], dim=1).float()             # [H, capacity]
        active = torch.cat([s.active for s in self.slots])                               # [capacity] bool, on the device
        logits = ops.router_logits(flat, W).masked_fill(~active, float("-inf"))          # [T, capacity], the fp32 router kernel on CUDA
        top = logits.argmax(dim=1, keepdim=True)
        probs = torch.softmax(torch.cat([logits, torch.zeros_like(logits[:, :1])], dim=1), dim=1)
        gate = probs[:, :n].gather(1, top)                                               # 0 where no slot is active
        out = None
        for i, s in enumerate(self.slots):
            weight = (gate * ((top == i) & active[i]).to(gate.dtype)).to(flat.dtype)
            y = s(flat) * weight
            out = y if out is None else out + y
        return out.reshape(x.shape)


class MemoryTier(nn.Module):
    def __init__(self, tier: MemoryTierDef, hidden: int, seed: int, init_std=None):
        super().__init__()
        self.name = tier.name
        self.feed_forward = build_ffn(tier.ffn, hidden, init_std)
        r = tier.reserve_experts
        self.reserve = LowRankExpertReserve(hidden, r.capacity, r.rank, r.top_k, seed)
        if tier.residual_init == "zero":
            with torch.no_grad():
                if isinstance(self.feed_forward, SparseMoe):
                    self.feed_forward.moe.experts.down_weight.zero_()
                    for sh in self.feed_forward.moe.shared_experts:
                        sh.down_proj.weight.zero_()
                else:
                    self.feed_forward.down_proj.weight.zero_()

    def forward(self, x: torch.Tensor, dream_seed: Optional[int] = None):
        if isinstance(self.feed_forward, SparseMoe):
            y, aux = self.feed_forward(x, dream_seed)
        else:
            y, aux = self.feed_forward(x), None
        return y + self.reserve(x), aux


class MemoryChain(nn.Module):
    """state = residual(state, tier(normalize(state))) for each tier, fast to slow.

    Every tier is normalised by the owning block's `ffn_norm` (passed in as
    `normalize`), so the chain adds no norm parameters of its own.
    """

    def __init__(self, memory: MemoryDef, hidden: int, layer_index: int, init_std=None):
        super().__init__()
        self.tiers = nn.ModuleList([MemoryTier(t, hidden, layer_index * 64 + i, init_std)
                                    for i, t in enumerate(memory.tiers)])

    def forward(self, state: torch.Tensor, normalize, residual, dream_seed: Optional[int] = None):
        """Returns (new stream, summed aux loss or None)."""
        aux_total = None
        for i, tier in enumerate(self.tiers):
            seed = None if dream_seed is None else dream_seed * 131 + i
            y, aux = tier(normalize(state), seed)
            state = residual(state, y)
            if aux is not None:
                aux_total = aux if aux_total is None else aux_total + aux
        return state, aux_total
