"""Training engine: flat parameter / gradient buffers, fused optimizer step,
data-parallel sharding.

Layout (per rank):
  * `params`  — one flat bf16 buffer holding every compute weight; the model's
    parameters are views into it.
  * `grads`   — one flat fp32 buffer; each parameter gets a `main_grad` view, and the
    weight-gradient GEMMs accumulate straight into it (TMA reduce-add), so gradient
    accumulation costs no extra pass.
  * `master`, `exp_avg`, `exp_avg_sq` — fp32, only for this rank's shard of the flat
    range (ZeRO-1 style).
With data parallelism both flat buffers live in symmetric memory: the fused kernel
in `summa_b200.parallel.dp` reads every peer's gradients for this rank's shard over
NVLink, reduces, clips, applies AdamW and writes the new bf16 weights into every
peer's parameter buffer — reduce-scatter, optimizer and all-gather in one launch.

Reference behaviour reproduced: AdamW(β 0.9/0.95, eps 1e-8, wd) with a global L2
gradient-norm clip before the update (`summa-train/src/trainer.rs:1123-1129,
1952-1975`, `summa-train/src/main.rs:667-694`).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional

import torch
import torch.nn as nn

from ..ops import native


@dataclass
class OptimConfig:
    lr: float = 3e-4
    beta1: float = 0.9
    beta2: float = 0.95
    eps: float = 1e-8
    weight_decay: float = 0.1
    max_grad_norm: float = 1.0       # <= 0 disables clipping


def _align(n: int, a: int) -> int:
    return (n + a - 1) // a * a


class FlatTrainEngine:
    """Owns the flat buffers of a model and performs optimizer steps.

    `dp` is an optional `summa_b200.parallel.dp.DataParallelGroup`; without it the
    engine runs single-device with the same buffers and the fused AdamW kernel.
    """

    def __init__(self, model: nn.Module, cfg: OptimConfig, dp=None, param_dtype=torch.bfloat16):
        self.model = model
        self.cfg = cfg
        self.dp = dp
        self.step_count = 0
        params = [(n, p) for n, p in model.named_parameters() if p.requires_grad]
        self.names = [n for n, _ in params]
        self.device = params[0][1].device
        world = dp.world_size if dp is not None else 1
        rank = dp.rank if dp is not None else 0
        # each parameter starts on a 16-byte boundary of the bf16 buffer (TMA base alignment)
        offsets, total = [], 0
        for _, p in params:
            offsets.append(total)
            total += _align(p.numel(), 8)
        self.numel = total
        self.padded = _align(total, world * 1024)
        self.shard = self.padded // world
        self.rank, self.world = rank, world
        if dp is not None:
            self.params_flat = dp.alloc_symmetric(self.padded, param_dtype, "params")
            self.grads_flat = dp.alloc_symmetric(self.padded, torch.float32, "grads")
        else:
            self.params_flat = torch.zeros(self.padded, device=self.device, dtype=param_dtype)
            self.grads_flat = torch.zeros(self.padded, device=self.device, dtype=torch.float32)
        self.offsets: Dict[str, int] = {}
        with torch.no_grad():
            for (name, p), off in zip(params, offsets):
                n = p.numel()
                self.params_flat[off:off + n].copy_(p.detach().reshape(-1).to(param_dtype))
                p.data = self.params_flat[off:off + n].view(p.shape)
                p.main_grad = self.grads_flat[off:off + n].view(p.shape)
                self.offsets[name] = off
        lo = rank * self.shard
        self.master = self.params_flat[lo:lo + self.shard].float().clone()
        self.exp_avg = torch.zeros(self.shard, device=self.device, dtype=torch.float32)
        self.exp_avg_sq = torch.zeros(self.shard, device=self.device, dtype=torch.float32)
        self._scratch = torch.zeros(4, device=self.device, dtype=torch.float32)
        if dp is not None:
            dp.barrier()

    # ------------------------------------------------------------------ gradient plumbing
    def zero_grad(self) -> None:
        self.grads_flat.zero_()
        for p in self.model.parameters():
            p.grad = None

    def fold_autograd_grads(self) -> None:
        """Gradients that arrived through autograd's `.grad` (ops without a fused
        main-grad epilogue) are added into the flat fp32 buffer."""
        for p in self.model.parameters():
            if p.grad is not None:
                p.main_grad.add_(p.grad.to(torch.float32).view_as(p.main_grad))
                p.grad = None

    # ------------------------------------------------------------------ step
    def step(self, lr: Optional[float] = None, grad_scale: float = 1.0) -> torch.Tensor:
        """Clip + AdamW over the flat buffers. Returns the (pre-clip) global gradient
        norm as a device scalar. `grad_scale` multiplies gradients first (e.g. 1/ga)."""
        self.fold_autograd_grads()
        cfg = self.cfg
        lr = cfg.lr if lr is None else lr
        self.step_count += 1
        bc1 = 1.0 - cfg.beta1 ** self.step_count
        bc2 = 1.0 - cfg.beta2 ** self.step_count
        if self.dp is not None:
            # the summed rank gradients become the gradient of the global-batch mean
            return self.dp.fused_step(self, lr, bc1, bc2, grad_scale / self.world)
        g = self.grads_flat
        sc = self._scratch
        sc.zero_()
        if g.is_cuda:
            native.call("sb_sumsq", g.data_ptr(), self.numel, sc.data_ptr(), native.stream())
            norm = sc[0].sqrt() * grad_scale
            # clip coefficient stays on the device: no host sync in the step
            if cfg.max_grad_norm > 0:
                coef = (cfg.max_grad_norm / (norm + 1e-6)).clamp(max=1.0) * grad_scale
            else:
                coef = torch.full((), grad_scale, device=g.device)
            sc[1] = coef
            native.call("sb_adamw", self.master.data_ptr(), self.exp_avg.data_ptr(), self.exp_avg_sq.data_ptr(),
                        g.data_ptr(), self.params_flat.data_ptr(), self.padded, sc[1:].data_ptr(), lr, cfg.beta1,
                        cfg.beta2, cfg.eps, cfg.weight_decay, bc1, bc2, native.stream())
            return norm
        # CPU path (same math in PyTorch)
        norm = g[:self.numel].norm() * grad_scale
        coef = grad_scale
        if cfg.max_grad_norm > 0:
            coef = float(min(1.0, cfg.max_grad_norm / (norm.item() + 1e-6))) * grad_scale
        gg = g * coef
        self.exp_avg.mul_(cfg.beta1).add_(gg, alpha=1 - cfg.beta1)
        self.exp_avg_sq.mul_(cfg.beta2).addcmul_(gg, gg, value=1 - cfg.beta2)
        upd = (self.exp_avg / bc1) / ((self.exp_avg_sq / bc2).sqrt() + cfg.eps)
        self.master.mul_(1 - lr * cfg.weight_decay).add_(upd, alpha=-lr)
        self.params_flat.copy_(self.master.to(self.params_flat.dtype))
        return norm

    # ------------------------------------------------------------------ state
    def state_dict(self) -> dict:
        return {"step": self.step_count, "master": self.master, "exp_avg": self.exp_avg,
                "exp_avg_sq": self.exp_avg_sq, "rank": self.rank, "world": self.world,
                "numel": self.numel, "offsets": dict(self.offsets)}

    def load_state_dict(self, sd: dict) -> None:
        self.step_count = int(sd["step"])
        self.master.copy_(sd["master"])
        self.exp_avg.copy_(sd["exp_avg"])
        self.exp_avg_sq.copy_(sd["exp_avg_sq"])
        lo = self.rank * self.shard
        self.params_flat[lo:lo + self.shard].copy_(self.master.to(self.params_flat.dtype))


def train_step(model, engine: FlatTrainEngine, tokens: torch.Tensor, targets: torch.Tensor,
               lr: Optional[float] = None, grad_accum: int = 1):
    """One optimizer step over `grad_accum` micro-batches stacked on dim 0 of tokens.
    Returns (mean loss, gradient norm) as device scalars."""
    engine.zero_grad()
    micro = tokens.shape[0] // grad_accum
    total = None
    for i in range(grad_accum):
        t = tokens[i * micro:(i + 1) * micro]
        y = targets[i * micro:(i + 1) * micro]
        out = model.forward_loss(t, y, with_router=True)
        loss, aux = out
        (loss + aux).backward()
        total = loss.detach() if total is None else total + loss.detach()
    norm = engine.step(lr, grad_scale=1.0 / grad_accum)
    return total / grad_accum, norm
