"""Batched Muon: momentum + Newton-Schulz orthogonalisation for the 2-D block matrices.

Reference semantics (`summa-train/src/muon.rs:12-15,182-283`): momentum 0.95 with a
Nesterov-style blend, five Newton-Schulz iterations with coefficients
(3.4445, -4.7750, 2.0315), update scaled by `lr * sqrt(max(1, rows / cols))`, no weight
decay; matrices of the same shape are stacked and iterated together (velocities are
stored per shape as `"{rows}x{cols}"`, rank-3 fp32). The Newton-Schulz products run in
bf16 on the tensor-core GEMM via batched matmul.
"""
from __future__ import annotations

from collections import defaultdict
from typing import Dict, List, Optional

import torch

NS_COEFFS = (3.4445, -4.7750, 2.0315)
NS_STEPS = 5
MOMENTUM = 0.95


def newton_schulz(G: torch.Tensor, steps: int = NS_STEPS) -> torch.Tensor:
    """Approximate orthogonalisation of a batch of matrices `[B, R, C]`."""
    a, b, c = NS_COEFFS
    X = G.to(torch.bfloat16) if G.is_cuda else G.float()
    transposed = X.shape[1] > X.shape[2]
    if transposed:
        X = X.transpose(1, 2)
    X = X / (X.float().norm(dim=(1, 2), keepdim=True).to(X.dtype) + 1e-7)
    for _ in range(steps):
        A = X @ X.transpose(1, 2)
        Bm = b * A + c * (A @ A)
        X = a * X + Bm @ X
    if transposed:
        X = X.transpose(1, 2)
    return X.float()


class BatchedMuon:
    def __init__(self, engine, names: List[str]):
        self.engine = engine
        params = dict(engine.model.named_parameters())
        self.groups: Dict[str, List[str]] = defaultdict(list)
        for n in names:
            p = params[n]
            self.groups[f"{p.shape[0]}x{p.shape[1]}"].append(n)
        self.params = params
        self.velocity = {k: torch.zeros(len(v), *params[v[0]].shape, device=engine.device, dtype=torch.float32)
                         for k, v in self.groups.items()}
        # Under data parallelism the engine's fp32 master is sharded by flat offset, but a
        # Muon update needs whole matrices: every rank then keeps full fp32 masters of the
        # Muon matrices and applies the identical update to them.
        self.own_master = engine.dp is not None
        self.master = {n: params[n].detach().float().clone() for n in names} if self.own_master else {}

    def step(self, lr: float, coef, grads: Optional[torch.Tensor] = None) -> None:
        """Applies the Muon update to its matrices (master + compute copies). The engine
        lays these matrices out after every AdamW-owned parameter, so the flat AdamW pass
        (and its weight decay) never touches them. `grads`: the rank-summed flat fp32
        gradient buffer (data parallelism); default is each parameter's own `main_grad`."""
        eng = self.engine
        scale = coef if not torch.is_tensor(coef) else coef.reshape(-1)[0]

        def grad_of(n):
            if grads is None:
                return self.params[n].main_grad
            off = eng.offsets[n]
            return grads[off:off + self.params[n].numel()].view_as(self.params[n])

        for key, names in self.groups.items():
            g = torch.stack([grad_of(n) for n in names]) * scale
            v = self.velocity[key]
            v.mul_(MOMENTUM).add_(g)
            upd = newton_schulz(g + MOMENTUM * v)
            rows, cols = g.shape[1], g.shape[2]
            step = lr * max(1.0, rows / cols) ** 0.5
            for i, n in enumerate(names):
                if self.own_master:
                    m = self.master[n]
                else:
                    off = eng.offsets[n]
                    m = eng.master[off:off + rows * cols].view(rows, cols)
                m.add_(upd[i], alpha=-step)
                self.params[n].data.copy_(m.to(self.params[n].dtype))
                self.params[n].main_grad.zero_()

    def state_tensors(self) -> Dict[str, torch.Tensor]:
        return dict(self.velocity)

    def load_state_tensors(self, t: Dict[str, torch.Tensor]) -> None:
        for k, v in t.items():
            if k in self.velocity:
                self.velocity[k].copy_(v.to(self.velocity[k].device))
