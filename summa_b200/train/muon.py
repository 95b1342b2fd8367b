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


def _bmm(a: torch.Tensor, b: torch.Tensor, trans_b: bool) -> torch.Tensor:
    """Batched product on this package's tcgen05 kernel for CUDA bf16 operands whose dimensions TMA can
    address (multiples of 8); plain matmul on the CPU oracle path."""
    if a.is_cuda and a.dtype == torch.bfloat16 and all(d % 8 == 0 for d in (*a.shape[1:], *b.shape[1:])):
        from ..ops import cuda_ops
        return cuda_ops.bmm(a, b, trans_b)
    return a @ (b.transpose(1, 2) if trans_b else b)


def newton_schulz(G: torch.Tensor, steps: int = NS_STEPS) -> torch.Tensor:
    """Approximate orthogonalisation of a batch of matrices `[B, R, C]`: five iterations of
    `X <- a X + (b A + c A A) X` with `A = X X^T`, in bf16 on the device. The three products of an iteration
    are batched GEMMs over all matrices of the shape group (`A` is symmetric, so `A A = A A^T` and both Gram
    products run in the transposed-operand layout without a copy)."""
    a, b, c = NS_COEFFS
    X = G.to(torch.bfloat16) if G.is_cuda else G.float()
    transposed = X.shape[1] > X.shape[2]
    if transposed:
        X = X.transpose(1, 2).contiguous()
    X = X / (X.float().norm(dim=(1, 2), keepdim=True).to(X.dtype) + 1e-7)
    for _ in range(steps):
        A = _bmm(X, X, True)                       # X X^T
        Bm = torch.add(b * A, _bmm(A, A, True), alpha=c)
        X = torch.add(_bmm(Bm, X, False), X, alpha=a)
    if transposed:
        X = X.transpose(1, 2)
    return X.float()


class BatchedMuon:
    """Muon for the block matrices, sharded BY MATRIX under data parallelism.

    Matrices of one shape form a group (`"{rows}x{cols}"`), as in the reference. With `world` ranks every
    group is cut into `world` contiguous chunks of whole matrices; a rank keeps the momentum only of ITS
    chunk, runs momentum + Newton-Schulz only on it (owner computes), and the orthogonalised updates (bf16,
    which is exactly what Newton-Schulz produces) are all-gathered so that every rank applies the identical
    update to its fp32 masters. The optimizer's tensor-core work and its momentum memory therefore drop by
    the rank count. Checkpoints hold whole-group velocities, so they resume on any number of ranks."""

    def __init__(self, engine, names: List[str]):
        self.engine = engine
        params = dict(engine.model.named_parameters())
        self.groups: Dict[str, List[str]] = defaultdict(list)
        for n in names:
            p = params[n]
            self.groups[f"{p.shape[0]}x{p.shape[1]}"].append(n)
        self.params = params
        self.world = engine.world if engine.dp is not None else 1
        self.rank = engine.rank if engine.dp is not None else 0
        # chunk of group `key` owned by this rank: [lo, hi) of `chunk` matrices (the last chunks may be short or empty)
        self.chunk = {k: -(-len(v) // self.world) for k, v in self.groups.items()}
        self.velocity = {k: torch.zeros(self._own(k)[1] - self._own(k)[0], *params[v[0]].shape, device=engine.device,
                                        dtype=torch.float32) for k, v in self.groups.items()}
        # Under data parallelism the engine's fp32 master is sharded by flat offset, but a
        # Muon update needs whole matrices: every rank then keeps full fp32 masters of the
        # Muon matrices and applies the identical update to them.
        self.own_master = engine.dp is not None
        self.master = {n: params[n].detach().float().clone() for n in names} if self.own_master else {}

    def _own(self, key: str):
        n, c = len(self.groups[key]), self.chunk[key]
        lo = min(n, self.rank * c)
        return lo, min(n, lo + c)

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
            rows, cols = self.params[names[0]].shape
            lo, hi = self._own(key)
            cuda = self.params[names[0]].is_cuda
            upd_dtype = torch.bfloat16 if cuda else torch.float32
            own = torch.zeros(self.chunk[key], rows, cols, device=eng.device, dtype=upd_dtype)
            if hi > lo:
                g = torch.stack([grad_of(n) for n in names[lo:hi]]) * scale
                v = self.velocity[key]
                v.mul_(MOMENTUM).add_(g)
                own[:hi - lo] = newton_schulz(g + MOMENTUM * v).to(upd_dtype)
            upd = own if self.world == 1 else eng.dp.all_gather(own.reshape(-1)).view(-1, rows, cols)
            step = lr * max(1.0, rows / cols) ** 0.5
            for i, n in enumerate(names):
                if self.own_master:
                    m = self.master[n]
                else:
                    off = eng.offsets[n]
                    m = eng.master[off:off + rows * cols].view(rows, cols)
                m.add_(upd[i].float(), alpha=-step)
                self.params[n].data.copy_(m.to(self.params[n].dtype))
                self.params[n].main_grad.zero_()

    def state_tensors(self) -> Dict[str, torch.Tensor]:
        """Whole-group velocities `[matrices, rows, cols]` (a collective under data parallelism)."""
        out = {}
        for key, names in self.groups.items():
            v = self.velocity[key]
            if self.world > 1:
                rows, cols = self.params[names[0]].shape
                pad = torch.zeros(self.chunk[key], rows, cols, device=v.device, dtype=v.dtype)
                pad[:v.shape[0]] = v
                v = self.engine.dp.all_gather(pad.reshape(-1)).view(-1, rows, cols)[:len(names)]
            out[key] = v
        return out

    def load_state_tensors(self, t: Dict[str, torch.Tensor]) -> None:
        for k, v in t.items():
            if k in self.velocity:
                lo, hi = self._own(k)
                self.velocity[k].copy_(v[lo:hi].to(self.velocity[k].device))
