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

from ..ops import native

NS_COEFFS = (3.4445, -4.7750, 2.0315)
NS_STEPS = 5
MOMENTUM = 0.95


def _bmm(a: torch.Tensor, b: torch.Tensor, trans_b: bool, trans_a: bool = False) -> torch.Tensor:
    """Batched product on this package's tcgen05 kernel for CUDA bf16 operands whose dimensions TMA can
    address (multiples of 8); plain matmul on the CPU oracle path."""
    if a.is_cuda and a.dtype == torch.bfloat16 and all(d % 8 == 0 for d in (*a.shape[1:], *b.shape[1:])):
        from ..ops import cuda_ops
        return cuda_ops.bmm(a, b, trans_b, trans_a=trans_a)
    return (a.transpose(1, 2) if trans_a else a) @ (b.transpose(1, 2) if trans_b else b)


def newton_schulz(G: torch.Tensor, steps: int = NS_STEPS) -> torch.Tensor:
    """Approximate orthogonalisation of a batch of matrices `[B, R, C]`: five iterations of
    `X <- a X + (b A + c A A) X` with `A = X X^T`, in bf16 on the device. The three products of an iteration
    are batched GEMMs over all matrices of the shape group (`A` is symmetric, so `A A = A A^T` and the Gram
    products run in the transposed-operand layouts without a copy). A tall matrix (R > C) iterates on the
    smaller Gram matrix `A = X^T X` instead, `X <- a X + X (b A + c A A)`: the same polynomial of the same
    singular values, again without transposing anything in memory."""
    a, b, c = NS_COEFFS
    X = G.to(torch.bfloat16) if G.is_cuda else G.float()
    tall = X.shape[1] > X.shape[2]
    X = X / (torch.linalg.vector_norm(X, dim=(1, 2), keepdim=True, dtype=torch.float32).to(X.dtype) + 1e-7)
    for _ in range(steps):
        A = _bmm(X, X, False, trans_a=True) if tall else _bmm(X, X, True)      # X^T X  or  X X^T
        Bm = torch.add(b * A, _bmm(A, A, True), alpha=c)
        X = torch.add(_bmm(X, Bm, False) if tall else _bmm(Bm, X, False), X, alpha=a)
    return X if X.is_cuda else X.float()          # bf16 on the device: that is what the update consumes


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
            p0 = self.params[names[0]]
            cuda = p0.is_cuda
            fused = cuda and p0.dtype == torch.bfloat16 and (rows * cols) % 8 == 0
            upd_dtype = torch.bfloat16 if cuda else torch.float32
            own = torch.zeros(self.chunk[key], rows, cols, device=eng.device, dtype=upd_dtype)
            if hi > lo:
                v = self.velocity[key]
                if fused and grads is None:
                    # one kernel: scale, momentum, Nesterov blend, bf16 operand of the chain, gradient zeroed
                    u = self._buffer(key, "u", (hi - lo, rows, cols), torch.bfloat16)
                    native.call("sb_muon_momentum", self._pointers(key, "grad", [grad_of(n) for n in names[lo:hi]]).data_ptr(),
                                v.data_ptr(), u.data_ptr(), hi - lo, rows * cols, self._scale(scale).data_ptr(), MOMENTUM,
                                native.stream())
                else:
                    g = torch.stack([grad_of(n) for n in names[lo:hi]]) * scale
                    v.mul_(MOMENTUM).add_(g)
                    u = g + MOMENTUM * v
                own[:hi - lo] = newton_schulz(u).to(upd_dtype)
            upd = own if self.world == 1 else eng.dp.all_gather(own.reshape(-1)).view(-1, rows, cols)
            step = lr * max(1.0, rows / cols) ** 0.5
            masters = []
            for n in names:
                if self.own_master:
                    masters.append(self.master[n])
                else:
                    off = eng.offsets[n]
                    masters.append(eng.master[off:off + rows * cols].view(rows, cols))
            if fused:
                # one kernel: fp32 master -= step * update, bf16 compute copy rewritten from the master
                native.call("sb_muon_apply", self._pointers(key, "master", masters).data_ptr(),
                            self._pointers(key, "param", [self.params[n].data for n in names]).data_ptr(),
                            upd.data_ptr(), len(names), rows * cols, float(step), native.stream())
                if grads is not None or not (hi > lo):
                    torch._foreach_zero_([self.params[n].main_grad for n in names])
                elif hi - lo < len(names):
                    torch._foreach_zero_([self.params[n].main_grad for n in names[:lo] + names[hi:]])
            else:
                # one multi-tensor launch per group and operation instead of three small kernels per matrix
                updates = list(upd[:len(names)].float().unbind(0))
                torch._foreach_add_(masters, updates, alpha=-step)
                torch._foreach_copy_([self.params[n].data for n in names], masters)
                torch._foreach_zero_([self.params[n].main_grad for n in names])

    # ------------------------------------------------------------------ helpers of the fused device path
    def _buffer(self, key: str, what: str, shape, dtype) -> torch.Tensor:
        bufs = self.__dict__.setdefault("_bufs", {})
        t = bufs.get((key, what))
        if t is None or tuple(t.shape) != tuple(shape):
            t = bufs[(key, what)] = torch.empty(shape, device=self.engine.device, dtype=dtype)
        return t

    def _pointers(self, key: str, what: str, tensors) -> torch.Tensor:
        """Device array of the tensors' addresses, built once per (group, role): the views it names (flat-buffer
        gradients, masters, parameters) never move."""
        cache = self.__dict__.setdefault("_ptrs", {})
        addrs = tuple(t.data_ptr() for t in tensors)
        hit = cache.get((key, what))
        if hit is None or hit[0] != addrs:
            assert all(a % 16 == 0 for a in addrs) and all(t.is_contiguous() for t in tensors)
            hit = cache[(key, what)] = (addrs, torch.tensor(addrs, dtype=torch.int64, device=self.engine.device))
        return hit[1]

    def _scale(self, scale) -> torch.Tensor:
        """The gradient scale as a device scalar (the clip coefficient already is one)."""
        if torch.is_tensor(scale):
            return scale.reshape(-1)[:1].float() if scale.dtype != torch.float32 else scale.reshape(-1)[:1]
        t = self._buffer("", "scale", (1,), torch.float32)
        t.fill_(float(scale))
        return t

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
