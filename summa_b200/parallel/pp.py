"""Pipeline parallelism over point-to-point sends (NCCL p2p on GPUs, gloo on CPU ranks).

The layer stack of a `Transformer` is cut into contiguous stages, one per rank. A step runs
the micro-batches through a one-forward-one-backward (1F1B) schedule: after a warm-up of
`stages - rank - 1` forwards every rank alternates one forward with one backward, so at most
`stages - rank` activations are alive per rank. Activations travel forward and their gradients
backward as `isend` / `irecv` pairs that are posted before the compute they overlap with and
waited on only where the data is needed. Pipeline transfers are small, latency-bound and
point-to-point, which is what the library's p2p path is for; the fused kernels of this package
cover the bandwidth-bound collectives. The reference has no pipeline parallelism
(`summa-llm/src/model/backend.rs:39-55`).
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence

import torch
import torch.distributed as dist


def split_layers(num_layers: int, stages: int) -> List[range]:
    """Contiguous, as-even-as-possible layer ranges (earlier stages take the remainder)."""
    if stages <= 0 or stages > num_layers:
        raise ValueError(f"cannot cut {num_layers} layers into {stages} stages")
    base, rem = divmod(num_layers, stages)
    out, start = [], 0
    for s in range(stages):
        n = base + (1 if s < rem else 0)
        out.append(range(start, start + n))
        start += n
    return out


class PipelineStage:
    """One rank's slice of a model: `first` embeds tokens, `last` computes the loss."""

    def __init__(self, model, group, micro_shape: Sequence[int], dtype=torch.float32):
        """`micro_shape` = shape of the activation that crosses a stage boundary for ONE
        micro-batch (`[B, S, H]`)."""
        self.model, self.group = model, group
        self.rank, self.stages = dist.get_rank(group), dist.get_world_size(group)
        self.layers = split_layers(len(model.layers), self.stages)[self.rank]
        self.first, self.last = self.rank == 0, self.rank == self.stages - 1
        self.micro_shape, self.dtype = tuple(micro_shape), dtype
        self.device = next(model.parameters()).device
        self.prev = dist.get_global_rank(group, self.rank - 1) if not self.first else None
        self.next = dist.get_global_rank(group, self.rank + 1) if not self.last else None

    def owned_parameters(self):
        """Parameters this stage updates (embedding on the first stage, head / final norm on the last)."""
        ps = []
        for i in self.layers:
            ps += list(self.model.layers[i].parameters())
        if self.first:
            ps += list(self.model.embedding.parameters())
        if self.last:
            ps += list(self.model.final_norm.parameters())
            if self.model.lm_head is not None:
                ps += list(self.model.lm_head.parameters())
        return ps

    # ------------------------------------------------------------------ compute of one micro-batch
    def _forward(self, x_in: Optional[torch.Tensor], tokens: Optional[torch.Tensor], targets: Optional[torch.Tensor]):
        m = self.model
        x = m.embed(tokens) if self.first else x_in
        rope = m.rope(self.device)
        aux_total = None
        for i in self.layers:
            x, aux = m.layers[i](x, rope, None, None)
            if aux is not None:
                aux_total = aux if aux_total is None else aux_total + aux
        if self.last:
            h = m.final_norm(x)
            loss = m.loss_from_hidden(h, targets)
            return loss if aux_total is None else loss + aux_total
        return x if aux_total is None else (x, aux_total)

    # ------------------------------------------------------------------ schedule
    def step(self, tokens: Optional[List[torch.Tensor]], targets: Optional[List[torch.Tensor]], n_micro: int) -> Optional[torch.Tensor]:
        """Runs `n_micro` micro-batches forward and backward (gradients accumulate in `.grad`,
        scaled by 1 / n_micro). `tokens` is needed on the first stage, `targets` on the last.
        Returns the mean loss on the last stage, None elsewhere."""
        warm = min(self.stages - self.rank - 1, n_micro)
        inputs, outputs = [], []           # per in-flight micro-batch: stage input (leaf) and output
        losses = []
        fwd_i = bwd_i = 0

        def recv_act():
            if self.first:
                return None
            buf = torch.empty(self.micro_shape, dtype=self.dtype, device=self.device)
            dist.recv(buf, src=self.prev, group=self.group)
            return buf.requires_grad_()

        def do_forward():
            nonlocal fwd_i
            x_in = recv_act()
            out = self._forward(x_in, tokens[fwd_i] if self.first else None, targets[fwd_i] if self.last else None)
            aux = None
            if not self.last and isinstance(out, tuple):
                out, aux = out
            if not self.last:
                if out.dtype != self.dtype or tuple(out.shape) != self.micro_shape:
                    raise ValueError(f"stage output is {tuple(out.shape)} {out.dtype}, the stage boundary was declared as "
                                     f"{self.micro_shape} {self.dtype}: the next stage would receive garbage")
                req = dist.isend(out.detach().contiguous(), dst=self.next, group=self.group)
                outputs.append((out, aux, req))
            else:
                losses.append(out.detach())
                outputs.append((out, None, None))
            inputs.append(x_in)
            fwd_i += 1

        def do_backward():
            nonlocal bwd_i
            out, aux, req = outputs.pop(0)
            x_in = inputs.pop(0)
            if self.last:
                (out / n_micro).backward()
            else:
                if req is not None:
                    req.wait()
                g = torch.empty(self.micro_shape, dtype=self.dtype, device=self.device)
                dist.recv(g, src=self.next, group=self.group)
                roots, grads = [out], [g]
                if aux is not None:                       # auxiliary (router) losses of this stage's layers
                    roots.append(aux / n_micro)
                    grads.append(torch.ones_like(aux))
                torch.autograd.backward(roots, grads)
            if not self.first:
                dist.send(x_in.grad.contiguous(), dst=self.prev, group=self.group)
            bwd_i += 1

        for _ in range(warm):
            do_forward()
        for _ in range(n_micro - warm):
            do_forward()
            do_backward()
        while bwd_i < n_micro:
            do_backward()
        return torch.stack(losses).mean() if self.last else None
