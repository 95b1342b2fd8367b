"""Inference engine: prefill + greedy decode over a KV cache, optionally tensor-parallel and
4-bit group-quantised.

`InferenceEngine.build` creates the model directly on the device (random-init or from a
state dict), shards it across the tensor-parallel group, quantises the block projections to
int4 g128 and allocates the KV cache. `prefill` uses the sequence-parallel fused
all-gather->GEMM / GEMM->reduce-scatter kernels when the token count allows and falls back
to the all-reduce form otherwise; `decode` runs one token per sequence per step: weight-
streaming int4 GEMV, split-KV decode attention, one-shot peer-memory all-reduce, device
argmax. The reference's generator is single-device (`summa-llm/src/generate.rs:127-250`).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from .transformer import Transformer


class InferenceEngine:
    def __init__(self, model: Transformer, tp=None):
        self.model = model
        self.tp = tp
        self.state = None
        self.device = model.embedding.weight.device

    @classmethod
    def build(cls, cfg, device: torch.device, tp_group=None, quantize: Optional[str] = "int4",
              init_std: float = 0.02, seed: int = 0, max_prefill_tokens: int = 0, state_dict=None,
              quantize_head: bool = False):
        torch.manual_seed(seed)                      # every rank draws the same full model, then keeps its shard
        with torch.device(device):
            model = Transformer(cfg, init_std=init_std)
        if state_dict is not None:
            model.load_state_dict(state_dict)
        model.prepare_inference(torch.bfloat16)
        tp = None
        if tp_group is not None:
            import torch.distributed as dist
            from ..parallel.tp import TensorParallelGroup, shard_model
            if dist.get_world_size(tp_group) > 1:
                mt = max_prefill_tokens
                if mt:
                    step = 128 * dist.get_world_size(tp_group)
                    mt = -(-mt // step) * step
                tp = TensorParallelGroup(tp_group, device, mode="fused", max_tokens=mt, hidden=cfg.hidden_size)
                shard_model(model, tp)
                torch.cuda.empty_cache()
        if quantize == "int4":
            from .quantized import quantize_model_int4
            quantize_model_int4(model, include_head=quantize_head)
            torch.cuda.empty_cache()
        elif quantize not in (None, "none"):
            raise ValueError(f"unknown quantisation `{quantize}`")
        return cls(model, tp)

    def reset(self, batch: int, capacity: int):
        self.state = self.model.make_state(batch, capacity)

    @torch.no_grad()
    def prefill(self, tokens: torch.Tensor) -> torch.Tensor:
        """Consumes the prompt `[B, S]`; returns the greedy next token `[B, 1]`."""
        if self.state is None:
            raise RuntimeError("call reset(batch, capacity) first")
        if self.tp is not None:
            from ..parallel.tp import prefill_sequence_parallel
            logits = prefill_sequence_parallel(self.model, self.tp, tokens, self.state)
        else:
            logits = self.model.forward_next_logits_with_state(tokens, self.state)
        return ops.argmax(logits).view(-1, 1)

    @torch.no_grad()
    def decode(self, first: torch.Tensor, steps: int) -> torch.Tensor:
        """Greedy-decodes `steps` tokens after `first` `[B, 1]`; returns `[B, steps]` (the
        tokens produced, not including `first`)."""
        out = []
        tok = first
        for _ in range(steps):
            logits = self.model.forward_next_logits_with_state(tok, self.state)
            tok = ops.argmax(logits).view(-1, 1)
            out.append(tok)
        return torch.cat(out, dim=1)
