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

import os

from .. import ops
from .transformer import Transformer

# SUMMA_DECODE_FUSED_EPILOGUES=0: separate RoPE-append and SwiGLU kernels behind plain decode projections instead
# of the cluster GEMV's fused epilogues
_FUSED_EPILOGUES = os.environ.get("SUMMA_DECODE_FUSED_EPILOGUES", "1") == "1"


class InferenceEngine:
    def __init__(self, model: Transformer, tp=None):
        self.model = model
        self.tp = tp
        self.state = None
        self.device = model.embedding.weight.device
        self.use_graph = True
        self._graph = None

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
        """Start a new set of sequences. A state of the same shape is recycled (the caches are
        overwritten as the new sequences grow), which also keeps the captured decode graph."""
        st = self.state
        if st is not None and st.capacity == capacity and st.layers and hasattr(st.layers[0], "k") \
                and st.layers[0].k.shape[0] == batch and all(hasattr(l, "length") for l in st.layers):
            for l in st.layers:
                l.length = 0
            st.pos = 0
            return
        self.state = self.model.make_state(batch, capacity)
        self._graph = None

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
        if self.use_graph and self.device.type == "cuda":
            if self._graph is None:
                self._graph = _GraphDecoder.try_build(self.model, self.state, steps)
            if self._graph is not None and self._graph.max_steps >= steps:
                return self._graph.run(first, steps)
        out = []
        tok = first
        for _ in range(steps):
            logits = self.model.forward_next_logits_with_state(tok, self.state)
            tok = ops.argmax(logits).view(-1, 1)
            out.append(tok)
        return torch.cat(out, dim=1)


class _GraphDecoder:
    """One decode step captured in a CUDA graph. Everything that changes from step to step (the
    token, the position, the output column) lives in device memory: RoPE + cache append and the
    split-KV attention read the position on the device, the tensor-parallel all-reduce keeps its
    call number on the device, so a replay needs no host input at all."""

    @classmethod
    def try_build(cls, model, state, max_steps: int):
        from .layers import FeedForward, MultiHeadAttention
        cfgm = model.cfg
        for blk in model.layers:
            a = blk.attention
            if (not isinstance(a, MultiHeadAttention) or not blk.pre_norm or not blk.residual or blk.memory is not None
                    or not isinstance(blk.feed_forward, FeedForward) or a.head_dim != 128 or a.window is not None
                    or a.q_norm is not None or not a.use_rope or not a.causal or a.num_heads // a.num_kv_heads > 8):
                return None
        if cfgm.embeddings.scale is not None or model.stream_dtype != torch.bfloat16:
            return None
        return cls(model, state, max_steps)

    def __init__(self, model, state, max_steps: int):
        from ..ops import native
        self.model, self.state, self.max_steps = model, state, max_steps
        st0 = state.layers[0]
        self.B, self.cap = st0.k.shape[0], st0.k.shape[1]
        dev = st0.k.device
        self.tok = torch.zeros(self.B, 1, dtype=torch.long, device=dev)
        self.pos = torch.zeros(1, dtype=torch.int32, device=dev)
        self.col = torch.zeros(1, 1, dtype=torch.long, device=dev)
        self.out = torch.zeros(self.B, max_steps, dtype=torch.long, device=dev)
        a0 = model.layers[0].attention
        self.splits = native.call_value("sb_attention_decode_splits", self.B, a0.num_kv_heads, self.cap)
        need = native.call_value("sb_attention_decode_workspace", self.B, a0.num_kv_heads, self.splits)
        self.ws = torch.empty(need, dtype=torch.float32, device=dev)
        P, I, L, F = native.P, native.I, native.L, native.F
        native.register("sb_decode_rope_append", [P] * 6 + [I, I, I, I, L, P, I, P])
        native.register("sb_attention_decode_dyn", [P] * 5 + [I, I, I, P, I, I, I] + [P] * 4 + [F, I, P])
        self.graph = None

    def _step(self):
        import ctypes
        from ..ops import native
        m, B = self.model, self.B
        h = torch.nn.functional.embedding(self.tok.view(-1), m.embedding.weight).to(torch.bfloat16)
        cos, sin = m.rope(h.device)
        for blk, st in zip(m.layers, self.state.layers):
            a = blk.attention
            cs = (ctypes.c_long * 3)(st.k.stride(0), st.k.stride(1), st.k.stride(2))
            if self._rope_fusable(blk, h):
                from ..ops import cuda_ops
                qkv = cuda_ops.int4_gemv_rope_append(h, a.qkv_proj.packed_k8(), a.qkv_proj.scales,
                                                     (blk.attn_norm.gamma, blk.attn_norm.eps), cos, sin, st.k, st.v,
                                                     self.pos, a.num_heads, a.num_kv_heads, a.head_dim, self.cap)
            else:
                qkv = self._norm_proj(blk.attn_norm, a.qkv_proj, h)
                native.call("sb_decode_rope_append", qkv.data_ptr(), cos.data_ptr(), sin.data_ptr(), st.k.data_ptr(),
                            st.v.data_ptr(), self.pos.data_ptr(), B, a.num_heads, a.num_kv_heads, a.head_dim,
                            qkv.stride(0), cs, self.cap, native.stream())
            o = torch.empty(B, a.q_dim, dtype=torch.bfloat16, device=h.device)
            qs = (ctypes.c_long * 2)(qkv.stride(0), a.head_dim)
            os_ = (ctypes.c_long * 2)(o.stride(0), a.head_dim)
            native.call("sb_attention_decode_dyn", qkv.data_ptr(), st.k.data_ptr(), st.v.data_ptr(), o.data_ptr(),
                        self.ws.data_ptr(), B, a.num_heads, a.num_kv_heads, self.pos.data_ptr(), 1, self.cap, a.head_dim,
                        qs, cs, cs, os_, 1.0 / a.head_dim ** 0.5, self.splits, native.stream())
            h = self._proj_add(a.o_proj, o, h)
            ff = blk.feed_forward
            if _FUSED_EPILOGUES and ff.gated and ff.act in ("swiglu", "silu") and getattr(blk.ffn_norm, "kind", None) == "rmsnorm" and h.shape[0] <= 4:
                from .quantized import in_proj_swiglu
                u = in_proj_swiglu(ff.in_proj, h, norm=(blk.ffn_norm.gamma, blk.ffn_norm.eps))
            else:
                u = self._norm_proj(blk.ffn_norm, ff.in_proj, h)
                u = ops.gated_act(u, ff.act) if ff.gated else ops.activation(ff.act, u)
            h = self._proj_add(ff.down_proj, u, h)
        logits = m.project_logits(m.final_norm(h))
        nxt = ops.argmax(logits).view(B, 1)
        self.out.scatter_(1, self.col.expand(B, 1), nxt)
        self.tok.copy_(nxt)
        self.pos += 1
        self.col += 1

    @staticmethod
    def _rope_fusable(blk, h) -> bool:
        """RMSNorm -> quantised qkv projection -> RoPE -> cache append as one kernel (<= 4 rows)."""
        from .quantized import QuantLinear
        a = blk.attention
        p = a.qkv_proj
        return (_FUSED_EPILOGUES and isinstance(p, QuantLinear) and p.bias is None and h.shape[0] <= 4
                and h.dtype == torch.bfloat16
                and getattr(blk.attn_norm, "kind", None) == "rmsnorm" and a.q_norm is None and a.k_norm is None
                and a.use_rope
                and p.d_in % 128 == 0 and p.d_in <= 20480 and h.is_contiguous()
                and p.d_out == (a.num_heads + 2 * a.num_kv_heads) * a.head_dim)

    @staticmethod
    def _norm_proj(norm, proj, h):
        """proj(norm(h)); an RMSNorm in front of a quantised projection runs inside its GEMV kernel."""
        from .quantized import QuantLinear
        if isinstance(proj, QuantLinear) and getattr(norm, "kind", None) == "rmsnorm" and h.shape[0] <= 4:
            return proj(h, norm=(norm.gamma, norm.eps))
        return proj(norm(h))

    @staticmethod
    def _proj_add(proj, x, h):
        """h + proj(x), with the add fused into the projection's epilogue when it can be."""
        from .quantized import QuantLinear
        from ..parallel.tp import RowParallelLinear
        if isinstance(proj, (QuantLinear, RowParallelLinear)):
            return proj(x, residual=h)
        return h + proj(x)

    def run(self, first: torch.Tensor, steps: int) -> torch.Tensor:
        start = self.state.layers[0].length
        if start + steps > self.cap:
            raise RuntimeError(f"KV cache overflow: {start + steps} > capacity {self.cap}")
        self.tok.copy_(first)
        self.pos.fill_(start)
        self.col.zero_()
        done = 0
        if self.graph is None:
            self._step()                                  # eager: warms every lazy allocation and attribute
            done = 1
            if steps > 1:
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    self._step()
                self.graph = g
        for _ in range(steps - done):
            self.graph.replay()
        for st in self.state.layers:
            st.length = start + steps
        self.state.pos += steps
        return self.out[:, :steps].clone()
