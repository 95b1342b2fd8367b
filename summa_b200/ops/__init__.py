"""Op layer: one function per hot operation.

CUDA tensors run the hand-written sm_100a kernels in `csrc/` (loaded by
`summa_b200.ops.native`); CPU tensors run the PyTorch oracles in `reference`.
There is no silent fallback on a GPU: if the native library is missing, a CUDA
call raises.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import reference
from .reference import rope_table as _rope_table_ref

__all__ = [
    "linear", "rmsnorm", "add_rmsnorm", "layernorm", "rope_table", "qk_norm_rope", "attention",
    "attention_dropout", "kv_append", "conv1d_silu", "selective_scan", "mul_silu", "gated_act",
    "activation", "router_logits", "moe_route", "moe_aux_loss", "moe_experts", "embedding",
    "linear_cross_entropy", "reference", "set_backend", "backend", "native_enabled",
]


def _cu():
    from . import cuda_ops
    return cuda_ops


_BACKEND = "native"


def set_backend(name: str) -> None:
    """`native` (default): CUDA bf16 tensors run this package's sm_100a kernels. `library`: they run
    stock PyTorch library ops instead (cuBLAS matmul, `scaled_dot_product_attention`, `F.rms_norm`,
    `F.cross_entropy`; see `library.py`). The library backend exists to MEASURE the baseline that the
    kernels have to beat on the same box (`bench.py --impl torch`); nothing in the product selects it."""
    global _BACKEND
    if name not in ("native", "library"):
        raise ValueError(f"unknown op backend `{name}`")
    _BACKEND = name


def backend() -> str:
    return _BACKEND


def native_enabled(t: torch.Tensor) -> bool:
    """True when `t` takes the hand-written kernels (a CUDA bf16 tensor under the native backend)."""
    return t.is_cuda and t.dtype == torch.bfloat16 and _BACKEND == "native"


def _lib(t: torch.Tensor) -> bool:
    return t.is_cuda and _BACKEND == "library"


def _library():
    from . import library
    return library


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x `[..., K]` @ weight `[K, N]` (+ bias). bf16 operands hit the tcgen05 GEMM."""
    if native_enabled(x):
        return _cu().linear(x, weight, bias)
    w = weight.to(x.dtype) if weight.dtype != x.dtype else weight
    y = x @ w
    if bias is not None:
        y = y + bias.to(y.dtype)
    return y


def rmsnorm(x, gamma, eps):
    if native_enabled(x):
        return _cu().rmsnorm(x, gamma, eps)
    if _lib(x):
        return _library().rmsnorm(x, gamma, eps)
    return reference.rmsnorm(x, gamma, eps)


def add_rmsnorm(x, residual, gamma, eps):
    """(rmsnorm(x + residual), x + residual)."""
    if native_enabled(x):
        return _cu().add_rmsnorm(x, residual, gamma, eps)
    s = x + residual
    return rmsnorm(s, gamma, eps), s


def layernorm(x, gamma, beta, eps):
    if native_enabled(x) and x.shape[-1] % 8 == 0:
        return _cu().layernorm(x, gamma, beta, eps)
    return reference.layernorm(x, gamma, beta, eps)


def rope_table(max_seq_len, head_dim, theta, scaling=None, device=None):
    return _rope_table_ref(max_seq_len, head_dim, theta, scaling, device)


def qk_norm_rope(q, k, q_gamma, k_gamma, eps, cos, sin, offset=0):
    if native_enabled(q) and cos is not None:
        return _cu().qk_norm_rope(q, k, q_gamma, k_gamma, eps, cos, sin, offset)
    return reference.qk_norm_rope(q, k, q_gamma, k_gamma, eps, cos, sin, offset)


def packed_qk_rope(qkv, q_gamma, k_gamma, eps, cos, sin, Hq, Hkv, D, offset=0):
    """QK-norm + RoPE applied to the q and k heads of a packed `[B, S, (Hq + 2 Hkv) * D]`
    projection (the v heads pass through); returns (q, k, v) views `[B, S, H, D]`."""
    B, S, _ = qkv.shape
    if native_enabled(qkv) and D in (64, 128) and cos is not None:
        out = _cu().qkv_rope(qkv, q_gamma, k_gamma, eps, cos, sin, Hq, Hkv, D, offset)
        q = out[..., :Hq * D].unflatten(-1, (Hq, D))
        k = out[..., Hq * D:(Hq + Hkv) * D].unflatten(-1, (Hkv, D))
        v = out[..., (Hq + Hkv) * D:].unflatten(-1, (Hkv, D))
        return q, k, v
    q = qkv[..., :Hq * D].unflatten(-1, (Hq, D))
    k = qkv[..., Hq * D:(Hq + Hkv) * D].unflatten(-1, (Hkv, D))
    v = qkv[..., (Hq + Hkv) * D:].unflatten(-1, (Hkv, D))
    q, k = qk_norm_rope(q, k, q_gamma, k_gamma, eps, cos, sin, offset)
    return q, k, v


def attention(q, k, v, causal=True, window=None, q_offset=0):
    if native_enabled(q):
        return _cu().attention(q, k, v, causal, window, q_offset)
    if _lib(q) and window is None and q_offset == 0:
        return _library().attention(q, k, v, causal)
    return reference.attention(q, k, v, causal, window, None, q_offset)


def packed_qkv_attention(qkv, q_gamma, k_gamma, eps, cos, sin, Hq, Hkv, D, causal, window):
    """CUDA-only fused path over the packed `[B, S, (Hq + 2 Hkv) D]` activation."""
    cu = _cu()
    qkv = cu.qkv_rope(qkv, q_gamma, k_gamma, eps, cos, sin, Hq, Hkv, D, 0)
    return cu.packed_attention(qkv, Hq, Hkv, D, causal, window)


def attention_dropout(q, k, v, causal, window, p):
    """Attention with dropout on the probabilities: materialises the scores, as the
    reference does on this (rare) path (`summa-llm/src/model/attention.rs:266-298`)."""
    import math
    B, Sq, H, D = q.shape
    g = H // k.shape[2]
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(g, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(g, dim=1)
    s = qf @ kf.transpose(-1, -2) / math.sqrt(D)
    m = reference.attention_mask(Sq, k.shape[1], causal, window, 0, q.device)
    if m is not None:
        s = s.masked_fill(m, float("-inf"))
    pr = torch.nn.functional.dropout(torch.softmax(s, dim=-1), p)
    return (pr @ vf).permute(0, 2, 1, 3).to(q.dtype)


def kv_append(k_cache, v_cache, k, v, offset):
    S = k.shape[1]
    k_cache[:, offset:offset + S].copy_(k)
    v_cache[:, offset:offset + S].copy_(v)


def conv1d_silu(x, weight, bias, state=None):
    """SiLU(causal depthwise conv(x))."""
    if native_enabled(x):
        return _cu().conv1d_silu(x, weight, bias, state)
    return torch.nn.functional.silu(reference.depthwise_conv1d(x, weight, bias, state))


def selective_scan(u, delta, A, Bm, Cm, D, h0=None, need_final_state=False):
    if native_enabled(u):
        return _cu().selective_scan(u, delta, A, Bm, Cm, D, h0, need_final_state)
    return reference.selective_scan(u, delta, A, Bm, Cm, D, h0)


def mul_silu(y, z):
    """y * silu(z), fp32 math."""
    if native_enabled(y):
        return _cu().mul_silu(y, z)
    return (y.float() * torch.nn.functional.silu(z.float())).to(y.dtype)


def gated_act(x, name="swiglu"):
    if native_enabled(x) and name in ("swiglu", "silu"):
        return _cu().swiglu(x)
    if _lib(x) and name in ("swiglu", "silu"):
        return _library().swiglu(x)
    if native_enabled(x) and name in _cu().ACT_IDS and x.shape[-1] % 16 == 0:
        return _cu().act(x, name, True)          # GeGLU / ReGLU: act(gate) * value on the same kernel family
    return reference.gated_act(x, name)


def activation(name, x):
    if native_enabled(x) and name in _cu().ACT_IDS and x.shape[-1] % 8 == 0:
        return _cu().act(x, name, False)
    return reference.activation(name, x.float()).to(x.dtype)


def router_logits(x, weight):
    """fp32 router logits `[T, E]`."""
    if native_enabled(x):
        return _cu().router_logits(x, weight)
    return x.float() @ weight.float()


def moe_route(logits, top_k):
    if logits.is_cuda and _BACKEND == "native":
        return _cu().moe_route(logits, top_k)
    return reference.moe_route(logits, top_k)


def moe_aux_loss(logits, idx, num_experts, lb_weight, z_weight):
    if lb_weight <= 0.0 and z_weight <= 0.0:
        return None
    if logits.is_cuda and _BACKEND == "native" and logits.dtype == torch.float32 and num_experts <= 256:
        return _cu().moe_aux_loss(logits, idx, num_experts, lb_weight, z_weight)
    return reference.moe_aux_loss(logits, idx, num_experts, lb_weight, z_weight)


def moe_experts(x, idx, gates, in_weight, down_weight, in_bias, down_bias, act, gated):
    """Dropless routed expert MLP: gather → grouped GEMM → act → grouped GEMM → combine."""
    if native_enabled(x) and in_bias is None and gated and act in ("swiglu", "silu"):
        return _cu().moe_experts(x, idx, gates, in_weight, down_weight)
    return _moe_experts_sorted(x, idx, gates, in_weight, down_weight, in_bias, down_bias, act, gated)


def _moe_experts_sorted(x, idx, gates, in_weight, down_weight, in_bias, down_bias, act, gated):
    """Compact per-expert loop over the stable route plan (differentiable)."""
    T, H = x.shape
    k = idx.shape[1]
    E = in_weight.shape[0]
    order, inverse, counts = reference.route_plan(idx, E)
    token_of_route = order // k
    routed = x.index_select(0, token_of_route)
    outs = []
    start = 0
    for e, c in enumerate(counts.tolist()):
        if c == 0:
            continue
        seg = routed[start:start + c]
        h = seg @ in_weight[e].to(seg.dtype)
        if in_bias is not None:
            h = h + in_bias[e].to(h.dtype)
        h = reference.gated_act(h, act) if gated else reference.activation(act, h.float()).to(h.dtype)
        y = h @ down_weight[e].to(h.dtype)
        if down_bias is not None:
            y = y + down_bias[e].to(y.dtype)
        outs.append(y)
        start += c
    routed_out = torch.cat(outs, dim=0)
    w = gates.reshape(-1).index_select(0, order).to(routed_out.dtype)
    out = torch.zeros(T, H, dtype=routed_out.dtype, device=x.device)
    return out.index_add(0, token_of_route, routed_out * w[:, None]).to(x.dtype)


def embedding(tokens, weight):
    return torch.nn.functional.embedding(tokens, weight)


def linear_cross_entropy(hidden, weight, bias, targets, vocab_size, chunks=4):
    if native_enabled(hidden):
        return _cu().linear_cross_entropy(hidden, weight, bias, targets, vocab_size, chunks)
    if _lib(hidden):
        return _library().linear_cross_entropy(hidden, weight, bias, targets, vocab_size, chunks)
    return reference.linear_cross_entropy(hidden, weight, bias, targets, vocab_size, chunks)


def int4_gemv(x, packed, scales, residual=None, packed_k8=None, norm=None):
    """x `[M<=64, K]` bf16 @ dequant(packed `[K/2, N]`, scales `[K/128, N]`) → `[M, N]` bf16.
    `packed_k8` (`reference.repack_int4_k8(packed)`) selects the tensor-core kernel (M > 4) or the
    one-launch cluster GEMV (M <= 4) on CUDA; `norm=(gamma, eps)` applies RMSNorm to x first."""
    if x.is_cuda:
        return _cu().int4_gemv(x, packed, scales, residual, packed_k8, norm)
    if norm is not None:
        x = rmsnorm(x, norm[0], norm[1])
    y = reference.int4_linear(x, packed, scales)
    return y if residual is None else y + residual


def int4_prefill_usable(x2, packed_k8, d_in: int, d_out: int) -> bool:
    """Whether `int4_matmul` takes this input: CUDA bf16 rows with 16-byte aligned, 8-element strided rows."""
    return bool(x2.is_cuda) and _cu().int4_prefill_usable(x2, packed_k8, d_in, d_out)


def int4_matmul(x, packed_k8, scales, residual=None):
    """x `[M > 64, K]` bf16 @ dequant(W) (+ residual) → `[M, N]` bf16 with the 4-bit weight expanded inside the
    tensor-core kernel (prefill); CUDA only, after `int4_prefill_usable`."""
    return _cu().int4_matmul(x, packed_k8, scales, residual)


def int4_dequant(packed, scales):
    if packed.is_cuda:
        return _cu().int4_dequant(packed, scales)
    return reference.dequantize_int4_g128(packed, scales).to(torch.bfloat16)


class _FakeQuantSTE(torch.autograd.Function):
    """Forward: dequant(quant(w)); backward: identity (straight-through estimator)."""

    @staticmethod
    def forward(ctx, w, fmt):
        return _cu().fake_quant_values(w, fmt)

    @staticmethod
    def backward(ctx, g):
        return g, None


def fake_quant(w, fmt: str):
    """`w + (q(w) - w).detach()` for the binary / ternary g128 codecs: one kernel on CUDA."""
    fmt_dev = "ternary_g128" if fmt == "ternary_entropy_g128" else fmt
    if w.is_cuda and w.dtype in (torch.bfloat16, torch.float32):
        return _FakeQuantSTE.apply(w, fmt_dev)
    return w + (reference.fake_quant_values(w, fmt) - w).detach()


def hquant_dequant(codes, scales, n: int, fmt: str, dtype=torch.bfloat16):
    """HQUANT binary / 2-bit ternary codes (uint8) + fp16 group scales -> `[n]` values."""
    if codes.is_cuda:
        return _cu().hquant_dequant(codes, scales, n, fmt, dtype)
    return reference.hquant_decode(codes, scales, n, fmt).to(dtype)


def hquant_gemv(x, codes, scales, d_out: int, fmt: str, residual=None):
    """x `[M, K]` @ decode(W `[K, d_out]`) from the group codes, d_out % 128 == 0."""
    if x.is_cuda and x.dtype == torch.bfloat16:
        return _cu().hquant_gemv(x, codes, scales, d_out, fmt, residual)
    K = x.shape[-1]
    y = (x.float() @ reference.hquant_decode(codes, scales, K * d_out, fmt).view(K, d_out)).to(x.dtype)
    return y if residual is None else y + residual


def argmax(logits):
    """Greedy token per row, `[rows]` int64."""
    if logits.is_cuda and logits.dim() == 2 and logits.stride(-1) == 1:
        return _cu().argmax_rows(logits)
    return logits.argmax(dim=-1)


def sample_rows(logits, seen=None, uniform=None, penalty=1.0, temperature=0.0, top_k=0):
    """Token selection with repetition penalty / temperature / top-k on the device (CUDA only)."""
    return _cu().sample_rows(logits, seen, uniform, penalty, temperature, top_k)


def seen_bitmap(tokens, vocab, device):
    return _cu().seen_bitmap(tokens, vocab, device)
