"""Plain-PyTorch oracles for every op in `summa_b200.ops`.

Each function here is the numerical definition that the sm_100a kernels are
tested against (fp32 math, no fusion, differentiable through autograd). They are
also the execution path for CPU tensors, which is how the whole model stack runs
in environments without a GPU.

Semantics follow the reference's CPU tensor-op implementations:
selective scan `summa-llm/src/model/scan/reference.rs:53-106`, chunked linear
cross-entropy `summa-llm/src/model/linear_cross_entropy/reference.rs:42-159`,
attention `summa-llm/src/model/fused_attention.rs:150-217`, masked-dense MoE
`summa-llm/src/model/ffn.rs:936-956`, norms `summa-llm/src/model/norm.rs:36-50`.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F


# ------------------------------------------------------------------ norms

def rmsnorm(x: torch.Tensor, gamma: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x / sqrt(mean(x^2) + eps) * gamma, statistics in fp32."""
    xf = x.float()
    inv = torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + eps)
    return (xf * inv * gamma.float()).to(x.dtype)


def layernorm(x: torch.Tensor, gamma: torch.Tensor, beta: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    mu = xf.mean(dim=-1, keepdim=True)
    var = (xf - mu).pow(2).mean(dim=-1, keepdim=True)
    return ((xf - mu) * torch.rsqrt(var + eps) * gamma.float() + beta.float()).to(x.dtype)


# ------------------------------------------------------------------ rope

def rope_table(max_seq_len: int, head_dim: int, theta: float, scaling: Optional[float] = None,
               device=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos/sin tables `[max_seq_len, head_dim // 2]` in fp32.

    Frequency i is `theta ** (-2 i / head_dim)`, divided by `scaling` when given
    (`summa-llm/src/model/transformer.rs:479-485`).
    """
    half = head_dim // 2
    inv = theta ** (-torch.arange(0, half, dtype=torch.float64, device=device) * 2.0 / head_dim)
    if scaling is not None:
        inv = inv / scaling
    pos = torch.arange(max_seq_len, dtype=torch.float64, device=device)
    ang = pos[:, None] * inv[None, :]
    return ang.cos().float(), ang.sin().float()


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, offset: int = 0) -> torch.Tensor:
    """Rotate ADJACENT pairs (x[2i], x[2i+1]) — the interleaved convention.

    x: `[B, S, H, D]`; cos/sin: `[max_seq, D/2]`; positions offset..offset+S-1.
    """
    B, S, H, D = x.shape
    xf = x.float().reshape(B, S, H, D // 2, 2)
    c = cos[offset:offset + S].view(1, S, 1, D // 2)
    s = sin[offset:offset + S].view(1, S, 1, D // 2)
    x0, x1 = xf[..., 0], xf[..., 1]
    out = torch.stack((x0 * c - x1 * s, x0 * s + x1 * c), dim=-1)
    return out.reshape(B, S, H, D).to(x.dtype)


def qk_norm_rope(q, k, q_gamma, k_gamma, eps, cos, sin, offset=0):
    """Optional per-head RMSNorm on q and k (before RoPE), then RoPE on both."""
    if q_gamma is not None:
        q = rmsnorm(q, q_gamma, eps)
        k = rmsnorm(k, k_gamma, eps)
    if cos is not None:
        q = apply_rope(q, cos, sin, offset)
        k = apply_rope(k, cos, sin, offset)
    return q, k


# ------------------------------------------------------------------ attention

def attention_mask(q_len: int, k_len: int, causal: bool, window: Optional[int], q_offset: int,
                   device) -> Optional[torch.Tensor]:
    """Boolean `[q_len, k_len]` mask, True = blocked.

    Query i sits at absolute position `q_offset + i`. Causal blocks j > pos;
    a window W blocks |pos - j| > W (`summa-llm/src/model/attention.rs:288-293`).
    """
    if not causal and window is None:
        return None
    qi = torch.arange(q_len, device=device)[:, None] + q_offset
    kj = torch.arange(k_len, device=device)[None, :]
    blocked = torch.zeros(q_len, k_len, dtype=torch.bool, device=device)
    if causal:
        blocked |= kj > qi
    if window is not None:
        blocked |= (qi - kj).abs() > window
    return blocked


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = True,
              window: Optional[int] = None, scale: Optional[float] = None, q_offset: int = 0,
              return_lse: bool = False):
    """Scaled-dot-product attention with native GQA.

    q `[B, Sq, H, D]`, k/v `[B, Sk, KV, D]`, H % KV == 0. Returns `[B, Sq, H, D]`
    (and the fp32 log-sum-exp `[B, H, Sq]` when asked).
    """
    B, Sq, H, D = q.shape
    Sk, KV = k.shape[1], k.shape[2]
    g = H // KV
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    qf = q.float().permute(0, 2, 1, 3)                       # B H Sq D
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(g, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(g, dim=1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    m = attention_mask(Sq, Sk, causal, window, q_offset, q.device)
    if m is not None:
        s = s.masked_fill(m, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse.unsqueeze(-1))
    o = torch.matmul(p, vf).permute(0, 2, 1, 3).to(q.dtype)
    if return_lse:
        return o, lse
    return o


# ------------------------------------------------------------------ activations

def activation(name: str, x: torch.Tensor) -> torch.Tensor:
    if name in ("swiglu", "silu"):
        return F.silu(x)
    if name == "gelu":
        return F.gelu(x)
    if name in ("gelu_new", "gelu_tanh"):
        return F.gelu(x, approximate="tanh")
    if name == "relu":
        return F.relu(x)
    raise ValueError(f"unknown activation {name}")


def gated_act(x: torch.Tensor, name: str = "swiglu") -> torch.Tensor:
    """`[.., 2I]` laid out as [gate | value] → act(gate) * value, fp32 math."""
    gate, value = x.float().chunk(2, dim=-1)
    return (activation(name, gate) * value).to(x.dtype)


# ------------------------------------------------------------------ cross entropy

def linear_cross_entropy(hidden: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor],
                         targets: torch.Tensor, vocab_size: int, chunks: int = 4,
                         return_logits: bool = False):
    """Mean CE of `hidden @ weight (+bias)` against targets over the LOGICAL vocab.

    hidden `[T, H]`, weight `[H, Vpad]`, targets `[T]` int64. Columns >= vocab_size
    are never read. Rows are processed in `chunks` chunks whose losses are weighted
    by chunk length, which equals the plain mean.
    """
    T = hidden.shape[0]
    rows = max(1, -(-T // max(1, chunks)))
    total = hidden.new_zeros((), dtype=torch.float32)
    all_logits = []
    for start in range(0, T, rows):
        h = hidden[start:start + rows].float()
        logits = h @ weight.float()[:, :vocab_size]
        if bias is not None:
            logits = logits + bias.float()[:vocab_size]
        if return_logits:
            all_logits.append(logits)
        total = total + F.cross_entropy(logits, targets[start:start + rows], reduction="sum")
    loss = total / T
    if return_logits:
        return loss, torch.cat(all_logits, dim=0)
    return loss


# ------------------------------------------------------------------ mamba

def depthwise_conv1d(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor],
                     state: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal depthwise conv over time.

    x `[B, T, C]`, weight `[C, 1, K]`, bias `[C]`; `state` `[B, C, K-1]` holds the
    K-1 inputs that precede x (zeros when None). Output `[B, T, C]`.
    """
    B, T, C = x.shape
    K = weight.shape[-1]
    xt = x.float().transpose(1, 2)                           # B C T
    if state is None:
        xt = F.pad(xt, (K - 1, 0))
    else:
        xt = torch.cat([state.float(), xt], dim=-1)
    y = F.conv1d(xt, weight.float(), bias.float() if bias is not None else None, groups=C)
    return y.transpose(1, 2).to(x.dtype)


def selective_scan(u: torch.Tensor, delta: torch.Tensor, A: torch.Tensor, Bm: torch.Tensor,
                   Cm: torch.Tensor, D: torch.Tensor, h0: Optional[torch.Tensor] = None):
    """Mamba-1 recurrence with softplus applied to `delta` inside the op.

    u, delta `[B, T, C]`; A `[C, N]` (already negative, = -exp(a_log)); Bm, Cm
    `[B, T, N]`; D `[C]`; h0 `[B, C, N]`.
        dt = softplus(delta); h_t = exp(dt*A) h_{t-1} + dt * B_t * u_t
        y_t = <h_t, C_t> + D u_t
    Returns (y `[B, T, C]` in u.dtype, h_T `[B, C, N]` fp32).
    """
    Bsz, T, C = u.shape
    N = A.shape[1]
    uf, dt = u.float(), F.softplus(delta.float())
    Af, Bf, Cf, Df = A.float(), Bm.float(), Cm.float(), D.float()
    h = h0.float() if h0 is not None else uf.new_zeros(Bsz, C, N)
    ys = []
    for t in range(T):
        dA = torch.exp(dt[:, t, :, None] * Af[None])                     # B C N
        dBu = dt[:, t, :, None] * Bf[:, t, None, :] * uf[:, t, :, None]
        h = dA * h + dBu
        ys.append((h * Cf[:, t, None, :]).sum(-1) + Df * uf[:, t])
    y = torch.stack(ys, dim=1)
    return y.to(u.dtype), h


# ------------------------------------------------------------------ MoE

def moe_route(router_logits: torch.Tensor, top_k: int):
    """Top-k on raw logits, softmax over the selected logits (fp32).

    Returns (indices `[T, k]` int64, gates `[T, k]` fp32).
    """
    vals, idx = torch.topk(router_logits.float(), top_k, dim=-1)
    gates = torch.softmax(vals, dim=-1)
    return idx, gates


def route_plan(indices: torch.Tensor, num_experts: int):
    """Stable sort of the flattened (token, slot) routes by expert.

    Returns `order` (route id at each sorted position), `inverse` (sorted position
    of each route id) and `counts` `[E]`. Route id = token * k + slot.
    """
    flat = indices.reshape(-1)
    order = torch.sort(flat, stable=True).indices
    inverse = torch.empty_like(order)
    inverse[order] = torch.arange(order.numel(), device=order.device)
    counts = torch.bincount(flat, minlength=num_experts)
    return order, inverse, counts


def moe_aux_loss(router_logits: torch.Tensor, indices: torch.Tensor, num_experts: int,
                 lb_weight: float, z_weight: float) -> torch.Tensor:
    """`lb_w * E * sum_e mean(p_e) * frac_e + z_w * mean(logsumexp^2)`."""
    lf = router_logits.float()
    aux = lf.new_zeros(())
    if lb_weight > 0.0:
        probs = torch.softmax(lf, dim=-1).mean(dim=0)
        frac = torch.bincount(indices.reshape(-1), minlength=num_experts).float() / indices.numel()
        aux = aux + lb_weight * num_experts * (probs * frac).sum()
    if z_weight > 0.0:
        aux = aux + z_weight * torch.logsumexp(lf, dim=-1).pow(2).mean()
    return aux


def moe_experts_dense(x: torch.Tensor, indices: torch.Tensor, gates: torch.Tensor,
                      in_weight: torch.Tensor, down_weight: torch.Tensor,
                      in_bias: Optional[torch.Tensor], down_bias: Optional[torch.Tensor],
                      act: str, gated: bool) -> torch.Tensor:
    """Masked-dense oracle: every expert sees every token, outputs are gated.

    x `[T, H]`; in_weight `[E, H, 2I or I]`; down_weight `[E, I, H]`.
    """
    T, H = x.shape
    E = in_weight.shape[0]
    out = x.new_zeros(T, H, dtype=torch.float32)
    xf = x.float()
    for e in range(E):
        w = (gates * (indices == e)).sum(dim=-1)              # [T]
        h = xf @ in_weight[e].float()
        if in_bias is not None:
            h = h + in_bias[e].float()
        h = gated_act(h, act) if gated else activation(act, h)
        y = h @ down_weight[e].float()
        if down_bias is not None:
            y = y + down_bias[e].float()
        out = out + y * w[:, None]
    return out.to(x.dtype)


# ------------------------------------------------------------------ quantisation

def quantize_int4_g128(w: torch.Tensor, group: int = 128):
    """Asymmetric-free (symmetric) 4-bit group quantisation along the input dim.

    w `[K, N]` (d_in, d_out). Groups run over K for each output column. Returns
    packed `[K // 2, N]` uint8 (low nibble = even k) and bf16 scales `[K // group, N]`.
    q in [-8, 7], w ≈ q * scale.
    """
    K, N = w.shape
    assert K % group == 0
    wf = w.float().view(K // group, group, N)
    scale = (wf.abs().amax(dim=1) / 7.0).clamp_min(1e-8)
    scale = scale.to(torch.bfloat16)
    q = torch.round(wf / scale.float()[:, None, :]).clamp_(-8, 7).to(torch.int8).view(K, N)
    u = (q + 8).to(torch.uint8)
    packed = u[0::2] | (u[1::2] << 4)
    return packed.contiguous(), scale.contiguous()


def repack_int4_k8(packed: torch.Tensor) -> torch.Tensor:
    """Canonical `[K/2, N]` bytes -> `[K/8, N]` int32 words for the tensor-core decode kernel: a
    word holds the 8 codes of 8 consecutive k of one column, even k in the low half-word and odd
    k in the high half-word (nibble i of each half = the pair (2i, 2i+1))."""
    K2, N = packed.shape
    assert K2 % 4 == 0
    b = packed.view(K2 // 4, 4, N).to(torch.int64)
    word = torch.zeros(K2 // 4, N, dtype=torch.int64, device=packed.device)
    for i in range(4):
        word |= (b[:, i] & 0xF) << (4 * i)
        word |= (b[:, i] >> 4) << (16 + 4 * i)
    word = torch.where(word >= (1 << 31), word - (1 << 32), word)
    return word.to(torch.int32).contiguous()


def dequantize_int4_g128(packed: torch.Tensor, scale: torch.Tensor, group: int = 128) -> torch.Tensor:
    K2, N = packed.shape
    K = K2 * 2
    lo = (packed & 0xF).to(torch.int16) - 8
    hi = (packed >> 4).to(torch.int16) - 8
    q = torch.stack((lo, hi), dim=1).reshape(K, N).float()
    s = scale.float().repeat_interleave(group, dim=0)
    return q * s


def int4_linear(x: torch.Tensor, packed: torch.Tensor, scale: torch.Tensor, group: int = 128) -> torch.Tensor:
    return (x.float() @ dequantize_int4_g128(packed, scale, group)).to(x.dtype)


def hquant_decode(codes: torch.Tensor, scales: torch.Tensor, n: int, fmt: str, group: int = 128) -> torch.Tensor:
    """HQUANT binary / 2-bit ternary group codes -> `[n]` fp32 (`summa-train/src/quantization.rs:447-501`):
    binary bit 1 -> +scale, bit 0 -> -scale (LSB first); ternary code 0 -> -scale, 1 -> 0, 2 -> +scale."""
    sc = scales.float()
    groups = sc.numel()
    dev = codes.device
    if fmt == "binary_g128":
        sh = torch.arange(8, dtype=torch.uint8, device=dev)
        bits = ((codes.view(groups, group // 8, 1) >> sh) & 1).reshape(groups, group)
        vals = (bits.float() * 2 - 1) * sc[:, None]
    elif fmt == "ternary_g128":
        sh = torch.arange(4, dtype=torch.uint8, device=dev) * 2
        c = ((codes.view(groups, group // 4, 1) >> sh) & 3).reshape(groups, group)
        vals = (c.float() - 1) * sc[:, None]
    else:
        raise ValueError(f"no device decode for {fmt}")
    return vals.reshape(-1)[:n]


def fake_quant_values(w: torch.Tensor, fmt: str, group: int = 128) -> torch.Tensor:
    """dequant(quant(w)) with the codec's scale estimators, groups over the flattened tensor
    (`summa-train/src/quantization.rs:691-771,934-978`)."""
    n = w.numel()
    groups = -(-n // group)
    flat = torch.zeros(groups * group, device=w.device, dtype=torch.float32)
    flat[:n] = w.detach().float().reshape(-1)
    G = flat.view(groups, group)
    if fmt == "binary_g128":
        cnt = torch.full((groups, 1), float(group), device=w.device)
        if n % group:
            cnt[-1, 0] = n % group
        scale = G.abs().sum(dim=1, keepdim=True) / cnt
        q = torch.where(G >= 0, scale, -scale)
    elif fmt in ("ternary_g128", "ternary_entropy_g128"):
        mag, _ = G.abs().sort(dim=1, descending=True)
        csum = mag.cumsum(dim=1)
        k = torch.arange(1, group + 1, device=w.device, dtype=torch.float32)
        best = (csum * csum / k).argmax(dim=1, keepdim=True)
        scale = csum.gather(1, best) / (best + 1).float()
        thresh = mag.gather(1, best)
        q = torch.where(G.abs() >= thresh, torch.sign(G) * scale, torch.zeros_like(G))
    else:
        raise ValueError(f"unknown format {fmt}")
    return q.reshape(-1)[:n].view(w.shape).to(w.dtype)
