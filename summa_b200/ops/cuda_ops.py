"""CUDA execution path of the op layer: autograd Functions over the native kernels.

Each Function's forward and backward launch hand-written sm_100a kernels from
`libsumma_b200.so`; PyTorch supplies only tensor allocation and the autograd tape.
Weights carrying a `main_grad` attribute (an fp32 view into a flat gradient
buffer, see `summa_b200.parallel.dp`) get their weight gradient accumulated in
place by the GEMM epilogue and receive `None` from autograd.
"""
from __future__ import annotations

import ctypes
import os
import math
from typing import Optional, Tuple

import torch

from . import native as N
from . import reference

BF16 = torch.bfloat16


def _rows(x: torch.Tensor) -> Tuple[torch.Tensor, int]:
    """2-D row view `[rows, last]` with unit inner stride; copies only when needed."""
    last = x.shape[-1]
    if x.dim() == 2 and x.stride(1) == 1 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0:
        return x, x.stride(0)
    if x.is_contiguous() and x.data_ptr() % 16 == 0:
        return x.view(-1, last), last
    # strided higher-rank views: collapse when all leading dims share one row stride
    if x.stride(-1) == 1 and x.dim() >= 2 and x.data_ptr() % 16 == 0:
        ok = True
        rs = x.stride(-2)
        expect = rs * x.shape[-2]
        for d in range(x.dim() - 3, -1, -1):
            if x.shape[d] != 1 and x.stride(d) != expect:
                ok = False
                break
            expect = expect * x.shape[d] if x.shape[d] != 1 else expect
        if ok and rs % 8 == 0:
            rows = x.numel() // last
            return torch.as_strided(x, (rows, last), (rs, 1)), rs
    c = x.contiguous()
    return c.view(-1, last), last


def gemm(A: torch.Tensor, B: torch.Tensor, M: int, Nn: int, K: int, lda: int, ldb: int, a_mn: bool, b_mn: bool,
         out: Optional[torch.Tensor] = None, out_dtype=BF16, accumulate: bool = False,
         bias: Optional[torch.Tensor] = None, tile_n: int = 0) -> torch.Tensor:
    """C[M,N] = A·B on the tcgen05 GEMM. See `csrc/gemm.cu` for the layout flags."""
    if out is None:
        out = torch.empty(M, Nn, device=A.device, dtype=out_dtype)
    assert out.stride(-1) == 1
    mode = 0 if out.dtype == BF16 else (2 if accumulate else 1)
    assert not (accumulate and out.dtype == BF16), "accumulation needs an fp32 output"
    if bias is not None and bias.dtype not in (BF16, torch.float32):
        bias = bias.float()
    N.call("sb_gemm_bf16", A.data_ptr(), B.data_ptr(), out.data_ptr(), N.ptr(bias),
           1 if (bias is not None and bias.dtype == BF16) else 0, M, Nn, K, lda, ldb, out.stride(0),
           1 if a_mn else 0, 1 if b_mn else 0, mode, tile_n, N.stream())
    return out


N.register("sb_gemm_bf16_batched", [N.P, N.P, N.P, N.I, N.L, N.L, N.L, N.I, N.I, N.I, N.I, N.I, N.I, N.I, N.I, N.I, N.P])


def bmm(A: torch.Tensor, B: torch.Tensor, trans_b: bool = False, out_dtype=BF16, trans_a: bool = False) -> torch.Tensor:
    """Batched `op(A[b]) @ op(B[b])` on the paired-CTA tcgen05 kernel, op = transpose with `trans_a` / `trans_b`
    (a layout flag of the kernel, no copy). A `[batch, M, K]` (`[batch, K, M]` with `trans_a`), B `[batch, K, N]`
    (`[batch, N, K]` with `trans_b`), contiguous bf16; returns `[batch, M, N]`."""
    assert A.dim() == 3 and B.dim() == 3 and A.dtype == BF16 and B.dtype == BF16
    A, B = A.contiguous(), B.contiguous()
    nb = A.shape[0]
    M, K = (A.shape[2], A.shape[1]) if trans_a else (A.shape[1], A.shape[2])
    Nn = B.shape[1] if trans_b else B.shape[2]
    assert B.shape[0] == nb and (B.shape[2] if trans_b else B.shape[1]) == K
    out = torch.empty(nb, M, Nn, device=A.device, dtype=out_dtype)
    mode = 0 if out_dtype == BF16 else 1
    N.call("sb_gemm_bf16_batched", A.data_ptr(), B.data_ptr(), out.data_ptr(), nb, M * K, B.shape[1] * B.shape[2],
           M * Nn, M, Nn, K, A.shape[2], B.shape[2], Nn, 1 if trans_a else 0, 0 if trans_b else 1, mode, N.stream())
    return out


def _weight_layout(w: torch.Tensor):
    """(b_mn, ld) for a logical `[K, N]` weight that is row-major or a transposed view."""
    if w.stride(1) == 1:
        return True, w.stride(0)
    assert w.stride(0) == 1, "weight must be row-major or a transposed view"
    return False, w.stride(1)


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias):
        K, Nn = weight.shape
        w = weight if weight.dtype == BF16 else weight.to(BF16)
        x2, lda = _rows(x)
        M = x2.shape[0]
        b_mn, ldb = _weight_layout(w)
        # the output is allocated in its final shape (not returned as a view of a 2-D buffer), so that a
        # following op may rotate / normalise it in place
        y = torch.empty(*x.shape[:-1], Nn, device=x.device, dtype=BF16)
        gemm(x2, w, M, Nn, K, lda, ldb, False, b_mn, out=y.view(M, Nn), bias=bias)
        ctx.save_for_backward(x, weight, bias)
        ctx.w_cast = w if w is not weight else None
        return y

    @staticmethod
    def backward(ctx, dy):
        x, weight, bias = ctx.saved_tensors
        K, Nn = weight.shape
        w = ctx.w_cast if ctx.w_cast is not None else weight
        dy2, ldd = _rows(dy)
        M = dy2.shape[0]
        b_mn, ldb = _weight_layout(w)
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            # dx[M,K] = dy[M,N] · W^T : contraction over N
            dx = gemm(dy2, w, M, K, Nn, ldd, ldb, False, not b_mn).view(x.shape)
        if ctx.needs_input_grad[1]:
            x2, lda = _rows(x)
            main = getattr(weight, "main_grad", None)
            if b_mn:   # memory [K, N]: dW = x^T · dy
                if main is not None:
                    gemm(x2, dy2, K, Nn, M, lda, ldd, True, True, out=main, accumulate=True)
                else:
                    dw = gemm(x2, dy2, K, Nn, M, lda, ldd, True, True,
                              out_dtype=BF16 if weight.dtype == BF16 else torch.float32)
            else:      # memory [N, K] (transposed view): store dW^T = dy^T · x
                if main is not None:
                    gemm(dy2, x2, Nn, K, M, ldd, lda, True, True, out=main, accumulate=True)
                else:
                    dwt = gemm(dy2, x2, Nn, K, M, ldd, lda, True, True,
                               out_dtype=BF16 if weight.dtype == BF16 else torch.float32)
                    dw = dwt.t()
        if bias is not None and ctx.needs_input_grad[2]:
            db = dy2.float().sum(dim=0).to(bias.dtype)
        return dx, dw, db


def linear(x, weight, bias=None):
    return _Linear.apply(x, weight, bias)


# ------------------------------------------------------------------ RMSNorm

def _gamma32(g: torch.Tensor) -> torch.Tensor:
    return g if g.dtype == torch.float32 else g.float()


class _RmsNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, residual, gamma, eps):
        H = x.shape[-1]
        xc = x.contiguous()
        rows = xc.numel() // H
        y = torch.empty_like(xc)
        rstd = torch.empty(rows, device=x.device, dtype=torch.float32)
        g = _gamma32(gamma)
        if residual is not None:
            rc = residual.contiguous()
            s = torch.empty_like(xc)
            N.call("sb_rmsnorm_fwd", xc.data_ptr(), rc.data_ptr(), g.data_ptr(), y.data_ptr(), s.data_ptr(),
                   rstd.data_ptr(), rows, H, eps, N.stream())
            ctx.save_for_backward(s, gamma, rstd)
            ctx.has_res = True
            return y, s
        N.call("sb_rmsnorm_fwd", xc.data_ptr(), None, g.data_ptr(), y.data_ptr(), None, rstd.data_ptr(), rows, H,
               eps, N.stream())
        ctx.save_for_backward(xc, gamma, rstd)
        ctx.has_res = False
        return y

    @staticmethod
    def backward(ctx, dy, dsum=None):
        x, gamma, rstd = ctx.saved_tensors
        H = x.shape[-1]
        rows = x.numel() // H
        g = _gamma32(gamma)
        dyc = dy.contiguous()
        dx = torch.empty_like(x)
        main = getattr(gamma, "main_grad", None)
        dgamma = main if main is not None else torch.zeros(H, device=x.device, dtype=torch.float32)
        dsc = dsum.contiguous() if (ctx.has_res and dsum is not None) else None
        N.call("sb_rmsnorm_bwd", x.data_ptr(), dyc.data_ptr(), N.ptr(dsc), g.data_ptr(), rstd.data_ptr(),
               dx.data_ptr(), dgamma.data_ptr(), rows, H, N.stream())
        dg = None if main is not None else dgamma.to(gamma.dtype)
        if ctx.has_res:
            return dx, dx, dg, None
        return dx, None, dg, None


def rmsnorm(x, gamma, eps):
    return _RmsNorm.apply(x, None, gamma, eps)


def add_rmsnorm(x, residual, gamma, eps):
    return _RmsNorm.apply(x, residual, gamma, eps)


# ------------------------------------------------------------------ SwiGLU / mul_silu

class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        x2, ldx = _rows(x)
        rows, two_i = x2.shape
        I = two_i // 2
        y = torch.empty(rows, I, device=x.device, dtype=BF16)
        N.call("sb_swiglu_fwd", x2.data_ptr(), y.data_ptr(), rows, I, ldx, N.stream())
        ctx.save_for_backward(x)
        return y.view(*x.shape[:-1], I)

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        x2, ldx = _rows(x)
        rows, two_i = x2.shape
        I = two_i // 2
        dyc = dy.contiguous()
        dx = torch.empty(rows, two_i, device=x.device, dtype=BF16)
        N.call("sb_swiglu_bwd", x2.data_ptr(), dyc.data_ptr(), dx.data_ptr(), rows, I, ldx, N.stream())
        return dx.view(x.shape)


def swiglu(x):
    return _SwiGLU.apply(x)


N.register("sb_act_fwd", [N.P, N.P, N.L, N.I, N.L, N.I, N.I, N.P])
N.register("sb_act_bwd", [N.P, N.P, N.P, N.L, N.I, N.L, N.I, N.I, N.P])
N.register("sb_layernorm_fwd", [N.P, N.P, N.P, N.P, N.P, N.P, N.I, N.I, N.F, N.P])
N.register("sb_layernorm_bwd", [N.P] * 8 + [N.I, N.I, N.P])

ACT_IDS = {"silu": 0, "swiglu": 0, "gelu": 1, "geglu": 1, "gelu_new": 2, "gelu_tanh": 2, "relu": 3, "reglu": 3}


class _Act(torch.autograd.Function):
    """act(x) (`gated=False`) or act(gate) * value for x = [gate | value] (`gated=True`), act in `ACT_IDS`."""

    @staticmethod
    def forward(ctx, x, act: int, gated: bool):
        x2, ldx = _rows(x)
        rows, width = x2.shape
        I = width // 2 if gated else width
        y = torch.empty(rows, I, device=x.device, dtype=BF16)
        N.call("sb_act_fwd", x2.data_ptr(), y.data_ptr(), rows, I, ldx, act, 1 if gated else 0, N.stream())
        ctx.save_for_backward(x)
        ctx.act, ctx.gated = act, gated
        return y.view(*x.shape[:-1], I)

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        x2, ldx = _rows(x)
        rows, width = x2.shape
        I = width // 2 if ctx.gated else width
        dyc = dy.contiguous()
        dx = torch.empty(rows, width, device=x.device, dtype=BF16)
        N.call("sb_act_bwd", x2.data_ptr(), dyc.data_ptr(), dx.data_ptr(), rows, I, ldx, ctx.act,
               1 if ctx.gated else 0, N.stream())
        return dx.view(x.shape), None, None


def act(x, name: str, gated: bool):
    return _Act.apply(x, ACT_IDS[name], gated)


class _LayerNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gamma, beta, eps):
        x2, ldx = _rows(x)
        if ldx != x2.shape[1]:
            x2 = x2.contiguous()
        rows, H = x2.shape
        g32 = _gamma32(gamma)
        b32 = _gamma32(beta) if beta is not None else None
        y = torch.empty(rows, H, device=x.device, dtype=BF16)
        mean = torch.empty(rows, device=x.device, dtype=torch.float32)
        rstd = torch.empty(rows, device=x.device, dtype=torch.float32)
        N.call("sb_layernorm_fwd", x2.data_ptr(), g32.data_ptr(), N.ptr(b32), y.data_ptr(), mean.data_ptr(),
               rstd.data_ptr(), rows, H, float(eps), N.stream())
        ctx.save_for_backward(x2, gamma, beta, mean, rstd)
        ctx.shape = x.shape
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, gamma, beta, mean, rstd = ctx.saved_tensors
        rows, H = x2.shape
        dyc = dy.reshape(rows, H).contiguous()
        dx = torch.empty(rows, H, device=dyc.device, dtype=BF16)
        need_p = ctx.needs_input_grad[1] or (beta is not None and ctx.needs_input_grad[2])
        dg = torch.zeros(H, device=dyc.device, dtype=torch.float32) if need_p else None
        db = torch.zeros(H, device=dyc.device, dtype=torch.float32) if (need_p and beta is not None) else None
        N.call("sb_layernorm_bwd", x2.data_ptr(), dyc.data_ptr(), _gamma32(gamma).data_ptr(), mean.data_ptr(),
               rstd.data_ptr(), dx.data_ptr(), N.ptr(dg), N.ptr(db), rows, H, N.stream())
        return (dx.view(ctx.shape), dg.to(gamma.dtype) if dg is not None else None,
                db.to(beta.dtype) if db is not None else None, None)


def layernorm(x, gamma, beta, eps):
    return _LayerNorm.apply(x, gamma, beta, eps)


class _MulSilu(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y, z):
        y2, ldy = _rows(y)
        z2, ldz = _rows(z)
        rows, C = y2.shape
        out = torch.empty(rows, C, device=y.device, dtype=BF16)
        N.call("sb_mul_silu_fwd", y2.data_ptr(), z2.data_ptr(), out.data_ptr(), rows, C, ldy, ldz, N.stream())
        ctx.save_for_backward(y, z)
        return out.view(y.shape)

    @staticmethod
    def backward(ctx, dout):
        y, z = ctx.saved_tensors
        y2, ldy = _rows(y)
        z2, ldz = _rows(z)
        rows, C = y2.shape
        d = dout.contiguous()
        dy = torch.empty(rows, C, device=y.device, dtype=BF16)
        dz = torch.empty(rows, C, device=y.device, dtype=BF16)
        N.call("sb_mul_silu_bwd", y2.data_ptr(), z2.data_ptr(), d.data_ptr(), dy.data_ptr(), dz.data_ptr(), rows, C,
               ldy, ldz, C, C, N.stream())
        return dy.view(y.shape), dz.view(z.shape)


def mul_silu(y, z):
    return _MulSilu.apply(y, z)


# ------------------------------------------------------------------ q/k norm + RoPE

class _QkRope(torch.autograd.Function):
    """Operates on the packed qkv activation `[B, S, (Hq + 2 Hkv) * D]`; returns a new
    packed tensor whose q and k heads are normalised + rotated and whose v heads are
    copied through untouched by reusing the input storage when no norm is needed."""

    @staticmethod
    def forward(ctx, qkv, q_gamma, k_gamma, eps, cos, sin, Hq, Hkv, D, offset):
        B, S, W = qkv.shape
        in_place_ok = qkv.is_contiguous() and not (qkv.is_leaf and qkv.requires_grad)
        qkv = qkv.contiguous()
        T = B * S
        norm = q_gamma is not None
        if not norm and in_place_ok:
            # Pure rotation: rotate the q and k heads where they are (the projection that produced `qkv`
            # keeps nothing of its output for backward), so the v heads are neither read nor copied.
            out = qkv
            ctx.mark_dirty(qkv)
        else:
            out = torch.empty_like(qkv)
            # v heads pass through
            out.view(T, W)[:, (Hq + Hkv) * D:].copy_(qkv.view(T, W)[:, (Hq + Hkv) * D:])
        rstd = torch.empty(T * (Hq + Hkv), device=qkv.device, dtype=torch.float32) if norm else None
        qg = _gamma32(q_gamma) if norm else None
        kg = _gamma32(k_gamma) if norm else None
        N.call("sb_qk_rope", qkv.data_ptr(), out.data_ptr(), None, N.ptr(qg), N.ptr(kg), N.ptr(rstd), None, None,
               cos.data_ptr(), sin.data_ptr(), T, S, Hq, Hkv, D, W, offset, eps, 0, N.stream())
        ctx.save_for_backward(qkv if norm else None, q_gamma, k_gamma, rstd, cos, sin)
        ctx.meta = (B, S, W, Hq, Hkv, D, offset, eps)
        return out

    @staticmethod
    def backward(ctx, dout):
        pre, q_gamma, k_gamma, rstd, cos, sin = ctx.saved_tensors
        B, S, W, Hq, Hkv, D, offset, eps = ctx.meta
        T = B * S
        norm = q_gamma is not None
        dout = dout.contiguous()
        dqkv = dout if not norm else torch.empty_like(dout)
        if norm:
            dqkv.view(T, W)[:, (Hq + Hkv) * D:].copy_(dout.view(T, W)[:, (Hq + Hkv) * D:])
        qg = _gamma32(q_gamma) if norm else None
        kg = _gamma32(k_gamma) if norm else None
        dqg = torch.zeros(D, device=dout.device, dtype=torch.float32) if norm else None
        dkg = torch.zeros(D, device=dout.device, dtype=torch.float32) if norm else None
        N.call("sb_qk_rope", dout.data_ptr(), dqkv.data_ptr(), N.ptr(pre), N.ptr(qg), N.ptr(kg), N.ptr(rstd),
               N.ptr(dqg), N.ptr(dkg), cos.data_ptr(), sin.data_ptr(), T, S, Hq, Hkv, D, W, offset, eps, 1,
               N.stream())
        return (dqkv, dqg.to(q_gamma.dtype) if norm else None, dkg.to(k_gamma.dtype) if norm else None,
                None, None, None, None, None, None, None)


def qkv_rope(qkv, q_gamma, k_gamma, eps, cos, sin, Hq, Hkv, D, offset=0):
    return _QkRope.apply(qkv, q_gamma, k_gamma, eps, cos, sin, Hq, Hkv, D, offset)


def qk_norm_rope(q, k, q_gamma, k_gamma, eps, cos, sin, offset=0):
    """Generic entry (separate q / k tensors): packs, runs the fused kernel, unpacks."""
    B, S, Hq, D = q.shape
    Hkv = k.shape[2]
    if D not in (64, 128):
        return reference.qk_norm_rope(q, k, q_gamma, k_gamma, eps, cos, sin, offset)
    packed = torch.cat([q.reshape(B, S, Hq * D), k.reshape(B, S, Hkv * D)], dim=-1)
    out = _QkRope.apply(packed, q_gamma, k_gamma, eps, cos, sin, Hq, Hkv, D, offset)
    return (out[..., :Hq * D].unflatten(-1, (Hq, D)), out[..., Hq * D:].unflatten(-1, (Hkv, D)))


# ------------------------------------------------------------------ attention

import ctypes as _ct

N.register("sb_attention_fwd", [N.P, N.P, N.P, N.P, N.P, N.I, N.I, N.I, N.I, N.I, N.I, N.P, N.P, N.P, N.P,
                                N.I, N.I, N.I, N.F, N.P])


def _bshd_strides(t: torch.Tensor):
    """(batch, seq, head) element strides of a `[B, S, H, D]` view with contiguous D."""
    assert t.stride(3) == 1, "head_dim must be contiguous"
    return (_ct.c_long * 3)(t.stride(0), t.stride(1), t.stride(2))


def _tma_ok(t: torch.Tensor) -> bool:
    return (t.stride(3) == 1 and t.data_ptr() % 16 == 0 and all(s % 8 == 0 for s in t.stride()[:3]))


def attention_fwd(q, k, v, causal=True, window=None, q_offset=0, scale=None, need_lse=True):
    """Flash attention forward. q `[B,Sq,Hq,D]`, k/v `[B,Sk,Hkv,D]` (any strides with
    contiguous D, 16-byte aligned). Returns (o `[B,Sq,Hq,D]`, lse `[B,Hq,Sq]` fp32)."""
    B, Sq, Hq, D = q.shape
    Sk, Hkv = k.shape[1], k.shape[2]
    q = q if _tma_ok(q) else q.contiguous()
    k = k if _tma_ok(k) else k.contiguous()
    v = v if _tma_ok(v) else v.contiguous()
    o = torch.empty(B, Sq, Hq, D, device=q.device, dtype=BF16)
    lse = torch.empty(B, Hq, Sq, device=q.device, dtype=torch.float32) if need_lse else None
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    N.call("sb_attention_fwd", q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), N.ptr(lse), B, Hq, Hkv, Sq, Sk,
           D, _bshd_strides(q), _bshd_strides(k), _bshd_strides(v), _bshd_strides(o), 1 if causal else 0,
           -1 if window is None else int(window), int(q_offset), float(scale), N.stream())
    return o, lse

N.register("sb_attention_bwd", [N.P] * 10 + [N.I] * 6 + [N.P] * 8 + [N.I, N.I, N.I, N.F, N.P])


def attention_bwd(q, k, v, o, dout, lse, dq, dk, dv, causal, window, q_offset, scale=None):
    """Writes dq/dk/dv (bf16, possibly strided views) for `attention_fwd`'s inputs."""
    B, Sq, Hq, D = q.shape
    Sk, Hkv = k.shape[1], k.shape[2]
    dout = dout if _tma_ok(dout) else dout.contiguous()
    delta = torch.empty(2 * B * Hq * (-(-Sq // 64) * 64), device=q.device, dtype=torch.float32)
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    N.call("sb_attention_bwd", q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), dout.data_ptr(),
           lse.data_ptr(), delta.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), B, Hq, Hkv, Sq, Sk, D,
           _bshd_strides(q), _bshd_strides(k), _bshd_strides(v), _bshd_strides(o), _bshd_strides(dout),
           _bshd_strides(dq), _bshd_strides(dk), _bshd_strides(dv), 1 if causal else 0,
           -1 if window is None else int(window), int(q_offset), float(scale), N.stream())


class _Attention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal, window, q_offset):
        q = q if _tma_ok(q) else q.contiguous()
        k = k if _tma_ok(k) else k.contiguous()
        v = v if _tma_ok(v) else v.contiguous()
        need = q.requires_grad or k.requires_grad or v.requires_grad
        o, lse = attention_fwd(q, k, v, causal, window, q_offset, need_lse=True)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.meta = (causal, window, q_offset)
        return o

    @staticmethod
    def backward(ctx, dout):
        q, k, v, o, lse = ctx.saved_tensors
        causal, window, q_offset = ctx.meta
        dq, dk, dv = torch.empty_like(q, memory_format=torch.contiguous_format), \
            torch.empty_like(k, memory_format=torch.contiguous_format), \
            torch.empty_like(v, memory_format=torch.contiguous_format)
        attention_bwd(q, k, v, o, dout, lse, dq, dk, dv, causal, window, q_offset)
        return dq, dk, dv, None, None, None


def attention(q, k, v, causal=True, window=None, q_offset=0):
    D = q.shape[-1]
    if D not in (64, 128):
        return reference.attention(q, k, v, causal, window, None, q_offset)
    if q.shape[1] <= 8 and not torch.is_grad_enabled():
        return decode_attention(q, k, v, causal, window, q_offset)
    return _Attention.apply(q, k, v, causal, window, q_offset)


N.register("sb_attention_decode", [N.P] * 5 + [N.I] * 6 + [N.P] * 4 + [N.F, N.I, N.P])
N.register("sb_attention_decode_workspace", [N.I, N.I, N.I], restype=ctypes.c_long)
N.register("sb_attention_decode_splits", [N.I, N.I, N.I])
_decode_ws = {}


def decode_attention(q, k, v, causal, window, q_offset, scale=None):
    """Few-query attention over a long cache (decode steps). One query token per sequence with
    head_dim 128 that sees the whole cache runs the split-KV tcgen05 kernel (the cache streams
    through TMA once for all query heads of a kv head); everything else uses the general kernel."""
    B, Sq, Hq, D = q.shape
    Sk, Hkv = k.shape[1], k.shape[2]
    sees_all = (not causal) or q_offset + Sq - 1 >= Sk - 1
    if not (Sq == 1 and D == 128 and window is None and sees_all and Hq // Hkv <= 8 and _tma_ok(k) and _tma_ok(v)):
        return _Attention.apply(q, k, v, causal, window, q_offset)
    q = q if q.stride(-1) == 1 and q.stride(2) % 8 == 0 else q.contiguous()
    o = torch.empty(B, 1, Hq, D, device=q.device, dtype=BF16)
    splits = N.call_value("sb_attention_decode_splits", B, Hkv, Sk)
    need = N.call_value("sb_attention_decode_workspace", B, Hkv, splits)
    key = (q.device.index, torch.cuda.current_stream().cuda_stream)
    ws = _decode_ws.get(key)
    if ws is None or ws.numel() < need:
        ws = torch.empty(max(need, 1 << 20), device=q.device, dtype=torch.float32)
        _decode_ws[key] = ws
    cap = Sk          # the views passed in are already cut to the live prefix
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    qs = (ctypes.c_long * 2)(q.stride(0), q.stride(2))
    os_ = (ctypes.c_long * 2)(o.stride(0), o.stride(2))
    N.call("sb_attention_decode", q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), ws.data_ptr(), B, Hq, Hkv, Sk,
           cap, D, qs, _bshd_strides(k), _bshd_strides(v), os_, float(scale), splits, N.stream())
    return o


class _PackedAttention(torch.autograd.Function):
    """Attention straight over the packed (already rotated) qkv activation
    `[B, S, (Hq + 2 Hkv) * D]`; the backward writes one packed dqkv buffer, so neither
    direction splits, copies or concatenates q/k/v."""

    @staticmethod
    def forward(ctx, qkv, Hq, Hkv, D, causal, window):
        qkv = qkv.contiguous()
        q, k, v = _split_packed(qkv, Hq, Hkv, D)
        o, lse = attention_fwd(q, k, v, causal, window, 0)
        ctx.save_for_backward(qkv, o, lse)
        ctx.meta = (Hq, Hkv, D, causal, window)
        return o

    @staticmethod
    def backward(ctx, dout):
        qkv, o, lse = ctx.saved_tensors
        Hq, Hkv, D, causal, window = ctx.meta
        q, k, v = _split_packed(qkv, Hq, Hkv, D)
        dqkv = torch.empty_like(qkv)
        dq, dk, dv = _split_packed(dqkv, Hq, Hkv, D)
        attention_bwd(q, k, v, o, dout, lse, dq, dk, dv, causal, window, 0)
        return dqkv, None, None, None, None, None


def _split_packed(qkv, Hq, Hkv, D):
    q = qkv[..., :Hq * D].unflatten(-1, (Hq, D))
    k = qkv[..., Hq * D:(Hq + Hkv) * D].unflatten(-1, (Hkv, D))
    v = qkv[..., (Hq + Hkv) * D:].unflatten(-1, (Hkv, D))
    return q, k, v


def packed_attention(qkv, Hq, Hkv, D, causal=True, window=None):
    return _PackedAttention.apply(qkv, Hq, Hkv, D, causal, window)


# ------------------------------------------------------------------ fused linear cross-entropy

N.register("sb_ce_rows", [N.P, N.P, N.P, N.P, N.I, N.I, N.I, N.L, N.L, N.F, N.P])

_CE_MAX_CHUNK_ROWS = 8192


class _LinearCrossEntropy(torch.autograd.Function):
    """mean CE(hidden @ W + b, targets) without a full `[T, V]` logits tensor.

    Row chunks: logits chunk (tcgen05 GEMM, fp32) → row kernel (loss + bf16 softmax
    gradient, already scaled by 1/T) → dH chunk = G·W^T and dW += H^T·G (tcgen05 GEMMs).
    The gradients are produced in the forward pass and scaled by the incoming gradient
    in backward, so the logits are never recomputed.
    """

    @staticmethod
    def forward(ctx, hidden, weight, bias, targets, vocab_size, chunks):
        T, H = hidden.shape
        Vpad = weight.shape[1]
        w = weight if weight.dtype == BF16 else weight.to(BF16)
        b_mn, ldb = _weight_layout(w)
        h2, ldh = _rows(hidden)
        need_grad = hidden.requires_grad or weight.requires_grad
        rows_per = min(_CE_MAX_CHUNK_ROWS, max(1, -(-T // max(1, chunks))))
        rows_per = -(-rows_per // 128) * 128
        row_loss = torch.empty(T, device=hidden.device, dtype=torch.float32)
        logits = torch.empty(min(rows_per, T), Vpad, device=hidden.device, dtype=torch.float32)
        dh = dw = db = None
        if need_grad:
            G = torch.empty(min(rows_per, T), Vpad, device=hidden.device, dtype=BF16)
            dh = torch.empty(T, H, device=hidden.device, dtype=BF16)
            # weight gradient in the weight's MEMORY layout, fp32
            dw = torch.zeros(weight.shape if b_mn else (Vpad, H), device=hidden.device, dtype=torch.float32)
            if bias is not None:
                db = torch.zeros(Vpad, device=hidden.device, dtype=torch.float32)
        tg = targets.contiguous()
        for r0 in range(0, T, rows_per):
            R = min(rows_per, T - r0)
            hc = h2[r0:r0 + R]
            gemm(hc, w, R, Vpad, H, ldh, ldb, False, b_mn, out=logits[:R], bias=bias)
            N.call("sb_ce_rows", logits.data_ptr(), tg[r0:].data_ptr(), row_loss[r0:].data_ptr(),
                   G.data_ptr() if need_grad else None, R, vocab_size, Vpad, Vpad, Vpad, 1.0 / T, N.stream())
            if need_grad:
                # dH_c[R,H] = G[R,V] · W^T
                gemm(G, w, R, H, Vpad, Vpad, ldb, False, not b_mn, out=dh[r0:r0 + R])
                if b_mn:    # dW[H,V] += H_c^T · G
                    gemm(hc, G, H, Vpad, R, ldh, Vpad, True, True, out=dw, accumulate=True)
                else:       # tied embedding memory [V,H]: dE += G^T · H_c
                    gemm(G, hc, Vpad, H, R, Vpad, ldh, True, True, out=dw, accumulate=True)
                if db is not None:
                    db += G[:R].float().sum(dim=0)
        loss = row_loss.sum() / T
        ctx.save_for_backward(dh, dw, db)
        ctx.weight = weight
        ctx.b_mn = b_mn
        ctx.hidden_shape = hidden.shape
        ctx.bias_dtype = bias.dtype if bias is not None else None
        return loss

    @staticmethod
    def backward(ctx, gout):
        dh, dw, db = ctx.saved_tensors
        weight = ctx.weight
        g_h = (dh * gout.to(dh.dtype)).view(ctx.hidden_shape) if dh is not None else None
        g_w = None
        if dw is not None and weight.requires_grad:
            main = getattr(weight, "main_grad", None)
            target_view = dw if ctx.b_mn else dw.t()
            if main is not None:        # main_grad has the weight's memory layout, like dw
                main.addcmul_(dw, gout.float().expand_as(dw))
            else:
                g_w = (target_view * gout.float()).to(weight.dtype)
        g_b = (db * gout.float()).to(ctx.bias_dtype) if (db is not None) else None
        return g_h, g_w, g_b, None, None, None


def linear_cross_entropy(hidden, weight, bias, targets, vocab_size, chunks=4):
    return _LinearCrossEntropy.apply(hidden, weight, bias, targets, vocab_size, chunks)


# ------------------------------------------------------------------ Mamba: conv1d + selective scan

N.register("sb_conv1d_fwd", [N.P, N.P, N.P, N.P, N.P, N.I, N.I, N.I, N.I, N.L, N.I, N.P])
N.register("sb_conv1d_bwd", [N.P, N.P, N.P, N.P, N.P, N.P, N.P, N.I, N.I, N.I, N.I, N.L, N.L, N.I, N.P])
N.register("sb_scan_fwd", [N.P] * 10 + [N.I] * 4 + [N.L] * 4 + [N.P])
N.register("sb_scan_bwd", [N.P] * 20 + [N.I] * 4 + [N.L] * 7 + [N.P])
N.register("sb_scan_ckpt_interval", [])

_SCAN_STATES = (8, 16, 32, 64, 128, 256)


def _btc(x: torch.Tensor):
    """`[B, T, C]` view with unit channel stride and one row stride for (b, t)."""
    B, T, C = x.shape
    if x.stride(2) == 1 and x.stride(0) == T * x.stride(1):
        return x, x.stride(1)
    c = x.contiguous()
    return c, C


class _Conv1dSilu(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, state):
        B, T, C = x.shape
        K = weight.shape[-1]
        xs, ldx = _btc(x)
        w32 = weight.reshape(C, K).float().contiguous()
        b32 = bias.float().contiguous() if bias is not None else None
        y = torch.empty(B, T, C, device=x.device, dtype=BF16)
        st = state.to(BF16).contiguous() if state is not None else None
        N.call("sb_conv1d_fwd", xs.data_ptr(), w32.data_ptr(), N.ptr(b32), N.ptr(st), y.data_ptr(), B, T, C, K, ldx,
               1, N.stream())
        ctx.save_for_backward(x, weight, bias)
        ctx.has_state = state is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        x, weight, bias = ctx.saved_tensors
        if ctx.has_state:
            raise RuntimeError("conv1d backward with a carried state is not supported")
        B, T, C = x.shape
        K = weight.shape[-1]
        xs, ldx = _btc(x)
        w32 = weight.reshape(C, K).float().contiguous()
        b32 = bias.float().contiguous() if bias is not None else None
        dyc = dy.contiguous()
        dx = torch.empty(B, T, C, device=x.device, dtype=BF16)
        dw = torch.zeros(C, K, device=x.device, dtype=torch.float32)
        db = torch.zeros(C, device=x.device, dtype=torch.float32)
        N.call("sb_conv1d_bwd", xs.data_ptr(), w32.data_ptr(), N.ptr(b32), dyc.data_ptr(), dx.data_ptr(),
               dw.data_ptr(), db.data_ptr(), B, T, C, K, ldx, C, 1, N.stream())
        return dx, dw.view(weight.shape).to(weight.dtype), (db.to(bias.dtype) if bias is not None else None), None


def conv1d_silu(x, weight, bias, state=None):
    K = weight.shape[-1]
    if x.shape[-1] % 8 != 0 or not (2 <= K <= 4):
        return torch.nn.functional.silu(reference.depthwise_conv1d(x, weight, bias, state))
    return _Conv1dSilu.apply(x, weight, bias, state)


class _SelectiveScan(torch.autograd.Function):
    @staticmethod
    def forward(ctx, u, delta, A, Bm, Cm, D, h0, need_final):
        B, T, C = u.shape
        Ns = A.shape[1]
        us, ld_u = _btc(u)
        ds, ld_d = _btc(delta)
        bs, ld_b = _btc(Bm)
        cs, ld_c = _btc(Cm)
        A32 = A.float().contiguous()
        D32 = D.float().contiguous()
        y = torch.empty(B, T, C, device=u.device, dtype=BF16)
        train = any(ctx.needs_input_grad[:6])
        nseg = -(-T // N.call_value("sb_scan_ckpt_interval"))
        ckpt = torch.empty(B, nseg, C, Ns, device=u.device, dtype=torch.float32) if train else None
        h_out = torch.empty(B, C, Ns, device=u.device, dtype=torch.float32) if need_final else None
        h0c = h0.float().contiguous() if h0 is not None else None
        N.call("sb_scan_fwd", us.data_ptr(), ds.data_ptr(), A32.data_ptr(), bs.data_ptr(), cs.data_ptr(),
               D32.data_ptr(), N.ptr(h0c), y.data_ptr(), N.ptr(ckpt), N.ptr(h_out), B, T, C, Ns, ld_u, ld_d, ld_b,
               ld_c, N.stream())
        ctx.save_for_backward(u, delta, A, Bm, Cm, D, ckpt)
        ctx.mark_non_differentiable(h_out) if h_out is not None else None
        return y, h_out

    @staticmethod
    def backward(ctx, dy, _dh):
        u, delta, A, Bm, Cm, D, ckpt = ctx.saved_tensors
        B, T, C = u.shape
        Ns = A.shape[1]
        us, ld_u = _btc(u)
        ds, ld_d = _btc(delta)
        bs, ld_b = _btc(Bm)
        cs, ld_c = _btc(Cm)
        dys, ld_dy = _btc(dy)
        A32 = A.float().contiguous()
        D32 = D.float().contiguous()
        tiles = -(-C // 32)
        ns = max(1, Ns // 64)
        dev = u.device
        part_dt = torch.empty(ns, B, T, C, device=dev, dtype=torch.float32)
        part_du = torch.empty(ns, B, T, C, device=dev, dtype=torch.float32)
        du = torch.empty(B, T, C, device=dev, dtype=BF16)
        dd = torch.empty(B, T, C, device=dev, dtype=BF16)
        part_b = torch.empty(tiles, B, T, Ns, device=dev, dtype=torch.float32)
        part_c = torch.empty(tiles, B, T, Ns, device=dev, dtype=torch.float32)
        dBm = torch.empty(B, T, Ns, device=dev, dtype=BF16)
        dCm = torch.empty(B, T, Ns, device=dev, dtype=BF16)
        dA = torch.zeros(C, Ns, device=dev, dtype=torch.float32)
        dD = torch.zeros(C, device=dev, dtype=torch.float32)
        N.call("sb_scan_bwd", us.data_ptr(), ds.data_ptr(), A32.data_ptr(), bs.data_ptr(), cs.data_ptr(),
               D32.data_ptr(), dys.data_ptr(), ckpt.data_ptr(), None, du.data_ptr(), dd.data_ptr(),
               part_b.data_ptr(), part_c.data_ptr(), part_dt.data_ptr(), part_du.data_ptr(), dBm.data_ptr(),
               dCm.data_ptr(), dA.data_ptr(), dD.data_ptr(),
               None, B, T, C, Ns, ld_u, ld_d, ld_b, ld_c, ld_dy, Ns, Ns, N.stream())
        return du, dd, dA.to(A.dtype), dBm, dCm, dD.to(D.dtype), None, None


def selective_scan(u, delta, A, Bm, Cm, D, h0=None, need_final_state=False):
    if A.shape[1] not in _SCAN_STATES or u.shape[-1] % 2:
        return reference.selective_scan(u, delta, A, Bm, Cm, D, h0)
    y, h = _SelectiveScan.apply(u, delta, A, Bm, Cm, D, h0, need_final_state)
    return y, h


# ------------------------------------------------------------------ mixture of experts

N.register("sb_router_logits", [N.P, N.P, N.P, N.I, N.I, N.I, N.L, N.P])
N.register("sb_moe_plan", [N.P] * 7 + [N.I] * 4 + [N.P])
N.register("sb_moe_gather", [N.P, N.P, N.P, N.P, N.I, N.I, N.I, N.L, N.I, N.P])
N.register("sb_moe_combine", [N.P, N.P, N.P, N.P, N.I, N.I, N.I, N.P])
N.register("sb_moe_combine_bwd", [N.P] * 7 + [N.I] * 4 + [N.P])
N.register("sb_moe_gather_bwd", [N.P, N.P, N.P, N.I, N.I, N.I, N.P])
N.register("sb_grouped_gemm_rows", [N.P, N.P, N.P, N.I, N.I, N.I, N.I, N.I, N.I, N.I, N.P, N.P, N.P])
N.register("sb_grouped_gemm_wgrad", [N.P, N.P, N.P, N.I, N.I, N.I, N.I, N.I, N.I, N.P, N.P])


class _RouterLogits(torch.autograd.Function):
    """fp32 logits = x(bf16) @ W(fp32) on a SIMT kernel; the backward products are tiny
    and run on the tensor-core GEMM in bf16 with fp32 accumulation."""

    @staticmethod
    def forward(ctx, x, w):
        x2, ldx = _rows(x)
        T, H = x2.shape
        E = w.shape[1]
        w32 = w.float().contiguous()
        out = torch.empty(T, E, device=x.device, dtype=torch.float32)
        N.call("sb_router_logits", x2.data_ptr(), w32.data_ptr(), out.data_ptr(), T, H, E, ldx, N.stream())
        ctx.save_for_backward(x, w)
        return out

    @staticmethod
    def backward(ctx, dl):
        x, w = ctx.saved_tensors
        x2, ldx = _rows(x)
        T, H = x2.shape
        E = w.shape[1]
        if E % 8 or H % 8 or x2.dtype != BF16 or ldx % 8:
            dlf = dl.float()
            dx = (dlf @ w.float().t()).to(x.dtype).view(x.shape) if ctx.needs_input_grad[0] else None
            dw = (x2.float().t() @ dlf).to(w.dtype) if ctx.needs_input_grad[1] else None
            return dx, dw
        dlb = dl.to(BF16).contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            # dx[T,H] = dl[T,E] · W^T: W is stored [H, E], i.e. the B operand K-major
            dx = gemm(dlb, w.to(BF16).contiguous(), T, H, E, E, E, False, False).view(x.shape)
        if ctx.needs_input_grad[1]:
            # dW[H,E] = x^T · dl: both operands as they lie in memory (M-major A, N-major B), fp32 out
            dw = gemm(x2, dlb, H, E, T, ldx, E, True, True, out_dtype=torch.float32).to(w.dtype)
        return dx, dw


def router_logits(x, w):
    if w.shape[1] > 256:
        return x.float() @ w.float()
    return _RouterLogits.apply(x, w)


class RoutePlan:
    """Device-resident routing plan of one MoE layer call (no host synchronisation)."""

    def __init__(self, logits: torch.Tensor, k: int):
        T, E = logits.shape
        dev = logits.device
        self.T, self.E, self.k = T, E, k
        self.max_rows = -(-(T * k + E * 127) // 128) * 128
        self.idx = torch.empty(T, k, device=dev, dtype=torch.int32)
        self.counts = torch.empty(E, device=dev, dtype=torch.int32)
        self.meta = torch.empty(E + 2, device=dev, dtype=torch.int32)
        self.tile_expert = torch.zeros(self.max_rows // 128, device=dev, dtype=torch.int32)
        self.dest = torch.empty(T * k, device=dev, dtype=torch.int32)
        self.row_route = torch.empty(self.max_rows, device=dev, dtype=torch.int32)
        lg = logits.detach().float().contiguous()
        N.call("sb_moe_plan", lg.data_ptr(), self.idx.data_ptr(), self.counts.data_ptr(), self.meta.data_ptr(),
               self.tile_expert.data_ptr(), self.dest.data_ptr(), self.row_route.data_ptr(), T, E, k, self.max_rows,
               N.stream())

    @property
    def num_m_tiles_ptr(self) -> int:
        return self.meta.data_ptr() + 4 * (self.E + 1)


N.register("sb_moe_aux_fwd", [N.P] * 6 + [N.I, N.I, N.I, N.F, N.F, N.P])
N.register("sb_moe_aux_bwd", [N.P] * 5 + [N.I, N.I, N.F, N.P])


class _MoeAuxLoss(torch.autograd.Function):
    """Load-balance + z loss of the fp32 router logits in two launches (row statistics with per-CTA partial sums,
    then one CTA that adds them in a fixed order); backward is one launch. `counts` is the routing plan's
    per-expert histogram, a constant for the gradient (`summa-llm/src/model/ffn.rs:626-710`)."""

    @staticmethod
    def forward(ctx, logits, counts, k, lb_w, z_w):
        T, E = logits.shape
        lg = logits.contiguous()
        dev = lg.device
        lse = torch.empty(T, device=dev, dtype=torch.float32)
        coef = torch.empty(E, device=dev, dtype=torch.float32)
        partial = torch.empty(-(-T // 64) * (E + 1), device=dev, dtype=torch.float32)
        aux = torch.empty((), device=dev, dtype=torch.float32)
        N.call("sb_moe_aux_fwd", lg.data_ptr(), counts.data_ptr(), lse.data_ptr(), coef.data_ptr(), partial.data_ptr(),
               aux.data_ptr(), T, E, int(k), float(lb_w), float(z_w), N.stream())
        ctx.save_for_backward(lg, lse, coef)
        ctx.z_w = float(z_w)
        return aux

    @staticmethod
    def backward(ctx, gout):
        lg, lse, coef = ctx.saved_tensors
        T, E = lg.shape
        grad = torch.empty_like(lg)
        g = gout.reshape(1).float().contiguous()
        N.call("sb_moe_aux_bwd", lg.data_ptr(), lse.data_ptr(), coef.data_ptr(), g.data_ptr(), grad.data_ptr(), T, E, ctx.z_w,
               N.stream())
        return grad, None, None, None, None


def moe_aux_loss(logits, idx, num_experts, lb_weight, z_weight):
    plan = getattr(idx, "_sb_plan", None)
    if plan is not None and plan.E == num_experts:
        counts = plan.counts
    else:
        counts = torch.bincount(idx.reshape(-1), minlength=num_experts).to(torch.int32)
    return _MoeAuxLoss.apply(logits, counts, idx.shape[1], max(lb_weight, 0.0), max(z_weight, 0.0))


def moe_route(logits, top_k):
    """(indices [T,k] int64, gates [T,k] fp32 = softmax over the selected logits). The
    selection runs in the top-k kernel; the gate softmax is differentiable torch math on
    the tiny `[T, k]` gather."""
    plan = RoutePlan(logits, top_k)
    idx = plan.idx.long()
    gates = torch.softmax(torch.gather(logits.float(), 1, idx), dim=-1)
    idx._sb_plan = plan
    return idx, gates


def _grouped_rows(a, w, plan: RoutePlan, n_out: int, k_in: int, w_kmajor: bool):
    out = torch.empty(plan.max_rows, n_out, device=a.device, dtype=BF16)
    N.call("sb_grouped_gemm_rows", a.data_ptr(), w.data_ptr(), out.data_ptr(), plan.max_rows, n_out, k_in, plan.E,
           a.stride(0), n_out, 1 if w_kmajor else 0, plan.tile_expert.data_ptr(), plan.num_m_tiles_ptr, N.stream())
    return out


def _grouped_wgrad(x, dy, plan: RoutePlan, out: torch.Tensor):
    E, M, Nn = out.shape
    N.call("sb_grouped_gemm_wgrad", x.data_ptr(), dy.data_ptr(), out.data_ptr(), plan.max_rows, M, Nn, E,
           x.stride(0), dy.stride(0), plan.meta.data_ptr(), N.stream())


class _MoeExperts(torch.autograd.Function):
    """gather → grouped GEMM → SwiGLU → grouped GEMM → weighted combine over the padded
    routed layout; the backward mirrors it with grouped dgrad / wgrad GEMMs."""

    @staticmethod
    def forward(ctx, x, gates, in_w, down_w, plan):
        T, H = x.shape
        E, _, I2 = in_w.shape
        I = I2 // 2
        k = plan.k
        x2, ldx = _rows(x)
        wi = in_w if in_w.dtype == BF16 else in_w.to(BF16)
        wd = down_w if down_w.dtype == BF16 else down_w.to(BF16)
        routed = torch.empty(plan.max_rows, H, device=x.device, dtype=BF16)
        N.call("sb_moe_gather", x2.data_ptr(), plan.row_route.data_ptr(), plan.meta.data_ptr(), routed.data_ptr(), E,
               H, k, ldx, plan.max_rows, N.stream())
        h = _grouped_rows(routed, wi, plan, I2, H, False)
        a = torch.empty(plan.max_rows, I, device=x.device, dtype=BF16)
        N.call("sb_swiglu_fwd", h.data_ptr(), a.data_ptr(), plan.max_rows, I, I2, N.stream())
        y = _grouped_rows(a, wd, plan, H, I, False)
        g32 = gates.detach().float().contiguous()
        out = torch.empty(T, H, device=x.device, dtype=BF16)
        N.call("sb_moe_combine", y.data_ptr(), plan.dest.data_ptr(), g32.data_ptr(), out.data_ptr(), T, H, k,
               N.stream())
        ctx.save_for_backward(x, g32, in_w, down_w, routed, h, a, y)
        ctx.plan = plan
        return out

    @staticmethod
    def backward(ctx, dout):
        x, g32, in_w, down_w, routed, h, a, y = ctx.saved_tensors
        plan = ctx.plan
        T, H = x.shape
        E, _, I2 = in_w.shape
        I = I2 // 2
        k = plan.k
        wi = in_w if in_w.dtype == BF16 else in_w.to(BF16)
        wd = down_w if down_w.dtype == BF16 else down_w.to(BF16)
        dout = dout.contiguous()
        dy = torch.empty(plan.max_rows, H, device=x.device, dtype=BF16)
        dgates = torch.zeros(T * k, device=x.device, dtype=torch.float32)
        N.call("sb_moe_combine_bwd", dout.data_ptr(), y.data_ptr(), plan.row_route.data_ptr(), g32.data_ptr(),
               plan.meta.data_ptr(), dy.data_ptr(), dgates.data_ptr(), E, H, k, plan.max_rows, N.stream())
        # down projection: da = dy · Wd^T (contraction over H), dWd += a^T · dy
        da = _grouped_rows(dy, wd, plan, I, H, True)
        dwd = _wgrad_target(down_w)
        _grouped_wgrad(a, dy, plan, dwd)
        dh = torch.empty(plan.max_rows, I2, device=x.device, dtype=BF16)
        N.call("sb_swiglu_bwd", h.data_ptr(), da.data_ptr(), dh.data_ptr(), plan.max_rows, I, I2, N.stream())
        dr = _grouped_rows(dh, wi, plan, H, I2, True)
        dwi = _wgrad_target(in_w)
        _grouped_wgrad(routed, dh, plan, dwi)
        dx = torch.empty(T, H, device=x.device, dtype=BF16)
        N.call("sb_moe_gather_bwd", dr.data_ptr(), plan.dest.data_ptr(), dx.data_ptr(), T, H, k, N.stream())
        return (dx.view(x.shape), dgates.view(T, k), _wgrad_result(in_w, dwi), _wgrad_result(down_w, dwd), None)


def _wgrad_target(w):
    main = getattr(w, "main_grad", None)
    return main if main is not None else torch.zeros(w.shape, device=w.device, dtype=torch.float32)


def _wgrad_result(w, buf):
    return None if getattr(w, "main_grad", None) is not None else buf.to(w.dtype)


def moe_experts(x, idx, gates, in_weight, down_weight):
    plan = getattr(idx, "_sb_plan", None)
    H, I2 = in_weight.shape[1], in_weight.shape[2]
    if plan is None or H % 64 != 0 or I2 % 128 != 0 or idx.shape[1] != plan.k:
        from . import _moe_experts_sorted
        return _moe_experts_sorted(x, idx, gates, in_weight, down_weight, None, None, "swiglu", True)
    return _MoeExperts.apply(x, gates, in_weight, down_weight, plan)


class _EpMoeExperts(torch.autograd.Function):
    """Expert-parallel form of `_MoeExperts`: the gather is fused with the NVLink dispatch, the
    owner runs the grouped GEMMs on its compact buffer and the rows travel back into the source
    layout before the local weighted combine. The backward runs the same two exchanges on the
    gradients; expert weight gradients stay on the owner."""

    @staticmethod
    def forward(ctx, x, gates, in_w, down_w, plan, ep):
        T, H = x.shape
        El, _, I2 = in_w.shape
        I = I2 // 2
        k = plan.k
        x2, ldx = _rows(x)
        wi = in_w if in_w.dtype == BF16 else in_w.to(BF16)
        wd = down_w if down_w.dtype == BF16 else down_w.to(BF16)
        recv, op = ep.exchange_to_owner(plan, x=x2)
        routed = recv.clone()                       # the symmetric buffer is reused by the next exchange
        h = _grouped_rows(routed, wi, op, I2, H, False)
        a = torch.empty(op.max_rows, I, device=x.device, dtype=BF16)
        N.call("sb_swiglu_fwd", h.data_ptr(), a.data_ptr(), op.max_rows, I, I2, N.stream())
        y_owner = _grouped_rows(a, wd, op, H, I, False)
        y = ep.exchange_to_source(y_owner, op)[:plan.max_rows].clone()
        g32 = gates.detach().float().contiguous()
        out = torch.empty(T, H, device=x.device, dtype=BF16)
        N.call("sb_moe_combine", y.data_ptr(), plan.dest.data_ptr(), g32.data_ptr(), out.data_ptr(), T, H, k,
               N.stream())
        ctx.save_for_backward(x, g32, in_w, down_w, routed, h, a, y)
        ctx.plan, ctx.ep = plan, ep
        return out

    @staticmethod
    def backward(ctx, dout):
        x, g32, in_w, down_w, routed, h, a, y = ctx.saved_tensors
        plan, ep = ctx.plan, ctx.ep
        T, H = x.shape
        El, _, I2 = in_w.shape
        I = I2 // 2
        k = plan.k
        wi = in_w if in_w.dtype == BF16 else in_w.to(BF16)
        wd = down_w if down_w.dtype == BF16 else down_w.to(BF16)
        dout = dout.contiguous()
        dy_src = torch.empty(plan.max_rows, H, device=x.device, dtype=BF16)
        dgates = torch.zeros(T * k, device=x.device, dtype=torch.float32)
        N.call("sb_moe_combine_bwd", dout.data_ptr(), y.data_ptr(), plan.row_route.data_ptr(), g32.data_ptr(),
               plan.meta.data_ptr(), dy_src.data_ptr(), dgates.data_ptr(), plan.E, H, k, plan.max_rows, N.stream())
        recv, op = ep.exchange_to_owner(plan, src_rows=dy_src)
        dy = recv.clone()
        da = _grouped_rows(dy, wd, op, I, H, True)
        dwd = _wgrad_target(down_w)
        _grouped_wgrad(a, dy, op, dwd)
        dh = torch.empty(op.max_rows, I2, device=x.device, dtype=BF16)
        N.call("sb_swiglu_bwd", h.data_ptr(), da.data_ptr(), dh.data_ptr(), op.max_rows, I, I2, N.stream())
        dr_owner = _grouped_rows(dh, wi, op, H, I2, True)
        dwi = _wgrad_target(in_w)
        _grouped_wgrad(routed, dh, op, dwi)
        dr = ep.exchange_to_source(dr_owner, op)
        dx = torch.empty(T, H, device=x.device, dtype=BF16)
        N.call("sb_moe_gather_bwd", dr.data_ptr(), plan.dest.data_ptr(), dx.data_ptr(), T, H, k, N.stream())
        return (dx.view(x.shape), dgates.view(T, k), _wgrad_result(in_w, dwi), _wgrad_result(down_w, dwd), None, None)


def ep_moe_experts(ep, x, gates, in_weight, down_weight, plan):
    return _EpMoeExperts.apply(x, gates, in_weight, down_weight, plan, ep)


# ------------------------------------------------------------------ int4 weights / sampling

N.register("sb_int4_gemv", [N.P] * 6 + [N.I, N.I, N.I, N.L, N.P])
N.register("sb_int4_dequant", [N.P, N.P, N.P, N.I, N.I, N.P])
N.register("sb_argmax_rows", [N.P, N.P, N.I, N.I, N.L, N.I, N.P])


N.register("sb_w4a16_gemm", [N.P] * 6 + [N.I, N.I, N.I, N.L, N.P])
N.register("sb_w4_gemv_small", [N.P] * 5 + [N.I, N.I, N.I, N.L, N.P])
N.register("sb_w4_gemv_cluster", [N.P] * 5 + [N.I, N.I, N.I, N.L, N.P, N.F, N.P])
N.register("sb_w4_gemv_mma", [N.P] * 5 + [N.I, N.I, N.I, N.L, N.P, N.F, N.P])
N.register("sb_w4_gemv_stream", [N.P] * 5 + [N.I, N.I, N.I, N.L, N.P, N.F, N.I, N.P])
# "cluster" (default): the CUDA-core GEMV with cluster split-K; "mma": nibble pairs go straight into warp-level
# mma fragments (1..8 rows). Measured on the 7B decode step: 348 tokens/s with "cluster", 124 with "mma".
W4_GEMV_KERNEL = os.environ.get("SUMMA_W4_GEMV", "cluster")
N.register("sb_w4_gemv_cluster_swiglu", [N.P] * 4 + [N.I, N.I, N.I, N.L, N.P, N.F, N.P])


N.register("sb_w4_gemv_cluster_rope", [N.P] * 4 + [N.I, N.I, N.I, N.L, N.P, N.F] + [N.P] * 5 + [N.I, N.I, N.I, N.P, N.I, N.P])


def int4_gemv_rope_append(x, packed_k8, scales, norm, cos, sin, k_cache, v_cache, pos, Hq, Hkv, D, cap):
    """The qkv projection of a decode step (x `[M <= 4, K]`, optional fused RMSNorm) with interleaved RoPE at the
    device-side position `pos` (int32 tensor) and the append of k / v to the caches in its epilogue. Returns
    `[M, (Hq + 2 Hkv) D]` whose q part is rotated (its k / v parts are not written)."""
    M, K = x.shape
    Nn = packed_k8.shape[1]
    x2, ldx = _rows(x)
    fuse = norm is not None and norm[0].dtype == torch.float32 and norm[0].is_contiguous()
    if norm is not None and not fuse:
        x2 = rmsnorm(x2, norm[0], norm[1])
        ldx = x2.stride(0)
    y = torch.empty(M, Nn, device=x.device, dtype=BF16)
    cs = (ctypes.c_long * 3)(k_cache.stride(0), k_cache.stride(1), k_cache.stride(2))
    N.call("sb_w4_gemv_cluster_rope", x2.data_ptr(), packed_k8.data_ptr(), scales.data_ptr(), y.data_ptr(), M, Nn, K,
           ldx, norm[0].data_ptr() if fuse else None, float(norm[1]) if fuse else 0.0, cos.data_ptr(), sin.data_ptr(),
           k_cache.data_ptr(), v_cache.data_ptr(), pos.data_ptr(), Hq, Hkv, D, cs, cap, N.stream())
    return y


def int4_gemv_swiglu(x, packed_k8, scales, norm=None):
    """silu(g) * v with [g | v] = (rmsnorm(x) or x) @ dequant(W `[K, 2I]`), x `[M <= 4, K]` -> `[M, I]`:
    the gated in-projection of a decode step in one launch."""
    M, K = x.shape
    Nn = packed_k8.shape[1]
    x2, ldx = _rows(x)
    fuse = norm is not None and norm[0].dtype == torch.float32 and norm[0].is_contiguous()
    if norm is not None and not fuse:
        x2 = rmsnorm(x2, norm[0], norm[1])
        ldx = x2.stride(0)
    y = torch.empty(M, Nn // 2, device=x.device, dtype=BF16)
    N.call("sb_w4_gemv_cluster_swiglu", x2.data_ptr(), packed_k8.data_ptr(), scales.data_ptr(), y.data_ptr(), M, Nn, K,
           ldx, norm[0].data_ptr() if fuse else None, float(norm[1]) if fuse else 0.0, N.stream())
    return y


def int4_gemv(x, packed, scales, residual=None, packed_k8=None, norm=None):
    """x `[M <= 64, K]` @ dequant(W) (+ residual). With the repacked weight (`reference.repack_int4_k8`)
    the product runs on the tensor cores (M > 4) or as the one-launch cluster GEMV (M <= 4);
    otherwise on the CUDA-core weight-streaming kernel. `norm=(gamma fp32 [K], eps)` applies RMSNorm
    to x first (fused into the GEMV for M <= 4)."""
    M, K = x.shape
    Nn = packed.shape[1]
    x2, ldx = _rows(x)
    y = torch.empty(M, Nn, device=x.device, dtype=BF16)
    res = residual.contiguous() if residual is not None else None
    use_mma = W4_GEMV_KERNEL == "mma"
    if (W4_GEMV_KERNEL == "stream" and packed_k8 is not None and M <= 4 and ldx % 8 == 0 and x2.data_ptr() % 16 == 0
            and K % 128 == 0 and Nn % 4 == 0 and K <= 16384):
        fuse = norm is not None and norm[0].dtype == torch.float32 and norm[0].is_contiguous()
        if norm is not None and not fuse:
            x2 = rmsnorm(x2, norm[0], norm[1])
            ldx = x2.stride(0)
        N.call("sb_w4_gemv_stream", x2.data_ptr(), packed_k8.data_ptr(), scales.data_ptr(), N.ptr(res), y.data_ptr(),
               M, Nn, K, ldx, norm[0].data_ptr() if fuse else None, float(norm[1]) if fuse else 0.0, 0, N.stream())
        return y
    if (packed_k8 is not None and M <= (8 if use_mma else 4) and ldx % 8 == 0 and x2.data_ptr() % 16 == 0
            and K % 128 == 0 and Nn % 4 == 0 and K <= (98304 if use_mma else 20480)):
        # batch 1..8 decode: one launch, K split over a thread-block cluster, no accumulator pass
        fuse = norm is not None and norm[0].dtype == torch.float32 and norm[0].is_contiguous()
        if norm is not None and not fuse:
            x2 = rmsnorm(x2, norm[0], norm[1])
            ldx = x2.stride(0)
        N.call("sb_w4_gemv_mma" if use_mma else "sb_w4_gemv_cluster", x2.data_ptr(), packed_k8.data_ptr(), scales.data_ptr(), N.ptr(res), y.data_ptr(),
               M, Nn, K, ldx, norm[0].data_ptr() if fuse else None, float(norm[1]) if fuse else 0.0, N.stream())
        return y
    if norm is not None:
        x2 = rmsnorm(x2, norm[0], norm[1])
        ldx = x2.stride(0)
    acc = torch.empty(max(M, 64), Nn, device=x.device, dtype=torch.float32)
    if packed_k8 is not None and ldx % 8 == 0 and x2.data_ptr() % 16 == 0:
        N.call("sb_w4a16_gemm", x2.data_ptr(), packed_k8.data_ptr(), scales.data_ptr(), acc.data_ptr(), N.ptr(res),
               y.data_ptr(), M, Nn, K, ldx, N.stream())
        return y
    N.call("sb_int4_gemv", x2.data_ptr(), packed.data_ptr(), scales.data_ptr(), acc.data_ptr(), N.ptr(res),
           y.data_ptr(), M, Nn, K, ldx, N.stream())
    return y


def int4_prefill_usable(x2, packed_k8, K: int, Nn: int) -> bool:
    return (packed_k8 is not None and x2.is_cuda and x2.dtype == BF16 and x2.dim() == 2 and x2.stride(1) == 1
            and x2.stride(0) % 8 == 0 and x2.data_ptr() % 16 == 0 and K % 128 == 0 and Nn % 4 == 0)


def int4_matmul(x, packed_k8, scales, residual=None):
    """x `[M > 64, K]` @ dequant(W) (+ residual) with the weight expanded inside the kernel: each 128 x MP output
    tile's CTA turns its 4-bit weight tiles into bf16 in registers and stores them to tensor memory as the MMA's A
    operand, so no bf16 copy of the weight is ever written. Callers check `int4_prefill_usable` first."""
    M, K = x.shape
    Nn = packed_k8.shape[1]
    y = torch.empty(M, Nn, device=x.device, dtype=BF16)
    res = residual.contiguous() if residual is not None else None
    N.call("sb_w4a16_gemm", x.data_ptr(), packed_k8.data_ptr(), scales.data_ptr(), None, N.ptr(res), y.data_ptr(),
           M, Nn, K, x.stride(0), N.stream())
    return y


def int4_dequant(packed, scales):
    K, Nn = packed.shape[0] * 2, packed.shape[1]
    out = torch.empty(K, Nn, device=packed.device, dtype=BF16)
    N.call("sb_int4_dequant", packed.data_ptr(), scales.data_ptr(), out.data_ptr(), K, Nn, N.stream())
    return out


N.register("sb_fake_quant", [N.P, N.P, N.L, N.I, N.I, N.P])
N.register("sb_hquant_dequant", [N.P, N.P, N.P, N.L, N.I, N.I, N.P])
N.register("sb_hquant_gemv", [N.P] * 6 + [N.I, N.I, N.I, N.L, N.I, N.P])
HQ_FMT = {"binary_g128": 0, "ternary_g128": 1}


def fake_quant_values(w, fmt: str):
    """dequant(quant(w)) over groups of 128 of the flattened tensor (no autograd)."""
    wc = w.detach().contiguous()
    if wc.dtype not in (BF16, torch.float32):
        wc = wc.float()
    out = torch.empty_like(wc)
    N.call("sb_fake_quant", wc.data_ptr(), out.data_ptr(), wc.numel(), HQ_FMT[fmt], 1 if wc.dtype == BF16 else 0,
           N.stream())
    return out.to(w.dtype)


def hquant_dequant(codes, scales, n: int, fmt: str, dtype=BF16):
    """`codes` uint8, `scales` fp16 (one per 128 flattened elements) -> `[n]` bf16 or fp32."""
    out = torch.empty(n, device=codes.device, dtype=dtype)
    N.call("sb_hquant_dequant", codes.data_ptr(), scales.data_ptr(), out.data_ptr(), n, HQ_FMT[fmt],
           1 if dtype == BF16 else 0, N.stream())
    return out


def hquant_gemv(x, codes, scales, Nn: int, fmt: str, residual=None):
    """x `[M, K]` bf16 @ decode(W `[K, Nn]`) straight from the group codes (Nn % 128 == 0)."""
    M, K = x.shape
    x2, ldx = _rows(x)
    acc = torch.zeros(M, Nn, device=x.device, dtype=torch.float32)
    y = torch.empty(M, Nn, device=x.device, dtype=BF16)
    res = residual.contiguous() if residual is not None else None
    N.call("sb_hquant_gemv", x2.data_ptr(), codes.data_ptr(), scales.data_ptr(), acc.data_ptr(), N.ptr(res),
           y.data_ptr(), M, Nn, K, ldx, HQ_FMT[fmt], N.stream())
    return y


def argmax_rows(logits):
    rows, vocab = logits.shape
    out = torch.empty(rows, device=logits.device, dtype=torch.int64)
    if logits.dtype not in (BF16, torch.float32):
        logits = logits.float()
    N.call("sb_argmax_rows", logits.data_ptr(), out.data_ptr(), rows, vocab, logits.stride(0),
           1 if logits.dtype == BF16 else 0, N.stream())
    return out


N.register("sb_sample_rows", [N.P, N.L, N.I, N.P, N.P, N.P, N.I, N.I, N.F, N.F, N.I, N.P])


def seen_bitmap(tokens, vocab: int, device) -> torch.Tensor:
    """`[rows, ceil(vocab / 32)]` int32 bit map with the bits of `tokens` (list of id lists) set."""
    words = (vocab + 31) // 32
    bm = torch.zeros(len(tokens), words, dtype=torch.int32)
    for r, ids in enumerate(tokens):
        for t in set(int(x) for x in ids):
            w, b = divmod(t, 32)
            v = int(bm[r, w]) | (1 << b)
            bm[r, w] = v - (1 << 32) if v >= (1 << 31) else v
    return bm.to(device)


def sample_rows(logits, seen=None, uniform=None, penalty: float = 1.0, temperature: float = 0.0, top_k: int = 0):
    """Device-side token selection (repetition penalty, temperature, top-k); updates `seen`."""
    rows, vocab = logits.shape
    lg = logits if logits.stride(-1) == 1 else logits.contiguous()
    if lg.dtype not in (torch.float32, BF16):
        lg = lg.float()
    out = torch.empty(rows, device=logits.device, dtype=torch.int64)
    if temperature > 0 and uniform is None:
        uniform = torch.rand(rows, device=logits.device)
    N.call("sb_sample_rows", lg.data_ptr(), lg.stride(0), 1 if lg.dtype == BF16 else 0, N.ptr(seen), N.ptr(uniform),
           out.data_ptr(), rows, vocab, float(penalty), float(temperature), int(top_k), N.stream())
    return out
