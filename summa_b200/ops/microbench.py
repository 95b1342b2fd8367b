"""Kernel microbenchmarks: `python -m summa_b200.ops.microbench <op> [--key value ...]`.

Every op is timed with CUDA events after warm-up, with an L2 flush (a write larger than
the L2) between timed launches, and reported as one JSON line with the achieved rate and
its fraction of the measured peaks (`MEASURED_PEAKS.json` beside the package's parent
directory when present, otherwise the stated fallback). `--once` runs two untimed
launches and exits: the small, bounded workload a profiler capture wants.

Ops: gemm, attention_fwd, attention_bwd, attention_decode, scan, rmsnorm, swiglu, cross_entropy, int4_gemv.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def peaks():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))),
                        "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "source": "measured"}
    return dict(FALLBACK_PEAKS)


_flush = None


def flush_l2():
    """Writes a buffer larger than L2, then reads a second one: the write evicts the timed kernel's operands, the read
    pushes the write's dirty lines out, so the next kernel does not share DRAM with their write-back."""
    global _flush
    if _flush is None:
        _flush = (torch.empty(256 << 20, dtype=torch.uint8, device="cuda"), torch.zeros(64 << 20, dtype=torch.int32, device="cuda"))
    _flush[0].zero_()
    _flush[1].sum()


def timeit(fn, iters=10, warmup=3, flush=True):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        if flush:
            flush_l2()
        s = torch.cuda.Event(enable_timing=True)
        e = torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        total += s.elapsed_time(e)
    return total / iters


def _report(name, ms, flops=None, nbytes=None, **extra):
    pk = peaks()
    out = {"op": name, "ms": round(ms, 5), **extra}
    if flops is not None:
        out["tflops"] = round(flops / ms / 1e9, 1)
        out[f"frac_of_{pk['source']}_bf16"] = round(out["tflops"] / pk["bf16_tflops"], 3)
    if nbytes is not None:
        out["gbs"] = round(nbytes / ms / 1e6, 1)
        out[f"frac_of_{pk['source']}_hbm"] = round(out["gbs"] / pk["hbm_gbs"], 3)
    print(json.dumps(out), flush=True)
    return out


def _gemm_case(M, N, K, layout, tile, iters, compare, once=False):
    """layout: fwd = x[M,K] @ w[K,N]; dgrad = dy[M,K] @ w[N,K]^T; wgrad = x[K,M]^T @ dy[K,N] into fp32 (+=)."""
    from . import cuda_ops
    if layout == "fwd":
        x = torch.randn(M, K, device="cuda").bfloat16()
        w = torch.randn(K, N, device="cuda").bfloat16()
        fn = lambda: cuda_ops.gemm(x, w, M, N, K, K, N, False, True, tile_n=tile)
        lib = lambda: x @ w
    elif layout == "dgrad":
        x = torch.randn(M, K, device="cuda").bfloat16()
        w = torch.randn(N, K, device="cuda").bfloat16()
        fn = lambda: cuda_ops.gemm(x, w, M, N, K, K, K, False, False, tile_n=tile)
        lib = lambda: x @ w.t()
    else:
        x = torch.randn(K, M, device="cuda").bfloat16()
        w = torch.randn(K, N, device="cuda").bfloat16()
        acc = torch.zeros(M, N, device="cuda")
        fn = lambda: cuda_ops.gemm(x, w, M, N, K, M, N, True, True, out=acc, accumulate=True, tile_n=tile)
        lib = lambda: x.t() @ w
    if once:
        fn(); fn(); return
    r = _report("gemm", timeit(fn, iters), flops=2.0 * M * N * K, M=M, N=N, K=K, layout=layout, tile=tile)
    if compare:
        r2 = _report("torch_matmul", timeit(lib, iters), flops=2.0 * M * N * K, M=M, N=N, K=K, layout=layout)
        print(json.dumps({"gemm_over_library": round(r2["ms"] / r["ms"], 3), "M": M, "N": N, "K": K,
                          "layout": layout, "tile": tile}), flush=True)


# the GEMM shapes of one llama-350m training step (16384 tokens, hidden 1024, FFN 2816)
TRAIN_SHAPES = [
    (16384, 3072, 1024, "fwd"), (16384, 1024, 1024, "fwd"), (16384, 5632, 1024, "fwd"), (16384, 1024, 2816, "fwd"),
    (16384, 1024, 3072, "dgrad"), (16384, 1024, 1024, "dgrad"), (16384, 1024, 5632, "dgrad"), (16384, 2816, 1024, "dgrad"),
    (1024, 3072, 16384, "wgrad"), (1024, 1024, 16384, "wgrad"), (1024, 5632, 16384, "wgrad"), (2816, 1024, 16384, "wgrad"),
]


def bench_gemm(a):
    if a.sweep:
        for (M, N, K, layout) in [(8192, 8192, 8192, "fwd")] + TRAIN_SHAPES:
            for tile in ([0] if a.tile < 0 else [a.tile]):
                _gemm_case(M, N, K, layout, tile, a.iters, a.compare)
        return
    _gemm_case(a.M, a.N, a.K, a.layout, max(a.tile, 0), a.iters, a.compare, once=a.once)


def _attn_inputs(a):
    B, S, H, KV, D = a.B, a.S, a.H, a.KV or a.H, a.D
    q = torch.randn(B, S, H, D, device="cuda").bfloat16()
    k = torch.randn(B, S, KV, D, device="cuda").bfloat16()
    v = torch.randn(B, S, KV, D, device="cuda").bfloat16()
    return q, k, v


def bench_attention_fwd(a):
    from . import cuda_ops
    q, k, v = _attn_inputs(a)
    fn = lambda: cuda_ops.attention_fwd(q, k, v, True)
    if a.once:
        fn(); fn(); return
    fl = 4.0 * a.B * a.H * a.S * a.S * a.D / 2
    _report("attention_fwd", timeit(fn, a.iters), flops=fl, B=a.B, S=a.S, H=a.H, D=a.D)
    if a.compare:
        qq, kk, vv = (t.transpose(1, 2) for t in (q, k, v))
        f2 = lambda: torch.nn.functional.scaled_dot_product_attention(qq, kk, vv, is_causal=True,
                                                                      enable_gqa=kk.shape[1] != qq.shape[1])
        _report("torch_sdpa_fwd", timeit(f2, a.iters), flops=fl)


def bench_attention_bwd(a):
    from . import cuda_ops
    q, k, v = _attn_inputs(a)
    o, lse = cuda_ops.attention_fwd(q, k, v, True)
    do = torch.randn_like(o)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    fn = lambda: cuda_ops.attention_bwd(q, k, v, o, do, lse, dq, dk, dv, True, None, 0)
    if a.once:
        fn(); fn(); return
    fl = 10.0 * a.B * a.H * a.S * a.S * a.D / 2
    _report("attention_bwd", timeit(fn, a.iters), flops=fl, B=a.B, S=a.S, H=a.H, D=a.D)
    if a.compare:
        qq, kk, vv = (t.transpose(1, 2).detach().requires_grad_() for t in (q, k, v))
        oo = torch.nn.functional.scaled_dot_product_attention(qq, kk, vv, is_causal=True,
                                                              enable_gqa=kk.shape[1] != qq.shape[1])
        g = torch.randn_like(oo)
        f2 = lambda: torch.autograd.grad(oo, (qq, kk, vv), g, retain_graph=True)
        _report("torch_sdpa_bwd", timeit(f2, a.iters), flops=fl)


def bench_scan(a):
    from .. import ops
    B, T, C, N = a.B, a.S, a.C, a.state
    u = torch.randn(B, T, C, device="cuda").bfloat16().requires_grad_()
    dt = (torch.rand(B, T, C, device="cuda") * 0.1).bfloat16().requires_grad_()
    A = -torch.rand(C, N, device="cuda").float().requires_grad_()
    Bm = torch.randn(B, T, N, device="cuda").bfloat16().requires_grad_()
    Cm = torch.randn(B, T, N, device="cuda").bfloat16().requires_grad_()
    Dp = torch.randn(C, device="cuda").float().requires_grad_()

    def fwd():
        with torch.no_grad():
            return ops.selective_scan(u, dt, A, Bm, Cm, Dp)

    def fwdbwd():
        y = ops.selective_scan(u, dt, A, Bm, Cm, Dp)[0]
        y.backward(torch.ones_like(y))

    if a.once:
        fwdbwd(); fwdbwd(); return
    nb = 2.0 * B * T * C * 3 + 2.0 * B * T * N * 2 * 2
    ms = timeit(fwd, a.iters)
    _report("scan_fwd", ms, nbytes=nb, B=B, T=T, C=C, N=N, tera_state_updates_per_s=round(B * T * C * N / ms / 1e9, 3))
    _report("scan_fwd_bwd", timeit(fwdbwd, a.iters), B=B, T=T, C=C, N=N)


def bench_rmsnorm(a):
    from .. import ops
    x = torch.randn(a.M, a.N, device="cuda").bfloat16()
    w = torch.ones(a.N, device="cuda")
    fn = lambda: ops.rmsnorm(x, w, 1e-5)
    if a.once:
        fn(); fn(); return
    _report("rmsnorm", timeit(fn, a.iters), nbytes=4.0 * a.M * a.N, M=a.M, N=a.N)


def bench_swiglu(a):
    from .. import ops
    x = torch.randn(a.M, 2 * a.N, device="cuda").bfloat16()
    fn = lambda: ops.gated_act(x, "swiglu")
    if a.once:
        fn(); fn(); return
    _report("swiglu", timeit(fn, a.iters), nbytes=6.0 * a.M * a.N, M=a.M, N=a.N)


def bench_cross_entropy(a):
    from .. import ops
    h = torch.randn(a.M, a.K, device="cuda").bfloat16()
    w = (torch.randn(a.K, a.N, device="cuda") * 0.02).bfloat16()
    t = torch.randint(0, a.N, (a.M,), device="cuda")
    fn = lambda: ops.linear_cross_entropy(h, w, None, t, a.N)
    if a.once:
        fn(); fn(); return
    _report("linear_cross_entropy_fwd", timeit(fn, a.iters), flops=2.0 * a.M * a.N * a.K, M=a.M, V=a.N, K=a.K)


def bench_int4_gemv(a):
    from .. import ops
    from . import reference
    packed, scales = reference.quantize_int4_g128(torch.randn(a.K, a.N) * 0.05)
    packed, scales = packed.cuda(), scales.cuda()
    k8 = reference.repack_int4_k8(packed)
    x = torch.randn(a.M, a.K, device="cuda").bfloat16()
    fn = lambda: ops.int4_gemv(x, packed, scales, None, k8)      # M <= 4: one-launch GEMV, else tcgen05 W4A16
    if a.once:
        fn(); fn(); return
    nbytes = a.K * a.N / 2 + a.K * a.N / 64
    _report("int4_gemv", timeit(fn, a.iters), nbytes=nbytes, M=a.M, N=a.N, K=a.K)
    if a.compare:
        old = lambda: ops.int4_gemv(x, packed, scales)           # CUDA-core split-K kernel + accumulator pass
        _report("int4_gemv_splitk_cuda_core", timeit(old, a.iters), nbytes=nbytes, M=a.M, N=a.N, K=a.K)
        if a.M <= 4:
            x64 = torch.randn(8, a.K, device="cuda").bfloat16()
            tc = lambda: ops.int4_gemv(x64, packed, scales, None, k8)
            _report("w4a16_tcgen05_m8", timeit(tc, a.iters), nbytes=nbytes, M=8, N=a.N, K=a.K)


def bench_int4_prefill(a):
    """Prefill-sized W4A16 product (M > 64): the fused dequant-GEMM against dequantise-to-bf16 + plain GEMM."""
    from .. import ops
    from . import reference
    packed, scales = reference.quantize_int4_g128(torch.randn(a.K, a.N) * 0.05)
    packed, scales = packed.cuda(), scales.cuda()
    k8 = reference.repack_int4_k8(packed)
    x = torch.randn(a.M, a.K, device="cuda").bfloat16()
    fn = lambda: ops.int4_matmul(x, k8, scales)
    if a.once:
        fn(); fn(); return
    flops = 2.0 * a.M * a.N * a.K
    _report("int4_prefill_fused", timeit(fn, a.iters), flops=flops, M=a.M, N=a.N, K=a.K)
    if a.compare:
        old = lambda: ops.linear(x, ops.int4_dequant(packed, scales), None)
        _report("int4_prefill_dequant_then_gemm", timeit(old, a.iters), flops=flops, M=a.M, N=a.N, K=a.K)


def bench_attention_decode(a):
    from . import cuda_ops
    B, Sk, H, KV, D = a.B, a.S, a.H, a.KV or a.H, 128
    q = torch.randn(B, 1, H, D, device="cuda").bfloat16()
    kc = torch.randn(B, Sk, KV, D, device="cuda").bfloat16()
    vc = torch.randn(B, Sk, KV, D, device="cuda").bfloat16()
    fn = lambda: cuda_ops.decode_attention(q, kc, vc, True, None, Sk - 1)
    if a.once:
        fn(); fn(); return
    _report("attention_decode", timeit(fn, a.iters), nbytes=4.0 * B * Sk * KV * D, B=B, Sk=Sk, H=H, KV=KV)


OPS = {"gemm": bench_gemm, "attention_decode": bench_attention_decode, "attention_fwd": bench_attention_fwd, "attention_bwd": bench_attention_bwd,
       "scan": bench_scan, "rmsnorm": bench_rmsnorm, "swiglu": bench_swiglu,
       "cross_entropy": bench_cross_entropy, "int4_gemv": bench_int4_gemv, "int4_prefill": bench_int4_prefill}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("op", choices=sorted(OPS))
    for name, default in (("M", 8192), ("N", 8192), ("K", 8192), ("B", 8), ("S", 2048), ("H", 16), ("KV", 0),
                          ("D", 64), ("C", 3072), ("state", 128), ("iters", 10)):
        ap.add_argument(f"--{name}", type=int, default=default)
    ap.add_argument("--tile", type=int, default=-1, help="gemm: 128 / 256 single-CTA tiles, 512 paired CTAs, 0 auto")
    ap.add_argument("--layout", default="fwd", choices=["fwd", "dgrad", "wgrad"], help="gemm operand layouts")
    ap.add_argument("--sweep", action="store_true", help="gemm: 8192^3 and the llama-350m training shapes")
    ap.add_argument("--once", action="store_true", help="two untimed launches, for a profiler capture")
    ap.add_argument("--compare", action="store_true", help="also time the library kernel of the same op")
    a = ap.parse_args(argv)
    if not torch.cuda.is_available():
        print(json.dumps({"error": "no CUDA device"}))
        return 1
    from . import native
    OPS[a.op](a)
    torch.cuda.synchronize()
    flag = native.read_error_flag()
    if flag:
        print(json.dumps({"device_error_word": flag}))
        return 2
    return 0


if __name__ == "__main__":
    sys.exit(main())
