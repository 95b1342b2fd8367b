"""Group-quantised linear layers for inference: 4-bit (`QuantLinear`) and the HQUANT binary /
ternary codecs (`HQuantLinear`), plus the loader of a quantised archive.

`QuantLinear` holds a `[d_in, d_out]` weight as packed int4 codes (group 128 along d_in,
bf16 scales). Decode-sized inputs (<= 64 rows) run the weight-streaming GEMV kernel, which
reads the packed weight once; inputs of up to 512 rows (short prefill chunks, speculative batches) run the
fused dequant-GEMM, which expands each 4-bit weight tile in registers on its way into tensor memory (no bf16
copy of the weight exists); longer prefill expands the weight once into a reused bf16 workspace and runs the
plain tensor-core GEMM, which is the faster form there (numbers beside `PREFILL_FUSED_MAX_ROWS`). The reference has only a host-side oracle for
quantised mat-vec (`summa-train/src/quantization.rs:626-654`); this is the device path.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from .. import ops
from ..ops import reference
from .layers import Linear

import os

GROUP = 128
_workspace = {}
# Inputs of 65 .. PREFILL_FUSED_MAX_ROWS rows run the fused dequant-GEMM (the 4-bit weight is expanded inside the
# kernel). Above that the weight is expanded once into a bf16 workspace and the plain GEMM runs: the expansion is
# then amortised over many rows and the paired-CTA GEMM reaches 0.85-0.88 of the measured bf16 peak where the fused
# kernel, whose tensor pipe waits on its eight expanding warps, reaches 0.61-0.66 (7B shapes, 8192 rows); at 512
# rows the fused kernel is 1.1-1.2 x faster, at 128 rows up to 1.7 x. 0 switches the fused form off.
PREFILL_FUSED_MAX_ROWS = int(os.environ.get("SUMMA_W4_PREFILL_FUSED_MAX_ROWS", "512"))


class QuantLinear(nn.Module):
    def __init__(self, packed: torch.Tensor, scales: torch.Tensor, bias: Optional[torch.Tensor] = None):
        super().__init__()
        self.d_in, self.d_out = packed.shape[0] * 2, packed.shape[1]
        self.register_buffer("packed", packed.contiguous())
        self.register_buffer("scales", scales.contiguous())
        self.register_buffer("bias", bias)
        self._k8 = None           # repacked copy for the tensor-core decode kernel (built on first use)

    def packed_k8(self) -> torch.Tensor:
        if self._k8 is None or self._k8.device != self.packed.device:
            self._k8 = reference.repack_int4_k8(self.packed)
        return self._k8

    @staticmethod
    def from_linear(lin: Linear) -> "QuantLinear":
        dev = lin.weight.device
        packed, scales = reference.quantize_int4_g128(lin.weight.detach(), GROUP)   # on the weight's device
        b = lin.bias.detach().to(torch.bfloat16) if lin.bias is not None else None
        return QuantLinear(packed.to(dev), scales.to(dev), b)

    def dequantized(self) -> torch.Tensor:
        if self.packed.is_cuda:
            return ops.int4_dequant(self.packed, self.scales)
        return reference.dequantize_int4_g128(self.packed, self.scales, GROUP)

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None, norm=None) -> torch.Tensor:
        """`residual` (same shape as the output) is added in the kernel epilogue on the decode path;
        `norm=(gamma, eps)` applies RMSNorm to `x` first (inside the GEMV kernel for <= 4 rows)."""
        lead = x.shape[:-1]
        x2 = x.reshape(-1, self.d_in)
        if x2.is_cuda and x2.dtype == torch.bfloat16:
            if x2.shape[0] <= 64:
                if residual is not None and self.bias is None:
                    return ops.int4_gemv(x2, self.packed, self.scales, residual.reshape(-1, self.d_out),
                                         self.packed_k8(), norm).view(*lead, self.d_out)
                y = ops.int4_gemv(x2, self.packed, self.scales, None, self.packed_k8(), norm)
            else:
                if norm is not None:
                    x2 = ops.rmsnorm(x2, norm[0], norm[1])
                k8 = self.packed_k8()
                if x2.shape[0] <= PREFILL_FUSED_MAX_ROWS and ops.int4_prefill_usable(x2, k8, self.d_in, self.d_out):
                    # prefill: the 4-bit weight is expanded inside the GEMM, on its way into tensor memory
                    fuse_res = residual is not None and self.bias is None
                    y = ops.int4_matmul(x2, k8, self.scales, residual.reshape(-1, self.d_out) if fuse_res else None)
                    if fuse_res:
                        return y.view(*lead, self.d_out)
                else:
                    y = ops.linear(x2, self.dequantized(), None)
        else:
            if norm is not None:
                x2 = ops.rmsnorm(x2, norm[0], norm[1])
            y = (x2.float() @ self.dequantized().float()).to(x.dtype)
        if self.bias is not None:
            y = y + self.bias.to(y.dtype)
        y = y.view(*lead, self.d_out)
        return y if residual is None else y + residual


def _swiglu_fusable(lin, x2) -> bool:
    return (isinstance(lin, QuantLinear) and lin.bias is None and x2.is_cuda and x2.dtype == torch.bfloat16
            and x2.shape[0] <= 4 and lin.d_in % GROUP == 0 and lin.d_out % 8 == 0 and lin.d_in <= 20480
            and x2.stride(-1) == 1 and x2.stride(0) % 8 == 0 and x2.data_ptr() % 16 == 0)


def in_proj_swiglu(lin, x: torch.Tensor, norm=None) -> torch.Tensor:
    """silu(gate) * value of a gated in-projection `[gate | value]`, with the optional RMSNorm of `x`
    in front: one kernel for <= 4 rows of a quantised projection, the separate ops otherwise."""
    x2 = x.reshape(-1, x.shape[-1])
    if _swiglu_fusable(lin, x2):
        from ..ops import cuda_ops
        return cuda_ops.int4_gemv_swiglu(x2, lin.packed_k8(), lin.scales, norm).view(*x.shape[:-1], lin.d_out // 2)
    if norm is not None:
        u = lin(x, norm=norm) if isinstance(lin, QuantLinear) else lin(ops.rmsnorm(x, norm[0], norm[1]))
    else:
        u = lin(x)
    return ops.gated_act(u, "swiglu")


def quantize_model_int4(model, include_head: bool = False) -> int:
    """Replace every block projection (and optionally the head) whose d_in is a multiple of
    128 by a `QuantLinear`. Returns the number of replaced layers."""
    n = 0
    for mod in list(model.modules()):
        for name, child in list(mod.named_children()):
            if isinstance(child, Linear) and child.d_in % GROUP == 0 and child.d_out % 4 == 0:
                if child is getattr(model, "lm_head", None) and not include_head:
                    continue
                setattr(mod, name, QuantLinear.from_linear(child))
                n += 1
    return n


class HQuantLinear(nn.Module):
    """`[d_in, d_out]` weight kept as HQUANT binary (1 bit) or ternary (2 bit) group codes with
    fp16 group scales (groups of 128 over the flattened tensor, `summa-train/src/quantization.rs:447-501`).
    Needs d_out % 128 == 0 so that a group lies inside one row. Decode-sized inputs stream the
    codes through the GEMV kernel; larger inputs expand the weight to bf16 for the tensor-core GEMM."""

    GEMV_ROWS = 16

    def __init__(self, codes: torch.Tensor, scales: torch.Tensor, d_in: int, d_out: int, fmt: str,
                 bias: Optional[torch.Tensor] = None):
        super().__init__()
        if fmt not in ("binary_g128", "ternary_g128") or d_out % GROUP:
            raise ValueError(f"HQuantLinear needs a binary / 2-bit ternary code and d_out % {GROUP} == 0")
        self.d_in, self.d_out, self.fmt = d_in, d_out, fmt
        self.register_buffer("codes", codes.contiguous())
        self.register_buffer("scales", scales.contiguous())
        self.register_buffer("bias", bias)

    @staticmethod
    def from_packed(pt, bias: Optional[torch.Tensor] = None, device=None) -> "HQuantLinear":
        """`pt`: a `train.quantization.PackedTensor` of rank 2."""
        codes = torch.from_numpy(pt.codes.copy())
        scales = torch.from_numpy(pt.scales.copy().view("float16"))
        out = HQuantLinear(codes, scales, pt.shape[0], pt.shape[1], pt.format, bias)
        return out.to(device) if device is not None else out

    def dequantized(self) -> torch.Tensor:
        return ops.hquant_dequant(self.codes, self.scales, self.d_in * self.d_out, self.fmt,
                                  torch.bfloat16).view(self.d_in, self.d_out)

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        lead = x.shape[:-1]
        x2 = x.reshape(-1, self.d_in)
        if x2.is_cuda and x2.dtype == torch.bfloat16 and x2.shape[0] <= self.GEMV_ROWS:
            r = residual.reshape(-1, self.d_out) if (residual is not None and self.bias is None) else None
            y = ops.hquant_gemv(x2, self.codes, self.scales, self.d_out, self.fmt, r)
            if r is not None:
                return y.view(*lead, self.d_out)
        elif x2.is_cuda and x2.dtype == torch.bfloat16:
            y = ops.linear(x2, self.dequantized(), None)
        else:
            w = ops.hquant_dequant(self.codes, self.scales, self.d_in * self.d_out, self.fmt, torch.float32)
            y = (x2.float() @ w.view(self.d_in, self.d_out)).to(x.dtype)
        if self.bias is not None:
            y = y + self.bias.to(y.dtype)
        y = y.view(*lead, self.d_out)
        return y if residual is None else y + residual


def load_archive(model, archive_dir: str) -> dict:
    """Loads a quantised archive (`train.quantization.export_archive`) into `model`: every file is
    checked against the manifest's sha256, the unquantised rest is copied into the parameters,
    projections whose codes a device kernel can consume become `QuantLinear` / `HQuantLinear`,
    and every other quantised tensor is decoded into its dense parameter. Returns counts."""
    import hashlib
    import json
    import os
    from ..train.quantization import PackedTensor, QuantError
    from . import weights as W
    with open(os.path.join(archive_dir, "archive-manifest.json")) as f:
        manifest = json.load(f)
    blobs = {}
    for ent in manifest["files"]:
        with open(os.path.join(archive_dir, ent["path"]), "rb") as f:
            data = f.read()
        if len(data) != ent["bytes"] or hashlib.sha256(data).hexdigest() != ent["sha256"]:
            raise QuantError(f"archive file {ent['path']} does not match the manifest")
        blobs[ent["path"]] = data
    params = dict(model.named_parameters())
    modules = dict(model.named_modules())
    rest = W.deserialize(blobs["rest.safetensors"])
    packed = {os.path.basename(k)[:-len(".hquant")]: PackedTensor.from_bytes(v)
              for k, v in blobs.items() if k.endswith(".hquant")}
    missing = sorted(set(params) - set(rest) - set(packed))
    if missing:
        raise QuantError(f"archive is missing {len(missing)} tensors, e.g. {missing[:3]}")
    with torch.no_grad():
        for name, t in rest.items():
            if name not in params or tuple(params[name].shape) != tuple(t.shape):
                raise QuantError(f"archive tensor {name} does not fit the model")
            params[name].copy_(t.to(device=params[name].device, dtype=params[name].dtype))
    swapped = decoded = 0
    for name, pt in sorted(packed.items()):
        p = params[name]
        if tuple(pt.shape) != tuple(p.shape):
            raise QuantError(f"archive tensor {name} has shape {tuple(pt.shape)}, the model {tuple(p.shape)}")
        mod_name, _, leaf = name.rpartition(".")
        mod = modules.get(mod_name)
        parent_name, _, child = mod_name.rpartition(".")
        parent = modules.get(parent_name) if mod_name else None
        new = None
        if isinstance(mod, Linear) and leaf == "weight" and parent is not None and mod is not getattr(model, "lm_head", None):
            bias = mod.bias.detach().to(torch.bfloat16) if mod.bias is not None else None
            if pt.format == "int4_g128" and mod.d_in % GROUP == 0 and mod.d_out % 4 == 0:
                K, N = pt.shape
                codes = torch.from_numpy(pt.codes.copy()).view(K // 2, N)
                scales = torch.from_numpy(pt.scales.copy().view("int16")).view(torch.bfloat16).view(K // GROUP, N)
                new = QuantLinear(codes.to(p.device), scales.to(p.device), bias)
            elif pt.format in ("binary_g128", "ternary_g128") and mod.d_out % GROUP == 0:
                new = HQuantLinear.from_packed(pt, bias, p.device)
        if new is not None:
            setattr(parent, child, new)
            swapped += 1
        else:
            with torch.no_grad():
                p.copy_(pt.decode().to(device=p.device, dtype=p.dtype))
            decoded += 1
    return {"format": manifest["format"], "kernel_layers": swapped, "decoded_tensors": decoded}
