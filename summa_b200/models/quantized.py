"""4-bit group-quantised linear layers for inference.

`QuantLinear` holds a `[d_in, d_out]` weight as packed int4 codes (group 128 along d_in,
bf16 scales). Decode-sized inputs (<= 64 rows) run the weight-streaming GEMV kernel, which
reads the packed weight once; larger inputs (prefill) dequantise the weight into a reused
bf16 workspace and run the tensor-core GEMM. The reference has only a host-side oracle for
quantised mat-vec (`summa-train/src/quantization.rs:626-654`); this is the device path.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from .. import ops
from ..ops import reference
from .layers import Linear

GROUP = 128
_workspace = {}


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

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        """`residual` (same shape as the output) is added in the kernel epilogue on the decode path."""
        lead = x.shape[:-1]
        x2 = x.reshape(-1, self.d_in)
        if x2.is_cuda and x2.dtype == torch.bfloat16:
            if x2.shape[0] <= 64:
                if residual is not None and self.bias is None:
                    return ops.int4_gemv(x2, self.packed, self.scales, residual.reshape(-1, self.d_out),
                                         self.packed_k8()).view(*lead, self.d_out)
                y = ops.int4_gemv(x2, self.packed, self.scales, None, self.packed_k8())
            else:
                y = ops.linear(x2, self.dequantized(), None)
        else:
            y = (x2.float() @ self.dequantized().float()).to(x.dtype)
        if self.bias is not None:
            y = y + self.bias.to(y.dtype)
        y = y.view(*lead, self.d_out)
        return y if residual is None else y + residual


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
