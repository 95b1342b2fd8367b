"""Low-bit group-quantised weights: HQUANT codecs, the 4-bit g128 format, STE fake
quantisation for QAT, archive export.

HQUANT tensor file (`summa-train/src/quantization.rs:34-38,416-523,691-771`):
    "HQUANT1\\0" | u16 codec version (1) | u8 format tag | u16 group size (128) | u8 rank |
    u64 dims... | u64 n_scales | u64 n_codes | fp16 scales (LE) | codes | u64 FNV-1a checksum
Formats: binary_g128 (tag 1: 1 bit / weight, LSB first, bit 1 = +scale, scale = mean|w|),
ternary_g128 (tag 2: 2 bits, 0 = -s, 1 = 0, 2 = +s), ternary_entropy_g128 (tag 3: five
trits per byte, base 3). Groups run over the FLATTENED tensor; the last group is
zero-padded in storage only. The ternary scale / support is the L2-optimal prefix of
the magnitudes sorted in descending order.

int4_g128 (tag 16) is this framework's addition for inference: symmetric 4-bit codes in
[-8, 7], groups of 128 along the INPUT dimension of a `[d_in, d_out]` matrix, bf16
scales `[d_in / 128, d_out]`, two codes per byte (low nibble = even row) — the layout
the dequant-GEMM kernels consume directly.
"""
from __future__ import annotations

import json
import os
import struct
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch

from .workflow import fnv1a64

MAGIC = b"HQUANT1\x00"
CODEC_VERSION = 1
GROUP = 128
TAGS = {"binary_g128": 1, "ternary_g128": 2, "ternary_entropy_g128": 3, "int4_g128": 16}
NAMES = {v: k for k, v in TAGS.items()}


class QuantError(ValueError):
    pass


@dataclass
class PackedTensor:
    format: str
    shape: Tuple[int, ...]
    group_size: int
    scales: np.ndarray        # uint16 bits (fp16; bf16 for int4_g128)
    codes: np.ndarray         # uint8

    def elements(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n

    def bits_per_weight(self) -> float:
        return 8.0 * (self.scales.size * 2 + self.codes.size) / self.elements()

    # ------------------------------------------------------------------ container
    def to_bytes(self) -> bytes:
        p = bytearray(MAGIC)
        p += struct.pack("<H", CODEC_VERSION)
        p += struct.pack("<B", TAGS[self.format])
        p += struct.pack("<H", self.group_size)
        p += struct.pack("<B", len(self.shape))
        for d in self.shape:
            p += struct.pack("<Q", d)
        p += struct.pack("<QQ", self.scales.size, self.codes.size)
        p += self.scales.astype("<u2").tobytes()
        p += self.codes.astype(np.uint8).tobytes()
        p += struct.pack("<Q", fnv1a64(bytes(p)))
        return bytes(p)

    @staticmethod
    def from_bytes(data: bytes) -> "PackedTensor":
        if len(data) < len(MAGIC) + 2 + 1 + 2 + 1 + 8:
            raise QuantError("quantized tensor is truncated")
        payload, chk = data[:-8], data[-8:]
        if struct.unpack("<Q", chk)[0] != fnv1a64(payload):
            raise QuantError("quantized tensor checksum mismatch")
        if payload[:8] != MAGIC:
            raise QuantError("not an HQUANT tensor")
        o = 8
        ver, tag, group, rank = struct.unpack_from("<HBHB", payload, o)
        o += 6
        if ver != CODEC_VERSION or tag not in NAMES:
            raise QuantError("unsupported HQUANT version or format")
        shape = struct.unpack_from(f"<{rank}Q", payload, o)
        o += 8 * rank
        ns, nc = struct.unpack_from("<QQ", payload, o)
        o += 16
        if len(payload) != o + 2 * ns + nc:
            raise QuantError("HQUANT payload size does not match its header")
        scales = np.frombuffer(payload, dtype="<u2", count=ns, offset=o).copy()
        codes = np.frombuffer(payload, dtype=np.uint8, count=nc, offset=o + 2 * ns).copy()
        return PackedTensor(NAMES[tag], tuple(shape), group, scales, codes)

    # ------------------------------------------------------------------ decode
    def decode(self) -> torch.Tensor:
        n = self.elements()
        if self.format == "int4_g128":
            K, N = self.shape
            packed = torch.from_numpy(self.codes.reshape(K // 2, N))
            scale = torch.from_numpy(self.scales.astype(np.int16)).view(torch.bfloat16).reshape(K // self.group_size, N)
            from ..ops.reference import dequantize_int4_g128
            return dequantize_int4_g128(packed, scale, self.group_size)
        scales = torch.from_numpy(self.scales.astype(np.int16)).view(torch.float16).float()
        g = self.group_size
        groups = scales.numel()
        codes = torch.from_numpy(self.codes)
        if self.format == "binary_g128":
            bits = ((codes.view(groups, g // 8, 1) >> torch.arange(8, dtype=torch.uint8)) & 1).reshape(groups, g)
            vals = (bits.float() * 2 - 1) * scales[:, None]
        elif self.format == "ternary_g128":
            c = ((codes.view(groups, g // 4, 1) >> (torch.arange(4, dtype=torch.uint8) * 2)) & 3).reshape(groups, g)
            if (c == 3).any():
                raise QuantError("reserved ternary code 3")
            vals = (c.float() - 1) * scales[:, None]
        else:
            bpg = -(-g // 5)
            b = codes.view(groups, bpg).to(torch.int32)
            if (b >= 243).any():
                raise QuantError("invalid base-3 packed byte")
            trits = torch.stack([(b // (3 ** i)) % 3 for i in range(5)], dim=-1).reshape(groups, bpg * 5)[:, :g]
            vals = (trits.float() - 1) * scales[:, None]
        return vals.reshape(-1)[:n].reshape(self.shape)

    def matrix_vector(self, x: torch.Tensor) -> torch.Tensor:
        """Host oracle: y = W^T-free product `x @ decode()` for a rank-2 tensor."""
        return x.float() @ self.decode().float()


def _optimal_ternary(groups: torch.Tensor):
    """Per row of `[G, 128]`: scale and {0,1,2} codes minimising the L2 error."""
    mag, order = groups.abs().sort(dim=1, descending=True)
    csum = mag.double().cumsum(dim=1)
    k = torch.arange(1, groups.shape[1] + 1, dtype=torch.float64)
    gain = csum * csum / k
    best = gain.argmax(dim=1)
    scale = (csum.gather(1, best[:, None]).squeeze(1) / (best + 1).double()).float()
    rank_of = torch.empty_like(order)
    rank_of.scatter_(1, order, torch.arange(groups.shape[1]).expand_as(order))
    support = rank_of <= best[:, None]
    trit = torch.where(support, torch.where(groups >= 0, 2, 0), 1).to(torch.uint8)
    trit = torch.where(support & (groups == 0), torch.ones_like(trit), trit)
    return scale, trit


def quantize_tensor(w: torch.Tensor, fmt: str, group_size: int = GROUP) -> PackedTensor:
    if group_size != GROUP:
        raise QuantError("only g128 is supported")
    if fmt not in TAGS:
        raise QuantError(f"unknown format {fmt}")
    wf = w.detach().float().cpu()
    if wf.numel() == 0 or not torch.isfinite(wf).all():
        raise QuantError("cannot quantize an empty or non-finite tensor")
    if fmt == "int4_g128":
        if wf.dim() != 2 or wf.shape[0] % group_size:
            raise QuantError("int4_g128 needs a [d_in, d_out] matrix with d_in % 128 == 0")
        from ..ops.reference import quantize_int4_g128
        packed, scale = quantize_int4_g128(wf, group_size)
        return PackedTensor(fmt, tuple(wf.shape), group_size,
                            scale.view(torch.int16).numpy().astype(np.uint16).reshape(-1), packed.numpy().reshape(-1))
    n = wf.numel()
    groups = -(-n // group_size)
    flat = torch.zeros(groups * group_size)
    flat[:n] = wf.reshape(-1)
    G = flat.view(groups, group_size)
    if fmt == "binary_g128":
        # the mean runs over the REAL elements of a ragged last group
        cnt = torch.full((groups,), float(group_size))
        if n % group_size:
            cnt[-1] = n % group_size
        scale = (G.abs().double().sum(dim=1) / cnt.double()).float()
        bits = (G >= 0).to(torch.uint8)
        if n % group_size:
            bits[-1, n % group_size:] = 0
        codes = (bits.view(groups, group_size // 8, 8) << torch.arange(8, dtype=torch.uint8)).sum(dim=-1).to(torch.uint8)
    else:
        if n % group_size:
            last = G[-1:, :n % group_size]
            s_last, t_last = _optimal_ternary(last)
            s_main, t_main = _optimal_ternary(G[:-1]) if groups > 1 else (torch.empty(0), torch.empty(0, group_size, dtype=torch.uint8))
            pad = torch.zeros(1, group_size, dtype=torch.uint8)
            pad[:, :n % group_size] = t_last
            if fmt == "ternary_entropy_g128":
                pad[:, n % group_size:] = 0
            scale = torch.cat([s_main, s_last])
            trit = torch.cat([t_main, pad])
        else:
            scale, trit = _optimal_ternary(G)
        if fmt == "ternary_g128":
            codes = (trit.view(groups, group_size // 4, 4) << (torch.arange(4, dtype=torch.uint8) * 2)).sum(dim=-1).to(torch.uint8)
        else:
            bpg = -(-group_size // 5)
            t = torch.zeros(groups, bpg * 5, dtype=torch.int32)
            t[:, :group_size] = trit.to(torch.int32)
            codes = (t.view(groups, bpg, 5) * torch.tensor([1, 3, 9, 27, 81], dtype=torch.int32)).sum(dim=-1).to(torch.uint8)
    s16 = scale.to(torch.float16)
    if not torch.isfinite(s16.float()).all():
        raise QuantError("a quantization group scale is outside the finite FP16 range")
    return PackedTensor(fmt, tuple(wf.shape), group_size,
                        s16.view(torch.int16).numpy().astype(np.uint16), codes.reshape(-1).numpy())


def fake_quantize(w: torch.Tensor, fmt: str, group_size: int = GROUP) -> torch.Tensor:
    """Device fake-quant with the straight-through estimator: `w + (q(w) − w).detach()`.
    Same code / scale estimator as the codec, scales kept in the training dtype. The binary
    and ternary forms are one kernel on CUDA (`ops/csrc/hquant.cu`)."""
    if group_size != GROUP:
        raise QuantError("only g128 is supported")
    if fmt in ("binary_g128", "ternary_g128", "ternary_entropy_g128"):
        from .. import ops
        return ops.fake_quant(w, fmt)
    if fmt == "int4_g128":
        if w.dim() != 2 or w.shape[0] % group_size:
            raise QuantError("int4_g128 needs a [d_in, d_out] matrix with d_in % 128 == 0")
        wf = w.detach().float().view(w.shape[0] // group_size, group_size, w.shape[1])
        s = (wf.abs().amax(dim=1, keepdim=True) / 7.0).clamp_min(1e-8)
        qq = (torch.round(wf / s).clamp_(-8, 7) * s).view(w.shape)
        return w + (qq.to(w.dtype) - w).detach()
    raise QuantError(f"unknown format {fmt}")


@torch.no_grad()
def fake_quant_values(w: torch.Tensor, fmt: str) -> torch.Tensor:
    """dequant(quant(w)) without the autograd wrapper."""
    return fake_quantize(w.detach(), fmt).detach()


def qat_parameter_names(model, include_embeddings: bool = True, include_head: bool = True) -> List[str]:
    """Every rank >= 2 parameter, optionally minus embeddings / head. A tied embedding / head is
    one tensor, so both switches must agree for it (`summa-train/src/quantization.rs:792-932`)."""
    tied = getattr(model, "lm_head", None) is None
    if tied and include_embeddings != include_head:
        raise QuantError("tied embedding / lm_head weights need the same embeddings and lm_head setting")
    return model.quant_parameter_names(include_embeddings, include_head)


def quantize_model(model, fmt: str, include_embeddings: bool = True, include_head: bool = True) -> Dict[str, PackedTensor]:
    names = model.quant_parameter_names(include_embeddings, include_head)
    params = dict(model.named_parameters())
    out = {}
    for n in names:
        p = params[n]
        if fmt == "int4_g128" and (p.dim() != 2 or p.shape[0] % GROUP):
            continue
        out[n] = quantize_tensor(p, fmt)
    return out


def export_archive(model, fmt: str, out_dir: str, include_embeddings=True, include_head=True) -> Dict[str, object]:
    """Writes `<out>/tensors/<name>.hquant` for every quantised tensor, the remaining
    parameters as `rest.safetensors`, and `archive-manifest.json` with sizes and hashes."""
    import hashlib
    from ..models import weights as W
    os.makedirs(os.path.join(out_dir, "tensors"), exist_ok=True)
    packed = quantize_model(model, fmt, include_embeddings, include_head)
    files = []
    total_bits, total_elems = 0.0, 0
    for name, pt in sorted(packed.items()):
        data = pt.to_bytes()
        rel = os.path.join("tensors", name + ".hquant")
        with open(os.path.join(out_dir, rel), "wb") as f:
            f.write(data)
        files.append({"path": rel, "bytes": len(data), "sha256": hashlib.sha256(data).hexdigest()})
        total_bits += 8.0 * len(data)
        total_elems += pt.elements()
    rest = {n: p.detach() for n, p in model.named_parameters() if n not in packed}
    rb = W.serialize(rest)
    with open(os.path.join(out_dir, "rest.safetensors"), "wb") as f:
        f.write(rb)
    files.append({"path": "rest.safetensors", "bytes": len(rb), "sha256": hashlib.sha256(rb).hexdigest()})
    manifest = {"version": 1, "format": fmt, "group_size": GROUP, "quantized_tensors": len(packed),
                "bits_per_quantized_weight": total_bits / max(total_elems, 1), "files": files}
    with open(os.path.join(out_dir, "archive-manifest.json"), "w") as f:
        json.dump(manifest, f, indent=2, sort_keys=True)
    return manifest


def quantize_command(args) -> Dict[str, object]:
    from .. import mal
    from ..models import Transformer
    from ..models import weights as W
    cfg = mal.load_model_def(args.model)
    if getattr(args, "tokenizer", None):
        from ..tokenizer import Tokenizer
        cfg.vocab_size = Tokenizer.from_file(args.tokenizer).vocab_size()
    model = Transformer(cfg)
    W.load_safetensors(model, args.checkpoint)
    manifest = export_archive(model, args.format, args.output, getattr(args, "quantize_embeddings", True), getattr(args, "quantize_lm_head", True))
    recipe = {"ternary_warmup_steps": int(getattr(args, "ternary_warmup_steps", 0) or 0),
              "distillation_weight": float(getattr(args, "distillation_weight", 0.0) or 0.0)}
    if recipe["ternary_warmup_steps"] < 0 or not (recipe["distillation_weight"] >= 0.0):
        raise ValueError("ternary warm-up steps and the distillation weight must be non-negative")
    with open(os.path.join(args.output, "training-recipe.json"), "w") as f:       # beside the sealed manifest, never inside it
        json.dump(recipe, f, sort_keys=True)
    return dict(manifest, training_recipe=recipe)
