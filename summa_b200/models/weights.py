"""safetensors weight I/O with the reference's discipline: strict loads (missing,
unused or mis-shaped tensors are errors and leave the model untouched), a canonical
header so identical weights serialise to identical bytes, atomic publication, and the
FFN → memory-chain key upgrade (`summa-llm/src/model/weights.rs:18-63,69-133,141-241`).

The container format is implemented here directly (8-byte little-endian header length,
JSON header, raw little-endian tensor bytes), which keeps the byte layout under our
control: header keys are emitted in sorted order, data is laid out in that same order
with no padding beyond the 8-byte header alignment.
"""
from __future__ import annotations

import hashlib
import json
import os
import struct
import tempfile
from typing import Dict, Iterable, Tuple

import torch

_DTYPES = {
    "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16, "F64": torch.float64,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
    "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class WeightsError(ValueError):
    pass


def serialize(tensors: Dict[str, torch.Tensor]) -> bytes:
    """Canonical safetensors bytes: keys sorted, offsets contiguous in key order."""
    header = {}
    chunks = []
    offset = 0
    for name in sorted(tensors):
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise WeightsError(f"unsupported dtype {t.dtype} for '{name}'")
        raw = t.view(torch.uint8).numpy().tobytes() if t.dtype != torch.bool else \
            t.to(torch.uint8).numpy().tobytes()
        if t.dtype == torch.bfloat16:
            raw = t.view(torch.int16).numpy().tobytes()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + len(raw)]}
        chunks.append(raw)
        offset += len(raw)
    hjson = json.dumps(header, separators=(",", ":"), sort_keys=True).encode("utf-8")
    pad = (8 - len(hjson) % 8) % 8
    hjson += b" " * pad
    return struct.pack("<Q", len(hjson)) + hjson + b"".join(chunks)


def deserialize(data: bytes) -> Dict[str, torch.Tensor]:
    if len(data) < 8:
        raise WeightsError("file too small for a safetensors header")
    (hlen,) = struct.unpack("<Q", data[:8])
    if hlen > len(data) - 8 or hlen > (1 << 27):
        raise WeightsError("invalid safetensors header length")
    try:
        header = json.loads(data[8:8 + hlen].decode("utf-8"))
    except Exception as e:
        raise WeightsError(f"invalid safetensors header: {e}")
    base = 8 + hlen
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        dt = _DTYPES.get(meta["dtype"])
        if dt is None:
            raise WeightsError(f"unsupported dtype {meta['dtype']} for '{name}'")
        lo, hi = meta["data_offsets"]
        shape = tuple(meta["shape"])
        n = 1
        for s in shape:
            n *= s
        esize = 1 if dt == torch.bool else torch.empty((), dtype=dt).element_size()
        if hi - lo != n * esize or base + hi > len(data):
            raise WeightsError(f"tensor '{name}' has inconsistent size")
        buf = bytearray(data[base + lo:base + hi])
        if dt == torch.bool:
            t = torch.frombuffer(buf, dtype=torch.uint8).to(torch.bool) if n else torch.empty(0, dtype=torch.bool)
        elif n:
            t = torch.frombuffer(buf, dtype=dt)
        else:
            t = torch.empty(0, dtype=dt)
        out[name] = t.reshape(shape).clone()
    return out


def model_tensors(model) -> Dict[str, torch.Tensor]:
    """Checkpointed tensors: every parameter (trainable or state flags); derived
    caches such as RoPE tables are never serialised."""
    return {name: p.detach() for name, p in model.named_parameters()}


def save_safetensors(model, path: str, dtype: torch.dtype = None) -> str:
    """Atomic save (write to a temp file in the same directory, fsync, rename). Returns
    the sha256 of the written bytes."""
    tensors = model_tensors(model)
    if dtype is not None:
        tensors = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
    data = serialize(tensors)
    d = os.path.dirname(os.path.abspath(path))
    os.makedirs(d, exist_ok=True)
    fd, tmp = tempfile.mkstemp(prefix=".weights-", dir=d)
    try:
        with os.fdopen(fd, "wb") as f:
            f.write(data)
            f.flush()
            os.fsync(f.fileno())
        os.replace(tmp, path)
    except BaseException:
        if os.path.exists(tmp):
            os.unlink(tmp)
        raise
    return hashlib.sha256(data).hexdigest()


def load_safetensors_bytes(model, data: bytes) -> None:
    """Strict load: validates everything first, mutates the model only on success."""
    tensors = deserialize(data)
    params = dict(model.named_parameters())
    missing = sorted(set(params) - set(tensors))
    unused = sorted(set(tensors) - set(params))
    if missing:
        raise WeightsError(f"checkpoint is missing {len(missing)} tensors, e.g. {missing[:3]}")
    if unused:
        raise WeightsError(f"checkpoint has {len(unused)} unused tensors, e.g. {unused[:3]}")
    for name, p in params.items():
        if tuple(tensors[name].shape) != tuple(p.shape):
            raise WeightsError(f"shape mismatch for '{name}': checkpoint {tuple(tensors[name].shape)} "
                               f"vs model {tuple(p.shape)}")
    with torch.no_grad():
        for name, p in params.items():
            p.copy_(tensors[name].to(device=p.device, dtype=p.dtype))


def load_safetensors(model, path: str) -> str:
    with open(path, "rb") as f:
        data = f.read()
    load_safetensors_bytes(model, data)
    return hashlib.sha256(data).hexdigest()


def upgrade_safetensors_to_memory(data: bytes, memory_model) -> bytes:
    """Remap a plain-FFN checkpoint onto a memory-chain model: `layers.N.feed_forward.*`
    becomes `layers.N.memory.tiers.0.feed_forward.*`; every tensor the memory model adds
    (later tiers, reserve slots) keeps the freshly initialised value of `memory_model`."""
    old = deserialize(data)
    new = {k: v.detach().cpu() for k, v in model_tensors(memory_model).items()}
    for key, t in old.items():
        parts = key.split(".")
        if len(parts) > 3 and parts[0] == "layers" and parts[2] == "feed_forward":
            mapped = ".".join(parts[:2] + ["memory", "tiers", "0"] + parts[2:])
            if mapped in new:
                key = mapped
        if key not in new:
            raise WeightsError(f"tensor '{key}' has no place in the memory model")
        if tuple(new[key].shape) != tuple(t.shape):
            raise WeightsError(f"shape mismatch for '{key}' during upgrade")
        new[key] = t
    return serialize(new)
