"""Generation-sealed checkpoints with an atomic `current.json` pointer.

Layout (`summa-train/src/checkpoint.rs:48-92,280-307,631-767,1202-1330`):

    <out>/current.json                         {version:1, generation, manifest_sha256}
    <out>/generations/sha256-<h>/
        weights.safetensors                    model parameters (canonical bytes)
        adamw-state.bpk, muon-state.bpk        optimizer state containers
        training-state.json                    TrainingState v2
        training-accounting.json               parameter / GPU-hour accounting
        generation-manifest.json               {version:1, training_state_version:2,
                                                global_step, phase, phase_id, files[]}

A generation directory is named after the sha256 of its manifest, is written in a
staging directory and renamed into place, and is verified (every file's size and
sha256) before `current.json` is replaced by rename. Resume verifies again before
anything is loaded.

Deviation: the reference's `.bpk` members are burn-pack records, whose byte layout
lives in an external crate that is not part of the reference tree. The members keep
their names; their content here is this module's own container (magic `SB200PK1`,
JSON index sorted by tensor name, raw little-endian data), which is byte-stable for
identical state.
"""
from __future__ import annotations

import hashlib
import json
import os
import shutil
import struct
import tempfile
from dataclasses import asdict, dataclass, field
from typing import Any, Dict, List, Optional

import torch

from ..models import weights as W

PACK_MAGIC = b"SB200PK1"
TRAINING_STATE_VERSION = 2


class CheckpointError(RuntimeError):
    pass


# ------------------------------------------------------------------ optimizer container

def pack_tensors(tensors: Dict[str, torch.Tensor], scalars: Dict[str, float] = None,
                 metadata: Dict[str, str] = None) -> bytes:
    index, chunks, off = [], [], 0
    for name in sorted(tensors):
        t = tensors[name].detach().cpu().contiguous()
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        index.append({"name": name, "dtype": str(t.dtype).replace("torch.", ""), "shape": list(t.shape),
                      "offset": off, "bytes": len(raw)})
        chunks.append(raw)
        off += len(raw)
    head = json.dumps({"tensors": index, "scalars": dict(sorted((scalars or {}).items())),
                       "metadata": dict(sorted((metadata or {}).items()))},
                      separators=(",", ":"), sort_keys=True).encode()
    return PACK_MAGIC + struct.pack("<Q", len(head)) + head + b"".join(chunks)


def unpack_tensors(data: bytes):
    if data[:8] != PACK_MAGIC:
        raise CheckpointError("optimizer container has a bad magic")
    (n,) = struct.unpack("<Q", data[8:16])
    head = json.loads(data[16:16 + n])
    base = 16 + n
    out = {}
    for e in head["tensors"]:
        dt = getattr(torch, e["dtype"])
        raw = bytearray(data[base + e["offset"]:base + e["offset"] + e["bytes"]])
        t = torch.frombuffer(raw, dtype=dt).clone() if e["bytes"] else torch.empty(0, dtype=dt)
        out[e["name"]] = t.reshape(e["shape"])
    return out, head["scalars"], head["metadata"]


# ------------------------------------------------------------------ training state

@dataclass
class RngStream:
    name: str
    seed: int
    counter: int


@dataclass
class TrainingState:
    version: int = TRAINING_STATE_VERSION
    global_step: int = 0
    phase: int = 0
    phase_id: str = ""
    phase_kind: str = "pretrain"
    epoch: int = 0
    records_in_phase: int = 0
    steps_in_phase: int = 0
    tokens_seen: int = 0
    metric_records: int = 0
    workflow_signature: str = ""
    data_manifest_hash: str = ""
    parameter_ids: Dict[str, str] = field(default_factory=dict)
    optimizer_states: List[Dict[str, Any]] = field(default_factory=list)
    memory_update: Optional[Dict[str, Any]] = None
    sleep: Optional[Dict[str, Any]] = None
    artifacts: Dict[str, str] = field(default_factory=dict)
    evaluator_hashes: Dict[str, str] = field(default_factory=dict)
    rng_streams: List[RngStream] = field(default_factory=list)
    wake_context_buffer: Optional[Dict[str, Any]] = None
    quantization: Optional[Dict[str, Any]] = None

    def to_json(self) -> str:
        return json.dumps(asdict(self), indent=2, sort_keys=True)

    @staticmethod
    def from_json(s: str) -> "TrainingState":
        d = json.loads(s)
        if d.get("version") != TRAINING_STATE_VERSION:
            raise CheckpointError(f"unsupported training state version {d.get('version')}")
        known = {f for f in TrainingState.__dataclass_fields__}
        unknown = set(d) - known
        if unknown:
            raise CheckpointError(f"unknown training-state fields {sorted(unknown)}")
        # The file keeps the reference's field names and version, but several containers have this package's
        # own shapes (maps where the reference has arrays, optional members where it has required ones). A
        # version-2 state written by the reference must therefore fail here, loudly, instead of being misread.
        shapes = {"global_step": int, "phase": int, "phase_id": str, "phase_kind": str, "epoch": int,
                  "records_in_phase": int, "steps_in_phase": int, "tokens_seen": int, "metric_records": int,
                  "workflow_signature": str, "data_manifest_hash": str, "parameter_ids": dict, "optimizer_states": list,
                  "memory_update": (dict, type(None)), "sleep": (dict, type(None)), "artifacts": dict,
                  "evaluator_hashes": dict, "rng_streams": list, "wake_context_buffer": (dict, type(None)),
                  "quantization": (dict, type(None))}
        for key, typ in shapes.items():
            if key in d and (not isinstance(d[key], typ) or isinstance(d[key], bool)):
                raise CheckpointError(f"training-state field `{key}` has type {type(d[key]).__name__}: this file was "
                                      "not written by this package (the reference's own containers differ in shape)")
        streams = []
        for r in d.get("rng_streams", []):
            if not isinstance(r, dict) or set(r) != {"name", "seed", "counter"}:
                raise CheckpointError("training-state rng_streams entries must be {name, seed, counter}")
            streams.append(RngStream(**r))
        d["rng_streams"] = streams
        return TrainingState(**d)


# ------------------------------------------------------------------ helpers

def _sha256_file(path: str) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for chunk in iter(lambda: f.read(1 << 20), b""):
            h.update(chunk)
    return h.hexdigest()


def _write_sync(path: str, data: bytes) -> None:
    with open(path, "wb") as f:
        f.write(data)
        f.flush()
        os.fsync(f.fileno())


def _fsync_dir(path: str) -> None:
    fd = os.open(path, os.O_RDONLY)
    try:
        os.fsync(fd)
    finally:
        os.close(fd)


MEMBERS = ["weights.safetensors", "adamw-state.bpk", "muon-state.bpk", "training-state.json",
           "training-accounting.json"]


def seal_generation(out_dir: str, model, state: TrainingState, adamw_state: bytes, muon_state: bytes,
                    accounting: Dict[str, Any]) -> str:
    """Writes one immutable generation and returns its name (`sha256-<manifest hash>`)."""
    gens = os.path.join(out_dir, "generations")
    os.makedirs(gens, exist_ok=True)
    staging = tempfile.mkdtemp(prefix=".staging-", dir=gens)
    try:
        wbytes = W.serialize(W.model_tensors(model))
        _write_sync(os.path.join(staging, "weights.safetensors"), wbytes)
        acc = dict(accounting)
        acc.update({"version": 1, "weights_bytes": len(wbytes), "weights_sha256": hashlib.sha256(wbytes).hexdigest()})
        _write_sync(os.path.join(staging, "training-accounting.json"),
                    json.dumps(acc, indent=2, sort_keys=True).encode())
        _write_sync(os.path.join(staging, "adamw-state.bpk"), adamw_state)
        _write_sync(os.path.join(staging, "muon-state.bpk"), muon_state)
        _write_sync(os.path.join(staging, "training-state.json"), state.to_json().encode())
        files = []
        for m in MEMBERS:
            p = os.path.join(staging, m)
            files.append({"path": m, "bytes": os.path.getsize(p), "sha256": _sha256_file(p)})
        manifest = {"version": 1, "training_state_version": TRAINING_STATE_VERSION,
                    "global_step": state.global_step, "phase": state.phase, "phase_id": state.phase_id,
                    "files": files}
        mbytes = json.dumps(manifest, indent=2, sort_keys=True).encode()
        _write_sync(os.path.join(staging, "generation-manifest.json"), mbytes)
        name = "sha256-" + hashlib.sha256(mbytes).hexdigest()
        final = os.path.join(gens, name)
        if os.path.exists(final):
            shutil.rmtree(staging)
        else:
            os.rename(staging, final)
        _fsync_dir(gens)
        return name
    except BaseException:
        shutil.rmtree(staging, ignore_errors=True)
        raise


def verify_generation(out_dir: str, name: str) -> Dict[str, Any]:
    """Checks the manifest hash and every member's size and sha256; returns the manifest."""
    d = os.path.join(out_dir, "generations", name)
    mp = os.path.join(d, "generation-manifest.json")
    if not os.path.isfile(mp):
        raise CheckpointError(f"generation {name} has no manifest")
    mbytes = open(mp, "rb").read()
    if "sha256-" + hashlib.sha256(mbytes).hexdigest() != name:
        raise CheckpointError(f"generation {name}: manifest hash does not match its directory name")
    manifest = json.loads(mbytes)
    listed = {f["path"] for f in manifest["files"]}
    present = {n for n in os.listdir(d) if n != "generation-manifest.json"}
    if listed != present:
        raise CheckpointError(f"generation {name}: members {sorted(present)} differ from manifest {sorted(listed)}")
    for f in manifest["files"]:
        p = os.path.join(d, f["path"])
        if os.path.islink(p) or not os.path.isfile(p):
            raise CheckpointError(f"generation {name}: {f['path']} is not a regular file")
        if os.path.getsize(p) != f["bytes"] or _sha256_file(p) != f["sha256"]:
            raise CheckpointError(f"generation {name}: {f['path']} failed verification")
    return manifest


def publish_current(out_dir: str, name: str) -> None:
    verify_generation(out_dir, name)
    mp = os.path.join(out_dir, "generations", name, "generation-manifest.json")
    ptr = {"version": 1, "generation": name, "manifest_sha256": _sha256_file(mp)}
    fd, tmp = tempfile.mkstemp(prefix=".current-", suffix=".tmp", dir=out_dir)
    with os.fdopen(fd, "wb") as f:
        f.write(json.dumps(ptr, indent=2, sort_keys=True).encode())
        f.flush()
        os.fsync(f.fileno())
    os.replace(tmp, os.path.join(out_dir, "current.json"))
    _fsync_dir(out_dir)


def read_current(out_dir: str) -> Optional[str]:
    p = os.path.join(out_dir, "current.json")
    if not os.path.exists(p):
        return None
    ptr = json.load(open(p))
    if ptr.get("version") != 1:
        raise CheckpointError("unsupported current.json version")
    return ptr["generation"]


def save_training_checkpoint(out_dir: str, model, state: TrainingState, adamw_state: bytes = b"",
                             muon_state: bytes = b"", accounting: Dict[str, Any] = None) -> str:
    name = seal_generation(out_dir, model, state, adamw_state or pack_tensors({}), muon_state or pack_tensors({}),
                           accounting or {})
    publish_current(out_dir, name)
    return name


def load_training_state(out_dir: str, model, stage_hook=None):
    """Verify → read → verify again → load. `stage_hook(stage_name, dir)` lets tests
    mutate files between stages to prove that a changed root is rejected.
    Returns (TrainingState, adamw bytes, muon bytes, generation name)."""
    name = read_current(out_dir)
    if name is None:
        raise CheckpointError(f"{out_dir} has no current.json")
    manifest = verify_generation(out_dir, name)
    d = os.path.join(out_dir, "generations", name)
    if stage_hook:
        stage_hook("verified", d)
    blobs = {}
    for f in manifest["files"]:
        data = open(os.path.join(d, f["path"]), "rb").read()
        if len(data) != f["bytes"] or hashlib.sha256(data).hexdigest() != f["sha256"]:
            raise CheckpointError(f"{f['path']} changed between verification and load")
        blobs[f["path"]] = data
    if stage_hook:
        stage_hook("read", d)
    state = TrainingState.from_json(blobs["training-state.json"].decode())
    if state.global_step != manifest["global_step"]:
        raise CheckpointError("training state and manifest disagree on global_step")
    W.load_safetensors_bytes(model, blobs["weights.safetensors"])
    return state, blobs["adamw-state.bpk"], blobs["muon-state.bpk"], name
