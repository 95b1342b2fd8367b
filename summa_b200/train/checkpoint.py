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


def _sha_identity(v: Optional[str]) -> Optional[str]:
    return None if not v else (v if v.startswith("sha256:") else "sha256:" + v)


def _strip_identity(v: Optional[str]) -> Optional[str]:
    return v[7:] if isinstance(v, str) and v.startswith("sha256:") else v


_STATE_SHAPES = {"optimizer_states": {"scope": str, "adamw": str, "muon": str, "gradient_accumulator": (str, type(None)), "update_clock": int},
                 "artifacts": {"kind": str, "manifest": str, "hash": str},
                 "rng_streams": {"name": str, "seed": int, "counter": int},
                 "wake_context_buffer": {"id": str, "optimizer_step": int, "token_ids": list}}
_QUANT_SHAPE = {"format": str, "fake_quant_active": bool, "calibration_step": int, "manifest": (str, type(None)),
                "candidate_weights_sha256": (str, type(None)), "teacher_hash": (str, type(None))}
MAX_WAKE_CONTEXT_RECORDS = 4096


@dataclass
class TrainingState:
    """`training-state.json` in the container shapes of `summa-train/src/checkpoint.rs:216-307`: every field is
    required on disk, `parameter_ids` / `artifacts` / `evaluator_hashes` / `wake_context_buffer` are arrays,
    `memory_update` is a tagged object (`ordinary` | `periodic_sleep` | `wake_only{config, optimizer_scopes}`), hashes
    use the `sha256:<hex>` identity form. In memory the signature and the data hash stay bare hex."""
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
    data_manifest_hash: Optional[str] = None
    parameter_ids: List[int] = field(default_factory=list)
    optimizer_states: List[Dict[str, Any]] = field(default_factory=list)
    memory_update: Dict[str, Any] = field(default_factory=lambda: {"type": "ordinary"})
    sleep: Optional[Dict[str, Any]] = None
    artifacts: List[Dict[str, str]] = field(default_factory=list)
    evaluator_hashes: List[str] = field(default_factory=list)
    rng_streams: List[RngStream] = field(default_factory=list)
    wake_context_buffer: List[Dict[str, Any]] = field(default_factory=list)
    quantization: Optional[Dict[str, Any]] = None

    def to_json(self) -> str:
        d = asdict(self)
        d["workflow_signature"] = _sha_identity(self.workflow_signature) or ""
        d["data_manifest_hash"] = _sha_identity(self.data_manifest_hash)
        return json.dumps(d, indent=2, sort_keys=True)

    @staticmethod
    def from_json(s: str) -> "TrainingState":
        d = json.loads(s)
        if not isinstance(d, dict) or d.get("version") != TRAINING_STATE_VERSION:
            raise CheckpointError(f"unsupported training state version {d.get('version') if isinstance(d, dict) else None}")
        known = set(TrainingState.__dataclass_fields__)
        unknown, missing = set(d) - known, known - set(d)
        if unknown:
            raise CheckpointError(f"unknown training-state fields {sorted(unknown)}")
        if missing:
            raise CheckpointError(f"training state lacks {sorted(missing)}: a version-{TRAINING_STATE_VERSION} state has no defaults")
        # files of earlier generations of this package: empty maps where arrays belong, null for the ordinary mode
        for key in ("parameter_ids", "artifacts", "evaluator_hashes"):
            if d[key] == {}:
                d[key] = []
        if d["memory_update"] is None:
            d["memory_update"] = {"type": "ordinary"}
        if d["wake_context_buffer"] is None:
            d["wake_context_buffer"] = []
        if d["data_manifest_hash"] == "":
            d["data_manifest_hash"] = None

        def bad(key: str, why: str):
            raise CheckpointError(f"training-state field `{key}` {why}")
        for key in ("global_step", "phase", "epoch", "records_in_phase", "steps_in_phase", "tokens_seen", "metric_records"):
            if not isinstance(d[key], int) or isinstance(d[key], bool) or d[key] < 0:
                bad(key, "must be a non-negative integer")
        for key in ("phase_id", "phase_kind", "workflow_signature"):
            if not isinstance(d[key], str) or not d[key].strip():
                bad(key, "must be a non-empty string")
        for key in ("workflow_signature", "data_manifest_hash"):
            v = _strip_identity(d[key])
            if v is not None and not (isinstance(v, str) and len(v) == 64 and all(c in "0123456789abcdef" for c in v)):
                bad(key, "must use the `sha256:<64 lowercase hex>` form")
            d[key] = v
        if not isinstance(d["parameter_ids"], list) or any(not isinstance(v, int) or isinstance(v, bool) or not 0 <= v < 1 << 64 for v in d["parameter_ids"]):
            bad("parameter_ids", "must be an array of unsigned 64-bit integers")
        if not isinstance(d["evaluator_hashes"], list) or any(not isinstance(v, str) for v in d["evaluator_hashes"]):
            bad("evaluator_hashes", "must be an array of strings")
        for key, shape in _STATE_SHAPES.items():
            if not isinstance(d[key], list):
                bad(key, "must be an array")
            for row in d[key]:
                if not isinstance(row, dict) or set(row) != set(shape) or any(not isinstance(row[k], t) or (t is int and isinstance(row[k], bool))
                                                                              for k, t in shape.items()):
                    bad(key, f"entries must be {{{', '.join(shape)}}} with the reference's types")
        if len(d["wake_context_buffer"]) > MAX_WAKE_CONTEXT_RECORDS:
            bad("wake_context_buffer", f"exceeds the {MAX_WAKE_CONTEXT_RECORDS}-record limit")
        mu = d["memory_update"]
        if not isinstance(mu, dict) or mu.get("type") not in ("ordinary", "periodic_sleep", "wake_only") or \
                set(mu) != ({"type", "config", "optimizer_scopes"} if mu.get("type") == "wake_only" else {"type"}):
            bad("memory_update", "must be {type: ordinary | periodic_sleep} or {type: wake_only, config, optimizer_scopes}")
        if d["sleep"] is not None and not isinstance(d["sleep"], dict):
            bad("sleep", "must be an object or null")
        q = d["quantization"]
        if q is not None and (not isinstance(q, dict) or set(q) != set(_QUANT_SHAPE) or any(not isinstance(q[k], t) for k, t in _QUANT_SHAPE.items())):
            bad("quantization", f"must be null or {{{', '.join(_QUANT_SHAPE)}}}")
        if d["global_step"] > 0 and d["tokens_seen"] == 0 and d["phase_kind"] != "evaluation":
            raise CheckpointError("non-evaluation checkpoint has optimizer progress but no token count")
        d["rng_streams"] = [RngStream(**r) for r in d["rng_streams"]]
        return TrainingState(**d)


def parameter_ids_of(model) -> List[int]:
    """Stable 64-bit identities of the model's parameters in registration order (the first eight bytes of the SHA-256
    of each qualified name): persisted so that a resume can tell a re-ordered or renamed parameter set."""
    return [int.from_bytes(hashlib.sha256(name.encode()).digest()[:8], "big") for name, _ in model.named_parameters()]


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
        if not state.parameter_ids and hasattr(model, "named_parameters"):
            state.parameter_ids = parameter_ids_of(model)
        state.optimizer_states = [r for r in state.optimizer_states if r.get("scope") != "wake"] + [
            {"scope": "wake", "adamw": "adamw-state.bpk", "muon": "muon-state.bpk", "gradient_accumulator": None,
             "update_clock": state.global_step}]
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


def verify_checkpoint_generation(directory: str, name: str, manifest_sha256: str) -> Dict[str, Any]:
    """One materialised generation directory (wherever it lies) against its content-addressed name and manifest digest:
    every member's size and hash, and the training state under the strict schema
    (`summa-train/src/main.rs:1722-1760`). Returns `{global_step, generation, manifest_sha256, metric_records, ...}`."""
    directory = os.path.normpath(directory)
    if os.path.basename(directory) != name:
        raise CheckpointError(f"generation directory {directory} is not named {name}")
    manifest = verify_generation(os.path.dirname(os.path.dirname(directory)), name) \
        if os.path.basename(os.path.dirname(directory)) == "generations" else _verify_loose_generation(directory, name)
    digest = _sha256_file(os.path.join(directory, "generation-manifest.json"))
    if digest != manifest_sha256.removeprefix("sha256:"):
        raise CheckpointError(f"generation {name}: manifest hashes to {digest}, expected {manifest_sha256}")
    with open(os.path.join(directory, "training-state.json"), "r", encoding="utf-8") as f:
        state = TrainingState.from_json(f.read())
    if state.global_step != manifest["global_step"]:
        raise CheckpointError("training state and manifest disagree on global_step")
    return {"global_step": state.global_step, "generation": name, "manifest_sha256": digest, "metric_records": state.metric_records,
            "phase": state.phase, "phase_id": state.phase_id, "tokens_seen": state.tokens_seen, "files": len(manifest["files"]),
            "workflow_signature": _sha_identity(state.workflow_signature)}


def _verify_loose_generation(directory: str, name: str) -> Dict[str, Any]:
    """`verify_generation` for a generation copied out of its `generations/` folder (a mirror's staging area)."""
    parent = os.path.dirname(directory)
    link_root = tempfile.mkdtemp(prefix=".verify-")
    try:
        os.makedirs(os.path.join(link_root, "generations"))
        os.symlink(os.path.abspath(directory), os.path.join(link_root, "generations", name))
        return verify_generation(link_root, name)
    finally:
        shutil.rmtree(link_root, ignore_errors=True)


def verify_checkpoint_root(out_dir: str) -> Dict[str, Any]:
    name = read_current(out_dir)
    if name is None:
        raise CheckpointError(f"{out_dir} has no current.json")
    with open(os.path.join(out_dir, "current.json")) as f:
        pointer = json.load(f)
    verified = verify_checkpoint_generation(os.path.join(out_dir, "generations", name), name, pointer.get("manifest_sha256", ""))
    return verified


def validate_checkpoint_metrics(verified: Dict[str, Any], metrics_path: str, exact: bool) -> None:
    """The journal's first `metric_records` records must be valid, in sequence and end at the checkpoint's step; with
    `exact`, nothing may follow them."""
    from .metrics import LogState, MetricsError, validate_record
    want, state, seen = verified["metric_records"], LogState(), 0
    try:
        with open(metrics_path, "r", encoding="utf-8") as f:
            for line in f:
                if seen >= want:
                    if exact and line.strip():
                        raise CheckpointError(f"{metrics_path} continues after the {want} records the checkpoint committed")
                    break
                rec = json.loads(line)
                validate_record(rec)
                state.accept(rec)
                seen += 1
    except (MetricsError, json.JSONDecodeError, OSError) as e:
        raise CheckpointError(f"{metrics_path}: record {seen} of the committed prefix is invalid: {e}")
    if seen != want:
        raise CheckpointError(f"{metrics_path}: checkpoint committed {want} records, journal has {seen}")
    if want and state.last_global_step is not None and state.last_global_step > verified["global_step"]:
        raise CheckpointError(f"{metrics_path}: the committed prefix reaches step {state.last_global_step}, the checkpoint step {verified['global_step']}")


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
    if state.parameter_ids and hasattr(model, "named_parameters") and any(r.get("scope") == "wake" for r in state.optimizer_states):
        # identities derived from names: only files of this package carry the `wake` scope, and for those the list must match
        if state.parameter_ids != parameter_ids_of(model):
            raise CheckpointError("the checkpoint's parameter identities differ from this model's (renamed or re-ordered parameters)")
    return state, blobs["adamw-state.bpk"], blobs["muon-state.bpk"], name
