"""Write-once publication of a trained QAT model together with its quantised archive.

A candidate key names one immutable artifact `root/<key>/{weights.safetensors, hquant/…,
candidate.json}`. Publication builds the canonical weights snapshot and the complete archive
in a private sibling directory, validates every member, writes the receipt and exposes the
whole candidate with ONE directory rename. A retry returns the existing candidate only when
the model bytes and the recipe match; a key is never rebound. Reopening re-derives the
archive from the stored weights (the encoding is deterministic), so hashes that are merely
self-consistent do not pass; `open_addressed` is the fast path for a receipt whose identity
an immutable checkpoint already seals (`summa-train/src/qat_candidate.rs:1-8,96-185,573-592`).
"""
from __future__ import annotations

import hashlib
import itertools
import json
import os
import shutil
from dataclasses import dataclass
from typing import Callable, Dict, Optional

import torch

from . import artifact_io as A
from . import quantization as Q

CANDIDATE_VERSION = 1
CANDIDATE_MANIFEST = "candidate.json"
WEIGHTS_FILE = "weights.safetensors"
ARCHIVE_DIRECTORY = "hquant"
ARCHIVE_MANIFEST = "archive-manifest.json"
MAX_QAT_JSON_BYTES = 16 * 1024 * 1024
_staging_sequence = itertools.count()


class CandidateError(RuntimeError):
    pass


@dataclass
class Recipe:
    format: str
    embeddings: bool = True
    lm_head: bool = True
    group_size: int = 128

    def validate(self) -> None:
        if self.format not in Q.TAGS:
            raise CandidateError(f"unknown quantization format {self.format!r}")
        if self.group_size != 128:
            raise CandidateError("quantization group_size must be 128")

    def to_json(self) -> Dict[str, object]:
        return {"format": self.format, "embeddings": self.embeddings, "lm_head": self.lm_head,
                "group_size": self.group_size}


@dataclass
class Publication:
    candidate_key: str
    candidate_root: str
    candidate_manifest_path: str
    candidate_manifest_sha256: str
    weights_path: str
    weights_sha256: str
    archive_path: str
    archive_manifest_sha256: str
    metrics: Dict[str, float]
    reused: bool = False


def validate_candidate_key(key: str) -> None:
    if not key or len(key.encode()) > 128:
        raise CandidateError("QAT candidate key must contain 1..=128 bytes")
    ok = all(c.isascii() and (c.isalnum() or c in "-_.") for c in key)
    if not ok or key in (".", ".."):
        raise CandidateError("QAT candidate key may contain only ASCII letters, digits, '.', '-', and '_'")


def _archive_metrics(model, packed: Dict[str, "Q.PackedTensor"]) -> Dict[str, float]:
    """Exact aggregates over every stored element: packed bytes include the group scales;
    the average bits per weight counts the tensors that stayed in their source dtype too."""
    q_elems = q_bytes = f_elems = f_bytes = f_tensors = 0
    sq_err, max_err = 0.0, 0.0
    for name, p in model.named_parameters():
        if name in packed:
            pt = packed[name]
            q_elems += pt.elements()
            q_bytes += len(pt.to_bytes())
            d = (pt.decode().double() - p.detach().double().cpu())
            sq_err += float(d.pow(2).sum())
            max_err = max(max_err, float(d.abs().max()))
        else:
            f_tensors += 1
            f_elems += p.numel()
            f_bytes += p.numel() * p.element_size()
    total_elems, total_bytes = q_elems + f_elems, q_bytes + f_bytes
    return {"quantized_tensors": len(packed), "quantized_elements": q_elems, "packed_bytes": q_bytes,
            "floating_tensors": f_tensors, "floating_elements": f_elems, "floating_bytes": f_bytes,
            "archive_weight_elements": total_elems, "archive_weight_bytes": total_bytes,
            "average_bits_per_weight": 8.0 * total_bytes / max(total_elems, 1),
            "weighted_mean_squared_error": sq_err / max(q_elems, 1), "maximum_absolute_error": max_err}


def _archive_content_identity(archive_dir: str, manifest: dict) -> str:
    h = hashlib.sha256()
    for ent in sorted(manifest["files"], key=lambda e: e["path"]):
        h.update(ent["path"].encode() + b"\0" + ent["sha256"].encode() + b"\0")
    return A.SHA256_PREFIX + h.hexdigest()


def _build(model, recipe: Recipe, directory: str) -> dict:
    """Weights snapshot + archive + receipt inside `directory` (staging)."""
    from ..models import weights as W
    weights_path = os.path.join(directory, WEIGHTS_FILE)
    W.save_safetensors(model, weights_path)
    A.sync_regular_file(weights_path, "QAT weights")
    weights_bytes, weights_id = A.hash_regular_file(weights_path)
    arch = os.path.join(directory, ARCHIVE_DIRECTORY)
    manifest = Q.export_archive(model, recipe.format, arch, recipe.embeddings, recipe.lm_head)
    for ent in manifest["files"]:                                   # validate every member as written
        size, ident = A.hash_regular_file(os.path.join(arch, ent["path"]))
        if size != ent["bytes"] or ident != A.SHA256_PREFIX + ent["sha256"]:
            raise CandidateError(f"archive member {ent['path']} does not match its manifest entry")
        A.sync_regular_file(os.path.join(arch, ent["path"]), "archive member")
    _, arch_manifest_id = A.hash_regular_file(os.path.join(arch, ARCHIVE_MANIFEST))
    packed = Q.quantize_model(model, recipe.format, recipe.embeddings, recipe.lm_head)
    return {"version": CANDIDATE_VERSION, "weights_file": WEIGHTS_FILE, "weights_bytes": weights_bytes,
            "weights_sha256": weights_id, "archive_directory": ARCHIVE_DIRECTORY, "archive_manifest": ARCHIVE_MANIFEST,
            "archive_manifest_sha256": arch_manifest_id,
            "archive_content_sha256": _archive_content_identity(arch, manifest),
            "recipe": recipe.to_json(), "metrics": _archive_metrics(model, packed)}


def _read_receipt(root: str, expected_identity: Optional[str] = None) -> (dict, str):
    data = A.read_regular_bounded(os.path.join(root, CANDIDATE_MANIFEST), MAX_QAT_JSON_BYTES, "QAT candidate manifest")
    ident = A.sha256_identity(data)
    if expected_identity is not None and ident != expected_identity:
        raise CandidateError(f"QAT candidate manifest is {ident}, the checkpoint sealed {expected_identity}")
    receipt = json.loads(data)
    allowed = {"version", "candidate_key", "weights_file", "weights_bytes", "weights_sha256", "archive_directory",
               "archive_manifest", "archive_manifest_sha256", "archive_content_sha256", "recipe", "metrics"}
    if set(receipt) != allowed or receipt["version"] != CANDIDATE_VERSION:
        raise CandidateError("QAT candidate manifest has an unknown layout")
    return receipt, ident


def _validate(root: str, key: str, model_factory: Optional[Callable[[], object]], reproduce: bool,
              expected_receipt_identity: Optional[str] = None) -> Publication:
    A.ensure_real_directory(root, "QAT candidate")
    receipt, receipt_id = _read_receipt(root, expected_receipt_identity)
    if receipt["candidate_key"] != key:
        raise CandidateError(f"candidate at {root} was published as '{receipt['candidate_key']}'")
    with A.PinnedDirectory.open(root, "QAT candidate") as pin:
        expected = {CANDIDATE_MANIFEST, WEIGHTS_FILE, ARCHIVE_DIRECTORY}
        if set(pin.entries()) != expected:
            raise CandidateError(f"QAT candidate {root} holds unexpected entries")
        size, wid = pin.hash_member(WEIGHTS_FILE)
        if size != receipt["weights_bytes"] or wid != receipt["weights_sha256"]:
            raise CandidateError("QAT candidate weights do not match the receipt")
        mdata = pin.read_bounded(f"{ARCHIVE_DIRECTORY}/{ARCHIVE_MANIFEST}", MAX_QAT_JSON_BYTES)
        if A.sha256_identity(mdata) != receipt["archive_manifest_sha256"]:
            raise CandidateError("QAT archive manifest does not match the receipt")
        manifest = json.loads(mdata)
        for ent in manifest["files"]:
            size, ident = pin.hash_member(f"{ARCHIVE_DIRECTORY}/{ent['path']}")
            if size != ent["bytes"] or ident != A.SHA256_PREFIX + ent["sha256"]:
                raise CandidateError(f"QAT archive member {ent['path']} does not match the archive manifest")
        if _archive_content_identity(os.path.join(root, ARCHIVE_DIRECTORY), manifest) != receipt["archive_content_sha256"]:
            raise CandidateError("QAT archive content identity does not match the receipt")
        pin.ensure_still_published(root)
    if reproduce:
        # the encoding is deterministic: rebuild the archive from the stored weights and compare
        if model_factory is None:
            raise CandidateError("reproducing a QAT candidate needs a model factory")
        from ..models import weights as W
        model = model_factory()
        W.load_safetensors(model, os.path.join(root, WEIGHTS_FILE))
        r = receipt["recipe"]
        packed = Q.quantize_model(model, r["format"], r["embeddings"], r["lm_head"])
        listed = {e["path"]: e["sha256"] for e in manifest["files"]}
        for name, pt in packed.items():
            rel = os.path.join("tensors", name + ".hquant")
            if listed.get(rel) != hashlib.sha256(pt.to_bytes()).hexdigest():
                raise CandidateError(f"QAT archive member {rel} is not the encoding of the stored weights")
        if len(packed) + 1 != len(listed):
            raise CandidateError("QAT archive lists members the stored weights do not produce")
    return Publication(key, root, os.path.join(root, CANDIDATE_MANIFEST), receipt_id,
                       os.path.join(root, WEIGHTS_FILE), receipt["weights_sha256"],
                       os.path.join(root, ARCHIVE_DIRECTORY), receipt["archive_manifest_sha256"], receipt["metrics"], True)


def publish(model, root: str, key: str, recipe: Recipe, model_factory: Callable[[], object],
            source_weights_sha256: Optional[str] = None, hook: Optional[Callable[[str, str], None]] = None) -> Publication:
    """Publishes `model` under `root/key`, or returns the existing candidate when it is bound to
    the same model bytes and recipe. `model_factory()` builds an empty model of the same
    architecture (for re-deriving an existing candidate). `hook(point, staging_dir)` is called
    at "weights_synced", "archive_verified" and "manifest_synced" (tests interrupt there)."""
    validate_candidate_key(key)
    recipe.validate()
    if source_weights_sha256 is not None:
        A.validate_sha256_identity(source_weights_sha256, "QAT source weights identity")
    A.ensure_directory(root, "QAT candidate root")
    final = os.path.join(root, key)
    if os.path.lexists(final):
        A.ensure_real_directory(final, "existing QAT candidate")

    def adopt(weights_identity: str) -> Publication:
        pub = _validate(final, key, model_factory, reproduce=True)
        if pub.weights_sha256 != weights_identity:
            raise CandidateError(f"QAT candidate key '{key}' is bound to different model weights")
        receipt, _ = _read_receipt(final)
        if receipt["recipe"] != recipe.to_json():
            raise CandidateError(f"QAT candidate key '{key}' is already bound to a different quantization recipe")
        return pub

    if source_weights_sha256 is not None and os.path.lexists(final):
        return adopt(source_weights_sha256)
    staging = None
    for _ in range(1024):
        cand = os.path.join(root, f".{key}.qat-tmp-{os.getpid()}-{next(_staging_sequence)}")
        try:
            os.mkdir(cand)
            staging = cand
            break
        except FileExistsError:
            continue
    if staging is None:
        raise CandidateError("could not allocate a QAT staging directory")
    try:
        receipt = _build(model, recipe, staging)
        receipt["candidate_key"] = key
        if source_weights_sha256 is not None and receipt["weights_sha256"] != source_weights_sha256:
            raise CandidateError(f"canonical QAT weights {receipt['weights_sha256']} differ from the authenticated source")
        if hook:
            hook("weights_synced", staging)
        if os.path.lexists(final):
            return adopt(receipt["weights_sha256"])
        if hook:
            hook("archive_verified", staging)
        A.write_new_synced(os.path.join(staging, CANDIDATE_MANIFEST),
                           json.dumps(receipt, sort_keys=True, indent=2).encode())
        A.sync_directory(os.path.join(staging, ARCHIVE_DIRECTORY, "tensors"))
        A.sync_directory(os.path.join(staging, ARCHIVE_DIRECTORY))
        A.sync_directory(staging)
        if hook:
            hook("manifest_synced", staging)
        try:
            os.rename(staging, final)                 # the one step that exposes the candidate
        except OSError:
            if os.path.lexists(final):                # a concurrent publisher won: adopt its result if it matches
                return adopt(receipt["weights_sha256"])
            raise
        staging = None
        A.sync_directory(root)
        pub = _validate(final, key, None, reproduce=False)
        pub.reused = False
        return pub
    finally:
        if staging is not None and os.path.isdir(staging):
            shutil.rmtree(staging, ignore_errors=True)


def open_candidate(candidate_root: str, model_factory: Callable[[], object]) -> Publication:
    """Reopens a published candidate and authenticates receipt, weights, archive manifest, every
    archive member, and that the archive is the encoding of the stored weights."""
    key = os.path.basename(os.path.normpath(candidate_root))
    validate_candidate_key(key)
    return _validate(candidate_root, key, model_factory, reproduce=True)


def open_addressed(candidate_root: str, expected_candidate_manifest_sha256: str) -> Publication:
    """Fast path when an immutable checkpoint seals the exact receipt bytes: the small receipt is
    authenticated before any weights or archive member is read."""
    A.validate_sha256_identity(expected_candidate_manifest_sha256, "QAT candidate manifest identity")
    key = os.path.basename(os.path.normpath(candidate_root))
    validate_candidate_key(key)
    return _validate(candidate_root, key, None, reproduce=False,
                     expected_receipt_identity=expected_candidate_manifest_sha256)
