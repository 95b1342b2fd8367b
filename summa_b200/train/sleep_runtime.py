"""The sleep-runtime configuration file (`--sleep-runtime <file> --sleep-runtime-sha256 sha256:...`).

A memory-enabled model trains with periodic sleep only when the operator hands the trainer this file together with
the `sha256:` identity of its bytes; the file pins every artifact the boundary work reads (each as `{path,
sha256}`), names where boundary state is written, and carries the rollout, tier-optimizer and dreaming settings.
Version 1, decoded strictly, in the two shapes of the reference (`summa-train/src/builtin_sleep_runtime.rs:45-260`,
`builtin_sleep_adapters.rs:95-150,336-385`, `builtin_dreaming.rs:56-200`, `tier_optimizer.rs:66-112`):

  periodic    (`sleep-runtime.periodic.example.json`) inside `train`: no wake journal, no initial tier / parameter-id
              artifacts (the integrated trainer seals those at each boundary);
  standalone  (`sleep-runtime.standalone.example.json`) for a `sleep` phase of `run-workflow`: the wake-context
              journal and the initial tier-optimizer / parameter-id artifacts are required, and dreaming must use the
              exact same pinned journal.

Relative paths resolve against the file. Output directories must be distinct. A pinned artifact is read with
`verify_bytes` / `verify_json`, which refuse a file whose bytes do not hash to the pin; an all-zero pin is a
placeholder and never verifies."""
from __future__ import annotations

import hashlib
import json
import math
import os
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .sleep import SleepError
from .sleep_state import MAX_SLEEP_RNG_STREAMS, check_sha256

SLEEP_RUNTIME_VERSION = 1
MAX_WAKE_CONTEXT_RECORDS = 4096
MAX_WAKE_CONTEXT_TOKENS = 65536
MAX_WAKE_CONTEXT_TOTAL_TOKENS = 4 * 1024 * 1024
MAX_ROLLOUT_CONTINUATION_TOKENS = 16384
MAX_ROLLOUT_TOP_K = 262144
MAX_IMITATION_GROUPS = 256
MAX_DREAM_NEW_TOKENS = 4096
MAX_DREAM_GRADIENT_DIMENSIONS = 4096
MAX_DREAM_LORA_STEPS = 1024
MAX_ARTIFACT_BYTES = 1 << 30


def _need(cond: bool, message: str) -> None:
    if not cond:
        raise SleepError(message)


def _object(value: Any, what: str, required: List[str], optional: List[str] = ()) -> Dict[str, Any]:
    _need(isinstance(value, dict), f"{what} must be an object")
    unknown = set(value) - set(required) - set(optional)
    if unknown:
        raise SleepError(f"unknown field `{sorted(unknown)[0]}` in {what}")
    for k in required:
        _need(k in value, f"missing field `{k}` in {what}")
    return value


def _uint(v: Any, what: str) -> int:
    _need(isinstance(v, int) and not isinstance(v, bool) and v >= 0, f"{what} must be a non-negative integer")
    return v


def _real(v: Any, what: str) -> float:
    _need(isinstance(v, (int, float)) and not isinstance(v, bool) and math.isfinite(float(v)), f"{what} must be a finite number")
    return float(v)


@dataclass
class PinnedArtifact:
    path: str
    sha256: str

    @staticmethod
    def decode(value: Any, what: str, base: str) -> "PinnedArtifact":
        d = _object(value, what, ["path", "sha256"])
        _need(isinstance(d["path"], str) and d["path"] != "", f"{what}: pinned artifact path is empty")
        check_sha256(d["sha256"], f"{what} hash")
        path = d["path"] if os.path.isabs(d["path"]) else os.path.join(base, d["path"])
        return PinnedArtifact(os.path.normpath(path), d["sha256"])

    def verify_bytes(self) -> bytes:
        check_sha256(self.sha256, "pinned artifact hash")
        st = os.lstat(self.path)
        import stat as _stat
        _need(_stat.S_ISREG(st.st_mode), f"pinned artifact {self.path} is not a regular file")
        _need(st.st_size <= MAX_ARTIFACT_BYTES, f"pinned artifact {self.path} is too large")
        with open(self.path, "rb") as f:
            data = f.read()
        seen = "sha256:" + hashlib.sha256(data).hexdigest()
        _need(seen == self.sha256, f"pinned artifact {self.path} changed: expected {self.sha256}, observed {seen}")
        return data

    def verify_json(self) -> Any:
        data = self.verify_bytes()
        try:
            return json.loads(data)
        except ValueError as e:
            raise SleepError(f"invalid pinned JSON artifact {self.path}: {e}")

    def to_json(self) -> Dict[str, str]:
        return {"path": self.path, "sha256": self.sha256}


@dataclass
class RolloutConfig:
    max_context_tokens: int
    continuation_tokens: int
    temperature: float = 0.8
    top_k: int = 32
    repetition_penalty: float = 1.05
    eos_token: Optional[int] = None
    imitation_groups: int = 1

    @staticmethod
    def decode(value: Any) -> "RolloutConfig":
        d = _object(value, "`rollouts`", ["max_context_tokens", "continuation_tokens"],
                    ["temperature", "top_k", "repetition_penalty", "eos_token", "imitation_groups"])
        r = RolloutConfig(_uint(d["max_context_tokens"], "`rollouts.max_context_tokens`"), _uint(d["continuation_tokens"], "`rollouts.continuation_tokens`"),
                          _real(d.get("temperature", 0.8), "`rollouts.temperature`"), _uint(d.get("top_k", 32), "`rollouts.top_k`"),
                          _real(d.get("repetition_penalty", 1.05), "`rollouts.repetition_penalty`"),
                          None if d.get("eos_token") is None else _uint(d["eos_token"], "`rollouts.eos_token`"),
                          _uint(d.get("imitation_groups", 1), "`rollouts.imitation_groups`"))
        _need(r.max_context_tokens > 0 and r.continuation_tokens > 0, "journal rollout context and continuation lengths must be positive")
        _need(r.max_context_tokens <= MAX_WAKE_CONTEXT_TOKENS, f"journal rollout context exceeds the {MAX_WAKE_CONTEXT_TOKENS}-token limit")
        _need(r.continuation_tokens <= MAX_ROLLOUT_CONTINUATION_TOKENS, f"journal rollout continuation exceeds the {MAX_ROLLOUT_CONTINUATION_TOKENS}-token limit")
        _need(r.temperature > 0.0, "journal rollout temperature must be finite and positive")
        _need(1 <= r.top_k <= MAX_ROLLOUT_TOP_K, f"journal rollout top_k must be in 1..={MAX_ROLLOUT_TOP_K}")
        _need(r.repetition_penalty >= 1.0, "journal rollout repetition penalty must be finite and at least one")
        _need(1 <= r.imitation_groups <= MAX_IMITATION_GROUPS, f"journal rollout imitation_groups must be in 1..={MAX_IMITATION_GROUPS}")
        return r


@dataclass
class TierOptimizerConfig:
    learning_rate: float = 3e-4
    beta_1: float = 0.9
    beta_2: float = 0.95
    epsilon: float = 1e-8
    weight_decay: float = 0.1

    @staticmethod
    def decode(value: Any) -> "TierOptimizerConfig":
        names = ["learning_rate", "beta_1", "beta_2", "epsilon", "weight_decay"]
        d = _object(value, "`tier_optimizer`", names)
        c = TierOptimizerConfig(*[_real(d[k], f"`tier_optimizer.{k}`") for k in names])
        _need(c.learning_rate > 0.0, "tier learning rate must be finite and positive")
        _need(0.0 <= c.beta_1 < 1.0, "tier AdamW beta_1 must be in [0, 1)")
        _need(0.0 <= c.beta_2 < 1.0, "tier AdamW beta_2 must be in [0, 1)")
        _need(c.epsilon > 0.0, "tier AdamW epsilon must be finite and positive")
        _need(c.weight_decay >= 0.0, "tier AdamW weight decay must be finite and non-negative")
        return c


@dataclass
class DreamingRuntimeConfig:
    artifact_directory: str
    reference_set: PinnedArtifact
    independent_evaluation_set: PinnedArtifact
    wake_context_journal: Optional[PinnedArtifact] = None
    initial_policy: Optional[PinnedArtifact] = None
    max_new_tokens: int = 32
    gradient_dimensions: int = 256
    lora_steps: int = 8
    lora_learning_rate: float = 1e-3
    restem_learning_rate: float = 0.1
    generation_temperature: float = 0.8
    generation_policy_rank: int = 64
    generation_policy_alpha: int = 128

    @staticmethod
    def decode(value: Any, base: str) -> "DreamingRuntimeConfig":
        opt = ["wake_context_journal", "initial_policy", "max_new_tokens", "gradient_dimensions", "lora_steps", "lora_learning_rate",
               "restem_learning_rate", "generation_temperature", "generation_policy_rank", "generation_policy_alpha"]
        d = _object(value, "`dreaming`", ["artifact_directory", "reference_set", "independent_evaluation_set"], opt)
        _need(isinstance(d["artifact_directory"], str) and d["artifact_directory"] != "", "Dreaming artifact directory is empty")
        pin = lambda k: PinnedArtifact.decode(d[k], f"`dreaming.{k}`", base) if d.get(k) is not None else None
        directory = d["artifact_directory"] if os.path.isabs(d["artifact_directory"]) else os.path.join(base, d["artifact_directory"])
        c = DreamingRuntimeConfig(os.path.normpath(directory), pin("reference_set"), pin("independent_evaluation_set"), pin("wake_context_journal"),
                                  pin("initial_policy"), _uint(d.get("max_new_tokens", 32), "`dreaming.max_new_tokens`"),
                                  _uint(d.get("gradient_dimensions", 256), "`dreaming.gradient_dimensions`"), _uint(d.get("lora_steps", 8), "`dreaming.lora_steps`"),
                                  _real(d.get("lora_learning_rate", 1e-3), "`dreaming.lora_learning_rate`"),
                                  _real(d.get("restem_learning_rate", 0.1), "`dreaming.restem_learning_rate`"),
                                  _real(d.get("generation_temperature", 0.8), "`dreaming.generation_temperature`"),
                                  _uint(d.get("generation_policy_rank", 64), "`dreaming.generation_policy_rank`"),
                                  _uint(d.get("generation_policy_alpha", 128), "`dreaming.generation_policy_alpha`"))
        _need(0 < c.max_new_tokens <= MAX_DREAM_NEW_TOKENS, f"Dreaming max_new_tokens must be in 1..={MAX_DREAM_NEW_TOKENS}")
        _need(0 < c.gradient_dimensions <= MAX_DREAM_GRADIENT_DIMENSIONS, f"Dreaming gradient dimensions must be in 1..={MAX_DREAM_GRADIENT_DIMENSIONS}")
        _need(0 < c.lora_steps <= MAX_DREAM_LORA_STEPS, f"Dreaming LoRA steps must be in 1..={MAX_DREAM_LORA_STEPS}")
        _need(c.lora_learning_rate > 0.0 and c.restem_learning_rate > 0.0, "Dreaming learning rates must be positive")
        _need(c.generation_temperature > 0.0, "Dreaming generation temperature must be positive")
        _need(c.generation_policy_rank > 0 and c.generation_policy_alpha > 0, "Dreaming generation-policy geometry must be positive")
        return c


_PINS = ("model_mal", "semantic_judge", "retention_evaluator", "retention_suite")
_OPTIONAL_PINS = ("wake_context_journal", "initial_tier_optimizer_state", "initial_model_parameter_ids")
_DIRECTORIES = ("tensor_transaction_directory", "prospective_directory", "tier_optimizer_directory", "candidate_directory",
                "rejection_report_directory")


@dataclass
class SleepRuntimeConfig:
    version: int
    workflow_signature: str
    pins: Dict[str, PinnedArtifact]
    rollouts: RolloutConfig
    tier_optimizer: TierOptimizerConfig
    directories: Dict[str, str]
    dreaming: Optional[DreamingRuntimeConfig] = None
    max_wake_context_records: int = 64
    rng_streams: int = 1
    identity: str = ""                       # `sha256:` of the file's bytes
    path: str = ""

    @staticmethod
    def decode(value: Any, base: str) -> "SleepRuntimeConfig":
        d = _object(value, "the sleep runtime", ["version", "workflow_signature", *_PINS, "rollouts", "tier_optimizer", *_DIRECTORIES],
                    [*_OPTIONAL_PINS, "dreaming", "max_wake_context_records", "rng_streams"])
        _need(d["version"] == SLEEP_RUNTIME_VERSION, f"unsupported built-in sleep runtime version {d['version']}")
        check_sha256(d["workflow_signature"], "workflow signature")
        pins = {k: PinnedArtifact.decode(d[k], f"`{k}`", base) for k in (*_PINS, *_OPTIONAL_PINS) if d.get(k) is not None}
        dirs = {}
        for k in _DIRECTORIES:
            _need(isinstance(d[k], str) and d[k] != "", "sleep runtime contains an empty output directory")
            dirs[k] = os.path.normpath(d[k] if os.path.isabs(d[k]) else os.path.join(base, d[k]))
        c = SleepRuntimeConfig(d["version"], d["workflow_signature"], pins, RolloutConfig.decode(d["rollouts"]),
                               TierOptimizerConfig.decode(d["tier_optimizer"]), dirs,
                               DreamingRuntimeConfig.decode(d["dreaming"], base) if d.get("dreaming") is not None else None,
                               _uint(d.get("max_wake_context_records", 64), "`max_wake_context_records`"), _uint(d.get("rng_streams", 1), "`rng_streams`"))
        c.validate()
        return c

    def validate(self) -> None:
        _need(1 <= self.rng_streams <= MAX_SLEEP_RNG_STREAMS, f"sleep runtime must contain 1..={MAX_SLEEP_RNG_STREAMS} RNG streams")
        _need(1 <= self.max_wake_context_records <= MAX_WAKE_CONTEXT_RECORDS, f"sleep runtime wake-context ring must contain 1..={MAX_WAKE_CONTEXT_RECORDS} records")
        _need(self.max_wake_context_records * self.rollouts.max_context_tokens <= MAX_WAKE_CONTEXT_TOTAL_TOKENS,
              f"sleep runtime wake-context ring exceeds the {MAX_WAKE_CONTEXT_TOTAL_TOKENS}-token limit")
        out = list(self.directories.values()) + ([self.dreaming.artifact_directory] if self.dreaming else [])
        _need(len(set(out)) == len(out), "sleep runtime output directories, including Dreaming artifacts, must be distinct")
        journal = self.pins.get("wake_context_journal")
        if self.dreaming and self.dreaming.wake_context_journal and journal:
            _need(self.dreaming.wake_context_journal == journal, "Dreaming and consolidation must use the same pinned wake journal")

    def validate_periodic(self) -> None:
        self.validate()
        _need(not any(k in self.pins for k in _OPTIONAL_PINS), "periodic sleep runtime must not contain standalone wake artifacts")
        _need(self.dreaming is None or self.dreaming.wake_context_journal is None, "periodic Dreaming must not contain a standalone wake_context_journal")

    def validate_standalone(self) -> None:
        self.validate()
        for k in _OPTIONAL_PINS:
            _need(k in self.pins, f"standalone sleep runtime requires {k}")
        if self.dreaming is not None:
            _need(self.dreaming.wake_context_journal == self.pins["wake_context_journal"],
                  "standalone Dreaming requires the exact consolidation wake_context_journal")


def load_sleep_runtime(path: str, expected_sha256: str, mode: str = "periodic") -> SleepRuntimeConfig:
    """Reads the file once, checks its bytes against the identity the operator supplied, decodes it strictly and
    applies the rules of its mode (`periodic` inside `train`, `standalone` for a `sleep` phase)."""
    check_sha256(expected_sha256, "sleep runtime identity")
    with open(path, "rb") as f:
        raw = f.read()
    seen = "sha256:" + hashlib.sha256(raw).hexdigest()
    _need(seen == expected_sha256, f"sleep runtime {path} is not the pinned file: expected {expected_sha256}, observed {seen}")
    try:
        value = json.loads(raw)
    except ValueError as e:
        raise SleepError(f"sleep runtime {path} is not valid JSON: {e}")
    cfg = SleepRuntimeConfig.decode(value, os.path.dirname(os.path.abspath(path)))
    _need(mode in ("periodic", "standalone"), f"unknown sleep runtime mode `{mode}`")
    (cfg.validate_periodic if mode == "periodic" else cfg.validate_standalone)()
    cfg.identity, cfg.path = seen, path
    return cfg


WAKE_CONTEXT_JOURNAL_VERSION = 1
MAX_WAKE_CONTEXT_ID_BYTES = 1024


class WakeContextJournal:
    """The model-owned contexts a standalone sleep phase replays (`builtin_sleep_adapters.rs:148-300`): records
    `{id, optimizer_step, token_ids}` with unique ids and non-decreasing optimizer steps, bound to the checkpoint they
    were collected under. Published once as an immutable file; read back only through its pin."""

    def __init__(self, source_checkpoint_sha256: str):
        self.version = WAKE_CONTEXT_JOURNAL_VERSION
        self.source_checkpoint_sha256 = check_sha256(source_checkpoint_sha256, "wake-context source checkpoint hash")
        self.records: List[Dict[str, Any]] = []

    @staticmethod
    def _check_record(r: Dict[str, Any]) -> None:
        _object(r, "wake context record", ["id", "optimizer_step", "token_ids"])
        _need(isinstance(r["id"], str) and r["id"].strip() != "" and len(r["id"].encode()) <= MAX_WAKE_CONTEXT_ID_BYTES,
              f"wake context id must contain 1..={MAX_WAKE_CONTEXT_ID_BYTES} bytes")
        _uint(r["optimizer_step"], "wake context optimizer_step")
        toks = r["token_ids"]
        _need(isinstance(toks, list) and len(toks) > 0, f"wake context `{r['id']}` has no tokens")
        _need(len(toks) <= MAX_WAKE_CONTEXT_TOKENS, f"wake context `{r['id']}` exceeds the {MAX_WAKE_CONTEXT_TOKENS}-token limit")
        _need(all(isinstance(t, int) and not isinstance(t, bool) and 0 <= t < (1 << 32) for t in toks),
              f"wake context `{r['id']}` contains a token outside the u32 vocabulary range")

    def push(self, record_id: str, optimizer_step: int, token_ids: List[int]) -> None:
        r = {"id": record_id, "optimizer_step": optimizer_step, "token_ids": list(token_ids)}
        self._check_record(r)
        _need(len(self.records) < MAX_WAKE_CONTEXT_RECORDS, f"wake context journal exceeds the {MAX_WAKE_CONTEXT_RECORDS}-record limit")
        _need(all(x["id"] != record_id for x in self.records), f"wake context journal repeats id `{record_id}`")
        _need(not self.records or self.records[-1]["optimizer_step"] <= optimizer_step, "wake context journal optimizer steps move backwards")
        self.records.append(r)

    def validate(self) -> None:
        _need(self.version == WAKE_CONTEXT_JOURNAL_VERSION, f"unsupported wake-context journal version {self.version}")
        check_sha256(self.source_checkpoint_sha256, "wake-context source checkpoint hash")
        _need(0 < len(self.records) <= MAX_WAKE_CONTEXT_RECORDS, "wake context journal is empty or exceeds its record limit")
        _need(sum(len(r["token_ids"]) for r in self.records) <= MAX_WAKE_CONTEXT_TOTAL_TOKENS,
              f"wake context journal exceeds the {MAX_WAKE_CONTEXT_TOTAL_TOKENS}-token limit")
        ids, previous = set(), 0
        for i, r in enumerate(self.records):
            self._check_record(r)
            _need(r["id"] not in ids, f"wake context journal repeats id `{r['id']}`")
            ids.add(r["id"])
            _need(i == 0 or r["optimizer_step"] >= previous, "wake context journal optimizer steps move backwards")
            previous = r["optimizer_step"]

    def to_json(self) -> Dict[str, Any]:
        return {"version": self.version, "source_checkpoint_sha256": self.source_checkpoint_sha256, "records": self.records}

    def publish(self, path: str) -> PinnedArtifact:
        """Writes the journal as a new file (never over an existing one) and returns its pin."""
        self.validate()
        body = (json.dumps(self.to_json(), indent=2) + "\n").encode()
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        fd = os.open(path, os.O_WRONLY | os.O_CREAT | os.O_EXCL, 0o644)
        try:
            os.write(fd, body)
            os.fsync(fd)
        finally:
            os.close(fd)
        return PinnedArtifact(path, "sha256:" + hashlib.sha256(body).hexdigest())

    @staticmethod
    def load(pin: PinnedArtifact) -> "WakeContextJournal":
        d = _object(pin.verify_json(), "wake-context journal", ["version", "source_checkpoint_sha256", "records"])
        j = WakeContextJournal(d["source_checkpoint_sha256"])
        j.version = d["version"]
        _need(isinstance(d["records"], list), "wake-context journal records must be an array")
        j.records = d["records"]
        j.validate()
        return j


REJECTION_REPORT_VERSION = 1


def write_rejection_report(directory: str, transaction, reason: str, metrics: Dict[str, Any]) -> str:
    """One immutable JSON per rejected boundary under the runtime's `rejection_report_directory`."""
    os.makedirs(directory, exist_ok=True)
    body = json.dumps({"version": REJECTION_REPORT_VERSION, "transaction_id": transaction.id, "trigger_clock": transaction.trigger_clock,
                       "sender": transaction.sender, "receiver": transaction.receiver, "terminal": transaction.terminal, "reason": reason,
                       "metrics": metrics}, sort_keys=True, indent=1).encode()
    path = os.path.join(directory, f"rejection-{transaction.id:012d}.json")
    fd = os.open(path, os.O_WRONLY | os.O_CREAT | os.O_EXCL, 0o644)
    try:
        os.write(fd, body)
        os.fsync(fd)
    finally:
        os.close(fd)
    return path
