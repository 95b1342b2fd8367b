"""Append-only `metrics.jsonl` (schema v2) with resume truncation.

Record shape (`summa-train/src/metrics.rs:25,307-449,586-856`):
    {schema_version: 2, sequence, emitted_at_unix_ms, run_id, global_step,
     phase: {index, name, kind}, checkpoint_hash?, event: {type, values}}
`run_id` is the FNV-1a64 of the run signature. Fourteen typed events exist; the two
core ones are `optimization` and `throughput`. On resume the journal is truncated to
the prefix that the checkpoint committed (`metric_records`), after validating that the
prefix is well formed and belongs to the same run.
"""
from __future__ import annotations

import json
import os
import time
from typing import Any, Dict, Optional

SCHEMA_VERSION = 2

EVENT_FIELDS = {
    "run_started": {"run_signature", "model", "parameters", "routed_active_parameters", "world_size"},
    "phase_started": {"planned_steps", "sequence_length", "batch_size", "gradient_accumulation"},
    "optimization": {"loss", "optimized_loss", "weighted_loss", "router_aux_loss", "retrieval_accuracy",
                     "learning_rate", "muon_learning_rate", "gradient_norm", "layer_norms", "tokens",
                     "supervised_tokens"},
    "throughput": {"tokens_per_second", "step_seconds", "input_wait_seconds", "host_to_device_seconds",
                   "gpu_busy_seconds"},
    "device_utilization": {"gpu_utilization", "memory_used_mib", "power_watts", "temperature_c", "sm_clock_mhz"},
    "quantization": {"format", "active", "fake_quantized_parameters"},
    "evaluation": {"name", "loss", "perplexity", "tokens", "top1", "mrr"},
    "checkpoint": {"generation", "global_step"},
    "phase_completed": {"steps", "tokens"},
    "sleep_boundary": {"clock", "due_tiers", "outcome"},
    "post_training": {"objective", "loss", "reward_mean", "kl"},
    "data_dropped": {"reason", "samples"},
    "warning": {"message"},
    "run_completed": {"global_step", "tokens_seen"},
}


class MetricsError(ValueError):
    pass


class MetricWriter:
    def __init__(self, path: str, run_id: int, sequence: int = 0):
        self.path = path
        self.run_id = run_id
        self.sequence = sequence
        self._f = open(path, "a", encoding="utf-8")
        self.phase = {"index": 0, "name": "", "kind": "pretrain"}
        self.global_step = 0

    @staticmethod
    def create(path: str, run_id: int) -> "MetricWriter":
        if os.path.exists(path) and os.path.getsize(path) > 0:
            raise MetricsError(f"{path} already exists; resume or choose a fresh output directory")
        return MetricWriter(path, run_id, 0)

    @staticmethod
    def resume_from_checkpoint(path: str, run_id: int, committed_records: int) -> "MetricWriter":
        """Validate the committed prefix and drop everything after it."""
        kept = []
        if os.path.exists(path):
            with open(path, "r", encoding="utf-8") as f:
                for i, line in enumerate(f):
                    if i >= committed_records:
                        break
                    try:
                        rec = json.loads(line)
                    except json.JSONDecodeError:
                        raise MetricsError(f"{path}: record {i} inside the committed prefix is corrupt")
                    validate_record(rec)
                    if rec["sequence"] != i or rec["run_id"] != run_id:
                        raise MetricsError(f"{path}: record {i} does not belong to this run's committed prefix")
                    kept.append(line if line.endswith("\n") else line + "\n")
        if len(kept) != committed_records:
            raise MetricsError(f"{path}: checkpoint committed {committed_records} records, journal has {len(kept)}")
        tmp = path + ".tmp"
        with open(tmp, "w", encoding="utf-8") as f:
            f.writelines(kept)
            f.flush()
            os.fsync(f.fileno())
        os.replace(tmp, path)
        return MetricWriter(path, run_id, committed_records)

    def set_context(self, global_step: int, phase_index: int, phase_name: str, phase_kind: str) -> None:
        self.global_step = global_step
        self.phase = {"index": phase_index, "name": phase_name, "kind": phase_kind}

    def emit(self, event_type: str, values: Dict[str, Any], checkpoint_hash: Optional[str] = None) -> None:
        if event_type not in EVENT_FIELDS:
            raise MetricsError(f"unknown metric event `{event_type}`")
        unknown = set(values) - EVENT_FIELDS[event_type]
        if unknown:
            raise MetricsError(f"event `{event_type}` has unknown fields {sorted(unknown)}")
        rec = {"schema_version": SCHEMA_VERSION, "sequence": self.sequence,
               "emitted_at_unix_ms": int(time.time() * 1000), "run_id": self.run_id,
               "global_step": self.global_step, "phase": dict(self.phase),
               "event": {"type": event_type, "values": values}}
        if checkpoint_hash is not None:
            rec["checkpoint_hash"] = checkpoint_hash
        self._f.write(json.dumps(rec, separators=(",", ":")) + "\n")
        self.sequence += 1

    def flush(self) -> None:
        self._f.flush()
        os.fsync(self._f.fileno())

    def close(self) -> None:
        self.flush()
        self._f.close()


def validate_record(rec: Dict[str, Any]) -> None:
    for k in ("schema_version", "sequence", "emitted_at_unix_ms", "run_id", "global_step", "phase", "event"):
        if k not in rec:
            raise MetricsError(f"metric record is missing `{k}`")
    if rec["schema_version"] != SCHEMA_VERSION:
        raise MetricsError(f"unsupported metrics schema {rec['schema_version']}")
    ev = rec["event"]
    if ev.get("type") not in EVENT_FIELDS or not isinstance(ev.get("values"), dict):
        raise MetricsError("malformed metric event")


def read_metrics(path: str):
    with open(path, "r", encoding="utf-8") as f:
        for line in f:
            if line.strip():
                rec = json.loads(line)
                validate_record(rec)
                yield rec
