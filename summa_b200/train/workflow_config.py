"""Typed sub-configurations of a WorkflowV2 phase, decoded as strictly as the reference decodes them.

The reference's phase carries serde structs with `deny_unknown_fields` for `post_training`
(`summa-train/src/posttrain.rs:211-247`, tagged by `algorithm`), `sleep` / `periodic_sleep`
(`summa-train/src/workflow.rs:183-206`, with `SleepSchedule` `summa-train/src/sleep.rs:68-150`,
`KnowledgeSeedingConfig` / `ImitationConfig` / `DreamingConfig` `sleep.rs:2421-2660`,
`RetentionGateConfig` `summa-train/src/tensor_sleep.rs:576-584`) and `memory_update_mode`
(`workflow.rs:327-372`, `TierOptimizerConfig` `summa-train/src/tier_optimizer.rs:66-121`). A workflow
file written for the reference must load here unchanged and a malformed one must fail in the same
place, so every decoder below checks: required fields present, JSON types exact (an integer field
rejects 1.0 and true), unknown fields rejected, documented defaults filled in, documented bounds
enforced. The decoders return plain dicts in the field order the reference serialises (what
`Workflow.to_json` and the workflow signature hash see), with every defaulted field made explicit
the way serde would re-serialise it.
"""
from __future__ import annotations

import math
import os
from typing import Any, Callable, Dict, List, Optional


class ConfigError(ValueError):
    pass


# ---------------------------------------------------------------------------- strict field decoding
_MISSING = object()


def _obj(v: Any, where: str) -> Dict[str, Any]:
    if not isinstance(v, dict):
        raise ConfigError(f"{where} must be an object")
    return v


def _deny_unknown(d: Dict[str, Any], allowed, where: str) -> None:
    extra = sorted(set(d) - set(allowed))
    if extra:
        raise ConfigError(f"unknown field `{extra[0]}` in {where}")


def _uint(d, key, where, default=_MISSING, hi: Optional[int] = None) -> int:
    v = d.get(key, _MISSING)
    if v is _MISSING:
        if default is _MISSING:
            raise ConfigError(f"missing field `{key}` in {where}")
        return default
    if not isinstance(v, int) or isinstance(v, bool) or v < 0 or (hi is not None and v > hi):
        raise ConfigError(f"`{key}` in {where} must be a non-negative integer")
    return v


def _float(d, key, where, default=_MISSING) -> float:
    v = d.get(key, _MISSING)
    if v is _MISSING:
        if default is _MISSING:
            raise ConfigError(f"missing field `{key}` in {where}")
        return default
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"`{key}` in {where} must be a number")
    return float(v)


def _bool(d, key, where, default=_MISSING) -> bool:
    v = d.get(key, _MISSING)
    if v is _MISSING:
        if default is _MISSING:
            raise ConfigError(f"missing field `{key}` in {where}")
        return default
    if not isinstance(v, bool):
        raise ConfigError(f"`{key}` in {where} must be a boolean")
    return v


def _str(d, key, where, default=_MISSING) -> Optional[str]:
    v = d.get(key, _MISSING)
    if v is _MISSING or (v is None and default is not _MISSING):
        if default is _MISSING:
            raise ConfigError(f"missing field `{key}` in {where}")
        return default
    if not isinstance(v, str):
        raise ConfigError(f"`{key}` in {where} must be a string")
    return v


def _enum(d, key, where, choices, default=_MISSING) -> str:
    v = _str(d, key, where, default)
    if v not in choices:
        raise ConfigError(f"`{key}` in {where}: unknown variant `{v}`, expected one of {', '.join(choices)}")
    return v


def _ensure(cond: bool, msg: str) -> None:
    if not cond:
        raise ConfigError(msg)


def validate_sha256_identity(s: Any, what: str) -> None:
    """`sha256:` + 64 lowercase hex characters (`summa-train/src/artifact_io.rs:42-76`)."""
    ok = isinstance(s, str) and s.startswith("sha256:") and len(s) == 71 and all(c in "0123456789abcdef" for c in s[7:])
    _ensure(ok, f"{what} must be `sha256:` followed by 64 lowercase hex characters")


def _frozen_identifier(v: str, field: str) -> None:
    _ensure(bool(v) and v.strip() == v and not any(ord(c) < 32 or ord(c) == 127 for c in v),
            f"{field} must be non-empty, trimmed, and contain no control characters")


# ---------------------------------------------------------------------------- post_training
MAX_ROLLOUTS_PER_PROMPT = 4_096
MAX_SEQUENCE_TOKENS = 1_048_576


def decode_frozen_model(v: Any, field: str) -> Dict[str, Any]:
    """`FrozenModelSpec`: an executor-owned frozen teacher / reference, pinned by hash or revision."""
    d = _obj(v, f"`{field}`")
    _deny_unknown(d, ("adapter", "artifact", "sha256", "revision", "parameters"), f"`{field}`")
    out: Dict[str, Any] = {"adapter": _str(d, "adapter", f"`{field}`")}
    _frozen_identifier(out["adapter"], f"`{field}.adapter`")
    artifact = _str(d, "artifact", f"`{field}`", None)
    sha = _str(d, "sha256", f"`{field}`", None)
    revision = _str(d, "revision", f"`{field}`", None)
    _ensure(artifact is None or artifact != "", f"`{field}.artifact` must not be empty when set")
    if revision is not None:
        _frozen_identifier(revision, f"`{field}.revision`")
    _ensure(artifact is None or sha is not None, f"`{field}.artifact` requires an exact `sha256`")
    if sha is not None:
        validate_sha256_identity(sha, f"`{field}.sha256`")
    _ensure(sha is not None or revision is not None, f"`{field}` must pin an exact sha256 or immutable revision")
    for k, val in (("artifact", artifact), ("sha256", sha), ("revision", revision)):
        if val is not None:
            out[k] = val
    params = d.get("parameters")
    if params is not None:
        _ensure(isinstance(params, dict), f"`{field}.parameters` must be an object")
        if params:
            out["parameters"] = dict(sorted(params.items()))
    return out


def decode_rollout_sampling(v: Any) -> Dict[str, Any]:
    d = _obj(v, "`sampling`")
    _deny_unknown(d, ("max_new_tokens", "temperature", "top_p"), "`sampling`")
    out = {"max_new_tokens": _uint(d, "max_new_tokens", "`sampling`"),
           "temperature": _float(d, "temperature", "`sampling`", 0.7),
           "top_p": _float(d, "top_p", "`sampling`", 0.95)}
    _ensure(1 <= out["max_new_tokens"] <= MAX_SEQUENCE_TOKENS, f"max_new_tokens must be in 1..={MAX_SEQUENCE_TOKENS}")
    _ensure(math.isfinite(out["temperature"]) and out["temperature"] > 0, "rollout temperature must be finite and positive")
    _ensure(math.isfinite(out["top_p"]) and 0 < out["top_p"] <= 1, "rollout top_p must be finite and in (0, 1]")
    return out


def decode_post_training(v: Any) -> Dict[str, Any]:
    """`PostTrainingConfig`, tagged by `algorithm`: dpo | forward_kl | grpo."""
    d = _obj(v, "`post_training`")
    algo = d.get("algorithm", _MISSING)
    if algo is _MISSING:
        raise ConfigError("missing field `algorithm` in `post_training`")
    if algo == "dpo":
        _deny_unknown(d, ("algorithm", "reference", "beta", "label_smoothing", "sequence_reduction"), "`post_training` (dpo)")
        if "reference" not in d:
            raise ConfigError("missing field `reference` in `post_training` (dpo)")
        out = {"algorithm": "dpo", "reference": decode_frozen_model(d["reference"], "reference"),
               "beta": _float(d, "beta", "`post_training`", 0.1),
               "label_smoothing": _float(d, "label_smoothing", "`post_training`", 0.0),
               "sequence_reduction": _enum(d, "sequence_reduction", "`post_training`", ("sum", "mean"), "sum")}
        _ensure(math.isfinite(out["beta"]) and out["beta"] > 0, "DPO beta must be finite and positive")
        _ensure(math.isfinite(out["label_smoothing"]) and 0 <= out["label_smoothing"] < 0.5,
                "DPO label_smoothing must be finite and in [0, 0.5)")
        return out
    if algo == "forward_kl":
        _deny_unknown(d, ("algorithm", "teacher", "temperature", "scale_by_temperature_squared"),
                      "`post_training` (forward_kl)")
        if "teacher" not in d:
            raise ConfigError("missing field `teacher` in `post_training` (forward_kl)")
        out = {"algorithm": "forward_kl", "teacher": decode_frozen_model(d["teacher"], "teacher"),
               "temperature": _float(d, "temperature", "`post_training`", 1.0),
               "scale_by_temperature_squared": _bool(d, "scale_by_temperature_squared", "`post_training`", True)}
        _ensure(math.isfinite(out["temperature"]) and out["temperature"] > 0,
                "distillation temperature must be finite and positive")
        return out
    if algo == "grpo":
        _deny_unknown(d, ("algorithm", "group_size", "clip_epsilon", "advantage_epsilon", "kl_coefficient", "reference",
                          "sampling"), "`post_training` (grpo)")
        out = {"algorithm": "grpo", "group_size": _uint(d, "group_size", "`post_training`", 8),
               "clip_epsilon": _float(d, "clip_epsilon", "`post_training`", 0.2),
               "advantage_epsilon": _float(d, "advantage_epsilon", "`post_training`", 1e-6),
               "kl_coefficient": _float(d, "kl_coefficient", "`post_training`", 0.04)}
        _ensure(2 <= out["group_size"] <= MAX_ROLLOUTS_PER_PROMPT, f"GRPO group_size must be in 2..={MAX_ROLLOUTS_PER_PROMPT}")
        _ensure(math.isfinite(out["clip_epsilon"]) and 0 < out["clip_epsilon"] < 1, "GRPO clip_epsilon must be finite and in (0, 1)")
        _ensure(math.isfinite(out["advantage_epsilon"]) and out["advantage_epsilon"] > 0,
                "GRPO advantage_epsilon must be finite and positive")
        _ensure(math.isfinite(out["kl_coefficient"]) and out["kl_coefficient"] >= 0,
                "GRPO kl_coefficient must be finite and non-negative")
        if d.get("reference") is not None:
            out["reference"] = decode_frozen_model(d["reference"], "reference")
        _ensure(out["kl_coefficient"] <= 0 or "reference" in out,
                "GRPO with positive kl_coefficient requires a frozen reference")
        if "sampling" not in d:
            raise ConfigError("missing field `sampling` in `post_training` (grpo)")
        out["sampling"] = decode_rollout_sampling(d["sampling"])
        return out
    raise ConfigError(f"unknown variant `{algo}` of `post_training.algorithm`, expected one of dpo, forward_kl, grpo")


def resolve_post_training_paths(cfg: Dict[str, Any], base: str) -> None:
    for key in ("reference", "teacher"):
        spec = cfg.get(key)
        if spec and spec.get("artifact") and not os.path.isabs(spec["artifact"]):
            spec["artifact"] = os.path.join(base, spec["artifact"])


# ---------------------------------------------------------------------------- sleep schedule
MAX_MEMORY_TIERS = 16
MAX_RESERVE_SLOTS_PER_TIER = 4_096
MAX_TOTAL_RESERVE_SLOTS = 16_384
MAX_MEMORY_TIER_ID_BYTES = 128


def decode_schedule(v: Any) -> Dict[str, Any]:
    d = _obj(v, "`schedule`")
    _deny_unknown(d, ("clock", "terminal_consolidation", "tiers"), "`schedule`")
    out = {"clock": _enum(d, "clock", "`schedule`", ("optimizer_steps", "model_tokens")),
           "terminal_consolidation": _enum(d, "terminal_consolidation", "`schedule`", ("distill_into_base_v1",))}
    tiers = d.get("tiers", _MISSING)
    if tiers is _MISSING:
        raise ConfigError("missing field `tiers` in `schedule`")
    _ensure(isinstance(tiers, list), "`schedule.tiers` must be an array")
    _ensure(2 <= len(tiers) <= MAX_MEMORY_TIERS, f"sleep requires 2..={MAX_MEMORY_TIERS} memory tiers")
    decoded: List[Dict[str, Any]] = []
    ids, total = set(), 0
    for i, t in enumerate(tiers):
        td = _obj(t, f"memory tier {i}")
        _deny_unknown(td, ("id", "update_period", "reserve_slots"), f"memory tier {i}")
        tier = {"id": _str(td, "id", f"memory tier {i}"), "update_period": _uint(td, "update_period", f"memory tier {i}"),
                "reserve_slots": _uint(td, "reserve_slots", f"memory tier {i}")}
        _ensure(tier["id"].strip() != "" and len(tier["id"].encode()) <= MAX_MEMORY_TIER_ID_BYTES,
                f"memory tier {i} id must contain 1..={MAX_MEMORY_TIER_ID_BYTES} bytes")
        _ensure(tier["id"] not in ids, f"duplicate memory tier id `{tier['id']}`")
        ids.add(tier["id"])
        _ensure(tier["update_period"] > 0, f"memory tier `{tier['id']}` update_period must be positive")
        _ensure(1 <= tier["reserve_slots"] <= MAX_RESERVE_SLOTS_PER_TIER,
                f"memory tier `{tier['id']}` reserve_slots must be in 1..={MAX_RESERVE_SLOTS_PER_TIER}")
        total += tier["reserve_slots"]
        _ensure(total <= MAX_TOTAL_RESERVE_SLOTS, f"sleep schedule exceeds the {MAX_TOTAL_RESERVE_SLOTS}-slot total reserve limit")
        if decoded:
            f = decoded[-1]
            _ensure(tier["update_period"] > f["update_period"],
                    f"memory tier `{tier['id']}` must update less often than `{f['id']}`")
            _ensure(tier["update_period"] % f["update_period"] == 0,
                    f"memory tier `{tier['id']}` period {tier['update_period']} must be divisible by faster tier "
                    f"`{f['id']}` period {f['update_period']}")
            per = tier["update_period"] // f["update_period"]
            _ensure(tier["reserve_slots"] >= per,
                    f"memory tier `{tier['id']}` needs at least {per} reserve slots to receive every `{f['id']}` "
                    "boundary before reclamation")
        decoded.append(tier)
    out["tiers"] = decoded
    return out


def decode_tier_optimizer(v: Any) -> Dict[str, Any]:
    if v is None:
        v = {"learning_rate": 3e-4, "beta_1": 0.9, "beta_2": 0.95, "epsilon": 1e-8, "weight_decay": 0.1}
    d = _obj(v, "`tier_optimizer`")
    names = ("learning_rate", "beta_1", "beta_2", "epsilon", "weight_decay")
    _deny_unknown(d, names, "`tier_optimizer`")
    out = {k: _float(d, k, "`tier_optimizer`") for k in names}
    _ensure(math.isfinite(out["learning_rate"]) and out["learning_rate"] > 0, "tier learning rate must be finite and positive")
    for k in ("beta_1", "beta_2"):
        _ensure(math.isfinite(out[k]) and 0 <= out[k] < 1, f"tier AdamW {k} must be in [0, 1)")
    _ensure(math.isfinite(out["epsilon"]) and out["epsilon"] > 0, "tier AdamW epsilon must be finite and positive")
    _ensure(math.isfinite(out["weight_decay"]) and out["weight_decay"] >= 0,
            "tier AdamW weight decay must be finite and non-negative")
    return out


def decode_memory_update_mode(v: Any, phase: str) -> Dict[str, Any]:
    d = _obj(v, "`memory_update_mode`")
    if d.get("type", _MISSING) is _MISSING:
        raise ConfigError("missing field `type` in `memory_update_mode`")
    if d["type"] != "wake_only":
        raise ConfigError(f"unknown variant `{d['type']}` of `memory_update_mode.type`, expected wake_only")
    _deny_unknown(d, ("type", "schedule", "tier_optimizer"), "`memory_update_mode`")
    if "schedule" not in d:
        raise ConfigError("missing field `schedule` in `memory_update_mode`")
    try:
        return {"type": "wake_only", "schedule": decode_schedule(d["schedule"]),
                "tier_optimizer": decode_tier_optimizer(d.get("tier_optimizer"))}
    except ConfigError as e:
        raise ConfigError(f"invalid wake_only memory update mode in workflow phase `{phase}`: {e}")


# ---------------------------------------------------------------------------- in-model sleep
def _decode_knowledge(v: Any) -> Dict[str, Any]:
    w = "`knowledge_seeding`"
    d = _obj(v, w)
    _deny_unknown(d, ("chunk_tokens", "teacher_rollouts", "detached_student_rollouts", "temperature", "forward_kl_weight"), w)
    out = {"chunk_tokens": _uint(d, "chunk_tokens", w), "teacher_rollouts": _uint(d, "teacher_rollouts", w),
           "detached_student_rollouts": _uint(d, "detached_student_rollouts", w),
           "temperature": _float(d, "temperature", w), "forward_kl_weight": _float(d, "forward_kl_weight", w)}
    _ensure(out["chunk_tokens"] > 0, "knowledge-seeding chunk_tokens must be positive")
    _ensure(out["chunk_tokens"] <= 16_384, "knowledge-seeding chunk_tokens exceeds the 16384-token operational limit")
    _ensure(out["teacher_rollouts"] > 0 and out["detached_student_rollouts"] > 0,
            "knowledge seeding requires teacher and detached-student rollouts")
    _ensure(out["teacher_rollouts"] + out["detached_student_rollouts"] <= 1_024,
            "knowledge-seeding rollout count exceeds the 1024-rollout operational limit")
    _ensure(math.isfinite(out["temperature"]) and out["temperature"] > 0, "knowledge-seeding temperature must be positive")
    _ensure(math.isfinite(out["forward_kl_weight"]) and out["forward_kl_weight"] >= 0,
            "knowledge-seeding KL weight must be non-negative")
    return out


def _decode_imitation(v: Any) -> Dict[str, Any]:
    w = "`imitation`"
    d = _obj(v, w)
    _deny_unknown(d, ("semantic_judge_hash", "semantic_weight", "maximum_edit_distance", "grpo_group_size"), w)
    out = {"semantic_judge_hash": _str(d, "semantic_judge_hash", w), "semantic_weight": _float(d, "semantic_weight", w),
           "maximum_edit_distance": _uint(d, "maximum_edit_distance", w), "grpo_group_size": _uint(d, "grpo_group_size", w)}
    validate_sha256_identity(out["semantic_judge_hash"], "imitation semantic-judge hash")
    _ensure(math.isfinite(out["semantic_weight"]) and 0 <= out["semantic_weight"] <= 1,
            "imitation semantic_weight must be in [0, 1]")
    _ensure(out["grpo_group_size"] >= 2, "imitation GRPO group must contain at least two samples")
    _ensure(out["maximum_edit_distance"] <= 4_096, "imitation maximum edit distance exceeds the 4096-token operational limit")
    _ensure(out["grpo_group_size"] <= 256, "imitation GRPO group size exceeds the 256-sample operational limit")
    return out


def _decode_dreaming(v: Any) -> Dict[str, Any]:
    w = "`dreaming`"
    d = _obj(v, w)
    ints = ("candidate_count", "retain_top", "retain_random", "lora_rank", "lora_alpha", "restem_iterations")
    strs = ("selector_version", "reference_set_hash", "trial_evaluator_hash")
    _deny_unknown(d, ints + strs, w)
    out: Dict[str, Any] = {k: _uint(d, k, w) for k in ints}
    out.update({k: _str(d, k, w) for k in strs})
    _ensure(0 < out["candidate_count"] <= 1_024, "dream candidate count must be in 1..=1024")
    retained = out["retain_top"] + out["retain_random"]
    _ensure(retained <= out["candidate_count"], "dream selection quotas exceed candidate count")
    _ensure(retained > 0, "dream selection must retain at least one candidate")
    _ensure(out["lora_rank"] > 0 and out["lora_alpha"] > 0, "dream LoRA geometry must be positive")
    _ensure(out["lora_rank"] <= 1_024, "dream LoRA rank exceeds the 1024-rank operational limit")
    _ensure(out["lora_alpha"] <= 65_536, "dream LoRA alpha exceeds the 65536 operational limit")
    _ensure(0 < out["restem_iterations"] <= 128, "ReSTEM iterations must be in 1..=128")
    _ensure(out["selector_version"].strip() != "", "dream selector version must not be empty")
    validate_sha256_identity(out["reference_set_hash"], "dream reference-set hash")
    validate_sha256_identity(out["trial_evaluator_hash"], "dream trial-evaluator hash")
    return out


def _decode_retention(v: Any) -> Dict[str, Any]:
    w = "`retention`"
    d = _obj(v, w)
    names = ("evaluator_hash", "suite_hash", "max_anchor_forward_kl", "max_anchor_regression", "min_incorporation_gain")
    _deny_unknown(d, names, w)
    out = {"evaluator_hash": _str(d, "evaluator_hash", w), "suite_hash": _str(d, "suite_hash", w),
           "max_anchor_forward_kl": _float(d, "max_anchor_forward_kl", w),
           "max_anchor_regression": _float(d, "max_anchor_regression", w),
           "min_incorporation_gain": _float(d, "min_incorporation_gain", w)}
    validate_sha256_identity(out["evaluator_hash"], "retention evaluator identity")
    validate_sha256_identity(out["suite_hash"], "retention suite identity")
    _ensure(math.isfinite(out["max_anchor_forward_kl"]) and out["max_anchor_forward_kl"] >= 0,
            "retention KL gate must be finite and non-negative")
    _ensure(math.isfinite(out["max_anchor_regression"]) and out["max_anchor_regression"] >= 0,
            "retention regression gate must be finite and non-negative")
    _ensure(math.isfinite(out["min_incorporation_gain"]), "incorporation gate is non-finite")
    return out


SLEEP_FIELDS = ("schedule", "standalone_trigger_clock", "knowledge_seeding", "imitation", "dreaming", "retention_suite",
                "retention_suite_sha256", "retention", "receiver_learning_rate", "receiver_weight_decay",
                "grpo_clip_epsilon", "grpo_advantage_epsilon", "grpo_kl_coefficient", "candidate_directory")


def decode_in_model_sleep(v: Any, phase: str, field: str) -> Dict[str, Any]:
    """`InModelSleepConfig` of a `sleep` phase or of a `periodic_sleep` hook."""
    w = f"`{field}`"
    d = _obj(v, w)
    _deny_unknown(d, SLEEP_FIELDS, w)
    try:
        for req in ("schedule", "knowledge_seeding", "imitation", "retention"):
            if req not in d:
                raise ConfigError(f"missing field `{req}` in {w}")
        out: Dict[str, Any] = {"schedule": decode_schedule(d["schedule"])}
        if d.get("standalone_trigger_clock") is not None:
            out["standalone_trigger_clock"] = _uint(d, "standalone_trigger_clock", w)
        out["knowledge_seeding"] = _decode_knowledge(d["knowledge_seeding"])
        out["imitation"] = _decode_imitation(d["imitation"])
        if d.get("dreaming") is not None:
            out["dreaming"] = _decode_dreaming(d["dreaming"])
        out["retention_suite"] = _str(d, "retention_suite", w)
        out["retention_suite_sha256"] = _str(d, "retention_suite_sha256", w)
        out["retention"] = _decode_retention(d["retention"])
        for k in ("receiver_learning_rate", "receiver_weight_decay", "grpo_clip_epsilon", "grpo_advantage_epsilon",
                  "grpo_kl_coefficient"):
            out[k] = _float(d, k, w)
        out["candidate_directory"] = _str(d, "candidate_directory", w)
        _ensure(out["retention_suite"] != "" and out["candidate_directory"] != "",
                f"sleep phase `{phase}` requires retention_suite and candidate_directory")
        validate_sha256_identity(out["retention_suite_sha256"], "sleep retention suite identity")
        _ensure(math.isfinite(out["receiver_learning_rate"]) and out["receiver_learning_rate"] > 0,
                "receiver learning rate must be finite and positive")
        _ensure(math.isfinite(out["receiver_weight_decay"]) and out["receiver_weight_decay"] >= 0,
                "receiver weight decay must be finite and non-negative")
        _ensure(math.isfinite(out["grpo_clip_epsilon"]) and 0 < out["grpo_clip_epsilon"] < 1,
                "GRPO clip epsilon must be in (0, 1)")
        _ensure(math.isfinite(out["grpo_advantage_epsilon"]) and out["grpo_advantage_epsilon"] > 0,
                "GRPO advantage epsilon must be positive")
        _ensure(math.isfinite(out["grpo_kl_coefficient"]) and out["grpo_kl_coefficient"] >= 0,
                "GRPO KL coefficient must be finite and non-negative")
        _ensure(out["retention"]["suite_hash"] == out["retention_suite_sha256"],
                f"sleep phase `{phase}` retention evaluator is not bound to retention_suite_sha256")
    except ConfigError as e:
        raise ConfigError(f"invalid {field} in workflow phase `{phase}`: {e}")
    return out


def resolve_sleep_paths(cfg: Dict[str, Any], base: str) -> None:
    for key in ("retention_suite", "candidate_directory"):
        if cfg.get(key) and not os.path.isabs(cfg[key]):
            cfg[key] = os.path.join(base, cfg[key])
