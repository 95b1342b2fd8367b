"""Append-only `metrics.jsonl`, schema version 2, in the reference's wire format.

Record (`summa-train/src/metrics.rs:437-449`, unknown fields denied):
    {schema_version: 2, sequence, emitted_at_unix_ms, run_id (string), global_step,
     phase: {index, name, kind}, checkpoint_hash?: "sha256:<64 hex>", event: {type, values}}
`event.type` is one of the fourteen typed events of `metrics.rs:419-435`; `values` carries exactly the
fields of that event's struct (`metrics.rs:92-418`): required fields present, optional ones either
absent or non-null, JSON types exact, enums by their snake_case names. The per-event consistency rules
of `metrics.rs:1650-2112` (time components within the elapsed time, rates equal to counts over time,
tier clocks on their period, objective-specific fields of a post-training update, ...) are enforced on
write and on read, so a journal written here is accepted by the reference's tooling (Model Lab, the
W&B sidecar) and a journal written there loads here. `run_id` is the 16-hex-digit FNV-1a64 of the run
signature (`summa-train/src/main.rs:1169-1171`).

Journal rules (`metrics.rs:1598-1627`): sequences count from 0 without gaps, one run id per file,
global steps and timestamps never rewind. On resume the journal is cut back to the prefix the
checkpoint committed, after that prefix has been validated record by record.

Things the trainer used to write as ad-hoc events (run / phase boundaries, checkpoints, dropped
samples) are expressed with the schema's own vocabulary: `phase_timing` records with a
`started | progress | completed | failed` boundary, and the record-level `checkpoint_hash`.
"""
from __future__ import annotations

import json
import math
import os
import time
from typing import Any, Dict, Iterator, List, Optional, Tuple

SCHEMA_VERSION = 2
MAX_METRIC_RECORD_BYTES = 16 * 1024 * 1024

PHASE_KINDS = ("pretrain", "continued_pretrain", "sft", "preference", "rl", "distillation", "sleep", "evaluation",
               "promotion", "quantization", "corpus_preparation")
MEMORY_TIERS = ("fast", "medium", "slow")

# field kinds
U32, U64, F64, BOOL, STR = "u32", "u64", "f64", "bool", "str"


def _enum(*names):
    return ("enum", names)


F64_LIST = "f64_list"

# event -> [(field, kind, required)] in the reference's declaration order
EVENTS: Dict[str, List[Tuple[str, Any, bool]]] = {
    "phase_timing": [("boundary", _enum("started", "progress", "completed", "failed"), True),
                     ("elapsed_seconds", F64, True), ("input_wait_seconds", F64, True), ("forward_seconds", F64, True),
                     ("backward_seconds", F64, True), ("optimizer_seconds", F64, True), ("checkpoint_seconds", F64, True)],
    "tier_update": [("transaction_id", STR, True), ("tier", _enum(*MEMORY_TIERS), True),
                    ("receiver_tier", _enum(*MEMORY_TIERS), False), ("tier_clock", U64, True), ("update_period", U64, True),
                    ("accumulated_micro_steps", U64, True),
                    ("outcome", _enum("prospective", "committed", "rolled_back", "skipped"), True),
                    ("update_l2_norm", F64, False), ("reserve_slot", U32, False), ("reserve_generation", U64, False),
                    ("optimizer_state_reset", BOOL, True)],
    "active_capacity": [("tier", _enum(*MEMORY_TIERS), True), ("active_base_experts", U32, True),
                        ("active_reserve_experts", U32, True), ("dormant_reserve_experts", U32, True),
                        ("routed_top_k", U32, True), ("reserve_routed_top_k", U32, True),
                        ("routed_active_parameters", U64, True), ("stored_parameters", U64, True),
                        ("dream_generation", BOOL, True), ("random_extra_expert", BOOL, True)],
    "wake_capacity_envelope": [("initial_wake_routed_active_parameters", U64, True),
                               ("completed_sleep_cycles_observed", U64, True),
                               ("minimum_observed_wake_routed_active_parameters", U64, True),
                               ("maximum_observed_wake_routed_active_parameters", U64, True),
                               ("stored_parameters", U64, True)],
    "distillation_divergence": [("transaction_id", STR, True), ("teacher_hash", STR, True), ("student_hash", STR, True),
                                ("chunk_index", U32, True), ("chunk_count", U32, True), ("selected_tokens", U64, True),
                                ("total_tokens", U64, True), ("forward_kl", F64, True), ("reverse_kl", F64, False),
                                ("teacher_entropy", F64, True), ("student_entropy", F64, True)],
    "imitation_reward": [("transaction_id", STR, True), ("semantic_judge_hash", STR, True), ("samples", U64, True),
                         ("semantic_score_mean", F64, True), ("normalized_levenshtein_mean", F64, True),
                         ("levenshtein_threshold", F64, True), ("reward_mean", F64, True), ("reward_stddev", F64, True),
                         ("grpo_kl", F64, True)],
    "dream_selection": [("transaction_id", STR, True), ("selector_version", STR, True), ("reference_set_hash", STR, True),
                        ("candidates_generated", U32, True), ("selected_by_alignment", U32, True),
                        ("selected_random", U32, True), ("random_quota", U32, True), ("gradient_cosine_mean", F64, True),
                        ("gradient_cosine_max", F64, True), ("selected_manifest_hash", STR, True)],
    "dream_trial": [("transaction_id", STR, True), ("candidate_hash", STR, True), ("adapter_hash", STR, True),
                    ("evaluator_hash", STR, True), ("lora_rank", U32, True), ("lora_alpha", F64, True),
                    ("independent_task_delta", F64, True), ("reward", F64, True), ("elapsed_seconds", F64, True),
                    ("accepted", BOOL, True), ("isolated", BOOL, True), ("shared_checkpoint_unchanged", BOOL, True)],
    "retention_delta": [("transaction_id", STR, True), ("suite", STR, True), ("metric", STR, True),
                        ("evaluator_hash", STR, True), ("direction", _enum("higher_is_better", "lower_is_better"), True),
                        ("baseline_score", F64, True), ("candidate_score", F64, True), ("improvement", F64, True),
                        ("maximum_allowed_regression", F64, True), ("passed", BOOL, True)],
    "quantization": [("stage", _enum("calibration", "fake_quantization", "export", "acceptance"), True),
                     ("format", _enum("binary_g128", "ternary_g128", "ternary_entropy_g128"), True),
                     ("group_size", U32, True), ("progress_fraction", F64, True), ("tensors_quantized", U64, True),
                     ("weights_quantized", U64, True), ("average_bits_per_weight", F64, False), ("packed_bytes", U64, False),
                     ("mean_squared_error", F64, False), ("max_absolute_error", F64, False),
                     ("distillation_forward_kl", F64, False), ("acceptance_delta", F64, False),
                     ("embeddings_quantized", BOOL, True), ("lm_head_quantized", BOOL, True)],
    "device_utilization": [("sampled_at_unix_ms", U64, True), ("device_index", U32, True),
                           ("sample_window_seconds", F64, True), ("gpu_utilization_percent", F64, True),
                           ("sm_active_percent", F64, False), ("tensor_core_active_percent", F64, False),
                           ("memory_bandwidth_percent", F64, False), ("memory_used_bytes", U64, True),
                           ("memory_total_bytes", U64, True), ("power_watts", F64, False),
                           ("temperature_celsius", F64, False)],
    "throughput": [("optimizer_steps", U64, True), ("compute_tokens", U64, True), ("supervised_tokens", U64, True),
                   ("examples", U64, True), ("elapsed_seconds", F64, True), ("tokens_per_second", F64, True),
                   ("examples_per_second", F64, True), ("input_wait_seconds", F64, True),
                   ("host_to_device_seconds", F64, True), ("gpu_busy_seconds", F64, True)],
    "optimization": [("objective", STR, True), ("loss", F64, True), ("optimized_loss", F64, True),
                     ("weighted_loss", F64, True), ("router_aux_loss", F64, False), ("retrieval_accuracy", F64, False),
                     ("learning_rate", F64, True), ("muon_learning_rate", F64, True), ("gradient_norm", F64, True),
                     ("layer_gradient_norms", F64_LIST, False), ("sequence_length", U32, True), ("batch_size", U32, True),
                     ("gradient_accumulation", U32, True), ("compute_tokens", U64, True), ("supervised_tokens", U64, True),
                     ("examples", U64, True), ("truncated_tokens", U64, True), ("retrieval_candidates", U64, True)],
    "post_training_update": [("transaction_id", STR, True), ("algorithm", _enum("dpo", "forward_kl", "grpo"), True),
                             ("epoch", U64, True), ("first_record", U64, True), ("records", U64, True),
                             ("optimizer_step", U64, True), ("rng_counter_start", U64, True), ("rng_counter_end", U64, True),
                             ("loss", F64, True), ("checkpoint_sha256", STR, True), ("optimizer_sha256", STR, True),
                             ("preference_accuracy", F64, False), ("implicit_reward_margin", F64, False),
                             ("forward_kl", F64, False), ("teacher_entropy", F64, False), ("top1_agreement", F64, False),
                             ("mean_reward", F64, False), ("reward_stddev", F64, False), ("mean_kl", F64, False),
                             ("clipped_fraction", F64, False)],
}
EVENT_TYPES = tuple(EVENTS)


class MetricsError(ValueError):
    pass


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise MetricsError(msg)


def _is_uint(v, bits: int) -> bool:
    return isinstance(v, int) and not isinstance(v, bool) and 0 <= v < (1 << bits)


def _is_num(v) -> bool:
    return isinstance(v, (int, float)) and not isinstance(v, bool)


def _identifier(name: str, value) -> None:
    _need(isinstance(value, str) and value.strip() != "", f"{name} must not be empty")
    _need("\n" not in value and "\r" not in value, f"{name} must not contain a newline")


def _sha(value, what: str) -> None:
    ok = (isinstance(value, str) and value.startswith("sha256:") and len(value) == 71
          and all(c in "0123456789abcdef" for c in value[7:]))
    _need(ok, f"{what} must be `sha256:` followed by 64 lowercase hex characters")


def _finite(name, v) -> None:
    _need(math.isfinite(v), f"{name} must be finite")


def _nonneg(name, v) -> None:
    _finite(name, v)
    _need(v >= 0.0, f"{name} must be non-negative")


def _unit(name, v) -> None:
    _finite(name, v)
    _need(0.0 <= v <= 1.0, f"{name} must be in [0, 1]")


def _signed_unit(name, v) -> None:
    _finite(name, v)
    _need(-1.0 <= v <= 1.0, f"{name} must be in [-1, 1]")


def _percent(name, v) -> None:
    _finite(name, v)
    _need(0.0 <= v <= 100.0, f"{name} must be in [0, 100]")


def _approx(a: float, b: float) -> bool:
    return abs(a - b) <= 1e-9 * max(1.0, abs(a), abs(b)) + 1e-12 or abs(a - b) <= 1e-6 * max(abs(a), abs(b))


def _timing_tolerance(elapsed: float) -> float:
    return max(1e-6, 1e-6 * abs(elapsed))


def validate_event(event_type: str, v: Dict[str, Any]) -> None:
    """Shape (fields, JSON types, enums) and the consistency rules of one event."""
    _need(event_type in EVENTS, f"unknown metric event `{event_type}`")
    _need(isinstance(v, dict), "metric event values must be an object")
    spec = EVENTS[event_type]
    known = {name for name, _, _ in spec}
    extra = sorted(set(v) - known)
    _need(not extra, f"unknown field `{extra[0] if extra else ''}` in `{event_type}` metrics")
    for name, kind, required in spec:
        if name not in v:
            _need(not required, f"missing field `{name}` in `{event_type}` metrics")
            continue
        x = v[name]
        _need(x is not None or not required, f"`{name}` of `{event_type}` must not be null")
        if x is None:
            continue
        if kind == U32:
            _need(_is_uint(x, 32), f"`{name}` of `{event_type}` must be an unsigned 32-bit integer")
        elif kind == U64:
            _need(_is_uint(x, 64), f"`{name}` of `{event_type}` must be an unsigned 64-bit integer")
        elif kind == F64:
            _need(_is_num(x), f"`{name}` of `{event_type}` must be a number")
        elif kind == BOOL:
            _need(isinstance(x, bool), f"`{name}` of `{event_type}` must be a boolean")
        elif kind == STR:
            _need(isinstance(x, str), f"`{name}` of `{event_type}` must be a string")
        elif kind == F64_LIST:
            _need(isinstance(x, list) and all(_is_num(e) for e in x), f"`{name}` of `{event_type}` must be an array of numbers")
        else:
            _need(isinstance(x, str) and x in kind[1], f"`{name}` of `{event_type}`: unknown variant `{x}`")
    g = v.get
    if event_type == "phase_timing":
        parts = ("input_wait_seconds", "forward_seconds", "backward_seconds", "optimizer_seconds", "checkpoint_seconds")
        _nonneg("elapsed_seconds", v["elapsed_seconds"])
        for k in parts:
            _nonneg(k, v[k])
        accounted = sum(v[k] for k in parts)
        _need(accounted <= v["elapsed_seconds"] + _timing_tolerance(v["elapsed_seconds"]),
              f"phase component time {accounted} exceeds elapsed time {v['elapsed_seconds']}")
    elif event_type == "tier_update":
        _identifier("transaction_id", v["transaction_id"])
        _need(v["update_period"] > 0, "update_period must be positive")
        _need(v["tier_clock"] % v["update_period"] == 0, "tier_clock must be on its update-period boundary")
        if g("update_l2_norm") is not None:
            _nonneg("update_l2_norm", v["update_l2_norm"])
        _need((g("reserve_slot") is None) == (g("reserve_generation") is None),
              "reserve_slot and reserve_generation must be present together")
        _need(not v["optimizer_state_reset"] or v["outcome"] == "committed",
              "only a committed tier update can reset optimizer state")
    elif event_type == "active_capacity":
        cap = v["active_reserve_experts"] + v["dormant_reserve_experts"]
        _need(0 < cap < (1 << 32), "sleep reserve capacity must be positive and fit u32")
        _need(v["routed_top_k"] > 0, "routed_top_k must be positive")
        _need(v["reserve_routed_top_k"] == 1, "sleep reserve route width must remain exactly one")
        _need(v["routed_top_k"] <= v["active_base_experts"], "routed_top_k exceeds persistent base experts")
        _need(0 < v["routed_active_parameters"] <= v["stored_parameters"],
              "routed and stored parameters must be positive, and routed parameters must not exceed stored parameters")
        _need(not v["random_extra_expert"] or v["dream_generation"],
              "random-extra-expert routing is only valid during dream generation")
        if v["random_extra_expert"]:
            _need(v["routed_top_k"] < v["active_base_experts"], "persistent base MoE has no expert outside ordinary top-k")
    elif event_type == "wake_capacity_envelope":
        init, lo, hi = (v["initial_wake_routed_active_parameters"], v["minimum_observed_wake_routed_active_parameters"],
                        v["maximum_observed_wake_routed_active_parameters"])
        _need(init > 0 and lo > 0 and hi > 0, "wake capacity measurements must be positive")
        _need(v["completed_sleep_cycles_observed"] > 0, "wake capacity envelope requires completed sleep-cycle observations")
        _need(lo <= hi, "wake capacity envelope is inverted")
        _need(lo == init == hi, "wake routed-active parameters changed across sleep cycles")
        _need(hi <= v["stored_parameters"], "wake routed parameters exceed stored parameters")
    elif event_type == "distillation_divergence":
        _identifier("transaction_id", v["transaction_id"])
        _sha(v["teacher_hash"], "teacher_hash")
        _sha(v["student_hash"], "student_hash")
        _need(v["chunk_count"] > 0, "chunk_count must be positive")
        _need(v["chunk_index"] < v["chunk_count"], "chunk_index must be less than chunk_count")
        _need(v["total_tokens"] > 0, "total_tokens must be positive")
        _need(0 < v["selected_tokens"] <= v["total_tokens"], "selected_tokens must be in 1..=total_tokens")
        _nonneg("forward_kl", v["forward_kl"])
        if g("reverse_kl") is not None:
            _nonneg("reverse_kl", v["reverse_kl"])
        _nonneg("teacher_entropy", v["teacher_entropy"])
        _nonneg("student_entropy", v["student_entropy"])
    elif event_type == "imitation_reward":
        _identifier("transaction_id", v["transaction_id"])
        _sha(v["semantic_judge_hash"], "semantic_judge_hash")
        _need(v["samples"] > 0, "imitation samples must be positive")
        for k in ("semantic_score_mean", "normalized_levenshtein_mean", "levenshtein_threshold"):
            _unit(k, v[k])
        _finite("reward_mean", v["reward_mean"])
        _nonneg("reward_stddev", v["reward_stddev"])
        _nonneg("grpo_kl", v["grpo_kl"])
    elif event_type == "dream_selection":
        _identifier("transaction_id", v["transaction_id"])
        _identifier("selector_version", v["selector_version"])
        _sha(v["reference_set_hash"], "reference_set_hash")
        _sha(v["selected_manifest_hash"], "selected_manifest_hash")
        _need(v["candidates_generated"] > 0, "dream selection requires generated candidates")
        _need(v["random_quota"] <= v["candidates_generated"], "random dream quota exceeds generated candidates")
        _need(v["selected_random"] <= v["random_quota"], "selected random dreams exceed the configured quota")
        sel = v["selected_by_alignment"] + v["selected_random"]
        _need(0 < sel <= v["candidates_generated"], "selected dream count must be in 1..=candidates_generated")
        _signed_unit("gradient_cosine_mean", v["gradient_cosine_mean"])
        _signed_unit("gradient_cosine_max", v["gradient_cosine_max"])
        _need(v["gradient_cosine_max"] >= v["gradient_cosine_mean"], "maximum gradient cosine is below the mean")
    elif event_type == "dream_trial":
        _identifier("transaction_id", v["transaction_id"])
        for k in ("candidate_hash", "adapter_hash", "evaluator_hash"):
            _sha(v[k], k)
        _need(v["lora_rank"] > 0, "LoRA rank must be positive")
        _finite("lora_alpha", v["lora_alpha"])
        _need(v["lora_alpha"] > 0.0, "LoRA alpha must be positive")
        _finite("independent_task_delta", v["independent_task_delta"])
        _finite("reward", v["reward"])
        _nonneg("elapsed_seconds", v["elapsed_seconds"])
        _need(v["isolated"], "dream trial must be isolated")
        _need(v["shared_checkpoint_unchanged"], "dream trial mutated the shared candidate checkpoint")
    elif event_type == "retention_delta":
        for k in ("transaction_id", "suite", "metric"):
            _identifier(k, v[k])
        _sha(v["evaluator_hash"], "evaluator_hash")
        for k in ("baseline_score", "candidate_score", "improvement"):
            _finite(k, v[k])
        _nonneg("maximum_allowed_regression", v["maximum_allowed_regression"])
        expected = (v["candidate_score"] - v["baseline_score"] if v["direction"] == "higher_is_better"
                    else v["baseline_score"] - v["candidate_score"])
        _need(_approx(expected, v["improvement"]),
              f"retention improvement {v['improvement']} does not match scores (expected {expected})")
        _need(v["passed"] == (v["improvement"] >= -v["maximum_allowed_regression"]),
              "retention passed flag disagrees with the configured regression gate")
    elif event_type == "quantization":
        _need(v["group_size"] > 0, "quantization group_size must be positive")
        _unit("progress_fraction", v["progress_fraction"])
        if g("average_bits_per_weight") is not None:
            _finite("average_bits_per_weight", v["average_bits_per_weight"])
            _need(v["average_bits_per_weight"] > 0.0, "average_bits_per_weight must be positive")
        for k in ("mean_squared_error", "max_absolute_error", "distillation_forward_kl"):
            if g(k) is not None:
                _nonneg(k, v[k])
        if g("acceptance_delta") is not None:
            _finite("acceptance_delta", v["acceptance_delta"])
        if v["stage"] == "export":
            _need(g("mean_squared_error") is not None and g("max_absolute_error") is not None,
                  "quantization export requires error measurements")
            if v["weights_quantized"] > 0:
                _need(g("average_bits_per_weight") is not None and g("packed_bytes") is not None,
                      "quantization export requires packed size and bits-per-weight")
                _need(v["tensors_quantized"] > 0 and v["packed_bytes"] > 0,
                      "non-empty quantization export requires tensors and packed bytes")
            _need(_approx(v["progress_fraction"], 1.0), "quantization export must report complete progress")
    elif event_type == "device_utilization":
        _finite("sample_window_seconds", v["sample_window_seconds"])
        _need(v["sample_window_seconds"] > 0.0, "device sample window must be positive")
        _percent("gpu_utilization_percent", v["gpu_utilization_percent"])
        for k in ("sm_active_percent", "tensor_core_active_percent", "memory_bandwidth_percent"):
            if g(k) is not None:
                _percent(k, v[k])
        _need(v["memory_used_bytes"] <= v["memory_total_bytes"], "used GPU memory exceeds total GPU memory")
        if g("power_watts") is not None:
            _nonneg("power_watts", v["power_watts"])
        if g("temperature_celsius") is not None:
            _finite("temperature_celsius", v["temperature_celsius"])
    elif event_type == "throughput":
        _need(v["optimizer_steps"] > 0, "optimizer_steps must be positive")
        _finite("elapsed_seconds", v["elapsed_seconds"])
        _need(v["elapsed_seconds"] > 0.0, "elapsed_seconds must be positive")
        _need(v["compute_tokens"] > 0 and v["examples"] > 0, "throughput window must contain tokens and examples")
        _need(v["supervised_tokens"] <= v["compute_tokens"], "throughput supervised tokens exceed compute tokens")
        for k in ("tokens_per_second", "examples_per_second", "input_wait_seconds", "host_to_device_seconds",
                  "gpu_busy_seconds"):
            _nonneg(k, v[k])
        _need(v["input_wait_seconds"] <= v["elapsed_seconds"], "input wait exceeds throughput window")
        _need(v["host_to_device_seconds"] <= v["elapsed_seconds"], "host-to-device time exceeds throughput window")
        _need(v["gpu_busy_seconds"] <= v["elapsed_seconds"], "GPU busy time exceeds throughput window")
        _need(_approx(v["compute_tokens"] / v["elapsed_seconds"], v["tokens_per_second"]),
              "tokens_per_second does not match compute_tokens / elapsed_seconds")
        _need(_approx(v["examples"] / v["elapsed_seconds"], v["examples_per_second"]),
              "examples_per_second does not match examples / elapsed_seconds")
    elif event_type == "optimization":
        _identifier("objective", v["objective"])
        for k in ("loss", "optimized_loss", "weighted_loss"):
            _finite(k, v[k])
        if g("router_aux_loss") is not None:
            _finite("router_aux_loss", v["router_aux_loss"])
        if g("retrieval_accuracy") is not None:
            _unit("retrieval_accuracy", v["retrieval_accuracy"])
        for k in ("learning_rate", "muon_learning_rate", "gradient_norm"):
            _nonneg(k, v[k])
        if g("layer_gradient_norms") is not None:
            _need(len(v["layer_gradient_norms"]) > 0, "layer_gradient_norms must not be empty")
            for n in v["layer_gradient_norms"]:
                _nonneg("layer_gradient_norm", n)
        _need(v["sequence_length"] > 0 and v["batch_size"] > 0 and v["gradient_accumulation"] > 0,
              "optimization geometry must be positive")
        _need(v["examples"] > 0 and v["compute_tokens"] > 0, "optimization batch is empty")
        _need(v["supervised_tokens"] <= v["compute_tokens"], "supervised tokens exceed compute tokens")
    elif event_type == "post_training_update":
        for k in ("transaction_id", "checkpoint_sha256", "optimizer_sha256"):
            _sha(v[k], k)
        _need(v["records"] > 0, "post-training update is empty")
        _need(v["first_record"] + v["records"] < (1 << 64), "post-training record interval overflows u64")
        _need(v["optimizer_step"] > 0, "optimizer_step must be positive")
        _need(v["rng_counter_end"] >= v["rng_counter_start"], "post-training RNG range is inverted")
        _finite("post_training_loss", v["loss"])
        dpo = [g("preference_accuracy"), g("implicit_reward_margin")]
        kl = [g("forward_kl"), g("teacher_entropy"), g("top1_agreement")]
        grpo = [g("mean_reward"), g("reward_stddev"), g("mean_kl"), g("clipped_fraction")]
        none = lambda xs: all(x is None for x in xs)     # noqa: E731
        full = lambda xs: all(x is not None for x in xs)  # noqa: E731
        rng = v["rng_counter_end"] - v["rng_counter_start"]
        if v["algorithm"] == "dpo":
            _nonneg("post_training_loss", v["loss"])
            _need(full(dpo) and none(kl) and none(grpo), "DPO metrics contain a missing or foreign objective field")
            _unit("preference_accuracy", dpo[0])
            _finite("implicit_reward_margin", dpo[1])
            _need(rng == 2 * v["records"], "DPO must reserve exactly two model RNG substreams per record")
        elif v["algorithm"] == "forward_kl":
            _nonneg("post_training_loss", v["loss"])
            _need(none(dpo) and full(kl) and none(grpo), "forward-KL metrics contain a missing or foreign objective field")
            _nonneg("forward_kl", kl[0])
            _nonneg("teacher_entropy", kl[1])
            _unit("top1_agreement", kl[2])
            _need(rng == v["records"], "forward-KL must reserve exactly one model RNG substream per record")
        else:
            _need(none(dpo) and none(kl) and full(grpo), "GRPO metrics contain a missing or foreign objective field")
            _finite("mean_reward", grpo[0])
            _nonneg("reward_stddev", grpo[1])
            _nonneg("mean_kl", grpo[2])
            _unit("clipped_fraction", grpo[3])
            _need(rng > 0, "GRPO must reserve rollout RNG")


RECORD_FIELDS = ("schema_version", "sequence", "emitted_at_unix_ms", "run_id", "global_step", "phase", "checkpoint_hash",
                 "event")


def validate_record(rec: Dict[str, Any]) -> None:
    _need(isinstance(rec, dict), "metric record must be an object")
    extra = sorted(set(rec) - set(RECORD_FIELDS))
    _need(not extra, f"unknown field `{extra[0] if extra else ''}` in metric record")
    for k in RECORD_FIELDS:
        _need(k in rec or k == "checkpoint_hash", f"metric record is missing `{k}`")
    _need(rec["schema_version"] == SCHEMA_VERSION,
          f"unsupported metric schema version {rec['schema_version']}; expected {SCHEMA_VERSION}")
    for k in ("sequence", "emitted_at_unix_ms", "global_step"):
        _need(_is_uint(rec[k], 64), f"`{k}` must be an unsigned integer")
    _identifier("run_id", rec["run_id"])
    ph = rec["phase"]
    _need(isinstance(ph, dict) and set(ph) == {"index", "name", "kind"}, "metric phase must be {index, name, kind}")
    _need(_is_uint(ph["index"], 32), "phase index must be an unsigned 32-bit integer")
    _identifier("phase name", ph["name"])
    _need(ph["kind"] in PHASE_KINDS, f"unknown metric phase kind `{ph['kind']}`")
    if rec.get("checkpoint_hash") is not None:
        _sha(rec["checkpoint_hash"], "checkpoint hash")
    else:
        _need("checkpoint_hash" not in rec, "checkpoint_hash must be absent rather than null")
    ev = rec["event"]
    _need(isinstance(ev, dict) and set(ev) == {"type", "values"}, "metric event must be {type, values}")
    validate_event(ev["type"], ev["values"])
    if ev["type"] == "device_utilization":
        _need(ev["values"]["sampled_at_unix_ms"] <= rec["emitted_at_unix_ms"],
              "device sample timestamp is later than its metric record")


class LogState:
    """Position rules of a journal (`MetricLogState`): gap-free sequences, one run, no rewinds."""

    def __init__(self):
        self.records = 0
        self.next_sequence = 0
        self.last_global_step: Optional[int] = None
        self.last_emitted_at_unix_ms: Optional[int] = None
        self.run_id: Optional[str] = None

    def accept(self, rec: Dict[str, Any]) -> None:
        _need(rec["sequence"] == self.next_sequence, f"expected metric sequence {self.next_sequence}, got {rec['sequence']}")
        if self.run_id is not None:
            _need(rec["run_id"] == self.run_id, f"metric run changed from `{self.run_id}` to `{rec['run_id']}`")
        if self.last_global_step is not None:
            _need(rec["global_step"] >= self.last_global_step,
                  f"metric global step rewound from {self.last_global_step} to {rec['global_step']}")
        if self.last_emitted_at_unix_ms is not None:
            _need(rec["emitted_at_unix_ms"] >= self.last_emitted_at_unix_ms,
                  f"metric timestamp rewound from {self.last_emitted_at_unix_ms} to {rec['emitted_at_unix_ms']}")
        self.records += 1
        self.next_sequence += 1
        self.last_global_step = rec["global_step"]
        self.last_emitted_at_unix_ms = rec["emitted_at_unix_ms"]
        self.run_id = rec["run_id"]


def run_id_from_signature(signature: str) -> str:
    """16 lowercase hex digits of FNV-1a64 over the signature text (`summa-train/src/main.rs:1169-1171`)."""
    h = 0xCBF29CE484222325
    for b in signature.encode():
        h ^= b
        h = (h * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
    return f"{h:016x}"


def _clean(values: Dict[str, Any]) -> Dict[str, Any]:
    """Optional fields that are None are omitted (serde `skip_serializing_if`)."""
    return {k: v for k, v in values.items() if v is not None}


class MetricWriter:
    def __init__(self, path: str, run_id: str, state: Optional[LogState] = None):
        _identifier("run_id", run_id)
        self.path = path
        self.run_id = run_id
        self.state = state or LogState()
        self._f = open(path, "a", encoding="utf-8")
        self.phase = {"index": 0, "name": "startup", "kind": "pretrain"}
        self.global_step = self.state.last_global_step or 0

    @property
    def sequence(self) -> int:
        return self.state.next_sequence

    @staticmethod
    def create(path: str, run_id: str) -> "MetricWriter":
        if os.path.exists(path) and os.path.getsize(path) > 0:
            raise MetricsError(f"{path} already exists; resume or choose a fresh output directory")
        parent = os.path.dirname(path)
        if parent:
            os.makedirs(parent, exist_ok=True)
        return MetricWriter(path, run_id)

    @staticmethod
    def resume_from_checkpoint(path: str, run_id: str, committed_records: int,
                               committed_global_step: Optional[int] = None) -> "MetricWriter":
        """Validate the committed prefix record by record and drop everything after it."""
        kept, state = [], LogState()
        if os.path.exists(path):
            with open(path, "r", encoding="utf-8") as f:
                for i, line in enumerate(f):
                    if i >= committed_records:
                        break
                    _need(len(line.encode()) <= MAX_METRIC_RECORD_BYTES, f"{path}: record {i} exceeds the record size limit")
                    try:
                        rec = json.loads(line)
                    except json.JSONDecodeError:
                        raise MetricsError(f"{path}: record {i} inside the committed prefix is corrupt")
                    validate_record(rec)
                    _need(rec["run_id"] == run_id, f"{path}: record {i} does not belong to this run's committed prefix")
                    state.accept(rec)
                    kept.append(line if line.endswith("\n") else line + "\n")
        if len(kept) != committed_records:
            raise MetricsError(f"{path}: checkpoint committed {committed_records} records, journal has {len(kept)}")
        if committed_records > 0 and committed_global_step is not None:
            _need(state.last_global_step == committed_global_step,
                  f"{path}: the committed prefix ends at step {state.last_global_step}, the checkpoint at {committed_global_step}")
        tmp = path + ".tmp"
        with open(tmp, "w", encoding="utf-8") as f:
            f.writelines(kept)
            f.flush()
            os.fsync(f.fileno())
        os.replace(tmp, path)
        return MetricWriter(path, run_id, state)

    def set_context(self, global_step: int, phase_index: int, phase_name: str, phase_kind: str) -> None:
        self.global_step = max(global_step, self.state.last_global_step or 0)
        self.phase = {"index": phase_index, "name": phase_name, "kind": phase_kind}

    def emit(self, event_type: str, values: Dict[str, Any], checkpoint_hash: Optional[str] = None) -> None:
        now = int(time.time() * 1000)
        if self.state.last_emitted_at_unix_ms is not None:
            now = max(now, self.state.last_emitted_at_unix_ms)
        rec = {"schema_version": SCHEMA_VERSION, "sequence": self.state.next_sequence, "emitted_at_unix_ms": now,
               "run_id": self.run_id, "global_step": self.global_step, "phase": dict(self.phase)}
        if checkpoint_hash is not None:
            rec["checkpoint_hash"] = checkpoint_hash
        rec["event"] = {"type": event_type, "values": _clean(values)}
        validate_record(rec)
        self.state.accept(rec)
        self._f.write(json.dumps(rec, separators=(",", ":")) + "\n")

    def phase_timing(self, boundary: str, elapsed: float, input_wait: float = 0.0, forward: float = 0.0,
                     backward: float = 0.0, optimizer: float = 0.0, checkpoint: float = 0.0,
                     checkpoint_hash: Optional[str] = None) -> None:
        """Phase boundary / progress record; the components are clamped into the elapsed time."""
        elapsed = max(float(elapsed), 0.0)
        parts = [max(float(x), 0.0) for x in (input_wait, forward, backward, optimizer, checkpoint)]
        total = sum(parts)
        if total > elapsed and total > 0.0:
            parts = [x * elapsed / total for x in parts]
        self.emit("phase_timing", {"boundary": boundary, "elapsed_seconds": elapsed, "input_wait_seconds": parts[0],
                                   "forward_seconds": parts[1], "backward_seconds": parts[2],
                                   "optimizer_seconds": parts[3], "checkpoint_seconds": parts[4]},
                  checkpoint_hash=checkpoint_hash)

    def flush(self) -> None:
        self._f.flush()
        os.fsync(self._f.fileno())

    def close(self) -> None:
        self.flush()
        self._f.close()


def tier_name(index: int, count: int) -> str:
    """The schema names three memory tiers; a schedule's tiers map onto them fastest first: index 0 is
    `fast`, the last tier `slow`, everything between `medium`."""
    if index <= 0:
        return "fast"
    return "slow" if index >= count - 1 else "medium"


def read_metrics(path: str, run_id: Optional[str] = None) -> Iterator[Dict[str, Any]]:
    """Validated records of a journal, in order (shape, event rules and position rules)."""
    state = LogState()
    with open(path, "r", encoding="utf-8") as f:
        for line in f:
            if not line.strip():
                continue
            _need(len(line.encode()) <= MAX_METRIC_RECORD_BYTES, "metric record exceeds the record size limit")
            rec = json.loads(line)
            validate_record(rec)
            if run_id is not None:
                _need(rec["run_id"] == run_id, f"metric record belongs to run `{rec['run_id']}`, expected `{run_id}`")
            state.accept(rec)
            yield rec
