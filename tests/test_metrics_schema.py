"""metrics.jsonl schema v2: one well-formed record per event type round-trips through the writer and the
reader, and the reference's shape and consistency rules (`summa-train/src/metrics.rs:1598-2112`) reject
malformed ones."""
import json
import os

import pytest

H = "sha256:" + "ab" * 32

GOOD = {
    "phase_timing": {"boundary": "progress", "elapsed_seconds": 10.0, "input_wait_seconds": 1.0, "forward_seconds": 3.0,
                     "backward_seconds": 4.0, "optimizer_seconds": 1.0, "checkpoint_seconds": 0.5},
    "tier_update": {"transaction_id": "txn-1", "tier": "fast", "receiver_tier": "medium", "tier_clock": 200,
                    "update_period": 100, "accumulated_micro_steps": 800, "outcome": "committed", "update_l2_norm": 0.5,
                    "reserve_slot": 1, "reserve_generation": 3, "optimizer_state_reset": True},
    "active_capacity": {"tier": "slow", "active_base_experts": 8, "active_reserve_experts": 1,
                        "dormant_reserve_experts": 7, "routed_top_k": 2, "reserve_routed_top_k": 1,
                        "routed_active_parameters": 1000, "stored_parameters": 5000, "dream_generation": True,
                        "random_extra_expert": True},
    "wake_capacity_envelope": {"initial_wake_routed_active_parameters": 10, "completed_sleep_cycles_observed": 2,
                               "minimum_observed_wake_routed_active_parameters": 10,
                               "maximum_observed_wake_routed_active_parameters": 10, "stored_parameters": 50},
    "distillation_divergence": {"transaction_id": "txn-1", "teacher_hash": H, "student_hash": H, "chunk_index": 0,
                                "chunk_count": 4, "selected_tokens": 100, "total_tokens": 512, "forward_kl": 0.1,
                                "teacher_entropy": 2.0, "student_entropy": 2.1},
    "imitation_reward": {"transaction_id": "txn-1", "semantic_judge_hash": H, "samples": 8, "semantic_score_mean": 0.7,
                         "normalized_levenshtein_mean": 0.2, "levenshtein_threshold": 0.5, "reward_mean": 0.6,
                         "reward_stddev": 0.1, "grpo_kl": 0.01},
    "dream_selection": {"transaction_id": "txn-1", "selector_version": "gradient-cosine-v1", "reference_set_hash": H,
                        "candidates_generated": 64, "selected_by_alignment": 8, "selected_random": 2, "random_quota": 2,
                        "gradient_cosine_mean": 0.1, "gradient_cosine_max": 0.6, "selected_manifest_hash": H},
    "dream_trial": {"transaction_id": "txn-1", "candidate_hash": H, "adapter_hash": H, "evaluator_hash": H,
                    "lora_rank": 64, "lora_alpha": 128.0, "independent_task_delta": 0.01, "reward": 0.2,
                    "elapsed_seconds": 3.0, "accepted": True, "isolated": True, "shared_checkpoint_unchanged": True},
    "retention_delta": {"transaction_id": "txn-1", "suite": "retention", "metric": "ppl", "evaluator_hash": H,
                        "direction": "lower_is_better", "baseline_score": 10.0, "candidate_score": 10.5,
                        "improvement": -0.5, "maximum_allowed_regression": 1.0, "passed": True},
    "quantization": {"stage": "export", "format": "ternary_g128", "group_size": 128, "progress_fraction": 1.0,
                     "tensors_quantized": 10, "weights_quantized": 1000, "average_bits_per_weight": 2.125,
                     "packed_bytes": 300, "mean_squared_error": 1e-4, "max_absolute_error": 0.1,
                     "embeddings_quantized": True, "lm_head_quantized": False},
    "device_utilization": {"sampled_at_unix_ms": 1, "device_index": 0, "sample_window_seconds": 1.0,
                           "gpu_utilization_percent": 97.0, "memory_used_bytes": 10, "memory_total_bytes": 100,
                           "power_watts": 900.0},
    "throughput": {"optimizer_steps": 1, "compute_tokens": 1000, "supervised_tokens": 1000, "examples": 10,
                   "elapsed_seconds": 2.0, "tokens_per_second": 500.0, "examples_per_second": 5.0,
                   "input_wait_seconds": 0.1, "host_to_device_seconds": 0.0, "gpu_busy_seconds": 1.5},
    "optimization": {"objective": "causal_lm", "loss": 3.0, "optimized_loss": 3.1, "weighted_loss": 3.1,
                     "router_aux_loss": 0.1, "learning_rate": 3e-4, "muon_learning_rate": 6e-3, "gradient_norm": 1.0,
                     "layer_gradient_norms": [0.1, 0.2], "sequence_length": 128, "batch_size": 8,
                     "gradient_accumulation": 1, "compute_tokens": 1024, "supervised_tokens": 1024, "examples": 8,
                     "truncated_tokens": 0, "retrieval_candidates": 0},
    "post_training_update": {"transaction_id": H, "algorithm": "dpo", "epoch": 0, "first_record": 0, "records": 4,
                             "optimizer_step": 1, "rng_counter_start": 0, "rng_counter_end": 8, "loss": 0.69,
                             "checkpoint_sha256": H, "optimizer_sha256": H, "preference_accuracy": 0.5,
                             "implicit_reward_margin": 0.0},
}


def test_all_fourteen_events_round_trip(tmp_path):
    from summa_b200.train.metrics import EVENT_TYPES, MetricWriter, read_metrics, run_id_from_signature
    assert set(GOOD) == set(EVENT_TYPES) and len(EVENT_TYPES) == 14
    rid = run_id_from_signature("a" * 64)
    assert len(rid) == 16 and int(rid, 16) >= 0
    path = str(tmp_path / "metrics.jsonl")
    w = MetricWriter.create(path, rid)
    w.set_context(3, 1, "phase-a", "continued_pretrain")
    for name in EVENT_TYPES:
        w.emit(name, GOOD[name], checkpoint_hash=H if name == "phase_timing" else None)
    w.close()
    recs = list(read_metrics(path, run_id=rid))
    assert [r["event"]["type"] for r in recs] == list(EVENT_TYPES)
    assert [r["sequence"] for r in recs] == list(range(14))
    for r in recs:
        assert r["schema_version"] == 2 and r["run_id"] == rid and r["event"]["values"] == GOOD[r["event"]["type"]]
        assert set(r) <= {"schema_version", "sequence", "emitted_at_unix_ms", "run_id", "global_step", "phase",
                          "checkpoint_hash", "event"}
        assert r["phase"] == {"index": 1, "name": "phase-a", "kind": "continued_pretrain"}
    assert recs[0]["checkpoint_hash"] == H and "checkpoint_hash" not in recs[1]
    # resume keeps exactly the committed prefix
    w2 = MetricWriter.resume_from_checkpoint(path, rid, 5, 3)
    assert w2.sequence == 5
    w2.emit("optimization", GOOD["optimization"])
    w2.close()
    assert len(list(read_metrics(path))) == 6


@pytest.mark.parametrize("event,patch,msg", [
    ("phase_timing", {"forward_seconds": 20.0}, "exceeds elapsed time"),
    ("tier_update", {"tier_clock": 150}, "update-period boundary"),
    ("tier_update", {"reserve_generation": None}, "present together"),
    ("tier_update", {"outcome": "skipped"}, "only a committed tier update"),
    ("active_capacity", {"reserve_routed_top_k": 2}, "exactly one"),
    ("distillation_divergence", {"chunk_index": 4}, "less than chunk_count"),
    ("dream_trial", {"isolated": False}, "must be isolated"),
    ("retention_delta", {"improvement": 0.5}, "does not match scores"),
    ("retention_delta", {"passed": False}, "passed flag"),
    ("quantization", {"mean_squared_error": None}, "requires error measurements"),
    ("quantization", {"format": "int8"}, "unknown variant"),
    ("device_utilization", {"memory_used_bytes": 1000}, "exceeds total"),
    ("throughput", {"tokens_per_second": 123.0}, "does not match"),
    ("optimization", {"loss": float("nan")}, "finite"),
    ("optimization", {"batch_size": 0}, "geometry"),
    ("optimization", {"tokens": 5}, "unknown field `tokens`"),
    ("optimization", {"examples": 1.5}, "unsigned 64-bit"),
    ("post_training_update", {"forward_kl": 0.1}, "foreign objective field"),
    ("post_training_update", {"rng_counter_end": 7}, "two model RNG"),
])
def test_event_rules_reject_malformed_values(event, patch, msg):
    from summa_b200.train.metrics import MetricsError, validate_event
    v = dict(GOOD[event])
    for k, val in patch.items():
        if val is None:
            v.pop(k, None)
        else:
            v[k] = val
    with pytest.raises(MetricsError, match=msg):
        validate_event(event, v)


def test_journal_position_rules(tmp_path):
    from summa_b200.train.metrics import MetricsError, MetricWriter, read_metrics
    path = str(tmp_path / "m.jsonl")
    w = MetricWriter.create(path, "run-1")
    w.set_context(1, 0, "p", "pretrain")
    w.emit("optimization", GOOD["optimization"])
    w.emit("throughput", GOOD["throughput"])
    w.close()
    lines = open(path).read().splitlines()
    for mutate, msg in [(lambda r: r.update(sequence=5), "expected metric sequence"),
                        (lambda r: r.update(run_id="run-2"), "run changed"),
                        (lambda r: r.update(global_step=0), "rewound"),
                        (lambda r: r.update(extra=1), "unknown field `extra`"),
                        (lambda r: r.update(run_id=7), "run_id"),
                        (lambda r: r.update(schema_version=1), "unsupported metric schema version")]:
        rec = json.loads(lines[1])
        mutate(rec)
        bad = str(tmp_path / "bad.jsonl")
        with open(bad, "w") as f:
            f.write(lines[0] + "\n" + json.dumps(rec) + "\n")
        with pytest.raises(MetricsError, match=msg):
            list(read_metrics(bad))
    with pytest.raises(MetricsError):
        MetricWriter.create(path, "run-1")           # a non-empty journal is never silently appended to
    with pytest.raises(MetricsError, match="committed 3 records"):
        MetricWriter.resume_from_checkpoint(path, "run-1", 3)
