"""The sleep-runtime configuration file: the reference's two example files decode under their modes, strictness,
pinned artifacts, and the trainer's `--sleep-runtime` / `--sleep-runtime-sha256` binding."""
import hashlib
import json
import os
import subprocess
import sys

import pytest

from summa_b200.train import sleep_runtime as R
from summa_b200.train.sleep import SleepError

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.environ.get("SUMMA_REFERENCE_TREE", os.path.join(os.sep, "root", "reference", "summa-train"))


def sha(data: bytes) -> str:
    return "sha256:" + hashlib.sha256(data).hexdigest()


@pytest.mark.skipif(not os.path.exists(os.path.join(REF, "sleep-runtime.periodic.example.json")), reason="reference tree not mounted")
def test_reference_example_files_decode_under_their_modes():
    per, sta = (os.path.join(REF, f"sleep-runtime.{k}.example.json") for k in ("periodic", "standalone"))
    p = R.load_sleep_runtime(per, sha(open(per, "rb").read()), "periodic")
    assert p.version == 1 and p.rng_streams == 4 and p.max_wake_context_records == 64 and p.rollouts.imitation_groups == 4
    assert p.tier_optimizer.weight_decay == 0.1 and p.dreaming.gradient_dimensions == 256 and p.dreaming.generation_policy_alpha == 128
    assert p.pins["model_mal"].path == os.path.normpath(os.path.join(REF, "../summa-mal/well-known/retriever_300m_moe_sleep.mal"))
    assert p.directories["candidate_directory"] == os.path.join(REF, "candidates") and "wake_context_journal" not in p.pins
    s = R.load_sleep_runtime(sta, sha(open(sta, "rb").read()), "standalone")
    assert s.pins["wake_context_journal"] == s.dreaming.wake_context_journal and "initial_model_parameter_ids" in s.pins
    with pytest.raises(SleepError, match="must not contain standalone wake artifacts"):
        R.load_sleep_runtime(sta, sha(open(sta, "rb").read()), "periodic")
    with pytest.raises(SleepError, match="requires wake_context_journal"):
        R.load_sleep_runtime(per, sha(open(per, "rb").read()), "standalone")
    with pytest.raises(SleepError, match="not the pinned file"):
        R.load_sleep_runtime(per, "sha256:" + "1" * 64, "periodic")


def minimal(**over):
    z = "sha256:" + "0" * 64
    cfg = {"version": 1, "workflow_signature": z, "model_mal": {"path": "m.mal", "sha256": z},
           "semantic_judge": {"path": "j.json", "sha256": z}, "retention_evaluator": {"path": "e.json", "sha256": z},
           "retention_suite": {"path": "s.json", "sha256": z}, "rollouts": {"max_context_tokens": 16, "continuation_tokens": 4},
           "tier_optimizer": {"learning_rate": 1e-2, "beta_1": 0.9, "beta_2": 0.95, "epsilon": 1e-8, "weight_decay": 0.0},
           "tensor_transaction_directory": "st/tx", "prospective_directory": "st/pro", "tier_optimizer_directory": "st/opt",
           "candidate_directory": "cand", "rejection_report_directory": "st/rej"}
    cfg.update(over)
    return cfg


def test_strict_decoding_limits_and_pins(tmp_path):
    base = str(tmp_path)
    c = R.SleepRuntimeConfig.decode(minimal(), base)
    assert c.rollouts.temperature == 0.8 and c.rollouts.top_k == 32 and c.rng_streams == 1 and c.dreaming is None
    c.validate_periodic()
    for bad, pat in [
        (minimal(extra=1), "unknown field `extra`"),
        (minimal(version=2), "unsupported built-in sleep runtime version 2"),
        (minimal(candidate_directory="st/tx"), "must be distinct"),
        (minimal(rng_streams=0), "RNG streams"),
        (minimal(max_wake_context_records=4096, rollouts={"max_context_tokens": 65536, "continuation_tokens": 4}), "token limit"),
        (minimal(rollouts={"max_context_tokens": 16, "continuation_tokens": 4, "temperature": 0}), "temperature"),
        (minimal(rollouts={"max_context_tokens": 16, "continuation_tokens": 4, "top_p": 0.9}), "unknown field `top_p`"),
        (minimal(tier_optimizer={"learning_rate": 1e-2, "beta_1": 1.0, "beta_2": 0.95, "epsilon": 1e-8, "weight_decay": 0.0}), "beta_1"),
        (minimal(model_mal={"path": "m.mal", "sha256": "sha256:xyz"}), "hash"),
        (minimal(workflow_signature="abc"), "workflow signature"),
        (minimal(dreaming={"artifact_directory": "cand", "reference_set": {"path": "r", "sha256": "sha256:" + "0" * 64},
                           "independent_evaluation_set": {"path": "i", "sha256": "sha256:" + "0" * 64}}), "must be distinct"),
    ]:
        with pytest.raises(SleepError, match=pat):
            R.SleepRuntimeConfig.decode(bad, base)
    art = tmp_path / "j.json"
    art.write_text('{"judge": 1}')
    pin = R.PinnedArtifact(str(art), sha(art.read_bytes()))
    assert pin.verify_json() == {"judge": 1}
    art.write_text('{"judge": 2}')
    with pytest.raises(SleepError, match="changed: expected"):
        pin.verify_bytes()
    with pytest.raises(SleepError, match="changed"):                       # an all-zero pin is a placeholder and never verifies
        R.PinnedArtifact(str(art), "sha256:" + "0" * 64).verify_bytes()


MEMORY_MAL = """attention a { num_heads: 2 } ffn f { hidden_dim: 64 }
  memory mm {
    tier fast { ffn: f reserve_experts { capacity: 2 rank: 4 top_k: 1 } }
    tier slow { ffn: f residual_init: zero reserve_experts { capacity: 2 rank: 4 top_k: 1 } }
  }
  block b { attention: a memory: mm norm: rmsnorm { eps: 1e-5 } }
  model t { max_seq_len: 64 hidden_size: 32 num_layers: 2 block: b }"""
ZERO = "sha256:" + "0" * 64


def _cli(*argv):
    return subprocess.run([sys.executable, "-m", "summa_b200.cli.train", *argv], capture_output=True, text=True, cwd=ROOT, timeout=600)


def test_trainer_binds_the_runtime_file_to_the_run(tmp_path):
    from summa_b200.tokenizer import Tokenizer
    (tmp_path / "tokenizer.json").write_text(Tokenizer.byte_level().to_json())
    (tmp_path / "train.jsonl").write_text("\n".join(json.dumps({"text": ("the quick brown fox %d jumps over the lazy dog. " % i) * 4}) for i in range(120)))
    (tmp_path / "mem.mal").write_text(MEMORY_MAL)
    sched = {"clock": "optimizer_steps", "terminal_consolidation": "distill_into_base_v1",
             "tiers": [{"id": "fast", "update_period": 2, "reserve_slots": 2}, {"id": "slow", "update_period": 4, "reserve_slots": 2}]}
    phase = {"name": "p0", "type": "pretrain", "task": {"type": "causal_lm"}, "data": "train.jsonl", "sequence_length": 32, "batch_size": 4,
             "gradient_accumulation": 1, "steps": 4, "shuffle_buffer": 16,
             "periodic_sleep": {"schedule": sched, "receiver_learning_rate": 2e-2, "receiver_weight_decay": 0.0,
                                "knowledge_seeding": {"chunk_tokens": 512, "teacher_rollouts": 4, "detached_student_rollouts": 1, "temperature": 1.0, "forward_kl_weight": 1.0},
                                "imitation": {"semantic_judge_hash": ZERO, "semantic_weight": 0.5, "maximum_edit_distance": 32, "grpo_group_size": 2},
                                "retention_suite": "retention.json", "retention_suite_sha256": ZERO,
                                "retention": {"evaluator_hash": ZERO, "suite_hash": ZERO, "max_anchor_forward_kl": 0.0, "max_anchor_regression": 1.0,
                                              "min_incorporation_gain": 0.0},
                                "grpo_clip_epsilon": 0.2, "grpo_advantage_epsilon": 1e-6, "grpo_kl_coefficient": 0.04, "candidate_directory": "candidates"}}
    (tmp_path / "wf.json").write_text(json.dumps({"version": 2, "phases": [phase]}))
    out = str(tmp_path / "run")
    common = ["train", "--model", str(tmp_path / "mem.mal"), "--tokenizer", str(tmp_path / "tokenizer.json"), "--workflow", str(tmp_path / "wf.json"),
              "--output", out, "--warmup", "1", "--lr", "3e-3", "--checkpoint-every", "2", "--device", "cpu", "--optimizer", "adamw"]
    sig = _cli(*common, "--print-run-signature")
    assert sig.returncode == 0, sig.stderr[-2000:]
    signature = sig.stdout.strip()
    runtime = minimal(workflow_signature="sha256:" + signature, model_mal={"path": "mem.mal", "sha256": sha((tmp_path / "mem.mal").read_bytes())},
                      max_wake_context_records=3, rng_streams=2)
    rt = tmp_path / "sleep-runtime.json"
    rt.write_text(json.dumps(runtime))
    ident = sha(rt.read_bytes())
    r = _cli(*common, "--sleep-runtime", str(rt))
    assert r.returncode != 0 and "go together" in r.stderr
    r = _cli(*common, "--sleep-runtime", str(rt), "--sleep-runtime-sha256", "sha256:" + "2" * 64)
    assert r.returncode != 0 and "not the pinned file" in r.stderr and not os.path.exists(out)
    other = tmp_path / "other.json"
    other.write_text(json.dumps(dict(runtime, workflow_signature="sha256:" + "3" * 64)))
    r = _cli(*common, "--sleep-runtime", str(other), "--sleep-runtime-sha256", sha(other.read_bytes()))
    assert r.returncode != 0 and "bound to workflow signature" in r.stderr
    r = _cli(*common, "--sleep-runtime", str(rt), "--sleep-runtime-sha256", ident)
    assert r.returncode == 0, r.stderr[-3000:]
    state = json.load(open(os.path.join(out, "sleep", "state.json")))
    assert len(state["rng_counters"]) == 2 and state["clock"] == 4
    # the retention gate of this workflow is impossible (a zero anchor KL bound): every transfer is rejected and reported
    reports = sorted(os.listdir(tmp_path / "st" / "rej"))
    assert reports and reports[0] == "rejection-000000000001.json"
    rep = json.load(open(tmp_path / "st" / "rej" / reports[0]))
    assert rep["version"] == 1 and rep["sender"] == 0 and rep["receiver"] == 1 and "anchor KL" in rep["reason"]
