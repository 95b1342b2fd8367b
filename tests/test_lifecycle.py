"""Binary-level lifecycle on CPU: train, preempt, resume, verify, eval, generate; workflow
validation; the phase runtime with a fake worker process."""
import hashlib
import json
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _fixture(tmp_path, steps=6):
    from summa_b200.tokenizer import Tokenizer
    tok = tmp_path / "tokenizer.json"
    tok.write_text(Tokenizer.byte_level().to_json())
    data = tmp_path / "train.jsonl"
    rows = [{"text": ("the quick brown fox %d jumps over the lazy dog. " % i) * 4} for i in range(200)]
    data.write_text("\n".join(json.dumps(r) for r in rows))
    wf = tmp_path / "workflow.json"
    wf.write_text(json.dumps({"version": 2, "phases": [
        {"name": "p0", "type": "pretrain", "task": {"type": "causal_lm"}, "data": "train.jsonl",
         "sequence_length": 32, "batch_size": 4, "gradient_accumulation": 2, "steps": steps, "shuffle_buffer": 16}]}))
    mal = tmp_path / "m.mal"
    mal.write_text("""attention a { num_heads: 2 } ffn f { hidden_dim: 64 }
      block b { attention: a ffn: f norm: rmsnorm { eps: 1e-5 } }
      model t { max_seq_len: 64 hidden_size: 32 num_layers: 2 block: b }""")
    return str(tok), str(data), str(wf), str(mal)


def _cli(*argv):
    return subprocess.run([sys.executable, "-m", "summa_b200.cli.train", *argv], capture_output=True, text=True,
                          cwd=ROOT, timeout=600)


def test_train_preempt_resume_eval_generate(tmp_path):
    tok, data, wf, mal = _fixture(tmp_path)
    out = str(tmp_path / "run")
    common = ["train", "--model", mal, "--tokenizer", tok, "--workflow", wf, "--output", out, "--warmup", "2",
              "--lr", "3e-3", "--checkpoint-every", "2", "--device", "cpu", "--optimizer", "adamw"]
    sig = _cli(*common, "--print-run-signature")
    assert sig.returncode == 0 and len(sig.stdout.strip()) == 64 and not os.path.exists(out)
    # "preempted" run: stops after 4 of 6 steps (checkpoint at step 4)
    r1 = _cli(*common, "--max-steps", "4")
    assert r1.returncode == 0, r1.stderr[-2000:]
    v = _cli("verify-checkpoint", out)
    assert v.returncode == 0 and json.loads(v.stdout)["global_step"] == 4
    n_before = sum(1 for _ in open(os.path.join(out, "metrics.jsonl")))
    # garbage after the committed prefix must be dropped on resume
    with open(os.path.join(out, "metrics.jsonl"), "a") as f:
        f.write('{"schema_version":2,"sequence":9999,"garbage":true}\n')
    # the strict verifier: root or materialised generation, committed metric prefix, automation-friendly TSV
    mpath = os.path.join(out, "metrics.jsonl")
    ok = _cli("verify-checkpoint", "--root", out, "--metrics", mpath)
    ver = json.loads(ok.stdout)
    assert ok.returncode == 0 and ver["global_step"] == 4 and 0 < ver["metric_records"] <= n_before and ver["workflow_signature"] == "sha256:" + sig.stdout.strip()
    exact = _cli("verify-checkpoint", "--root", out, "--metrics", mpath, "--exact-metrics")
    assert exact.returncode != 0 and "continues after" in exact.stderr
    tsv = _cli("verify-checkpoint", "--generation", os.path.join(out, "generations", ver["generation"]), "--generation-name", ver["generation"],
               "--manifest-sha256", ver["manifest_sha256"], "--format", "tsv")
    assert tsv.returncode == 0 and tsv.stdout.strip().split("\t") == ["4", ver["generation"], ver["manifest_sha256"], str(ver["metric_records"])]
    assert _cli("verify-checkpoint", "--generation", os.path.join(out, "generations", ver["generation"])).returncode != 0
    assert _cli("verify-checkpoint", "--generation", os.path.join(out, "generations", ver["generation"]), "--generation-name", ver["generation"],
                "--manifest-sha256", "0" * 64).returncode != 0
    r2 = _cli(*common, "--resume")
    assert r2.returncode == 0, r2.stderr[-2000:]
    res = json.loads(r2.stdout.strip().splitlines()[-1])
    assert res["global_step"] == 6
    from summa_b200.train.metrics import read_metrics
    recs = list(read_metrics(os.path.join(out, "metrics.jsonl")))
    assert [r["sequence"] for r in recs] == list(range(len(recs))) and len(recs) > n_before - 1
    losses = [r["event"]["values"]["loss"] for r in recs if r["event"]["type"] == "optimization"]
    assert len(losses) == 6 and losses[-1] < losses[0]
    # a different recipe must not resume from this directory
    r3 = _cli(*[c if c != "3e-3" else "1e-3" for c in common], "--resume")
    assert r3.returncode != 0 and "signature" in r3.stderr
    gen = json.load(open(os.path.join(out, "current.json")))["generation"]
    ckpt = os.path.join(out, "generations", gen, "weights.safetensors")
    e = _cli("eval", "--model", mal, "--tokenizer", tok, "--checkpoint", ckpt, "--data", data,
             "--sequence-length", "32", "--batch-size", "4", "--device", "cpu")
    assert e.returncode == 0, e.stderr[-2000:]
    rep = json.loads(e.stdout)
    assert rep["version"] == 3 and rep["objective"] == "causal_lm" and rep["supervised_tokens"] > 0
    assert rep["causal_lm"]["loss"] < 5.6 and rep["checkpoint_sha256"] and rep["data"][0]["identity"].startswith("sha256:")
    g = subprocess.run([sys.executable, "-m", "summa_b200.cli.llm", "generate", "--model", mal, "--tokenizer", tok,
                        "--weights", ckpt, "--prompt", "the quick", "--max-new-tokens", "8", "--device", "cpu"],
                       capture_output=True, text=True, cwd=ROOT, timeout=300)
    assert g.returncode == 0, g.stderr[-2000:]


def test_second_trainer_is_locked_out(tmp_path):
    from summa_b200.train.trainer import OutputLock
    a = OutputLock(str(tmp_path / "o"))
    with pytest.raises(RuntimeError):
        OutputLock(str(tmp_path / "o"))
    a.release()
    OutputLock(str(tmp_path / "o")).release()


def test_workflow_validation_rules(tmp_path):
    from summa_b200.train.workflow import WorkflowError, parse_workflow, wake_plan
    base = {"name": "p", "type": "pretrain", "task": {"type": "causal_lm"}, "data": "d.jsonl",
            "sequence_length": 8, "batch_size": 2, "gradient_accumulation": 1, "steps": 1}
    ok = parse_workflow(json.dumps({"version": 2, "phases": [base]}), str(tmp_path))
    assert ok.phases[0].data == os.path.join(str(tmp_path), "d.jsonl") and len(ok.signature()) == 64
    for bad, msg in [
        ({"version": 1, "phases": [base]}, "version"),
        ({"version": 2, "phases": [dict(base, bogus=1)]}, "unknown field"),
        ({"version": 2, "phases": [dict(base, max_steps=3)]}, "both steps and max_steps"),
        ({"version": 2, "phases": [{k: v for k, v in base.items() if k != "gradient_accumulation"}]},
         "requires gradient_accumulation"),
        ({"version": 2, "phases": [dict(base, post_training={"algorithm": "dpo"})]}, "missing field `reference`"),
        ({"version": 2, "phases": [dict(base, type="sft")]}, "supervised-generation"),
        ({"version": 2, "phases": [dict(base, type="quantization")]}, "requires quantization settings"),
        ({"version": 2, "phases": [dict(base, batch_size=70000)]}, "batch_size"),
        ({"version": 2, "phases": [base, base]}, "duplicate phase"),
        ({"version": 2, "phases": [dict(base, task={"type": "causal_lm", "x": 1})]}, "unknown field"),
    ]:
        with pytest.raises(WorkflowError) as e:
            parse_workflow(json.dumps(bad))
        assert msg in str(e.value), (msg, str(e.value))
    frozen = {"adapter": "summa_checkpoint", "artifact": "ref.json", "sha256": "sha256:" + "0" * 64}
    pref = dict(base, type="preference", task={"type": "pairwise_preference"},
                post_training={"algorithm": "dpo", "reference": frozen})
    wf = parse_workflow(json.dumps({"version": 2, "phases": [pref]}), str(tmp_path))
    pt = wf.phases[0].post_training
    assert pt["beta"] == 0.1 and pt["label_smoothing"] == 0.0 and pt["sequence_reduction"] == "sum"      # serde defaults
    assert pt["reference"]["artifact"] == os.path.join(str(tmp_path), "ref.json")
    with pytest.raises(WorkflowError):
        wake_plan(wf)
    for bad_pt, msg in [({"type": "dpo"}, "missing field `algorithm`"),
                        ({"algorithm": "dpo", "reference": frozen, "gamma": 1}, "unknown field `gamma`"),
                        ({"algorithm": "dpo", "reference": dict(frozen, sha256="abc")}, "64 lowercase hex"),
                        ({"algorithm": "dpo", "reference": frozen, "beta": "0.1"}, "must be a number"),
                        ({"algorithm": "grpo", "kl_coefficient": 0.0, "sampling": {"max_new_tokens": 4}}, "requires a DPO")]:
        with pytest.raises(WorkflowError) as e:
            parse_workflow(json.dumps({"version": 2, "phases": [dict(pref, post_training=bad_pt)]}))
        assert msg in str(e.value), (msg, str(e.value))


FAKE_WORKER = r'''
import json, sys
req = json.loads(sys.stdin.readline())
i = req["phase_index"]
print(json.dumps({"type": "metric", "record": {"phase_index": i, "x": 1}}), flush=True)
if req["phase"]["type"] == "evaluation":
    print(json.dumps({"type": "complete", "product": {"type": "assessment", "report": {"ok": True}}}), flush=True)
elif req["resume_state"] is None and i == 1:
    print(json.dumps({"type": "yielded", "resume_state": {"half": True}}), flush=True)
else:
    print(json.dumps({"type": "complete", "product": {"type": "model_candidate",
          "checkpoint": {"uri": "ckpt-%d" % i, "sha256": ("%064x" % (i + 1))}}}), flush=True)
'''


def test_runtime_state_machine_with_external_worker(tmp_path):
    from summa_b200.train import runtime as R
    from summa_b200.train.workflow import parse_workflow
    worker = tmp_path / "worker.py"
    worker.write_text(FAKE_WORKER)
    base = {"task": {"type": "causal_lm"}, "data": "d.jsonl", "sequence_length": 8, "batch_size": 2}
    wf = parse_workflow(json.dumps({"version": 2, "phases": [
        dict(base, name="a", type="pretrain", steps=1, gradient_accumulation=1),
        dict(base, name="b", type="continued_pretrain", steps=1, gradient_accumulation=1),
        dict(base, name="c", type="evaluation")]}))
    ex = R.ExternalPhaseExecutor([sys.executable, str(worker)], 60.0)
    reg = R.ExecutorRegistry()
    for k in ("pretrain", "continued_pretrain", "evaluation"):
        reg.register(k, ex)
    with pytest.raises(R.RuntimeError_):
        reg.register("pretrain", ex)
    store = R.AtomicRuntimeCheckpoint(str(tmp_path / "state.json"), ex.identity())
    rt = R.WorkflowRuntime(wf, reg, store)
    assert rt.run_until_yield_or_complete() == "yielded" and rt.state.next_phase == 1
    # a fresh process picks the run up from the persisted state and finishes it
    rt2 = R.WorkflowRuntime(wf, reg, store)
    assert rt2.state.active["resume_state"] == {"half": True}
    assert rt2.run_until_yield_or_complete() == "complete"
    assert rt2.state.current_checkpoint["uri"] == "ckpt-1" and len(rt2.state.completed) == 3
    # a prepared-but-uncommitted phase commits without re-running the executor
    st = store.load()
    st.next_phase, st.completed = 2, st.completed[:2]
    st.active = {"phase_index": 2, "boundary": "prepared", "resume_state": None,
                 "prepared_product": {"type": "assessment", "report": {"ok": 1}}}
    store.store(st)
    rt3 = R.WorkflowRuntime(wf, R.ExecutorRegistry(), store)       # empty registry: executing would fail
    assert rt3.run_until_yield_or_complete() == "complete"
    # product legality
    with pytest.raises(R.RuntimeError_):
        R.validate_product(wf.phases[1], R.Checkpoint("u", "s"), {"type": "model_candidate",
                                                                 "checkpoint": {"uri": "u", "sha256": "t"}})
    with pytest.raises(R.RuntimeError_):
        R.AtomicRuntimeCheckpoint(str(tmp_path / "state.json"), "other").load()


@pytest.mark.parametrize("optimizer", ["adamw", "muon"])
def test_data_parallel_trainer_matches_single_rank_and_resumes_anywhere(tmp_path, optimizer):
    """`torch.distributed.run` with 2 gloo ranks: same losses as one rank on the same recipe (the
    global micro-batch is cut into rank slices), one journal / one checkpoint owned by rank 0,
    and the 2-rank checkpoint resumes on a single rank."""
    from summa_b200.train.metrics import read_metrics
    tok, data, wf, mal = _fixture(tmp_path)

    def common(out):
        return ["train", "--model", mal, "--tokenizer", tok, "--workflow", wf, "--output", out, "--warmup", "2",
                "--lr", "3e-3", "--checkpoint-every", "2", "--device", "cpu", "--optimizer", optimizer]

    def losses(out):
        recs = list(read_metrics(os.path.join(out, "metrics.jsonl")))
        assert [r["sequence"] for r in recs] == list(range(len(recs)))
        return [r["event"]["values"]["loss"] for r in recs if r["event"]["type"] == "optimization"]

    one = str(tmp_path / "one")
    r1 = _cli(*common(one))
    assert r1.returncode == 0, r1.stderr[-2000:]
    two = str(tmp_path / "two")
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    launch = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
              "127.0.0.1", "--master-port", "29547", "-m", "summa_b200.cli.train"]
    r2 = subprocess.run(launch + common(two) + ["--max-steps", "4"], capture_output=True, text=True, cwd=ROOT, env=env,
                        timeout=600)
    assert r2.returncode == 0, r2.stderr[-3000:]
    l1, l2 = losses(one), losses(two)
    assert len(l1) == 6 and len(l2) == 4
    assert all(abs(a - b) < 2e-3 * max(1.0, abs(a)) for a, b in zip(l1, l2)), (l1, l2)
    v = _cli("verify-checkpoint", two)
    assert v.returncode == 0 and json.loads(v.stdout)["global_step"] == 4
    # finish the 2-rank run on one rank: the optimizer state is stored whole
    r3 = _cli(*common(two), "--resume")
    assert r3.returncode == 0, r3.stderr[-2000:]
    l3 = losses(two)
    assert len(l3) == 6
    assert all(abs(a - b) < 5e-3 * max(1.0, abs(a)) for a, b in zip(l1, l3)), (l1, l3)


MEMORY_MAL = """attention a { num_heads: 2 } ffn f { hidden_dim: 64 }
  memory mm {
    tier fast { ffn: f reserve_experts { capacity: 2 rank: 4 top_k: 1 } }
    tier slow { ffn: f residual_init: zero reserve_experts { capacity: 2 rank: 4 top_k: 1 } }
  }
  block b { attention: a memory: mm norm: rmsnorm { eps: 1e-5 } }
  model t { max_seq_len: 64 hidden_size: 32 num_layers: 2 block: b }"""
ZERO_HASH = "sha256:" + "0" * 64
SCHEDULE = {"clock": "optimizer_steps", "terminal_consolidation": "distill_into_base_v1",
            "tiers": [{"id": "fast", "update_period": 2, "reserve_slots": 2},
                      {"id": "slow", "update_period": 4, "reserve_slots": 2}]}


@pytest.mark.parametrize("mode", ["wake_only", "periodic_sleep"])
def test_memory_model_update_policies_in_the_trainer(tmp_path, mode):
    """A two-tier memory model under both update policies: tier parameters move only at their
    boundaries; with periodic sleep the fast tier's update is consolidated into a slot of the slow
    tier by a persisted transaction; the tier banks survive a preempt / resume."""
    from summa_b200.train.metrics import read_metrics
    tok, data, _, _ = _fixture(tmp_path)
    mal = tmp_path / "mem.mal"
    mal.write_text(MEMORY_MAL)
    phase = {"name": "p0", "type": "pretrain", "task": {"type": "causal_lm"}, "data": "train.jsonl",
             "sequence_length": 32, "batch_size": 4, "gradient_accumulation": 1, "steps": 6, "shuffle_buffer": 16}
    if mode == "wake_only":
        phase["memory_update_mode"] = {"type": "wake_only", "schedule": SCHEDULE,
                                       "tier_optimizer": {"learning_rate": 1e-2, "beta_1": 0.9, "beta_2": 0.95,
                                                          "epsilon": 1e-8, "weight_decay": 0.0}}
    else:
        phase["periodic_sleep"] = {
            "schedule": SCHEDULE, "receiver_learning_rate": 2e-2, "receiver_weight_decay": 0.0,
            "knowledge_seeding": {"chunk_tokens": 512, "teacher_rollouts": 8, "detached_student_rollouts": 1,
                                  "temperature": 1.0, "forward_kl_weight": 1.0},
            "imitation": {"semantic_judge_hash": ZERO_HASH, "semantic_weight": 0.5, "maximum_edit_distance": 32,
                          "grpo_group_size": 2},
            "retention_suite": "retention.json", "retention_suite_sha256": ZERO_HASH,
            "retention": {"evaluator_hash": ZERO_HASH, "suite_hash": ZERO_HASH, "max_anchor_forward_kl": 10.0,
                          "max_anchor_regression": 1.0, "min_incorporation_gain": 0.0},
            "grpo_clip_epsilon": 0.2, "grpo_advantage_epsilon": 1e-6, "grpo_kl_coefficient": 0.04,
            "candidate_directory": "candidates"}
    wf = tmp_path / "wf.json"
    wf.write_text(json.dumps({"version": 2, "phases": [phase]}))
    out = str(tmp_path / "run")
    common = ["train", "--model", str(mal), "--tokenizer", tok, "--workflow", str(wf), "--output", out, "--warmup", "1",
              "--lr", "3e-3", "--checkpoint-every", "3", "--device", "cpu", "--optimizer", "adamw"]
    r1 = _cli(*common, "--max-steps", "3")
    assert r1.returncode == 0, r1.stderr[-3000:]
    r2 = _cli(*common, "--resume")
    assert r2.returncode == 0, r2.stderr[-3000:]
    recs = list(read_metrics(os.path.join(out, "metrics.jsonl")))
    ups = [x["event"]["values"] for x in recs if x["event"]["type"] == "tier_update"]
    assert all(u["update_period"] == (2 if u["tier"] == "fast" else 4) for u in ups)
    assert [(u["tier_clock"], u["tier"]) for u in ups if u["tier"] == "fast"] == [(2, "fast"), (4, "fast"), (6, "fast")]
    slow = [u for u in ups if u["tier"] == "slow"]
    assert all(u["tier_clock"] == 4 for u in slow)
    if mode == "wake_only":
        assert len(slow) == 1 and all(u["outcome"] == "committed" and "receiver_tier" not in u for u in ups)
    else:
        fast = [u for u in ups if u["tier"] == "fast"]
        # one transaction of the durable state machine per boundary; the terminal tier's own update and the
        # distillation of its reserves are ONE transaction, and while a rejected terminal boundary waits for its
        # retry the faster tiers' transfers are held back
        assert len(slow) == 1 and slow[0]["outcome"] in ("committed", "rolled_back") and "receiver_tier" not in slow[0]
        assert all(u["receiver_tier"] == "slow" for u in fast)
        assert [u["outcome"] in ("committed", "rolled_back") for u in fast[:2]] == [True, True]
        assert fast[2]["outcome"] == ("skipped" if slow[0]["outcome"] == "rolled_back" else fast[2]["outcome"])
        for u in fast:
            assert (u["outcome"] == "committed") == ("reserve_slot" in u), u
        ids = [u["transaction_id"] for u in ups if u["outcome"] != "skipped"]
        assert ids == [f"sleep-{i + 1}" for i in range(len(ids))]            # attempt ids are consumed in order, never reused
        saved = json.load(open(os.path.join(out, "sleep", "state.json")))
        assert saved["clock"] == 6 and saved["phase"] == "wake" and saved["pending"] is None and saved["cycle"] == len(ids)
        assert saved["completed_count"] == sum(u["outcome"] == "committed" for u in ups)
    losses = [x["event"]["values"]["loss"] for x in recs if x["event"]["type"] == "optimization"]
    assert len(losses) == 6 and all(l == l for l in losses)
    # the optimizer container carries the tier banks
    from summa_b200.train import checkpoint as C
    gen = json.load(open(os.path.join(out, "current.json")))["generation"]
    t, _, _ = C.unpack_tensors(open(os.path.join(out, "generations", gen, "adamw-state.bpk"), "rb").read())
    assert "extra.tier0.clock" in t and any(k.startswith("extra.tier1.w.") for k in t)
    ts = json.load(open(os.path.join(out, "generations", gen, "training-state.json")))
    scopes = {r["scope"]: r for r in ts["optimizer_states"]}                       # one optimizer scope per tier, each with its own clock
    assert set(scopes) == {"wake", "tier0", "tier1"} and scopes["wake"]["update_clock"] == 6 and scopes["tier0"]["gradient_accumulator"]
    assert ts["memory_update"]["type"] == mode and ts["workflow_signature"].startswith("sha256:") and len(ts["parameter_ids"]) > 0
    if mode == "wake_only":
        sc = ts["memory_update"]["optimizer_scopes"]
        owned = [i for t in sc["tiers"] for i in t["parameter_ids"]]
        assert len(set(owned)) == len(owned) and not set(owned) & set(sc["wake_parameter_ids"])
        assert sorted(owned + sc["wake_parameter_ids"]) == sorted(ts["parameter_ids"])
        # every tier's optimizer and pending gradients are sealed as an immutable bundle that the scopes name
        for t in sc["tiers"]:
            body = open(os.path.join(out, "tier-optimizers", t["artifact"]["path"]), "rb").read()
            assert "sha256:" + hashlib.sha256(body).hexdigest() == t["artifact"]["sha256"] and scopes[f"tier{t['tier']}"]["gradient_accumulator"] == t["artifact"]["path"]
    if mode == "periodic_sleep":      # the sealed generation carries the sleep state machine; the resumed half continued from it
        assert ts["sleep"]["clock"] == 6 and ts["sleep"]["completed_chain_hash"] == saved["completed_chain_hash"]


def test_signatures_are_read_only_and_cover_what_changes_the_run(tmp_path):
    """Behaviour of `summa-train/tests/trainer_lifecycle.rs:264-456`: printing a signature creates nothing; the output
    location is not part of it, the learning rate, explicit telemetry settings and the BYTES of the initial checkpoint
    are; `validate-workflow --signature-only` prints the workflow's identity alone; periodic sleep on an ordinary model
    and reserve capacities that drift from the model are refused before any state exists."""
    tok, data, wf, mal = _fixture(tmp_path)
    base = ["train", "--model", mal, "--tokenizer", tok, "--workflow", wf, "--device", "cpu", "--optimizer", "adamw"]

    def sig(out, *extra):
        r = _cli(*base, "--output", str(tmp_path / out), "--print-run-signature", *extra)
        assert r.returncode == 0 and not os.path.exists(tmp_path / out), r.stderr[-1500:]
        return r.stdout.strip()
    first = sig("a")
    assert sig("b") == first and sig("c", "--lr", "0.0004") != first
    assert sig("d", "--gpu-metrics-interval-ms", "2500", "--gpu-physical-device", "GPU-1234-abcd") != first
    fast = _cli(*base, "--output", str(tmp_path / "g"), "--print-run-signature", "--gpu-metrics-interval-ms", "50")
    assert fast.returncode != 0 and "at least 100" in fast.stderr
    init = tmp_path / "initial.safetensors"
    init.write_bytes(b"first checkpoint identity")
    with_ckpt = sig("e", "--checkpoint", str(init))
    init.write_bytes(b"second checkpoint identity")
    assert with_ckpt != first and sig("f", "--checkpoint", str(init)) != with_ckpt

    before = sorted(os.listdir(tmp_path))
    v = _cli("validate-workflow", "--workflow", wf, "--signature-only")
    from summa_b200.train.workflow import load_workflow
    assert v.returncode == 0 and v.stdout.strip() == "sha256:" + load_workflow(wf).signature() and sorted(os.listdir(tmp_path)) == before
    h = _cli("validate-workflow", "--help")
    assert "--signature-only" in h.stdout and "--config" in h.stdout
    h = _cli("train", "--help")
    assert all(flag in h.stdout for flag in ("--print-run-signature", "--gpu-metrics-interval-ms", "--gpu-physical-device"))

    # periodic sleep needs a memory hierarchy in the model ...
    sleepy = json.loads(open(wf).read())
    sleepy["phases"][0]["memory_update_mode"] = {"type": "wake_only", "schedule": json.loads(json.dumps(SCHEDULE)),
                                                 "tier_optimizer": {"learning_rate": 1e-2, "beta_1": 0.9, "beta_2": 0.95, "epsilon": 1e-8,
                                                                    "weight_decay": 0.0}}
    sw = tmp_path / "sleepy.json"
    sw.write_text(json.dumps(sleepy))
    r = _cli("train", "--model", mal, "--tokenizer", tok, "--workflow", str(sw), "--device", "cpu", "--output", str(tmp_path / "never"))
    assert r.returncode != 0 and "explicit memory" in r.stderr and not os.path.exists(tmp_path / "never")
    # ... and its reserve capacities must be the model's
    mem = tmp_path / "mem.mal"
    mem.write_text("""attention a { num_heads: 2 } ffn f { hidden_dim: 64 }
      memory m { tier fast { ffn: f reserve_experts { capacity: 2 rank: 4 top_k: 1 } }
                 tier slow { ffn: f reserve_experts { capacity: 3 rank: 4 top_k: 1 } } }
      block b { attention: a memory: m norm: rmsnorm { eps: 1e-5 } }
      model t { max_seq_len: 64 hidden_size: 32 num_layers: 2 block: b }""")
    r = _cli("validate-workflow", "--workflow", str(sw), "--config", str(mem))
    assert r.returncode != 0 and "preallocates" in r.stderr
    sleepy["phases"][0]["memory_update_mode"]["schedule"]["tiers"][1]["reserve_slots"] = 3
    sw.write_text(json.dumps(sleepy))
    r = _cli("validate-workflow", "--workflow", str(sw), "--config", str(mem))
    assert r.returncode == 0, r.stderr[-1500:]


def test_killed_run_resumes_and_finetune_resume_needs_its_checkpoint(tmp_path):
    """`summa-train/tests/trainer_lifecycle.rs:713-853`: a trainer killed outright after its first published generation
    resumes to the planned step count; a fine-tune started from `--checkpoint` resumes only when the same file is named
    again; `--layer-metrics-every` adds per-layer gradient norms to every N-th optimization record."""
    import signal
    import time
    from summa_b200.train.metrics import read_metrics
    tok, data, _, mal = _fixture(tmp_path)
    rows = [{"tokens": list(range(r % 200 + 1, r % 200 + 13))} for r in range(48)]
    (tmp_path / "stream.jsonl").write_text("\n".join(json.dumps(r) for r in rows))
    wf = tmp_path / "wake.json"
    wf.write_text(json.dumps({"version": 2, "phases": [{
        "name": "wake", "type": "continued_pretrain", "task": {"type": "causal_lm"}, "data": "stream.jsonl", "sequence_length": 4,
        "batch_size": 1, "gradient_accumulation": 1, "epochs": 1, "shuffle_buffer": 1, "steps": 12}]}))
    out = tmp_path / "run"
    cmd = [sys.executable, "-m", "summa_b200.cli.train", "train", "--config", mal, "--tokenizer", tok, "--workflow", str(wf),
           "--output", str(out), "--warmup-steps", "0", "--checkpoint-every", "1", "--device", "cpu", "--optimizer", "adamw",
           "--layer-metrics-every", "2"]
    child = subprocess.Popen(cmd, cwd=ROOT, stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL, start_new_session=True)
    try:
        for _ in range(2400):
            if (out / "current.json").is_file() or child.poll() is not None:
                break
            time.sleep(0.025)
    finally:
        if child.poll() is None:
            os.killpg(child.pid, signal.SIGKILL)                                     # the process group this test started
        child.wait()
    assert (out / "current.json").is_file(), "the trainer published no resumable generation to preempt"

    def step():
        gen = json.load(open(out / "current.json"))["generation"]
        return json.load(open(out / "generations" / gen / "training-state.json"))["global_step"]
    assert step() >= 1
    r = subprocess.run(cmd + ["--resume"], cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-3000:]
    assert step() == 12
    opt = [x["event"]["values"] for x in read_metrics(str(out / "metrics.jsonl")) if x["event"]["type"] == "optimization"]
    with_layers = [v for v in opt if v.get("layer_gradient_norms")]
    assert len(opt) == 12 and 1 <= len(with_layers) <= 6 and all(len(v["layer_gradient_norms"]) == 2 for v in with_layers)
    assert all(n >= 0 and max(v["layer_gradient_norms"]) <= v["gradient_norm"] * 1.0001 for v in with_layers for n in v["layer_gradient_norms"])

    # fine-tune from the finished run's weights
    gen = json.load(open(out / "current.json"))["generation"]
    initial = str(out / "generations" / gen / "weights.safetensors")
    ft = tmp_path / "finetune"
    base = ["train", "--model", mal, "--tokenizer", tok, "--workflow", str(wf), "--output", str(ft), "--warmup", "0", "--device", "cpu",
            "--optimizer", "adamw"]
    first = _cli(*base, "--checkpoint", initial)
    assert first.returncode == 0, first.stderr[-3000:]
    bare = _cli(*base, "--resume")
    assert bare.returncode != 0 and "must repeat the same `--checkpoint`" in bare.stderr
    again = _cli(*base, "--resume", "--checkpoint", initial)
    assert again.returncode == 0, again.stderr[-3000:]


def test_run_workflow_command_with_executor_spelling_and_pinned_initial_checkpoint(tmp_path, capsys):
    """`run-workflow --executor X --executor-arg Y --executor-timeout-seconds N --initial-checkpoint-uri U
    --initial-checkpoint-sha256 H` (`summa-train/src/main.rs`, RunWorkflowArgs): the worker runs every phase, the initial
    checkpoint must hash to the pinned identity."""
    import hashlib
    from summa_b200.cli import train as cli
    worker = tmp_path / "worker.py"
    worker.write_text(FAKE_WORKER)
    (tmp_path / "d.jsonl").write_text(json.dumps({"text": "x"}))
    base = {"task": {"type": "causal_lm"}, "data": "d.jsonl", "sequence_length": 8, "batch_size": 2}
    wf = tmp_path / "wf.json"
    wf.write_text(json.dumps({"version": 2, "phases": [dict(base, name="a", type="continued_pretrain", steps=1, gradient_accumulation=1),
                                                         dict(base, name="c", type="evaluation")]}))
    init = tmp_path / "init.safetensors"
    init.write_bytes(b"initial weights")
    digest = hashlib.sha256(b"initial weights").hexdigest()
    argv = ["run-workflow", "--workflow", str(wf), "--state", str(tmp_path / "state.json"), "--executor", sys.executable, "--executor-arg", str(worker),
            "--executor-timeout-seconds", "60", "--initial-checkpoint-uri", str(init)]
    with pytest.raises(SystemExit, match="expected"):
        cli.main(argv + ["--initial-checkpoint-sha256", "sha256:" + "0" * 64])
    outcomes = []
    for _ in range(4):
        assert cli.main(argv + ["--initial-checkpoint-sha256", "sha256:" + digest]) == 0
        outcomes.append(json.loads(capsys.readouterr().out.strip().splitlines()[-1])["outcome"])
        if outcomes[-1] == "complete":
            break
    assert outcomes[-1] == "complete"
    with pytest.raises(SystemExit):
        cli.main(argv + ["--worker", "x"])


def test_llm_command_line_accepts_the_reference_spellings(tmp_path):
    """`summa-llm generate|trace` with `--config -c -t -p -m --no-eos --trace-tokens --channel-bins --attention-heads
    --metrics-points -o` (`summa-llm/src/main.rs`: InferenceArtifacts, SamplingControls, TraceLimits)."""
    from summa_b200 import mal as mal_mod
    from summa_b200.models import Transformer
    from summa_b200.models import weights as W
    tok, _, _, mal = _fixture(tmp_path)
    cfg = mal_mod.load_model_def(mal)
    from summa_b200.tokenizer import Tokenizer
    cfg.vocab_size = Tokenizer.from_file(tok).vocab_size()
    torch.manual_seed(0)
    ckpt = tmp_path / "w.safetensors"
    ckpt.write_bytes(W.serialize(W.model_tensors(Transformer(cfg))))
    llm = lambda *a: subprocess.run([sys.executable, "-m", "summa_b200.cli.llm", *a], capture_output=True, text=True, cwd=ROOT, timeout=300)
    g = llm("generate", "--config", mal, "-c", str(ckpt), "-t", tok, "-p", "the quick", "-m", "6", "--no-eos", "--temperature", "0.9", "--top-k", "5",
            "--seed", "3", "--device", "cpu")
    assert g.returncode == 0 and len(g.stdout.strip()) > 0, g.stderr[-2000:]
    out = tmp_path / "trace.json"
    t = llm("trace", "--config", mal, "--checkpoint", str(ckpt), "--tokenizer", tok, "--prompt", "the quick", "--max-tokens", "3", "-o", str(out),
            "--trace-tokens", "8", "--channel-bins", "4", "--attention-heads", "1", "--metrics-points", "10", "--device", "cpu")
    assert t.returncode == 0, t.stderr[-2000:]
    bundle = json.loads(out.read_text())
    sampling = bundle["inference"]["sampling"]
    assert sampling["max_new_tokens"] == 3 and sampling["stop_at_eos"] is True and bundle["capture"]["requested_token_limit"] == 8


def test_phase_without_steps_runs_its_natural_epoch(tmp_path):
    """No `steps`: floor(floor(samples / batch) / accumulation) * epochs optimizer steps; a `max_steps` above that is a
    cap, not a request; a phase that cannot complete one step is refused before any output exists."""
    tok, _, _, mal = _fixture(tmp_path)
    (tmp_path / "tokens.jsonl").write_text("\n".join(json.dumps({"tokens": list(range(1, 9))}) for _ in range(22)))   # 22 x (8 + eos) tokens
    phase = {"name": "p", "type": "pretrain", "task": {"type": "causal_lm"}, "data": "tokens.jsonl", "sequence_length": 8, "batch_size": 2,
             "gradient_accumulation": 3, "epochs": 1, "shuffle_buffer": 1}
    # 198 tokens -> 24 windows of 9 with stride 8 -> 12 batches -> 4 steps
    for extra, want in [({}, 4), ({"max_steps": 3}, 3), ({"max_steps": 200}, 4), ({"epochs": 2}, 8)]:
        wf = tmp_path / "wf.json"
        wf.write_text(json.dumps({"version": 2, "phases": [dict(phase, **extra)]}))
        out = tmp_path / f"run-{len(extra)}-{want}"
        r = _cli("train", "--model", mal, "--tokenizer", tok, "--workflow", str(wf), "--output", str(out), "--warmup", "0", "--device", "cpu",
                 "--optimizer", "adamw")
        assert r.returncode == 0, r.stderr[-3000:]
        assert json.loads(r.stdout.strip().splitlines()[-1])["global_step"] == want, (extra, r.stdout[-300:])
    wf.write_text(json.dumps({"version": 2, "phases": [dict(phase, batch_size=64)]}))
    r = _cli("train", "--model", mal, "--tokenizer", tok, "--workflow", str(wf), "--output", str(tmp_path / "none"), "--device", "cpu")
    assert r.returncode != 0 and "zero complete optimizer steps" in r.stderr and not os.path.exists(tmp_path / "none")
