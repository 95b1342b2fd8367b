"""The embedded workflow host: fail-closed routing, dispatch identity, and a distillation -> preference -> RL
run through the in-process post-training executor on a tiny model (CPU), with a yield / resume in between
and a metric journal whose `post_training_update` records satisfy the schema's objective-specific rules."""
import hashlib
import json
import os

import pytest
import torch

MAL = """attention a { num_heads: 2 } ffn f { hidden_dim: 64 }
block b { attention: a ffn: f norm: rmsnorm { eps: 1e-5 } }
model t { max_seq_len: 64 hidden_size: 32 num_layers: 2 block: b }"""


def _setup(tmp_path):
    from summa_b200 import mal
    from summa_b200.models import Transformer
    from summa_b200.models import weights as W
    from summa_b200.tokenizer import Tokenizer
    tok = Tokenizer.byte_level()
    cfg = mal.parse_mal(MAL)
    cfg.vocab_size = tok.vocab_size()
    torch.manual_seed(0)
    model = Transformer(cfg, init_std=0.05)
    init = str(tmp_path / "init.safetensors")
    W.save_safetensors(model, init)
    torch.manual_seed(1)
    frozen = str(tmp_path / "frozen.safetensors")
    W.save_safetensors(Transformer(cfg, init_std=0.05), frozen)
    sha = "sha256:" + hashlib.sha256(open(frozen, "rb").read()).hexdigest()
    spec = {"adapter": "summa_checkpoint", "artifact": "frozen.safetensors", "sha256": sha}
    (tmp_path / "kl.jsonl").write_text("\n".join(json.dumps({"prompt": f"q{i} ", "response": f"a{i}"}) for i in range(4)))
    (tmp_path / "pref.jsonl").write_text("\n".join(
        json.dumps({"prompt": f"say {i}: ", "chosen": "yes", "rejected": "no"}) for i in range(4)))
    (tmp_path / "rl.jsonl").write_text("\n".join(
        json.dumps({"prompt": f"{i}+0=", "verifier_payload": {}, "reference_answer": str(i)}) for i in range(2)))
    geo = {"sequence_length": 24, "batch_size": 2, "gradient_accumulation": 1}
    wf = {"version": 2, "phases": [
        dict(geo, name="distill", type="distillation", task={"type": "instruction_tuning"}, data="kl.jsonl", steps=2,
             post_training={"algorithm": "forward_kl", "teacher": spec, "temperature": 1.5}),
        dict(geo, name="prefer", type="preference", task={"type": "pairwise_preference"}, data="pref.jsonl", steps=2,
             post_training={"algorithm": "dpo", "reference": spec}),
        dict(geo, name="reason", type="rl", task={"type": "verifiable_rl", "verifier": {"adapter": "exact_answer"}},
             data="rl.jsonl", steps=1,
             post_training={"algorithm": "grpo", "group_size": 2, "reference": spec,
                            "sampling": {"max_new_tokens": 3, "temperature": 1.0, "top_p": 0.9}})]}
    path = tmp_path / "wf.json"
    path.write_text(json.dumps(wf))
    return cfg, tok, init, str(path)


def test_routing_is_fail_closed_and_identity_pins_adapters(tmp_path):
    from summa_b200.train import native_host as NH
    from summa_b200.train.runtime import ExternalPhaseExecutor
    from summa_b200.train.workflow import load_workflow, parse_workflow
    cfg, tok, init, wf_path = _setup(tmp_path)
    wf = load_workflow(wf_path)
    empty = NH.NativeWorkflowAdapters()
    with pytest.raises(NH.NativeHostError, match="requires a registered native post-training context factory"):
        empty.dispatch_plan(wf)
    with pytest.raises(NH.NativeHostError):       # nothing is created when routing is incomplete
        NH.NativeWorkflowHost.start(wf, empty, str(tmp_path / "state.json"))
    assert not os.path.exists(tmp_path / "state.json")
    ad = NH.NativeWorkflowAdapters()
    ad.register_post_training_factory(NH.TorchPostTrainingFactory(cfg, tok, str(tmp_path / "out")))
    with pytest.raises(NH.NativeHostError, match="already registered"):
        ad.register_post_training_factory(NH.TorchPostTrainingFactory(cfg, tok, str(tmp_path / "out")))
    assert [r["dispatch"] for r in ad.dispatch_plan(wf)] == ["native_post_training"] * 3
    ident = ad.dispatch_identity(wf)
    assert ident.startswith("sha256:") and len(ident) == 71
    ad.register_external(ExternalPhaseExecutor(["/bin/true"], 5.0))
    assert ad.dispatch_identity(wf) != ident          # another adapter set is another run
    plain = parse_workflow(json.dumps({"version": 2, "phases": [
        {"name": "p", "type": "pretrain", "task": {"type": "causal_lm"}, "data": "d.jsonl", "sequence_length": 8,
         "batch_size": 2, "gradient_accumulation": 1, "steps": 1},
        {"name": "e", "type": "evaluation", "task": {"type": "causal_lm"}, "data": "d.jsonl", "sequence_length": 8,
         "batch_size": 2}]}))
    assert [r["dispatch"] for r in ad.dispatch_plan(plain)] == ["external_worker", "external_worker"]
    with pytest.raises(NH.NativeHostError, match="no registered native route"):
        NH.NativeWorkflowAdapters().dispatch_plan(plain)


def test_post_training_phases_run_in_process_with_yield_and_resume(tmp_path):
    from summa_b200.train import native_host as NH
    from summa_b200.train.metrics import read_metrics
    from summa_b200.train.runtime import Checkpoint
    from summa_b200.train.workflow import load_workflow
    cfg, tok, init, wf_path = _setup(tmp_path)
    wf = load_workflow(wf_path)

    def adapters():
        ad = NH.NativeWorkflowAdapters()
        ad.register_post_training_factory(NH.TorchPostTrainingFactory(cfg, tok, str(tmp_path / "out"), lr=1e-3))
        return ad

    state, metrics = str(tmp_path / "state.json"), (str(tmp_path / "metrics.jsonl"), "run-native")
    first = Checkpoint(init, hashlib.sha256(open(init, "rb").read()).hexdigest())
    host = NH.NativeWorkflowHost.start(wf, adapters(), state, metrics, first, update_budget=1)
    assert host.run_until_yield_or_complete() == "yielded"            # one update of the first phase, then yield
    host.close()
    with pytest.raises(NH.NativeHostError, match="already exists"):
        NH.NativeWorkflowHost.start(wf, adapters(), state, None, first)
    outcome, rounds = "yielded", 0
    while outcome == "yielded":
        host = NH.NativeWorkflowHost.resume(wf, adapters(), state, metrics, update_budget=2)
        outcome = host.run_until_yield_or_complete()
        host.close()
        rounds += 1
        assert rounds < 10
    assert outcome == "complete" and host.runtime.state.next_phase == 3
    cur = host.runtime.state.current_checkpoint
    assert os.path.exists(cur["uri"]) and cur["sha256"] != first.sha256
    recs = [r for r in read_metrics(metrics[0], run_id="run-native")]
    ups = [r["event"]["values"] for r in recs if r["event"]["type"] == "post_training_update"]
    assert [u["algorithm"] for u in ups] == ["forward_kl", "forward_kl", "dpo", "dpo", "grpo"]
    assert [u["optimizer_step"] for u in ups] == [1, 2, 1, 2, 1]
    assert all(u["records"] == 2 for u in ups)
    assert "forward_kl" in ups[0] and "preference_accuracy" in ups[2] and "mean_reward" in ups[4]
    assert [r["phase"]["kind"] for r in recs] == ["distillation"] * 2 + ["preference"] * 2 + ["rl"]
    # a different adapter configuration may not adopt this run's state
    other = NH.NativeWorkflowAdapters()
    other.register_post_training_factory(NH.TorchPostTrainingFactory(cfg, tok, str(tmp_path / "out"), lr=5e-4))
    with pytest.raises(Exception, match="different executor configuration"):
        NH.NativeWorkflowHost.resume(wf, other, state)


def test_run_workflow_cli_native_mode_runs_and_resumes(tmp_path, capsys):
    """`run-workflow --native` registers the first-party adapters, refuses an incomplete routing before any
    state exists, yields on the update budget and completes after `--resume`."""
    from summa_b200.cli import train as cli
    cfg, tok, init, wf_path = _setup(tmp_path)
    mal_path = tmp_path / "model.mal"
    mal_path.write_text(MAL.replace("model t {", f"model t {{ vocab_size: {tok.vocab_size()}"))
    state, out = str(tmp_path / "state.json"), str(tmp_path / "out")
    base = ["run-workflow", "--workflow", wf_path, "--state", state, "--native", "--model", str(mal_path),
            "--output", out, "--metrics", str(tmp_path / "metrics.jsonl"), "--lr", "1e-3"]
    cli.main(base + ["--initial-checkpoint", init, "--update-budget", "1"])
    first = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert first["outcome"] == "yielded" and first["routes"] == ["native_post_training"] * 3
    outcome, rounds = first["outcome"], 0
    while outcome == "yielded":
        cli.main(base + ["--resume", "--update-budget", "2"])
        res = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
        outcome, rounds = res["outcome"], rounds + 1
        assert rounds < 10
    assert res["next_phase"] == 3 and os.path.exists(res["current_checkpoint"]["uri"])
    assert res["dispatch_sha256"] == first["dispatch_sha256"]
    # a phase with no native route and no --worker: refused before a state file is created
    from summa_b200.train import native_host as NH
    wf = json.loads(open(wf_path).read())
    wf["phases"] = [{"name": "wake", "type": "pretrain", "task": {"type": "causal_lm"}, "data": "kl.jsonl",
                     "steps": 1, "sequence_length": 24, "batch_size": 2, "gradient_accumulation": 1}]
    plain = tmp_path / "plain.json"
    plain.write_text(json.dumps(wf))
    state2 = str(tmp_path / "state2.json")
    with pytest.raises(NH.NativeHostError, match="no registered native route"):
        cli.main(["run-workflow", "--workflow", str(plain), "--state", state2, "--native", "--model", str(mal_path),
                  "--output", out])
    assert not os.path.exists(state2)


MEMORY_MAL = """attention a { num_heads: 2 } ffn f { hidden_dim: 64 }
  memory mm {
    tier fast { ffn: f reserve_experts { capacity: 2 rank: 4 top_k: 1 } }
    tier slow { ffn: f residual_init: zero reserve_experts { capacity: 2 rank: 4 top_k: 1 } }
  }
  block b { attention: a memory: mm norm: rmsnorm { eps: 1e-5 } }
  model t { vocab_size: 257 max_seq_len: 64 hidden_size: 32 num_layers: 2 block: b }"""
ZERO = "sha256:" + "0" * 64


def test_standalone_sleep_phase_runs_on_the_state_machine_from_a_pinned_wake_journal(tmp_path, capsys):
    """`run-workflow --native` with a standalone sleep-runtime file: the replay windows come from the pinned
    wake-context journal (bound to the phase's input checkpoint), the due tier is consolidated as a transaction of the
    durable state machine whose state is persisted beside the candidate, and the `tier_update` event names the
    receiver slot. A journal of another checkpoint and a runtime bound to another workflow are refused."""
    from summa_b200 import mal
    from summa_b200.cli import train as cli
    from summa_b200.models import Transformer
    from summa_b200.models import weights as W
    from summa_b200.train import native_host as NH
    from summa_b200.train.sleep_runtime import WakeContextJournal
    from summa_b200.train.workflow import load_workflow
    mal_path = tmp_path / "mem.mal"
    mal_path.write_text(MEMORY_MAL)
    torch.manual_seed(0)
    init = str(tmp_path / "init.safetensors")
    W.save_safetensors(Transformer(mal.parse_mal(MEMORY_MAL), init_std=0.08), init)
    init_sha = "sha256:" + hashlib.sha256(open(init, "rb").read()).hexdigest()
    sched = {"clock": "optimizer_steps", "terminal_consolidation": "distill_into_base_v1",
             "tiers": [{"id": "fast", "update_period": 2, "reserve_slots": 2}, {"id": "slow", "update_period": 4, "reserve_slots": 2}]}
    sleep = {"schedule": sched, "standalone_trigger_clock": 2, "receiver_learning_rate": 2e-2, "receiver_weight_decay": 0.0,
             "knowledge_seeding": {"chunk_tokens": 512, "teacher_rollouts": 6, "detached_student_rollouts": 1, "temperature": 1.0, "forward_kl_weight": 1.0},
             "imitation": {"semantic_judge_hash": ZERO, "semantic_weight": 0.5, "maximum_edit_distance": 32, "grpo_group_size": 2},
             "retention_suite": "retention.json", "retention_suite_sha256": ZERO,
             "retention": {"evaluator_hash": ZERO, "suite_hash": ZERO, "max_anchor_forward_kl": 10.0, "max_anchor_regression": 1.0, "min_incorporation_gain": 0.0},
             "grpo_clip_epsilon": 0.2, "grpo_advantage_epsilon": 1e-6, "grpo_kl_coefficient": 0.04, "candidate_directory": "candidates"}
    wf_path = tmp_path / "wf.json"
    wf_path.write_text(json.dumps({"version": 2, "phases": [{"name": "nap", "type": "sleep", "sleep": sleep}]}))
    signature = "sha256:" + load_workflow(str(wf_path)).signature()
    g = torch.Generator().manual_seed(3)
    journal = WakeContextJournal(init_sha)
    for i in range(4):
        journal.push(f"ctx-{i}", i, torch.randint(0, 257, (20,), generator=g).tolist())
    with pytest.raises(Exception, match="repeats id"):
        journal.push("ctx-0", 9, [1, 2])
    with pytest.raises(Exception, match="move backwards"):
        journal.push("late", 1, [1, 2])
    pin = journal.publish(str(tmp_path / "art" / "wake-journal.json"))
    assert WakeContextJournal.load(pin).to_json() == journal.to_json()
    art = lambda name: {"path": f"art/{name}", "sha256": ZERO}
    runtime = {"version": 1, "workflow_signature": signature, "model_mal": {"path": "mem.mal", "sha256": "sha256:" + hashlib.sha256(mal_path.read_bytes()).hexdigest()},
               "wake_context_journal": {"path": "art/wake-journal.json", "sha256": pin.sha256}, "semantic_judge": art("judge.json"),
               "retention_evaluator": art("evaluator.json"), "retention_suite": art("suite.json"),
               "initial_tier_optimizer_state": art("tier.snapshot"), "initial_model_parameter_ids": art("ids.json"),
               "rollouts": {"max_context_tokens": 16, "continuation_tokens": 4, "imitation_groups": 1},
               "tier_optimizer": {"learning_rate": 2e-2, "beta_1": 0.9, "beta_2": 0.95, "epsilon": 1e-8, "weight_decay": 0.0},
               "tensor_transaction_directory": "st/tx", "prospective_directory": "st/pro", "tier_optimizer_directory": "st/opt",
               "candidate_directory": "cand", "rejection_report_directory": "st/rej", "max_wake_context_records": 8, "rng_streams": 2}
    rt = tmp_path / "sleep-runtime.json"
    rt.write_text(json.dumps(runtime))
    ident = "sha256:" + hashlib.sha256(rt.read_bytes()).hexdigest()
    state, out, metrics = str(tmp_path / "state.json"), str(tmp_path / "out"), str(tmp_path / "metrics.jsonl")
    base = ["run-workflow", "--workflow", str(wf_path), "--state", state, "--native", "--model", str(mal_path), "--output", out, "--metrics", metrics,
            "--initial-checkpoint", init]
    cli.main(base + ["--sleep-runtime", str(rt), "--sleep-runtime-sha256", ident])
    res = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert res["outcome"] == "complete" and res["routes"] == ["native_sleep"]
    saved = json.load(open(os.path.join(out, "000-nap", "sleep", "state.json")))
    assert saved["clock"] == 2 and saved["phase"] == "wake" and len(saved["rng_counters"]) == 2 and saved["cycle"] == 1
    from summa_b200.train.metrics import read_metrics
    ups = [r["event"]["values"] for r in read_metrics(metrics) if r["event"]["type"] == "tier_update"]
    assert len(ups) == 1 and ups[0]["tier"] == "fast" and ups[0]["receiver_tier"] == "slow" and ups[0]["tier_clock"] == 2
    if ups[0]["outcome"] == "committed":
        assert ups[0]["reserve_slot"] == 0 and ups[0]["reserve_generation"] == 1 and saved["completed_count"] == 1
        assert res["current_checkpoint"]["uri"].endswith("candidate.safetensors")
    # refusals: runtime bound to another workflow; a journal collected under another checkpoint
    other = tmp_path / "other-runtime.json"
    other.write_text(json.dumps(dict(runtime, workflow_signature=ZERO)))
    with pytest.raises(Exception, match="bound to workflow signature"):
        cli.main(["run-workflow", "--workflow", str(wf_path), "--state", str(tmp_path / "s2.json"), "--native", "--model", str(mal_path), "--output", out,
                  "--initial-checkpoint", init, "--sleep-runtime", str(other), "--sleep-runtime-sha256", "sha256:" + hashlib.sha256(other.read_bytes()).hexdigest()])
    foreign = WakeContextJournal("sha256:" + "9" * 64)
    foreign.push("x", 0, [1, 2, 3])
    foreign.push("y", 1, [4, 5, 6])
    fpin = foreign.publish(str(tmp_path / "art" / "foreign.json"))
    fr = tmp_path / "foreign-runtime.json"
    fr.write_text(json.dumps(dict(runtime, wake_context_journal={"path": "art/foreign.json", "sha256": fpin.sha256})))
    with pytest.raises(Exception, match="another checkpoint"):
        cli.main(["run-workflow", "--workflow", str(wf_path), "--state", str(tmp_path / "s3.json"), "--native", "--model", str(mal_path), "--output", out,
                  "--initial-checkpoint", init, "--sleep-runtime", str(fr), "--sleep-runtime-sha256", "sha256:" + hashlib.sha256(fr.read_bytes()).hexdigest()])
