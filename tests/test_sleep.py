"""Sleep schedule, consolidation transaction (resume + rollback), imitation reward and the
tier optimizer bank."""
import json

import pytest
import torch

from summa_b200.train import sleep


def test_schedule_and_due_senders():
    s = sleep.TierSchedule([4, 8, 32])
    assert s.due_senders(0) == [] and s.due_senders(4) == [0] and s.due_senders(8) == [0, 1]
    assert s.due_senders(32) == [0, 1, 2] and s.due_senders(6) == []
    assert s.next_boundary(5) == 8
    with pytest.raises(sleep.SleepError):
        sleep.TierSchedule([4, 6])
    with pytest.raises(sleep.SleepError):
        sleep.TierSchedule([])


def test_transaction_resume_and_rollback(tmp_path):
    path = str(tmp_path / "txn.json")
    calls = []

    def ok(name):
        def h(ctx):
            calls.append(name)
            return sleep.PhaseResult(True, {"x": 1.0})
        return h

    def crash(ctx):
        calls.append("imitation-crash")
        raise KeyboardInterrupt          # a real crash: not caught by the transaction

    txn = sleep.ConsolidationTxn(path, 8, 0, 1, dreaming=False)
    assert txn.phases() == ["prospective_update", "knowledge_seeding", "imitation", "retention_validation", "commit",
                            "candidate"]
    handlers = {p: ok(p) for p in txn.phases()}
    handlers["imitation"] = crash
    with pytest.raises(KeyboardInterrupt):
        txn.run(handlers, lambda: calls.append("restore"))
    assert json.load(open(path))["phase_index"] == 2            # resumes AT the phase that was running
    txn2 = sleep.ConsolidationTxn(path, 8, 0, 1)
    handlers["imitation"] = ok("imitation")
    st = txn2.run(handlers, lambda: calls.append("restore"))
    assert st.status == "committed" and "restore" not in calls
    assert calls.count("prospective_update") == 1 and calls[-1] == "candidate"
    with pytest.raises(sleep.SleepError):
        sleep.ConsolidationTxn(path, 16, 0, 1)
    # rejection (and handler exceptions) roll back and restore the teacher
    path2 = str(tmp_path / "txn2.json")
    t3 = sleep.ConsolidationTxn(path2, 8, 1, 2, dreaming=True)
    assert "dream_trials" in t3.phases()
    restored = []
    st3 = t3.run({"retention_validation": lambda c: sleep.PhaseResult(False, {"anchor_kl": 9.0}, "anchor KL too high")},
                 lambda: restored.append(1))
    assert st3.status == "rolled_back" and restored == [1] and st3.history[-1]["reason"] == "anchor KL too high"
    t4 = sleep.ConsolidationTxn(str(tmp_path / "t4.json"), 8, 0, 1)
    st4 = t4.run({"commit": lambda c: 1 / 0}, lambda: restored.append(2))
    assert st4.status == "rolled_back" and "ZeroDivisionError" in st4.history[-1]["reason"]


def test_driver_runs_due_tiers(tmp_path):
    d = sleep.SleepDriver(sleep.TierSchedule([2, 4]), str(tmp_path), dreaming_from_tier=1)
    seen = []
    out = d.run_boundary(4, lambda tier: {"commit": lambda c: (seen.append((tier, c["clock"])), sleep.PhaseResult())[1]},
                         lambda tier: None)
    assert [s.sender for s in out] == [0, 1] and all(s.status == "committed" for s in out)
    assert seen == [(0, 4), (1, 4)] and out[1].dreaming and not out[0].dreaming
    assert d.run_boundary(4, lambda t: {"commit": lambda c: 1 / 0}, lambda t: None)[0].status == "committed"  # idempotent


def test_reward_and_levenshtein():
    assert sleep.levenshtein([1, 2, 3], [1, 3]) == 1 and sleep.levenshtein([], [1, 2]) == 2
    assert sleep.imitation_reward([1, 2, 3, 4], [1, 2, 3, 4], semantic=0.5, gamma=0.5) == pytest.approx(0.75)
    assert sleep.imitation_reward([1], [2], semantic=0.2, gamma=0.5, threshold=0.5) == 0.0


def test_gradient_partition_and_tier_bank():
    ps = {"layers.0.attention.o_proj.weight": torch.nn.Parameter(torch.ones(2, 2)),
          "layers.0.memory.tiers.0.ffn.down_proj.weight": torch.nn.Parameter(torch.ones(2, 2)),
          "layers.0.memory.tiers.1.reserve.a": torch.nn.Parameter(torch.ones(2, 2)),
          "layers.0.memory.tiers.1.reserve.slot3": torch.nn.Parameter(torch.ones(2, 2))}
    for n, p in ps.items():
        p.grad = torch.full_like(p, 0.5) if "slot3" not in n else None
    scopes = sleep.partition_gradients(ps.items(), dormant=["layers.0.memory.tiers.1.reserve.slot3"])
    assert scopes["wake"] == ["layers.0.attention.o_proj.weight"] and len(scopes["tier0"]) == 1 and len(scopes["tier1"]) == 1
    ps["layers.0.memory.tiers.1.reserve.slot3"].grad = torch.ones(2, 2)
    with pytest.raises(sleep.SleepError):
        sleep.partition_gradients(ps.items(), dormant=["layers.0.memory.tiers.1.reserve.slot3"])
    bank = sleep.TierOptimizerBank(ps.items(), lr=0.1)
    bank.accumulate(0); bank.accumulate(0 if False else 1)
    before = ps["layers.0.memory.tiers.0.ffn.down_proj.weight"].detach().clone()
    assert bank.apply(0) == 1 and bank.clocks() == {0: 1, 1: 0}
    assert not torch.equal(before, ps["layers.0.memory.tiers.0.ffn.down_proj.weight"].detach())
    assert torch.equal(ps["layers.0.memory.tiers.1.reserve.a"].detach(), torch.ones(2, 2))   # tier 1 not applied yet
