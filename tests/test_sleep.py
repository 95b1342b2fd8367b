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


def _sleep_model():
    from summa_b200 import mal
    from summa_b200.models import Transformer
    cfg = mal.parse_mal("""
      attention a { num_heads: 2 }
      ffn f { hidden_dim: 64 }
      memory mm {
        tier fast { ffn: f reserve_experts { capacity: 2 rank: 4 top_k: 1 } }
        tier slow { ffn: f residual_init: zero reserve_experts { capacity: 2 rank: 4 top_k: 1 } }
      }
      block b { attention: a memory: mm norm: rmsnorm { eps: 1e-5 } }
      model t { vocab_size: 64 max_seq_len: 32 hidden_size: 32 num_layers: 2 block: b }""")
    torch.manual_seed(0)
    return Transformer(cfg, init_std=0.08)


def _accumulate_wake_gradient(model, bank, data, steps=3):
    for tok in data[:steps]:
        model.train()
        model.zero_grad(set_to_none=True)
        model.forward_loss(tok[:, :-1], tok[:, 1:]).backward()
        bank.accumulate(0)


def test_builtin_consolidation_commits_and_rolls_back(tmp_path):
    """The built-in handlers on a two-tier memory model: the sender's accumulated update is distilled
    into a newly activated slot of the receiver tier (KL to the prospective teacher drops), the
    transaction commits and clears the accumulator; with an impossible retention gate the same
    transaction rolls back to the exact pre-consolidation weights."""
    from summa_b200.train.builtin_sleep import BuiltinConsolidation, ConsolidationConfig
    g = torch.Generator().manual_seed(1)
    replay = [torch.randint(0, 64, (4, 17), generator=g) for _ in range(3)]
    anchors = [torch.randint(0, 64, (4, 17), generator=g)]

    def run(cfg, name):
        model = _sleep_model()
        bank = sleep.TierOptimizerBank(model.named_parameters(), lr=2e-2)
        _accumulate_wake_gradient(model, bank, replay)
        before = {n: p.detach().clone() for n, p in model.named_parameters()}
        bc = BuiltinConsolidation(model, bank, 0, 1, [t[:, :-1] for t in replay], [t[:, :-1] for t in anchors], cfg)
        txn = sleep.ConsolidationTxn(str(tmp_path / name), clock=4, sender=0, receiver=1)
        st = txn.run(bc.handlers(), bc.restore_teacher, {"clock": 4})
        return model, bank, before, st

    model, bank, before, st = run(ConsolidationConfig(seeding_steps=30, seeding_lr=2e-2, imitation_steps=1,
                                                      imitation_group=3, imitation_new_tokens=4, max_anchor_kl=5.0), "a.json")
    hist = {h["phase"]: h for h in st.history}
    assert st.status == "committed", st.history
    seed = hist["knowledge_seeding"]["metrics"]
    assert seed["kl_after"] < seed["kl_before"] and seed["activated_slots"] == 2.0
    assert hist["retention_validation"]["metrics"]["incorporation_gain"] >= 0.05
    assert 0.0 <= hist["imitation"]["metrics"]["reward_mean"] <= 1.0
    for blk in model.layers:
        assert blk.memory.tiers[1].reserve.active_slots() == [0] and blk.memory.tiers[0].reserve.active_slots() == []
    assert all(float(a.abs().sum()) == 0.0 for a in bank.state[0]["acc"])
    # only the activated slots moved; the sender tier kept its pre-update weights
    for n, p in model.named_parameters():
        if ".tiers.1.reserve.slots.0." in n:
            continue
        assert torch.equal(p.detach(), before[n]), n

    model, bank, before, st = run(ConsolidationConfig(seeding_steps=3, imitation_steps=0, max_anchor_kl=-1.0), "b.json")
    assert st.status == "rolled_back" and st.history[-1]["phase"] == "retention_validation"
    assert "anchor KL" in st.history[-1]["reason"]
    for n, p in model.named_parameters():
        assert torch.equal(p.detach(), before[n]), n
    assert any(float(a.abs().sum()) > 0.0 for a in bank.state[0]["acc"])       # the update is still pending


def test_builtin_dreaming_phases_run_after_consolidation(tmp_path):
    """A dreaming transaction: consolidation handlers followed by the four dream phases; the model is
    only changed by the policy update, and only in the receiver tier's active slots."""
    from summa_b200.train.builtin_sleep import BuiltinConsolidation, BuiltinDreaming, ConsolidationConfig, DreamConfig
    g = torch.Generator().manual_seed(2)
    replay = [torch.randint(0, 64, (4, 17), generator=g) for _ in range(2)]
    reference = [torch.randint(0, 64, (4, 13), generator=g)]
    model = _sleep_model()
    bank = sleep.TierOptimizerBank(model.named_parameters(), lr=2e-2)
    _accumulate_wake_gradient(model, bank, replay, steps=2)
    bc = BuiltinConsolidation(model, bank, 0, 1, [t[:, :-1] for t in replay], [],
                              ConsolidationConfig(seeding_steps=10, seeding_lr=2e-2, imitation_steps=0, max_anchor_kl=5.0))
    dream = BuiltinDreaming(model, [t[:1, :6] for t in replay], reference,
                            cfg=DreamConfig(candidates_per_prompt=3, new_tokens=5, keep=3, trial_steps=3, policy_steps=2))
    txn = sleep.ConsolidationTxn(str(tmp_path / "d.json"), clock=8, sender=0, receiver=1, dreaming=True)
    handlers = dict(bc.handlers(), **dream.handlers())
    snap = {}

    def remember(ctx):                                   # weights as the consolidation left them
        snap.update({n: p.detach().clone() for n, p in model.named_parameters()})
        return bc.commit(ctx)
    handlers["commit"] = remember
    st = txn.run(handlers, bc.restore_teacher, {"clock": 8})
    assert st.status == "committed", st.history
    hist = {h["phase"]: h["metrics"] for h in st.history}
    assert hist["dream_generation"]["candidates"] == 6.0 and hist["dream_ranking"]["kept"] == 3.0
    assert -1.0 <= hist["dream_ranking"]["best_cosine"] <= 1.0
    assert hist["dream_trials"]["accepted"] <= 3.0
    changed = [n for n, p in model.named_parameters() if not torch.equal(p.detach(), snap[n])]
    assert all(".tiers.1.reserve.slots.0." in n for n in changed), changed
    if hist["dream_trials"]["accepted"] > 0:
        assert changed and hist["dream_policy_update"]["trained_on"] == hist["dream_trials"]["accepted"]


def test_terminal_tier_distils_its_reserves_into_the_base():
    from summa_b200.train.builtin_sleep import distill_into_base
    model = _sleep_model()
    g = torch.Generator().manual_seed(5)
    batches = [torch.randint(0, 64, (4, 16), generator=g) for _ in range(2)]
    with torch.no_grad():                                   # give the slow tier's slots something to say
        for blk in model.layers:
            r = blk.memory.tiers[1].reserve
            r.activate(0)
            r.slots[0].b.normal_(0, 0.05, generator=g)
            r.slots[0].router.weight.normal_(0, 0.5, generator=g)
    before = {n: p.detach().clone() for n, p in model.named_parameters()}
    rejected = distill_into_base(model, 1, batches, steps=1, lr=1e-5, max_kl=0.0)
    assert not rejected.accepted and rejected.metrics["freed_slots"] == 2.0
    for n, p in model.named_parameters():
        assert torch.equal(p.detach(), before[n]), n        # exact rollback, slots active again
    res = distill_into_base(model, 1, batches, steps=60, lr=5e-3, max_kl=1.0)
    assert res.accepted and res.metrics["kl"] < res.metrics["kl_before"]
    for blk in model.layers:
        assert blk.memory.tiers[1].reserve.active_slots() == []
    moved = [n for n, p in model.named_parameters() if not torch.equal(p.detach(), before[n])]
    reclaimed = (".active", ".generation", ".b", ".router.weight")          # the freed slots wake up as the identity next time
    assert moved and all(".tiers.1.feed_forward." in n or (".tiers.1.reserve.slots.0" in n and n.endswith(reclaimed)) for n in moved), moved


def test_builtin_consolidation_under_the_durable_state_machine():
    """The same tensor work driven by `sleep_state.run_consolidation`: the state machine names the receiver slot
    and reserves the RNG ranges, the commit flips the slot masks in the metadata exactly as the model's reserves
    flipped, and a retention rejection restores the weights and consumes the attempt id."""
    from summa_b200.train import sleep_state as SS
    from summa_b200.train.builtin_sleep import BuiltinConsolidation, ConsolidationConfig, StateMachineConsolidation, parameter_fingerprint
    g = torch.Generator().manual_seed(1)
    replay = [torch.randint(0, 64, (4, 17), generator=g) for _ in range(3)]
    anchors = [torch.randint(0, 64, (4, 17), generator=g)]
    sched = SS.SleepSchedule("optimizer_steps", "distill_into_base_v1", [SS.TierSpec("fast", 4, 2), SS.TierSpec("slow", 8, 2)])

    def run(cfg):
        model = _sleep_model()
        bank = sleep.TierOptimizerBank(model.named_parameters(), lr=2e-2)
        _accumulate_wake_gradient(model, bank, replay)
        before = {n: p.detach().clone() for n, p in model.named_parameters()}
        state = SS.SleepState(sched, 1)
        state.advance_clock(sched, 4)
        teacher = parameter_fingerprint(model)
        state.begin(0, "memory://teacher", teacher, "memory://student", teacher, SS.ZERO_HASH)
        be = StateMachineConsolidation(BuiltinConsolidation(model, bank, 0, 1, [t[:, :-1] for t in replay], [t[:, :-1] for t in anchors], cfg))
        return model, before, state, be, SS.run_consolidation(state, be)

    model, before, state, be, ok = run(ConsolidationConfig(seeding_steps=30, seeding_lr=2e-2, imitation_steps=1, imitation_group=3,
                                                          imitation_new_tokens=4, max_anchor_kl=5.0))
    assert ok and state.pending.committed and state.pending.receiver_slot == 0
    assert state.tiers[1].slots[0].active and state.tiers[1].slots[0].generation == 1
    for blk in model.layers:
        assert blk.memory.tiers[1].reserve.active_slots() == [0]
    assert state.pending.candidate_hash == parameter_fingerprint(model) != state.pending.teacher_hash
    assert state.pending.knowledge_rng.count == 30 and state.pending.imitation_rng.count == 12 and state.rng_counters == [42]
    assert be.metrics["knowledge_seeding"]["kl_after"] < be.metrics["knowledge_seeding"]["kl_before"]
    state.transition("candidate")
    state.finish_candidate()
    assert state.completed_count == 1 and state.phase == "wake"

    model, before, state, be, ok = run(ConsolidationConfig(seeding_steps=3, imitation_steps=0, max_anchor_kl=-1.0))
    assert not ok and state.phase == "wake" and state.cycle == 1 and not state.tiers[1].slots[0].active
    assert "anchor KL" in be.metrics["retention_validation"]["reason"]
    for n, p in model.named_parameters():
        assert torch.equal(p.detach(), before[n]), n


def test_builtin_dreaming_under_the_durable_state_machine():
    """Consolidation then dreaming, both driven by the state machine: the shared candidate's fingerprint is the same
    before and after every backend call (trials and the policy step never write it), the kept dreams each get one
    isolated trial under their own RNG receipt, the policy state is installed only after the transaction retires,
    and a backend that lost its in-memory candidates regenerates the recorded manifest."""
    from summa_b200.train import sleep_state as SS
    from summa_b200.train.builtin_sleep import (BuiltinConsolidation, BuiltinDreaming, ConsolidationConfig, DreamConfig,
                                                StateMachineConsolidation, StateMachineDreaming, parameter_fingerprint)
    g = torch.Generator().manual_seed(1)
    replay = [torch.randint(0, 64, (4, 17), generator=g) for _ in range(3)]
    anchors = [torch.randint(0, 64, (4, 17), generator=g)]
    sched = SS.SleepSchedule("optimizer_steps", "distill_into_base_v1", [SS.TierSpec("fast", 4, 2), SS.TierSpec("slow", 8, 2)])
    model = _sleep_model()
    bank = sleep.TierOptimizerBank(model.named_parameters(), lr=2e-2)
    _accumulate_wake_gradient(model, bank, replay)
    state = SS.SleepState(sched, 1)
    state.advance_clock(sched, 4)
    fp = parameter_fingerprint(model)
    state.begin(0, "memory://teacher", fp, "memory://student", fp, SS.ZERO_HASH)
    cons = StateMachineConsolidation(BuiltinConsolidation(model, bank, 0, 1, [t[:, :-1] for t in replay], [t[:, :-1] for t in anchors],
                                                          ConsolidationConfig(seeding_steps=10, seeding_lr=2e-2, imitation_steps=0, max_anchor_kl=5.0)))
    assert SS.run_consolidation(state, cons)
    committed = parameter_fingerprint(model)
    ev = "sha256:" + "e" * 64
    cfg = SS.DreamingConfig(candidate_count=6, retain_top=2, retain_random=1, lora_rank=4, lora_alpha=8, trial_evaluator_hash=ev)
    inner = BuiltinDreaming(model, [r[:1, :6] for r in replay], anchors, cfg=DreamConfig(new_tokens=5, trial_steps=3, policy_steps=2))
    be = StateMachineDreaming(inner, ev)
    events = []

    class Sink:
        def persist(self, st):
            pass

        def metric(self, kind, fields):
            events.append(kind)

    accepted = SS.run_dreaming(state, cfg, be, Sink())
    t = state.pending
    assert state.phase == "candidate" and parameter_fingerprint(model) == committed == t.dream_shared_checkpoint_hash
    assert len(t.dream_selected) == 3 and len(t.dream_trials) == 3 and len({r.start for _, r in t.dream_trial_rngs}) == 3
    assert events == ["dream_selection"] + ["dream_trial"] * 3 and all(x.independent_task_improvement > 0 for x in accepted)
    # a fresh backend (process restart) regenerates the same candidates from the recorded RNG range
    again = StateMachineDreaming(BuiltinDreaming(model, [r[:1, :6] for r in replay], anchors, cfg=DreamConfig(new_tokens=5)), ev)
    assert [d.artifact_hash for d in again.load_generated_dreams(t, t.generated_manifest)] == [d.artifact_hash for d in be.generated[t.generated_manifest]]
    done = state.finish_candidate()
    assert done.dream_policy_receipt == be.receipts[done.id] and state.phase == "wake"
    moved = be.install_policy_state()
    assert (moved > 0) == bool(accepted) and (parameter_fingerprint(model) != committed) == bool(accepted)


def test_three_tier_chain_reclaims_sender_slots_and_keeps_model_and_metadata_in_step():
    """fast -> mid -> slow: the mid tier's reserves (filled by the fast tier's boundaries) are reclaimed when the mid
    tier itself consolidates into the slow tier, so it never runs out of slots; after every retired transaction the
    masks and generations in every memory block equal the sleep state's."""
    from summa_b200 import mal
    from summa_b200.models import Transformer
    from summa_b200.train import sleep_state as SS
    from summa_b200.train.builtin_sleep import (BuiltinConsolidation, ConsolidationConfig, StateMachineConsolidation, TerminalConsolidation,
                                                validate_model_memory_state)
    cfg = mal.parse_mal("""
      attention a { num_heads: 2 } ffn f { hidden_dim: 32 }
      memory mm {
        tier fast { ffn: f reserve_experts { capacity: 1 rank: 2 top_k: 1 } }
        tier mid { ffn: f residual_init: zero reserve_experts { capacity: 2 rank: 2 top_k: 1 } }
        tier slow { ffn: f residual_init: zero reserve_experts { capacity: 2 rank: 2 top_k: 1 } }
      }
      block b { attention: a memory: mm norm: rmsnorm { eps: 1e-5 } }
      model t { vocab_size: 64 max_seq_len: 32 hidden_size: 16 num_layers: 2 block: b }""")
    torch.manual_seed(0)
    model = Transformer(cfg, init_std=0.08)
    sched = SS.SleepSchedule("optimizer_steps", "distill_into_base_v1",
                             [SS.TierSpec("fast", 2, 1), SS.TierSpec("mid", 4, 2), SS.TierSpec("slow", 8, 2)])
    state = SS.SleepState(sched, 1)
    bank = sleep.TierOptimizerBank(model.named_parameters(), lr=1e-2)
    g = torch.Generator().manual_seed(2)
    replay = [torch.randint(0, 64, (2, 13), generator=g) for _ in range(2)]
    ccfg = ConsolidationConfig(seeding_steps=2, imitation_steps=0, max_anchor_kl=100.0, min_incorporation_gain=-1e9)
    log = []
    for clock in range(1, 9):
        model.train()
        model.zero_grad(set_to_none=True)
        model.forward_loss(replay[0][:, :-1], replay[0][:, 1:]).backward()
        for t in (0, 1, 2):
            bank.accumulate(t)
        state.advance_clock(sched, clock)
        while state.next_due() is not None:
            sender, trigger = state.next_due()
            txn = state.begin(sender, "m://t", SS.ZERO_HASH, "m://s", SS.ZERO_HASH, SS.ZERO_HASH)
            if sender < 2:
                be = StateMachineConsolidation(BuiltinConsolidation(model, bank, sender, sender + 1, [r[:, :-1] for r in replay], [], ccfg),
                                               publish=lambda t, m: ("m://c", SS.ZERO_HASH))
            else:
                be = TerminalConsolidation(model, bank, 2, [r[:, :-1] for r in replay], publish=lambda t, m: ("m://c", SS.ZERO_HASH))
            ok = SS.run_consolidation(state, be)
            log.append((trigger, sender, ok, list(txn.sender_slots_to_reset), txn.receiver_slot))
            if ok:
                state.transition("candidate")
                state.finish_candidate()
            validate_model_memory_state(model, state)
    by_clock = {(c, s): (ok, reset, slot) for c, s, ok, reset, slot in log}
    assert by_clock[(2, 0)] == (True, [], 0) and by_clock[(4, 0)] == (True, [], 1)           # the mid tier fills both slots
    assert by_clock[(4, 1)][0] and by_clock[(4, 1)][1] == [0, 1] and by_clock[(4, 1)][2] == 0     # ... and is emptied into the slow tier
    assert by_clock[(6, 0)] == (True, [], 0)                                                    # so the fast tier can transfer again
    assert by_clock[(8, 1)][1] == [0, 1] and by_clock[(8, 1)][2] == 1
    mid = [(s.active, s.generation) for s in state.tiers[1].slots]
    assert [a for a, _ in mid] == [False, False] and all(gen == 4 for _, gen in mid)           # woken and reclaimed twice each
    # the terminal boundary at 8 either folded the slow tier's two reserves into its base or left everything as it was
    ok8, reset8, _ = by_clock[(8, 2)]
    assert reset8 == [0, 1] and [s.active for s in state.tiers[2].slots] == ([False, False] if ok8 else [True, True])
    # tampering with one layer's mask is caught
    model.layers[1].memory.tiers[1].reserve.activate(0)
    with pytest.raises(sleep.SleepError, match="differ from the sleep state"):
        validate_model_memory_state(model, state)


def test_tier_bank_snapshots_and_checkpoint_scopes(tmp_path):
    """`summa-train/tests/trainer_lifecycle.rs:911-987`: identical state gives identical bytes, a restored bank snapshots
    to the same bytes, every tier is sealed as its own immutable bundle, and a failed restore leaves the bank untouched."""
    import os
    from summa_b200 import mal
    from summa_b200.models import Transformer
    from summa_b200.train.sleep import TierOptimizerBank
    cfg = mal.parse_mal("""attention a { num_heads: 2 } ffn f { hidden_dim: 32 }
      memory mm { tier fast { ffn: f reserve_experts { capacity: 2 rank: 4 top_k: 1 } }
                  tier slow { ffn: f residual_init: zero reserve_experts { capacity: 2 rank: 4 top_k: 1 } } }
      block b { attention: a memory: mm norm: rmsnorm { eps: 1e-5 } }
      model t { vocab_size: 64 max_seq_len: 16 hidden_size: 16 num_layers: 2 block: b }""")
    torch.manual_seed(7)
    model = Transformer(cfg)
    bank = TierOptimizerBank(model.named_parameters(), lr=1e-2)
    x = torch.tensor([[1, 2, 3, 4]])
    model.forward_loss(x, torch.tensor([[2, 3, 4, 5]])).backward() if hasattr(model, "forward_loss") else model(x).logits.sum().backward()
    for t in (0, 1):
        bank.accumulate(t)
    assert [bank.state[t]["count"] for t in (0, 1)] == [1, 1]
    bank.apply(0)
    snap = bank.snapshot_bytes()
    assert snap == bank.snapshot_bytes()
    other = TierOptimizerBank(model.named_parameters(), lr=1e-2)
    other.restore_bytes(snap)
    assert other.snapshot_bytes() == snap and other.clocks() == {0: 1, 1: 0}
    scopes = bank.publish_checkpoint_scopes(str(tmp_path / "tier-optimizers"))
    assert [t["accumulated_micro_steps"] for t in scopes["tiers"]] == [0, 1] and all(t["artifact"]["sha256"].startswith("sha256:") for t in scopes["tiers"])
    assert bank.publish_checkpoint_scopes(str(tmp_path / "tier-optimizers")) == scopes             # write once, content addressed
    assert len(os.listdir(tmp_path / "tier-optimizers" / "generations")) == 2
    fresh = TierOptimizerBank(model.named_parameters(), lr=1e-2)
    fresh.restore_scopes(str(tmp_path / "tier-optimizers"), scopes)
    assert fresh.snapshot_bytes() == snap
    # a bundle that changed, foreign settings and a lying clock are all refused, and the bank keeps its state
    before = fresh.snapshot_bytes()
    lying = {"tiers": [dict(scopes["tiers"][0], update_clock=9), scopes["tiers"][1]]}
    with pytest.raises(ValueError, match="clocks differ"):
        fresh.restore_scopes(str(tmp_path / "tier-optimizers"), lying)
    path = tmp_path / "tier-optimizers" / scopes["tiers"][1]["artifact"]["path"]
    body = bytearray(path.read_bytes())
    body[-1] ^= 1
    path.write_bytes(bytes(body))
    with pytest.raises(ValueError, match="recorded identity"):
        fresh.restore_scopes(str(tmp_path / "tier-optimizers"), scopes)
    with pytest.raises(ValueError, match="other optimizer settings"):
        TierOptimizerBank(model.named_parameters(), lr=3e-4).restore_bytes(snap)
    assert fresh.snapshot_bytes() == before


def test_tier_window_joins_the_global_clip():
    """Tier gradients wait in a window, contribute their squared norm to the step's one global norm and enter the
    accumulators scaled by the same clip coefficient as the wake gradients."""
    from summa_b200 import mal
    from summa_b200.models import Transformer
    from summa_b200.train.engine import FlatTrainEngine, OptimConfig
    from summa_b200.train.sleep import TierOptimizerBank, tier_of_parameter
    cfg = mal.parse_mal("""attention a { num_heads: 2 } ffn f { hidden_dim: 32 }
      memory mm { tier fast { ffn: f reserve_experts { capacity: 2 rank: 4 top_k: 1 } } }
      block b { attention: a memory: mm norm: rmsnorm { eps: 1e-5 } }
      model t { vocab_size: 64 max_seq_len: 16 hidden_size: 16 num_layers: 1 block: b }""")
    torch.manual_seed(3)
    model = Transformer(cfg)
    bank = TierOptimizerBank(model.named_parameters(), lr=1e-2)
    eng = FlatTrainEngine(model, OptimConfig(lr=1e-3, max_grad_norm=0.05), param_dtype=torch.float32,
                          exclude=lambda n: tier_of_parameter(n) is not None)
    x = torch.tensor([[1, 2, 3, 4, 5, 6]])
    eng.zero_grad()
    model.forward_loss(x[:, :-1], x[:, 1:]).backward() if hasattr(model, "forward_loss") else None
    tier_grads = [None if p.grad is None else p.grad.detach().float().clone() for _, p in bank.params[0]]
    assert any(g is not None and float(g.abs().sum()) > 0 for g in tier_grads), "the tier parameters received no gradient"
    eng.fold_autograd_grads()
    wake_sq = float(eng.grads_flat[:eng.numel].pow(2).sum() + eng.small_grads.pow(2).sum())
    bank.accumulate(0, staged=True)
    tier_sq = float(sum(g.pow(2).sum() for g in tier_grads if g is not None))
    assert abs(float(bank.window_sumsq()) - tier_sq) <= 1e-6 * max(tier_sq, 1.0) and all(float(a.abs().sum()) == 0.0 for a in bank.state[0]["acc"])
    eng.extra_sumsq = bank.window_sumsq()
    norm = float(eng.step(1e-3))
    assert abs(norm - (wake_sq + tier_sq) ** 0.5) <= 1e-4 * norm and eng.extra_sumsq is None and norm > 0.05
    c = min(1.0, 0.05 / (norm + 1e-6))
    bank.commit_window(c)
    for acc, g in zip(bank.state[0]["acc"], tier_grads):
        assert torch.allclose(acc, torch.zeros_like(acc) if g is None else g * c, rtol=1e-5, atol=1e-9)
    assert float(bank.window_sumsq()) == 0.0 and bank.state[0]["count"] == 1
