"""The durable sleep state machine: schedule rules, clock and due queue, transaction life cycle, RNG receipts,
failure atomicity, the audit chain, and the consolidation / dreaming drivers against scripted backends
(the cases of `summa-train/src/sleep.rs:3486-4600`, restated for this package's API)."""
import copy
import json

import pytest

from summa_b200.train import sleep_state as S
from summa_b200.train.sleep import SleepError


def H(d):
    return "sha256:" + str(d) * 64


def schedule(periods=(2, 4, 8), slots=(2, 2, 2)):
    return S.SleepSchedule("optimizer_steps", "distill_into_base_v1",
                           [S.TierSpec(n, p, k) for n, p, k in zip(("fast", "mid", "slow"), periods, slots)])


def begun(clock=2):
    st = S.SleepState(schedule(), 2)
    st.advance_clock(schedule(), clock)
    st.begin(0, "teacher", H(1), "student", H(2), H(3))
    return st


def test_schedule_rules_and_due_order():
    sc = schedule()
    sc.validate()
    assert sc.due_senders(2) == [0] and sc.due_senders(4) == [0, 1] and sc.due_senders(8) == [0, 1, 2] and sc.due_senders(0) == []
    with pytest.raises(SleepError, match="divisible"):
        schedule(periods=(2, 3, 9)).validate()
    with pytest.raises(SleepError, match="less often"):
        schedule(periods=(2, 2, 8)).validate()
    with pytest.raises(SleepError, match="at least 4 reserve slots"):
        schedule(periods=(2, 8, 16), slots=(2, 2, 2)).validate()
    with pytest.raises(SleepError, match="2..=16"):
        S.SleepSchedule("optimizer_steps", "distill_into_base_v1", [S.TierSpec("only", 2, 1)]).validate()
    with pytest.raises(SleepError, match="duplicate"):
        S.SleepSchedule("optimizer_steps", "distill_into_base_v1", [S.TierSpec("a", 2, 1), S.TierSpec("a", 4, 2)]).validate()
    with pytest.raises(SleepError, match="exactly"):
        S.SleepSchedule.from_json({"clock": "optimizer_steps", "terminal_consolidation": "distill_into_base_v1", "tiers": [], "extra": 1})
    again = S.SleepSchedule.from_json(sc.to_json())
    assert again == sc
    with pytest.raises(SleepError, match="RNG streams"):
        S.SleepState(sc, 0)


def test_clock_advance_queues_boundaries_and_refuses_coarse_steps():
    sc, st = schedule(), S.SleepState(schedule(), 1)
    st.advance_clock(sc, 1)
    assert st.next_due() is None
    st.advance_clock(sc, 2)
    assert st.next_due() == (0, 2)
    with pytest.raises(SleepError, match="finishing every due sender"):
        st.advance_clock(sc, 3)
    fresh = S.SleepState(sc, 1)
    before = json.dumps(fresh.to_json(), sort_keys=True)
    with pytest.raises(SleepError, match="crosses multiple `fast` boundaries"):
        fresh.advance_clock(sc, 4)
    assert json.dumps(fresh.to_json(), sort_keys=True) == before          # refused without touching the scheduler
    with pytest.raises(SleepError, match="backwards"):
        st2 = S.SleepState(sc, 1)
        st2.advance_clock(sc, 1)
        st2.advance_clock(sc, 0)


def test_rng_receipts_are_phase_bound_idempotent_and_failure_atomic():
    st = S.SleepState(schedule(), 2)
    snap = st.to_json()
    with pytest.raises(SleepError, match="requires the knowledge_seeding phase"):
        st.reserve_rng("knowledge", 0, 4)
    assert st.to_json() == snap
    st = begun()
    with pytest.raises(SleepError, match="requires the knowledge_seeding phase"):
        st.reserve_rng("knowledge", 0, 4)                                   # still in prospective_update
    assert st.rng_counters == [0, 0]
    st.transition("knowledge_seeding")
    r = st.reserve_rng("knowledge", 1, 5)
    assert (r.stream, r.start, r.count) == (1, 0, 5) and st.rng_counters == [0, 5]
    assert st.reserve_rng("knowledge", 1, 5) == r and st.rng_counters == [0, 5]      # a resumed sub-phase gets the same draws
    with pytest.raises(SleepError, match="differs on retry"):
        st.reserve_rng("knowledge", 1, 6)
    with pytest.raises(SleepError, match="does not exist"):
        st2 = begun()
        st2.transition("knowledge_seeding")
        st2.reserve_rng("knowledge", 9, 1)
    with pytest.raises(SleepError, match="invalid sleep transition"):
        st.transition("commit")
    with pytest.raises(SleepError, match="before atomic consolidation commit"):
        st3 = begun()
        for ph in ("knowledge_seeding", "imitation", "retention_validation", "commit"):
            st3.transition(ph)
        st3.transition("candidate")


def _to_commit(st):
    st.transition("knowledge_seeding")
    st.reserve_rng("knowledge", 0, 3)
    st.transition("imitation")
    st.reserve_rng("imitation", 0, 2)
    st.transition("retention_validation")
    st.transition("commit")


def test_commit_activates_receiver_reclaims_sender_and_chains_the_audit_hash():
    sc = schedule()
    st = begun()
    _to_commit(st)
    with pytest.raises(SleepError, match="no published candidate"):
        st.commit_consolidation()
    st.record_committed_candidate("cand-1", H(4))
    st.record_committed_candidate("cand-1", H(4))                            # same receipt again: fine
    with pytest.raises(SleepError, match="changed during retry"):
        st.record_committed_candidate("cand-2", H(5))
    st.commit_consolidation()
    st.commit_consolidation()                                                # idempotent
    assert st.tiers[1].slots[0].active and st.tiers[1].slots[0].generation == 1 and st.cycle == 1 and not st.due
    assert st.tiers[0].last_update_clock == 2
    with pytest.raises(SleepError, match="cannot be rolled back"):
        st.rollback()
    st.transition("candidate")
    done = st.finish_candidate()
    assert done.id == 1 and st.phase == "wake" and st.pending is None and st.completed_count == 1
    assert st.completed_chain_hash != S.ZERO_HASH
    first_hash = st.completed_chain_hash
    # second boundary of the fast tier lands in the mid tier's second slot; at clock 4 the mid tier is due as well
    st.advance_clock(sc, 4)
    assert st.due == [(4, 0), (4, 1)]
    t2 = st.begin(0, "teacher", H(1), "student", H(2), H(3))
    assert (t2.id, t2.receiver, t2.receiver_slot, t2.sender_slots_to_reset) == (2, 1, 1, [])
    _to_commit(st)
    st.record_committed_candidate("cand-2", H(5))
    st.commit_consolidation()
    st.transition("candidate")
    st.finish_candidate()
    t3 = st.begin(1, "teacher", H(1), "student", H(2), H(3))                # the mid tier sends both active reserves on
    assert t3.sender_slots_to_reset == [0, 1] and (t3.receiver, t3.receiver_slot) == (2, 0)
    _to_commit(st)
    st.record_committed_candidate("cand-3", H(6))
    st.commit_consolidation()
    assert [s.active for s in st.tiers[1].slots] == [False, False] and [s.generation for s in st.tiers[1].slots] == [2, 2]
    assert st.tiers[2].slots[0].active
    st.transition("candidate")
    st.finish_candidate()
    assert st.completed_count == 3 and st.completed_chain_hash != first_hash
    # the checkpoint form round-trips and re-validates; tampering is caught
    data = json.loads(json.dumps(st.to_json()))
    again = S.SleepState.from_json(data)
    assert again.to_json() == st.to_json()
    bad = copy.deepcopy(data)
    bad["completed_transactions"][1]["id"] = 1
    with pytest.raises(SleepError, match="alias attempt ids"):
        S.SleepState.from_json(bad)
    bad = copy.deepcopy(data)
    bad["completed_transactions"][0]["knowledge_rng"]["count"] = 99
    with pytest.raises(SleepError, match="exceeds its persisted stream counter"):
        S.SleepState.from_json(bad)
    bad = copy.deepcopy(data)
    bad["completed_transactions"][2]["terminal"] = True
    with pytest.raises(SleepError, match="topology"):
        S.SleepState.from_json(bad)
    bad = copy.deepcopy(data)
    bad["unknown"] = 1
    with pytest.raises(SleepError, match="missing or unknown"):
        S.SleepState.from_json(bad)


def test_rollback_consumes_the_attempt_id_and_a_rejected_terminal_boundary_retries_first():
    sc = schedule()
    st = begun()
    t = st.rollback()
    assert t.id == 1 and st.cycle == 1 and st.phase == "wake" and not st.due and st.tiers[0].last_boundary_clock == 2
    assert st.tiers[0].last_update_clock == 0                                # nothing was consolidated
    st.advance_clock(sc, 4)
    assert st.begin(0, "t", H(1), "s", H(2), H(3)).id == 2                  # the id of the rejected attempt is never reused
    st.rollback()
    st.begin(1, "t", H(1), "s", H(2), H(3))
    st.rollback()
    st.advance_clock(sc, 6)
    st.begin(0, "t", H(1), "s", H(2), H(3))
    st.rollback()
    st.advance_clock(sc, 8)
    assert st.due == [(8, 0), (8, 1), (8, 2)]
    for sender in (0, 1):
        st.begin(sender, "t", H(1), "s", H(2), H(3))
        st.rollback()
    st.begin(2, "t", H(1), "s", H(2), H(3))
    assert st.pending.terminal and st.pending.receiver == 2
    st.rollback()                                                            # terminal consolidation rejected
    assert st.tiers[2].last_update_clock < st.tiers[2].last_boundary_clock
    st.advance_clock(sc, 10)
    assert st.due == [] and st.tiers[0].last_boundary_clock == 10           # transfers held back until the terminal retry
    st.advance_clock(sc, 12)
    assert st.due == []
    st.advance_clock(sc, 14)
    st.advance_clock(sc, 16)
    assert st.due[0] == (16, 2) and [s for _, s in st.due] == [2, 0, 1]     # the terminal tier goes first now
    st.begin(2, "t", H(1), "s", H(2), H(3))
    st.rollback()
    assert st.due == [] and st.tiers[0].last_boundary_clock == 16           # rejected again: the queue behind it is shelved


class Backend:
    def __init__(self, retain=True, fail_at=None):
        self.calls, self.retain, self.fail_at, self.restored = [], retain, fail_at, 0

    def _step(self, name):
        self.calls.append(name)
        if self.fail_at == name:
            raise RuntimeError(f"{name} exploded")

    def knowledge_rng_count(self):
        return 7

    def imitation_rng_count(self):
        return 3

    def compute_prospective_update(self, txn):
        self._step("prospective")

    def stage_student(self, txn):
        self._step("stage")

    def knowledge_seed(self, txn):
        assert txn.knowledge_rng.count == 7
        self._step("seed")

    def learn_to_imitate(self, txn):
        assert txn.imitation_rng.count == 3
        self._step("imitate")

    def retention_passes(self, txn):
        self._step("retention")
        return self.retain

    def commit(self, txn):
        self._step("commit")
        return f"candidate-{txn.id}", H(7)

    def restore_teacher(self, txn):
        self.restored += 1


class Journal:
    def __init__(self, fail_after=None):
        self.states, self.metrics, self.fail_after = [], [], fail_after

    def persist(self, state):
        if self.fail_after is not None and len(self.states) >= self.fail_after:
            raise OSError("disk full")
        self.states.append(json.dumps(state.to_json(), sort_keys=True))

    def metric(self, kind, fields):
        self.metrics.append((kind, fields))


def test_consolidation_driver_commits_rejects_recovers_and_resumes():
    st, be, jr = begun(), Backend(), Journal()
    assert S.run_consolidation(st, be, jr) is True
    assert be.calls == ["prospective", "stage", "seed", "imitate", "retention", "commit"]
    assert st.phase == "commit" and st.pending.committed and st.rng_counters == [10, 0] and st.pending.candidate_checkpoint == "candidate-1"
    assert S.run_consolidation(st, be, jr) is True and be.calls.count("commit") == 1           # re-entry after the commit does nothing
    # rejected by retention: teacher restored, metadata rolled back, id consumed
    st, be = begun(), Backend(retain=False)
    assert S.run_consolidation(st, be, Journal()) is False
    assert be.restored == 1 and st.phase == "wake" and st.pending is None and st.cycle == 1 and "commit" not in be.calls
    # a backend error before the commit does the same and re-raises
    st, be = begun(), Backend(fail_at="imitate")
    with pytest.raises(RuntimeError, match="imitate exploded"):
        S.run_consolidation(st, be, Journal())
    assert be.restored == 1 and st.phase == "wake" and st.cycle == 1
    # a journal that fails while persisting the ROLLBACK leaves the caller's transaction pending (retryable)
    st, be = begun(), Backend(retain=False)
    with pytest.raises(OSError, match="disk full"):
        S.run_consolidation(st, be, Journal(fail_after=6))
    assert be.restored == 1 and st.pending is not None and st.phase == "retention_validation"
    # resume from a checkpointed sub-phase: only the remaining steps run, with the recorded receipts
    st, be, jr = begun(), Backend(fail_at=None), Journal()
    st.transition("knowledge_seeding")
    st.reserve_rng("knowledge", 0, 7)
    resumed = S.SleepState.from_json(json.loads(json.dumps(st.to_json())))
    assert S.run_consolidation(resumed, be, jr) is True
    assert be.calls == ["seed", "imitate", "retention", "commit"] and resumed.rng_counters == [10, 0]
    # a persistence failure AFTER the in-memory commit must not roll back
    st, be = begun(), Backend()
    with pytest.raises(SleepError, match="without rolling back"):
        S.run_consolidation(st, be, Journal(fail_after=7))
    assert be.restored == 0 and st.pending.committed


class DreamBackend:
    def __init__(self, n=6, mutate_in=None):
        self.fingerprint, self.sealed, self.n, self.mutate_in, self.calls, self.policy = H("a"), H("a"), n, mutate_in, [], {}
        self.dreams = [S.GeneratedDream(f"d{i}", H(i % 10), [1.0, float(i) - 2.0, 0.5], diversity_key=(i * 7919) % 101) for i in range(n)]

    def _touch(self, name):
        self.calls.append(name)
        if self.mutate_in == name:
            self.fingerprint = H("b")

    def verify_committed_candidate(self, txn):
        assert txn.candidate_hash == H(7)

    def shared_checkpoint_hash(self):
        return self.fingerprint

    def generate_from_wake_contexts(self, txn, count, random_extra_expert):
        self._touch("generate")
        assert count == self.n and random_extra_expert and txn.dream_generation_rng.count == self.n
        return H("c"), list(self.dreams)

    def load_generated_dreams(self, txn, manifest):
        assert manifest == H("c")
        return list(self.dreams)

    def reference_gradient(self, txn, reference_set_hash):
        self._touch("reference")
        return [1.0, 1.0, 0.0]

    def isolated_lora_trial(self, txn, dream, rank, alpha):
        self._touch(f"trial-{dream.id}")
        assert any(c == dream.id for c, _ in txn.dream_trial_rngs)
        return S.DreamTrial(dream.id, H("d"), H("e"), 0.25 if dream.id != "d3" else -0.1)

    def restem_update(self, txn, accepted, iterations):
        self._touch("policy")
        return self.policy.setdefault(txn.id, H("f"))

    def restore_shared_candidate(self, txn):
        self.calls.append("restore")
        self.fingerprint = self.sealed


def _committed():
    st = begun()
    assert S.run_consolidation(st, Backend(), Journal())
    return st


def test_dreaming_driver_selects_trials_and_guards_the_shared_candidate():
    cfg = S.DreamingConfig(candidate_count=6, retain_top=2, retain_random=1, lora_rank=4, lora_alpha=8, trial_evaluator_hash=H("e"))
    st, be, jr = _committed(), DreamBackend(), Journal()
    accepted = S.run_dreaming(st, cfg, be, jr)
    t = st.pending
    assert st.phase == "candidate" and t.generated_manifest == H("c") and t.dream_shared_checkpoint_hash == H("a")
    assert len(t.dream_selected) == 3 and {"d3", "d4"} <= set(t.dream_selected)       # the two best cosines, plus one by diversity key
    assert {x.candidate_id for x in accepted} == set(t.dream_selected) - {"d3"} and t.dream_policy_receipt == H("f")
    kinds = [k for k, _ in jr.metrics]
    assert kinds == ["dream_selection"] + ["dream_trial"] * 3
    from summa_b200.train import metrics as M
    for kind, fields in jr.metrics:                                            # the driver's events fit the journal schema
        M.validate_event(kind, fields)
    done = st.finish_candidate()
    assert done.dream_policy_receipt == H("f") and st.to_json()["artifact_manifests"] == [H("c")]
    S.SleepState.from_json(json.loads(json.dumps(st.to_json())))
    # a trial that changes the shared candidate is detected, the candidate restored, the run fails
    st, be = _committed(), DreamBackend(mutate_in="trial-d4")
    with pytest.raises(SleepError, match="mutated the shared checkpoint"):
        S.run_dreaming(st, cfg, be, Journal())
    assert be.calls[-1] == "restore" and be.fingerprint == H("a") and st.phase == "dream_trials"
    # ... and the run resumes from the persisted sub-phase without repeating finished trials
    be.mutate_in = None
    finished = [c for c in be.calls if c.startswith("trial-") and c != "trial-d4"]
    S.run_dreaming(st, cfg, be, Journal())
    assert st.phase == "candidate" and sorted(x.candidate_id for x in st.pending.dream_trials) == sorted(st.pending.dream_selected)
    assert all(be.calls.count(c) == 1 for c in finished) and be.calls.count("trial-d4") == 2
    # a frozen evaluator other than the configured one is refused
    st = _committed()
    with pytest.raises(SleepError, match="evaluator other than the frozen"):
        S.run_dreaming(st, S.DreamingConfig(candidate_count=6, retain_top=2, retain_random=1, trial_evaluator_hash=H(9)), DreamBackend(), Journal())
    with pytest.raises(SleepError, match="retain at least one"):
        S.DreamingConfig(candidate_count=4, retain_top=0, retain_random=0).validate()
    with pytest.raises(SleepError, match="unsupported dream selector"):
        S.DreamingConfig(selector_version="magic").validate()


def test_scalar_helpers():
    assert S.normalized_levenshtein_reward([1, 2, 3], [1, 2, 3], 0) == 1.0
    assert S.normalized_levenshtein_reward([1, 2, 3, 4], [1, 2, 9, 4], 2) == 0.75
    assert S.normalized_levenshtein_reward([1, 2, 3, 4], [9, 9, 9, 9], 2) == 0.0 and S.normalized_levenshtein_reward([], [], 0) == 1.0
    assert S.blended_imitation_reward(True, 0.5, 0.25) == pytest.approx(0.625)
    with pytest.raises(SleepError):
        S.blended_imitation_reward(True, 1.5, 0.5)
    assert S.gradient_cosine([1, 0], [1, 0]) == pytest.approx(1.0) and S.gradient_cosine([1, 0], [0, 1]) == 0.0
    assert S.gradient_cosine([0, 0], [1, 1]) == 0.0
    with pytest.raises(SleepError, match="non-finite"):
        S.gradient_cosine([float("nan")], [1.0])
    cands = [("a", 0.9, 5), ("b", 0.9, 1), ("c", 0.1, 0), ("d", 0.5, 9)]
    assert S.select_dreams(cands, 1, 1) == ["a", "c"] and S.select_dreams(list(reversed(cands)), 1, 1) == ["a", "c"]
    with pytest.raises(SleepError, match="exceeds candidate count"):
        S.select_dreams(cands, 3, 2)
    with pytest.raises(SleepError, match="unique"):
        S.select_dreams([("a", 1.0, 0), ("a", 0.5, 1)], 1, 0)
    adv = S.group_relative_advantages([1.0, 2.0, 3.0], 1e-6)
    assert sum(adv) == pytest.approx(0.0) and adv[2] == pytest.approx(-adv[0]) and S.group_relative_advantages([2.0, 2.0], 0.5) == [0.0, 0.0]
