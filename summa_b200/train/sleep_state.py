"""Durable sleep lifecycle: the schedule of parameter-memory tiers, the checkpointed state machine of one
consolidation boundary (reserve-slot masks and generations, the due queue, RNG receipts, the audit chain of
completed transactions) and the two drivers that walk a tensor backend through consolidation and dreaming.

Semantics follow the reference's metadata layer (`summa-train/src/sleep.rs:47-300` schedule and state,
`:955-996,1553-1830` clock / begin / transition / RNG receipts, `:1960-2250` commit / finish / rollback,
`:2369-2420,2551-2760` backend contracts, `:2732-3010` dreaming, `:3177-3283` consolidation,
`:3286-3450` scalar helpers); the code is this package's own: plain dataclasses, strict JSON decoding, and one
rule for failure atomicity: every mutating method works on a copy of the state and installs it only when the
whole method succeeded, so a refused call can never leave a half-applied transaction behind.

`train/sleep.py` keeps the tensor-side pieces (tier optimizer bank, gradient partition) and the compact
file-backed driver the built-in handlers use; this module is the full state machine that a checkpoint carries."""
from __future__ import annotations

import copy
import hashlib
import json
import math
from dataclasses import asdict, dataclass, field, fields
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

from .sleep import SleepError, levenshtein

MAX_MEMORY_TIERS = 16
MAX_RESERVE_SLOTS_PER_TIER = 4096
MAX_TOTAL_RESERVE_SLOTS = 16384
MAX_SLEEP_RNG_STREAMS = 1024
MAX_TIER_ID_BYTES = 128
MAX_LOCATION_BYTES = 16 * 1024
MAX_CANDIDATE_ID_BYTES = 1024
MAX_GRADIENT_DIMENSIONS = 4096
COMPLETED_TAIL = 64
U64_MAX = (1 << 64) - 1
ZERO_HASH = "sha256:" + "0" * 64

PHASES = ("wake", "prospective_update", "knowledge_seeding", "imitation", "retention_validation", "commit",
          "dream_generation", "dream_ranking", "dream_trials", "dream_policy_update", "candidate")
_NEXT = {"prospective_update": ("knowledge_seeding",), "knowledge_seeding": ("imitation",), "imitation": ("retention_validation",),
         "retention_validation": ("commit",), "commit": ("dream_generation", "candidate"), "dream_generation": ("dream_ranking",),
         "dream_ranking": ("dream_trials",), "dream_trials": ("dream_policy_update",), "dream_policy_update": ("candidate",)}
_AFTER_COMMIT = {"dream_generation", "dream_ranking", "dream_trials", "dream_policy_update", "candidate"}
# RNG receipt kind -> (phase that may reserve it, transaction field, fixed count or None)
_RNG_KINDS = {"knowledge": ("knowledge_seeding", "knowledge_rng", None), "imitation": ("imitation", "imitation_rng", None),
              "dream_generation": ("dream_generation", "dream_generation_rng", None),
              "dream_selection": ("dream_ranking", "dream_selection_rng", 1), "dream_trial": ("dream_trials", None, 1)}


def _need(cond: bool, message: str) -> None:
    if not cond:
        raise SleepError(message)


def check_sha256(value: Any, label: str) -> str:
    _need(isinstance(value, str) and len(value) == 71 and value.startswith("sha256:")
          and all(c in "0123456789abcdef" for c in value[7:]), f"{label} must be `sha256:` + 64 lower-case hex digits")
    return value


def _location(value: Any, label: str) -> str:
    _need(isinstance(value, str) and value.strip() != "" and len(value.encode()) <= MAX_LOCATION_BYTES, f"{label} is empty or too long")
    return value


# ------------------------------------------------------------------------------------------------ schedule
@dataclass
class TierSpec:
    id: str
    update_period: int
    reserve_slots: int


@dataclass
class SleepSchedule:
    """Ordered fast-to-slow tiers; index 0 is the fastest. The last tier is terminal: its boundary distils its
    reserves into its own base instead of transferring to a slower tier."""
    clock: str
    terminal_consolidation: str
    tiers: List[TierSpec]

    @staticmethod
    def from_json(data: Dict[str, Any]) -> "SleepSchedule":
        _need(isinstance(data, dict) and set(data) == {"clock", "terminal_consolidation", "tiers"},
              "sleep schedule needs exactly clock, terminal_consolidation and tiers")
        tiers = []
        for t in data["tiers"]:
            _need(isinstance(t, dict) and set(t) == {"id", "update_period", "reserve_slots"},
                  "memory tier needs exactly id, update_period and reserve_slots")
            tiers.append(TierSpec(t["id"], t["update_period"], t["reserve_slots"]))
        s = SleepSchedule(data["clock"], data["terminal_consolidation"], tiers)
        s.validate()
        return s

    def to_json(self) -> Dict[str, Any]:
        return asdict(self)

    def validate(self) -> None:
        _need(self.clock in ("optimizer_steps", "model_tokens"), f"unknown update clock `{self.clock}`")
        _need(self.terminal_consolidation == "distill_into_base_v1", f"unknown terminal consolidation `{self.terminal_consolidation}`")
        _need(2 <= len(self.tiers) <= MAX_MEMORY_TIERS, f"sleep requires 2..={MAX_MEMORY_TIERS} memory tiers")
        seen, total = set(), 0
        for i, t in enumerate(self.tiers):
            _need(isinstance(t.id, str) and t.id.strip() != "" and len(t.id.encode()) <= MAX_TIER_ID_BYTES,
                  f"memory tier {i} id must contain 1..={MAX_TIER_ID_BYTES} bytes")
            _need(t.id not in seen, f"duplicate memory tier id `{t.id}`")
            seen.add(t.id)
            _need(isinstance(t.update_period, int) and 0 < t.update_period <= U64_MAX, f"memory tier `{t.id}` update_period must be positive")
            _need(isinstance(t.reserve_slots, int) and 1 <= t.reserve_slots <= MAX_RESERVE_SLOTS_PER_TIER,
                  f"memory tier `{t.id}` reserve_slots must be in 1..={MAX_RESERVE_SLOTS_PER_TIER}")
            total += t.reserve_slots
            _need(total <= MAX_TOTAL_RESERVE_SLOTS, f"sleep schedule exceeds the {MAX_TOTAL_RESERVE_SLOTS}-slot total reserve limit")
            if i:
                fast = self.tiers[i - 1]
                _need(t.update_period > fast.update_period, f"memory tier `{t.id}` must update less often than `{fast.id}`")
                _need(t.update_period % fast.update_period == 0,
                      f"memory tier `{t.id}` period {t.update_period} must be divisible by faster tier `{fast.id}` period {fast.update_period}")
                transfers = t.update_period // fast.update_period
                _need(t.reserve_slots >= transfers,
                      f"memory tier `{t.id}` needs at least {transfers} reserve slots to receive every `{fast.id}` boundary before reclamation")

    def due_senders(self, clock: int) -> List[int]:
        """Sender indexes due at this clock, fastest first (the terminal tier runs last)."""
        return [] if clock == 0 else [i for i, t in enumerate(self.tiers) if clock % t.update_period == 0]


# ------------------------------------------------------------------------------------------------ records
@dataclass
class RngReservation:
    stream: int
    start: int
    count: int

    def end(self) -> int:
        return self.start + self.count


@dataclass
class DreamTrial:
    candidate_id: str
    adapter_hash: str
    evaluator_hash: str
    independent_task_improvement: float


@dataclass
class GeneratedDream:
    id: str
    artifact_hash: str
    gradient: List[float]
    diversity_key: int


@dataclass
class Transaction:
    """Identity and mutation plan of one consolidation boundary, plus the receipts each sub-phase leaves."""
    id: int
    trigger_clock: int
    sender: int
    receiver: int
    receiver_slot: int
    terminal: bool
    sender_slots_to_reset: List[int]
    teacher_checkpoint: str
    teacher_hash: str
    student_checkpoint: str
    student_hash: str
    prospective_update_hash: str
    candidate_checkpoint: Optional[str] = None
    candidate_hash: Optional[str] = None
    knowledge_rng: Optional[RngReservation] = None
    imitation_rng: Optional[RngReservation] = None
    dream_generation_rng: Optional[RngReservation] = None
    dream_selection_rng: Optional[RngReservation] = None
    dream_trial_rngs: List[Tuple[str, RngReservation]] = field(default_factory=list)
    tensor_transaction_generation: Optional[str] = None
    tensor_transaction_manifest_hash: Optional[str] = None
    generated_manifest: Optional[str] = None
    dream_shared_checkpoint_hash: Optional[str] = None
    dream_selected: List[str] = field(default_factory=list)
    dream_trials: List[DreamTrial] = field(default_factory=list)
    dream_policy_receipt: Optional[str] = None
    committed: bool = False

    def to_json(self) -> Dict[str, Any]:
        d = asdict(self)
        d["dream_trial_rngs"] = [{"candidate_id": cid, "reservation": asdict(r)} for cid, r in self.dream_trial_rngs]
        return d

    @staticmethod
    def from_json(d: Dict[str, Any]) -> "Transaction":
        names = {f.name for f in fields(Transaction)}
        _need(isinstance(d, dict) and set(d) <= names, f"sleep transaction has unknown fields {sorted(set(d) - names) if isinstance(d, dict) else ''}")
        d = dict(d)
        for k in ("knowledge_rng", "imitation_rng", "dream_generation_rng", "dream_selection_rng"):
            if d.get(k) is not None:
                d[k] = RngReservation(**d[k])
        d["dream_trial_rngs"] = [(t["candidate_id"], RngReservation(**t["reservation"])) for t in d.get("dream_trial_rngs", [])]
        d["dream_trials"] = [DreamTrial(**t) for t in d.get("dream_trials", [])]
        try:
            return Transaction(**d)
        except TypeError as e:
            raise SleepError(f"sleep transaction is incomplete: {e}")

    def reservations(self) -> List[RngReservation]:
        out = [r for r in (self.knowledge_rng, self.imitation_rng, self.dream_generation_rng, self.dream_selection_rng) if r]
        return out + [r for _, r in self.dream_trial_rngs]


@dataclass
class SlotState:
    active: bool = False
    generation: int = 0           # raised on activation AND on reclamation: stale optimizer state cannot alias a slot


@dataclass
class TierState:
    id: str
    last_update_clock: int = 0
    last_boundary_clock: int = 0
    slots: List[SlotState] = field(default_factory=list)


def _atomic(method):
    """The method runs against a deep copy; its changes are installed only if it returns."""
    def wrapper(self, *args, **kwargs):
        trial = copy.deepcopy(self)
        out = method(trial, *args, **kwargs)
        self.__dict__.update(trial.__dict__)
        return out
    wrapper.__name__, wrapper.__doc__ = method.__name__, method.__doc__
    return wrapper


# ------------------------------------------------------------------------------------------------ state
class SleepState:
    def __init__(self, schedule: SleepSchedule, rng_streams: int = 1):
        schedule.validate()
        _need(1 <= rng_streams <= MAX_SLEEP_RNG_STREAMS, f"sleep requires 1..={MAX_SLEEP_RNG_STREAMS} RNG streams")
        self.cycle = 0                 # highest attempt id handed out; commits AND roll-backs consume one
        self.clock = 0
        self.phase = "wake"
        self.tiers = [TierState(t.id, 0, 0, [SlotState() for _ in range(t.reserve_slots)]) for t in schedule.tiers]
        self.due: List[Tuple[int, int]] = []          # (trigger clock, sender), in execution order
        self.pending: Optional[Transaction] = None
        self.rng_counters = [0] * rng_streams
        self.evaluator_hashes: List[str] = []
        self.completed: List[Transaction] = []        # bounded tail; `completed_chain_hash` commits to the whole history
        self.completed_count = 0
        self.completed_chain_hash = ZERO_HASH

    # ---- serialisation
    def to_json(self) -> Dict[str, Any]:
        return {"cycle": self.cycle, "clock": self.clock, "phase": self.phase, "tiers": [asdict(t) for t in self.tiers],
                "due_senders": [s for _, s in self.due], "due_clocks": [c for c, _ in self.due],
                "pending": self.pending.to_json() if self.pending else None, "rng_counters": list(self.rng_counters),
                "evaluator_hashes": list(self.evaluator_hashes), "artifact_manifests": self.artifact_manifests(),
                "completed_transactions": [t.to_json() for t in self.completed], "completed_count": self.completed_count,
                "completed_chain_hash": self.completed_chain_hash}

    @staticmethod
    def from_json(d: Dict[str, Any]) -> "SleepState":
        keys = {"cycle", "clock", "phase", "tiers", "due_senders", "due_clocks", "pending", "rng_counters", "evaluator_hashes",
                "artifact_manifests", "completed_transactions", "completed_count", "completed_chain_hash"}
        _need(isinstance(d, dict) and set(d) == keys, "sleep state has missing or unknown fields")
        s = SleepState.__new__(SleepState)
        s.cycle, s.clock, s.phase = d["cycle"], d["clock"], d["phase"]
        s.tiers = [TierState(t["id"], t["last_update_clock"], t["last_boundary_clock"], [SlotState(**x) for x in t["slots"]]) for t in d["tiers"]]
        _need(len(d["due_senders"]) == len(d["due_clocks"]), "sleep due queue is not paired")
        s.due = list(zip(d["due_clocks"], d["due_senders"]))
        s.pending = Transaction.from_json(d["pending"]) if d["pending"] is not None else None
        s.rng_counters = list(d["rng_counters"])
        s.evaluator_hashes = list(d["evaluator_hashes"])
        s.completed = [Transaction.from_json(t) for t in d["completed_transactions"]]
        s.completed_count, s.completed_chain_hash = d["completed_count"], d["completed_chain_hash"]
        s.validate_resume()
        _need(d["artifact_manifests"] == s.artifact_manifests(), "sleep artifact-manifest index differs from its transactions")
        return s

    def artifact_manifests(self) -> List[str]:
        txns = self.completed + ([self.pending] if self.pending else [])
        return sorted({t.generated_manifest for t in txns if t.generated_manifest})

    # ---- invariants a checkpoint must satisfy on its own (topology against the model is checked elsewhere)
    def validate_resume(self) -> None:
        _need(2 <= len(self.tiers) <= MAX_MEMORY_TIERS, f"sleep checkpoint must contain 2..={MAX_MEMORY_TIERS} tiers")
        _need(self.phase in PHASES, f"unknown sleep phase `{self.phase}`")
        _need(1 <= len(self.rng_counters) <= MAX_SLEEP_RNG_STREAMS and all(isinstance(c, int) and 0 <= c <= U64_MAX for c in self.rng_counters),
              "sleep RNG counters are out of range")
        for t in self.tiers:
            _need(1 <= len(t.slots) <= MAX_RESERVE_SLOTS_PER_TIER, f"memory tier `{t.id}` has an invalid slot count")
            _need(t.last_update_clock <= t.last_boundary_clock <= self.clock, f"memory tier `{t.id}` clocks are ahead of the sleep clock")
        senders = [s for _, s in self.due]
        _need(len(set(senders)) == len(senders), "sleep due queue holds several unconsumed boundaries for one sender")
        _need(all(0 <= s < len(self.tiers) and 0 < c <= self.clock for c, s in self.due), "sleep due queue entry is out of range")
        _need((self.pending is None) == (self.phase == "wake"), "sleep phase and pending transaction disagree")
        if self.pending is not None:
            p = self.pending
            self._check_topology(p)
            _need(p.id == self.cycle + 1 or (p.committed and p.id == self.cycle), "pending sleep transaction id does not follow the cycle counter")
            _need(bool(self.due) and self.due[0] == (p.trigger_clock, p.sender) or p.committed, "pending sleep transaction is not first in the due queue")
            _need(p.committed or self.phase not in _AFTER_COMMIT, f"sleep phase `{self.phase}` requires a committed transaction")
            self._check_receipts(p)
        _need(len(self.completed) <= COMPLETED_TAIL and self.completed_count >= len(self.completed), "sleep completed-transaction tail is out of bounds")
        ids = [t.id for t in self.completed]
        _need(ids == sorted(set(ids)) and all(i <= self.cycle for i in ids), "completed sleep receipts can alias attempt ids")
        for t in self.completed:
            _need(t.committed, "completed sleep transaction is not committed")
            self._check_topology(t)
            self._check_receipts(t, completed=True)
        check_sha256(self.completed_chain_hash, "sleep audit-chain hash")
        for h in self.evaluator_hashes:
            check_sha256(h, "sleep evaluator hash")

    def _check_topology(self, t: Transaction) -> None:
        n = len(self.tiers)
        _need(0 <= t.sender < n and 0 <= t.receiver < n, "sleep transaction tier is out of range")
        _need(t.terminal == (t.sender + 1 == n) and ((t.terminal and t.receiver == t.sender) or (not t.terminal and t.receiver == t.sender + 1)),
              "sleep transaction has an invalid sender/receiver topology")
        _need(t.terminal or 0 <= t.receiver_slot < len(self.tiers[t.receiver].slots), "sleep transaction receiver slot is out of range")
        r = t.sender_slots_to_reset
        _need(all(0 <= s < len(self.tiers[t.sender].slots) for s in r) and r == sorted(set(r)), "sleep transaction has an invalid sender reset plan")
        _need(t.trigger_clock > 0, "sleep transaction has no trigger clock")
        _location(t.teacher_checkpoint, "teacher checkpoint")
        _location(t.student_checkpoint, "student checkpoint")
        for h, label in ((t.teacher_hash, "teacher hash"), (t.student_hash, "student hash"), (t.prospective_update_hash, "prospective-update hash")):
            check_sha256(h, label)

    def _check_receipts(self, t: Transaction, completed: bool = False) -> None:
        rs = sorted(t.reservations(), key=lambda r: (r.stream, r.start))
        for r in rs:
            _need(r.count > 0 and 0 <= r.stream < len(self.rng_counters) and r.end() <= self.rng_counters[r.stream],
                  "sleep RNG reservation exceeds its persisted stream counter")
        _need(all(a.stream != b.stream or a.end() <= b.start for a, b in zip(rs, rs[1:])), "sleep transaction has overlapping RNG receipts")
        _need((t.tensor_transaction_generation is None) == (t.tensor_transaction_manifest_hash is None), "sleep tensor transaction identity is incomplete")
        if t.tensor_transaction_generation is not None:
            _check_generation(t.tensor_transaction_generation, t.tensor_transaction_manifest_hash)
        _need((t.candidate_checkpoint is None) == (t.candidate_hash is None), "sleep transaction has a partial candidate identity")
        if t.candidate_hash is not None:
            check_sha256(t.candidate_hash, "candidate hash")
        sel, trials, trial_rngs = set(t.dream_selected), {x.candidate_id for x in t.dream_trials}, {c for c, _ in t.dream_trial_rngs}
        _need(len(sel) == len(t.dream_selected) and len(trials) == len(t.dream_trials) and len(trial_rngs) == len(t.dream_trial_rngs)
              and all(i.strip() and len(i.encode()) <= MAX_CANDIDATE_ID_BYTES for i in sel), "sleep transaction has invalid dream candidate ids")
        _need(trials <= sel and trial_rngs <= sel, "dream trial evidence is not for a selected candidate")
        for x in t.dream_trials:
            _need(math.isfinite(x.independent_task_improvement), "dream trial has invalid evidence")
            check_sha256(x.adapter_hash, "dream adapter hash")
            check_sha256(x.evaluator_hash, "dream evaluator hash")
        if not completed:
            return
        _need(t.candidate_hash is not None and t.knowledge_rng is not None and t.imitation_rng is not None,
              "completed sleep transaction lacks its candidate or RNG receipts")
        if t.generated_manifest is None:
            _need(not (t.dream_generation_rng or t.dream_selection_rng or t.dream_trial_rngs or t.dream_shared_checkpoint_hash or t.dream_selected
                       or t.dream_trials or t.dream_policy_receipt), "completed transaction contains partial dreaming evidence")
        else:
            check_sha256(t.generated_manifest, "completed dream manifest")
            check_sha256(t.dream_shared_checkpoint_hash, "completed dream shared-checkpoint hash")
            check_sha256(t.dream_policy_receipt, "completed dream policy receipt")
            _need(t.dream_generation_rng is not None and t.dream_selection_rng is not None and sel and len(sel) <= t.dream_generation_rng.count
                  and trials == sel and trial_rngs == sel, "completed dream selection / trial evidence is incomplete")

    # ---- wake clock
    @_atomic
    def advance_clock(self, schedule: SleepSchedule, clock: int) -> None:
        """Moves the wake clock and queues the boundaries it reached. One advance may reach at most one boundary
        per tier (a tier's gradient accumulator can supply one update); the host splits longer advances."""
        schedule.validate()
        _need(self.pending is None, "cannot advance wake clock during consolidation")
        _need(not self.due, "cannot advance sleep clock before finishing every due sender")
        _need(len(schedule.tiers) == len(self.tiers) and all(c.id == s.id and c.reserve_slots == len(s.slots) for c, s in zip(schedule.tiers, self.tiers)),
              "sleep schedule topology differs from checkpoint state")
        _need(isinstance(clock, int) and self.clock <= clock <= U64_MAX, "sleep clock cannot move backwards")
        due = []
        for sender, spec in enumerate(schedule.tiers):
            first = (self.tiers[sender].last_boundary_clock // spec.update_period + 1) * spec.update_period
            if first <= clock:
                _need(first + spec.update_period > clock,
                      f"sleep clock advance from {self.clock} to {clock} crosses multiple `{spec.id}` boundaries ({first} and "
                      f"{first + spec.update_period}); the host must split the advance at a boundary")
                due.append((first, sender))
        due.sort()
        # A rejected terminal boundary left its reserves full: it retries first at its next boundary, and until then
        # ordinary transfers are held back (their logical boundaries pass, their accumulated gradients stay)
        last = len(self.tiers) - 1
        if self.tiers[last].last_update_clock < self.tiers[last].last_boundary_clock:
            retry = [e for e in due if e[1] == last]
            if retry:
                due = retry + [e for e in due if e[1] != last]
            else:
                for trigger, sender in due:
                    self.tiers[sender].last_boundary_clock = trigger
                due = []
        self.clock, self.due = clock, due

    def next_due(self) -> Optional[Tuple[int, int]]:
        """(sender, trigger clock) of the next boundary to consolidate."""
        return (self.due[0][1], self.due[0][0]) if self.due else None

    def next_transaction_id(self) -> int:
        _need(self.cycle < U64_MAX, "sleep consolidation transaction id overflows")
        return self.cycle + 1

    # ---- transaction life cycle
    @_atomic
    def begin(self, sender: int, teacher_checkpoint: str, teacher_hash: str, student_checkpoint: str, student_hash: str,
              prospective_update_hash: str) -> Transaction:
        _need(self.pending is None and self.phase == "wake", "a consolidation transaction is already active")
        _need(isinstance(sender, int) and 0 <= sender < len(self.tiers), f"sender tier {sender} is out of range")
        nxt = self.next_due()
        _need(nxt is not None, f"sender tier {sender} has no paired due boundary at sleep clock {self.clock}")
        _need(nxt[0] == sender, f"sender tier {sender} is not next at sleep clock {self.clock}")
        terminal = sender + 1 == len(self.tiers)
        receiver = sender if terminal else sender + 1
        slot = 0
        if not terminal:
            free = [i for i, s in enumerate(self.tiers[receiver].slots) if not s.active]
            _need(bool(free), f"memory tier `{self.tiers[receiver].id}` has exhausted its reserve slots")
            slot = free[0]
        txn = Transaction(self.next_transaction_id(), nxt[1], sender, receiver, slot, terminal,
                          [i for i, s in enumerate(self.tiers[sender].slots) if s.active],
                          _location(teacher_checkpoint, "teacher checkpoint"), check_sha256(teacher_hash, "teacher hash"),
                          _location(student_checkpoint, "student checkpoint"), check_sha256(student_hash, "student hash"),
                          check_sha256(prospective_update_hash, "prospective-update hash"))
        self.phase, self.pending = "prospective_update", txn
        return copy.deepcopy(txn)

    @_atomic
    def transition(self, nxt: str) -> None:
        _need(nxt in _NEXT.get(self.phase, ()), f"invalid sleep transition {self.phase} -> {nxt}")
        _need(self.pending is not None, "sleep transition has no transaction")
        _need(nxt not in _AFTER_COMMIT or self.pending.committed, f"sleep cannot enter {nxt} before atomic consolidation commit")
        self.phase = nxt

    @_atomic
    def reserve_rng(self, kind: str, stream: int, count: int = 1, candidate_id: Optional[str] = None) -> RngReservation:
        """Reserves `count` draws of a persisted stream for one sub-phase and records the receipt in the transaction.
        Asking again with the same arguments returns the recorded receipt (a resumed sub-phase replays the same
        draws); different arguments are refused."""
        _need(kind in _RNG_KINDS, f"unknown sleep RNG receipt `{kind}`")
        phase, attr, fixed = _RNG_KINDS[kind]
        _need(self.pending is not None and self.phase == phase, f"{kind} RNG reservation requires the {phase} phase")
        count = fixed if fixed is not None else count
        txn = self.pending
        if kind == "dream_trial":
            _need(isinstance(candidate_id, str) and candidate_id.strip() != "" and len(candidate_id.encode()) <= MAX_CANDIDATE_ID_BYTES,
                  "dream candidate id is empty or too long")
            _need(candidate_id in txn.dream_selected, "dream-trial RNG reservation is not for a selected candidate")
            old = next((r for c, r in txn.dream_trial_rngs if c == candidate_id), None)
        else:
            old = getattr(txn, attr)
        if old is not None:
            _need(old.stream == stream and old.count == count, f"{kind} RNG reservation differs on retry")
            return copy.copy(old)
        _need(isinstance(count, int) and count > 0, "sleep RNG reservation count must be positive")
        _need(isinstance(stream, int) and 0 <= stream < len(self.rng_counters), f"sleep RNG stream {stream} does not exist")
        r = RngReservation(stream, self.rng_counters[stream], count)
        _need(r.end() <= U64_MAX, "sleep RNG counter overflow")
        self.rng_counters[stream] = r.end()
        if kind == "dream_trial":
            txn.dream_trial_rngs.append((candidate_id, r))
        else:
            setattr(txn, attr, r)
        return copy.copy(r)

    @_atomic
    def record_committed_candidate(self, checkpoint: str, digest: str) -> None:
        """Binds the exact weights a tensor commit published, before any mask or clock changes; repeating the same
        receipt is fine, another candidate is refused."""
        _need(self.phase == "commit" and self.pending is not None, "candidate identity can be recorded only in commit phase")
        _location(checkpoint, "candidate checkpoint")
        check_sha256(digest, "published candidate hash")
        t = self.pending
        if t.candidate_checkpoint is None and t.candidate_hash is None:
            t.candidate_checkpoint, t.candidate_hash = checkpoint, digest
        else:
            _need((t.candidate_checkpoint, t.candidate_hash) == (checkpoint, digest), "committed candidate identity changed during retry")

    @_atomic
    def commit_consolidation(self) -> None:
        """Activates the receiver slot, reclaims the sender's active slots (every touched slot's generation rises),
        consumes the boundary. Idempotent; every check runs before the first change."""
        _need(self.phase == "commit" and self.pending is not None, "consolidation can commit only in commit phase")
        t = self.pending
        if t.committed:
            return
        self._check_topology(t)
        _need(t.candidate_checkpoint is not None and t.candidate_checkpoint.strip() != "", "consolidation has no published candidate checkpoint")
        check_sha256(t.candidate_hash, "published candidate hash")
        _need(bool(self.due) and self.due[0] == (t.trigger_clock, t.sender), f"committed boundary ({t.trigger_clock}, {t.sender}) is not first in the due queue")
        sender = self.tiers[t.sender]
        _need(t.sender_slots_to_reset == [i for i, s in enumerate(sender.slots) if s.active],
              "consolidation sender reset plan does not contain the exact active-slot set")
        if not t.terminal:
            slot = self.tiers[t.receiver].slots[t.receiver_slot]
            _need(not slot.active, "receiver slot is already active")
            _need(slot.generation < U64_MAX, "receiver reserve generation overflows")
        _need(all(sender.slots[i].generation < U64_MAX for i in t.sender_slots_to_reset), "sender reserve generation overflows")
        self.due.pop(0)
        if not t.terminal:
            slot.active, slot.generation = True, slot.generation + 1
        for i in t.sender_slots_to_reset:
            sender.slots[i].active, sender.slots[i].generation = False, sender.slots[i].generation + 1
        sender.last_update_clock = sender.last_boundary_clock = t.trigger_clock
        self.cycle, t.committed = t.id, True

    @_atomic
    def record_tensor_transaction(self, generation: str, manifest_hash: str) -> None:
        _need(self.pending is not None, "no consolidation transaction for tensor snapshot")
        _check_generation(generation, manifest_hash)
        self.pending.tensor_transaction_generation, self.pending.tensor_transaction_manifest_hash = generation, manifest_hash

    @_atomic
    def record_generated_manifest(self, manifest: str) -> None:
        check_sha256(manifest, "generated manifest")
        _need(self.phase == "dream_generation" and self.pending is not None, "generated manifest can be recorded only during dream generation")
        _need(self.pending.generated_manifest in (None, manifest), "generated manifest identity changed during retry")
        self.pending.generated_manifest = manifest
        _need(len(self.artifact_manifests()) <= COMPLETED_TAIL + 1, "sleep artifact-manifest tail exceeds its bounded transaction history")

    @_atomic
    def record_dream_evidence(self, shared_checkpoint_hash: Optional[str] = None, selected: Optional[Sequence[str]] = None,
                              trial: Optional[DreamTrial] = None, policy_receipt: Optional[str] = None) -> None:
        """The four receipts dreaming leaves, each only in its own sub-phase."""
        _need(self.pending is not None and self.pending.committed, "dream evidence needs a committed transaction")
        t = self.pending
        if shared_checkpoint_hash is not None:
            _need(self.phase == "commit", "the shared-checkpoint hash is recorded when dreaming starts")
            t.dream_shared_checkpoint_hash = check_sha256(shared_checkpoint_hash, "shared-checkpoint hash")
        if selected is not None:
            _need(self.phase == "dream_ranking", "dream selection is recorded during ranking")
            _need(len(selected) > 0 and len(set(selected)) == len(selected), "dreaming requires a non-empty unambiguous selection")
            t.dream_selected = list(selected)
        if trial is not None:
            _need(self.phase == "dream_trials" and trial.candidate_id in t.dream_selected, "dream trial is not for a selected candidate")
            _need(all(x.candidate_id != trial.candidate_id for x in t.dream_trials), f"dream trial `{trial.candidate_id}` is already recorded")
            t.dream_trials.append(trial)
        if policy_receipt is not None:
            _need(self.phase == "dream_policy_update", "the policy receipt is recorded during the policy update")
            t.dream_policy_receipt = check_sha256(policy_receipt, "dream policy receipt")

    @_atomic
    def finish_candidate(self) -> Transaction:
        """Retires the committed transaction into the audit chain and returns to wake."""
        _need(self.phase == "candidate", "sleep cycle is not a candidate")
        _need(self.pending is not None and self.pending.committed, "sleep candidate is not atomically committed")
        t = self.pending
        _need(self.completed_count < U64_MAX, "sleep completed-transaction count overflow")
        body = json.dumps(t.to_json(), sort_keys=True, separators=(",", ":")).encode()
        h = hashlib.sha256()
        h.update(b"summa-sleep-audit-chain-v1\0")
        h.update(self.completed_chain_hash.encode())
        h.update(len(body).to_bytes(8, "little"))
        h.update(body)
        self.completed = (self.completed + [t])[-COMPLETED_TAIL:]
        self.completed_chain_hash, self.completed_count = "sha256:" + h.hexdigest(), self.completed_count + 1
        self.pending, self.phase = None, "wake"
        self.validate_resume()
        return copy.deepcopy(t)

    @_atomic
    def rollback(self) -> Transaction:
        """Metadata half of a rejected boundary (the backend restores the teacher first). The attempt id stays
        consumed; a rejected terminal boundary also shelves the transfers queued behind it."""
        _need(self.pending is not None, "no consolidation transaction")
        t = self.pending
        _need(not t.committed, "a committed consolidation cannot be rolled back")
        _need(0 <= t.sender < len(self.tiers), "rolled-back sender tier is out of range")
        _need(bool(self.due) and self.due[0] == (t.trigger_clock, t.sender), f"rolled-back boundary ({t.trigger_clock}, {t.sender}) is not first in the due queue")
        _need(all(0 <= s < len(self.tiers) for _, s in self.due), "rolled-back boundary has an invalid trailing due queue")
        self.due.pop(0)
        self.tiers[t.sender].last_boundary_clock = t.trigger_clock
        if t.terminal:
            for trigger, sender in self.due:
                self.tiers[sender].last_boundary_clock = trigger
            self.due = []
        self.cycle, self.pending, self.phase = t.id, None, "wake"
        return copy.deepcopy(t)


def _check_generation(generation: Any, manifest_hash: Any) -> None:
    _need(isinstance(generation, str) and generation.startswith("sha256-"), "tensor transaction generation has an unsafe name")
    check_sha256("sha256:" + generation[7:], "tensor transaction generation")
    check_sha256(manifest_hash, "tensor transaction manifest hash")
    _need(manifest_hash[7:] == generation[7:], "tensor transaction generation does not match its manifest hash")


# ------------------------------------------------------------------------------------------------ scalar helpers
def normalized_levenshtein_reward(generated: Sequence[int], teacher: Sequence[int], maximum_distance: int) -> float:
    """1 - distance / max length, and 0 beyond the distance threshold."""
    d = levenshtein(generated, teacher)
    if d > maximum_distance:
        return 0.0
    n = max(len(generated), len(teacher))
    return 1.0 if n == 0 else 1.0 - d / n


def blended_imitation_reward(semantic_equivalent: bool, edit_reward: float, gamma: float) -> float:
    _need(math.isfinite(gamma) and 0.0 <= gamma <= 1.0, "semantic reward weight must be in [0, 1]")
    _need(math.isfinite(edit_reward) and 0.0 <= edit_reward <= 1.0, "edit reward must be in [0, 1]")
    return gamma * float(bool(semantic_equivalent)) + (1.0 - gamma) * edit_reward


def gradient_cosine(candidate: Sequence[float], reference: Sequence[float]) -> float:
    """Cosine between a dream's gradient sketch and the training-only reference gradient; 0 for a zero vector."""
    _need(len(candidate) > 0 and len(candidate) == len(reference), "gradient vectors must have the same positive length")
    _need(all(math.isfinite(x) for x in candidate) and all(math.isfinite(x) for x in reference), "gradient contains non-finite value")
    dot = math.fsum(a * b for a, b in zip(candidate, reference))
    na, nb = math.fsum(a * a for a in candidate), math.fsum(b * b for b in reference)
    return 0.0 if na == 0.0 or nb == 0.0 else dot / (math.sqrt(na) * math.sqrt(nb))


def select_dreams(candidates: Sequence[Tuple[str, float, int]], top: int, random: int) -> List[str]:
    """Candidates are (id, importance, diversity key). Keeps the `top` most important plus the `random` smallest
    diversity keys among the rest; ids break ties, so the answer does not depend on input order. Sorted ids."""
    _need(top >= 0 and random >= 0 and top + random <= len(candidates), "dream selection exceeds candidate count")
    _need(all(math.isfinite(c[1]) for c in candidates), "dream importance must be finite")
    ids = [c[0] for c in candidates]
    _need(len(set(ids)) == len(ids) and all(isinstance(i, str) and i.strip() and len(i.encode()) <= MAX_CANDIDATE_ID_BYTES for i in ids),
          "dream candidates must have unique, non-empty ids")
    chosen = {c[0] for c in sorted(candidates, key=lambda c: (-c[1], c[0]))[:top]}
    rest = sorted((c for c in candidates if c[0] not in chosen), key=lambda c: (c[2], c[0]))
    chosen.update(c[0] for c in rest[:random])
    return sorted(chosen)


def group_relative_advantages(rewards: Sequence[float], epsilon: float) -> List[float]:
    _need(len(rewards) > 0, "reward group is empty")
    _need(math.isfinite(epsilon) and epsilon > 0, "epsilon must be positive")
    _need(all(math.isfinite(r) for r in rewards), "reward is non-finite")
    mean = sum(rewards) / len(rewards)
    scale = max(math.sqrt(sum((r - mean) ** 2 for r in rewards) / len(rewards)), epsilon)
    return [(r - mean) / scale for r in rewards]


# ------------------------------------------------------------------------------------------------ dreaming config
@dataclass
class DreamingConfig:
    candidate_count: int = 64
    retain_top: int = 8
    retain_random: int = 2
    lora_rank: int = 64
    lora_alpha: int = 128
    restem_iterations: int = 1
    selector_version: str = "gradient-cosine-v1"
    reference_set_hash: str = ZERO_HASH
    trial_evaluator_hash: str = ZERO_HASH

    MAX_CANDIDATES = 1024
    MAX_LORA_RANK = 1024
    MAX_LORA_ALPHA = 65536
    MAX_RESTEM_ITERATIONS = 128

    def validate(self) -> None:
        _need(0 < self.candidate_count <= self.MAX_CANDIDATES, f"dream candidate count must be in 1..={self.MAX_CANDIDATES}")
        kept = self.retain_top + self.retain_random
        _need(self.retain_top >= 0 and self.retain_random >= 0 and 0 < kept <= self.candidate_count,
              "dream selection must retain at least one candidate and no more than were generated")
        _need(0 < self.lora_rank <= self.MAX_LORA_RANK and 0 < self.lora_alpha <= self.MAX_LORA_ALPHA, "dream LoRA geometry is out of range")
        _need(0 < self.restem_iterations <= self.MAX_RESTEM_ITERATIONS, "policy iterations are out of range")
        _need(self.selector_version == "gradient-cosine-v1", f"unsupported dream selector `{self.selector_version}`")
        check_sha256(self.reference_set_hash, "dream reference-set hash")
        check_sha256(self.trial_evaluator_hash, "dream trial-evaluator hash")


def validate_generated_dreams(dreams: Sequence[GeneratedDream], expected: int) -> None:
    _need(len(dreams) == expected, f"dream generator returned {len(dreams)} candidates; expected {expected}")
    ids, dims = set(), None
    for d in dreams:
        _need(isinstance(d.id, str) and d.id.strip() != "" and len(d.id.encode()) <= MAX_CANDIDATE_ID_BYTES
              and 0 < len(d.gradient) <= MAX_GRADIENT_DIMENSIONS and all(math.isfinite(g) for g in d.gradient),
              "generated dream has incomplete identity or gradient")
        _need(dims in (None, len(d.gradient)), "generated dreams use inconsistent gradient dimensions")
        dims = len(d.gradient)
        check_sha256(d.artifact_hash, "generated dream artifact hash")
        _need(d.id not in ids, f"duplicate dream candidate `{d.id}`")
        ids.add(d.id)


# ------------------------------------------------------------------------------------------------ drivers
class NullProgress:
    def persist(self, state: SleepState) -> None:
        pass

    def metric(self, kind: str, fields_: Dict[str, Any]) -> None:
        pass


def run_consolidation(state: SleepState, backend, progress=None) -> bool:
    """Walks a begun transaction from its checkpointed sub-phase to the commit. `backend` supplies
    `knowledge_rng_count()`, `imitation_rng_count()`, `compute_prospective_update(txn)`, `stage_student(txn)`,
    `knowledge_seed(txn)`, `learn_to_imitate(txn)`, `retention_passes(txn) -> bool`, `commit(txn) -> (checkpoint,
    sha256)` (idempotent per transaction id) and `restore_teacher(txn)`. `progress.persist(state)` makes each step
    durable. Returns True when committed (the transaction stays pending for dreaming / `finish_candidate`), False
    when retention rejected it: the teacher is restored first, then the rolled-back metadata is persisted, and only
    then does the caller's state change. An error before the commit does the same and re-raises; an error after the
    in-memory commit never rolls back (the caller retries persistence)."""
    progress = progress or NullProgress()
    state.validate_resume()
    progress.persist(state)
    _need(state.pending is not None, "no consolidation transaction")
    txn = copy.deepcopy(state.pending)

    def walk() -> bool:
        while True:
            ph = state.phase
            if ph == "prospective_update":
                backend.compute_prospective_update(txn)
                backend.stage_student(txn)
                state.transition("knowledge_seeding")
            elif ph == "knowledge_seeding":
                state.reserve_rng("knowledge", 0, backend.knowledge_rng_count())
                progress.persist(state)
                backend.knowledge_seed(copy.deepcopy(state.pending))
                state.transition("imitation")
            elif ph == "imitation":
                state.reserve_rng("imitation", 0, backend.imitation_rng_count())
                progress.persist(state)
                backend.learn_to_imitate(copy.deepcopy(state.pending))
                state.transition("retention_validation")
            elif ph == "retention_validation":
                if not backend.retention_passes(txn):
                    return False
                state.transition("commit")
            elif ph == "commit":
                if not state.pending.committed:
                    checkpoint, digest = backend.commit(txn)
                    state.record_committed_candidate(checkpoint, digest)
                    state.commit_consolidation()
                    progress.persist(state)
                return True
            elif ph in _AFTER_COMMIT:
                return True
            else:
                raise SleepError("consolidation transaction is in wake phase")
            progress.persist(state)

    def undo() -> None:
        backend.restore_teacher(txn)
        restored = copy.deepcopy(state)
        restored.rollback()
        progress.persist(restored)              # a failed persist leaves the caller's state pending
        state.__dict__.update(restored.__dict__)

    try:
        ok = walk()
    except Exception as error:
        if state.pending is not None and state.pending.committed:
            raise SleepError(f"consolidation committed in memory but durable state publication failed; retry persistence "
                             f"without rolling back: {error}") from error
        try:
            undo()
        except Exception as second:
            raise SleepError(f"consolidation failed: {error}; restoring the teacher also failed: {second}") from error
        raise
    if not ok:
        undo()
    return ok


def run_dreaming(state: SleepState, config: DreamingConfig, backend, progress=None) -> List[DreamTrial]:
    """Dreaming over the committed candidate: generate from the model's own wake contexts, rank by gradient cosine
    against a reference set, keep the top and a random quota, run one isolated low-rank trial per kept dream, feed
    the improving ones to the policy update. Every backend call sits between two checks that the shared candidate's
    fingerprint is still the one recorded when dreaming started; a mismatch restores the candidate and fails.
    Resumes from any sub-phase; returns the trials that improved the independent task.

    `backend`: `verify_committed_candidate(txn)`, `shared_checkpoint_hash()`, `generate_from_wake_contexts(txn, n,
    random_extra_expert) -> (manifest, dreams)`, `load_generated_dreams(txn, manifest)`, `reference_gradient(txn,
    reference_set_hash)`, `isolated_lora_trial(txn, dream, rank, alpha) -> DreamTrial`, `restem_update(txn, accepted,
    iterations) -> receipt` (idempotent per transaction), `restore_shared_candidate(txn)`."""
    progress = progress or NullProgress()
    config.validate()
    state.validate_resume()
    _need(state.pending is not None and state.pending.committed, "dreaming requires committed transaction metadata")
    try:
        backend.verify_committed_candidate(state.pending)
    except Exception as first:
        backend.restore_shared_candidate(state.pending)
        backend.verify_committed_candidate(state.pending)
        raise SleepError(f"dreaming did not start from the committed candidate ({first}); immutable candidate was restored")

    def fingerprint_is(txn, expected: str, what: str) -> None:
        try:
            seen = check_sha256(backend.shared_checkpoint_hash(), "observed shared-checkpoint hash")
            problem = None if seen == expected else f"mutated the shared checkpoint from {expected} to {seen}"
        except Exception as e:
            problem = f"left the shared checkpoint unverifiable ({e})"
        if problem is None:
            return
        backend.restore_shared_candidate(txn)
        _need(check_sha256(backend.shared_checkpoint_hash(), "restored shared-checkpoint hash") == expected,
              f"{what} did not preserve the shared checkpoint and restoration recovered a different candidate")
        raise SleepError(f"{what} {problem}; immutable candidate was restored")

    def guarded(txn, what: str, action: Callable[[], Any]) -> Any:
        expected = txn.dream_shared_checkpoint_hash
        _need(expected is not None, "dream transaction has no shared checkpoint hash")
        fingerprint_is(txn, expected, f"before {what}")
        try:
            out, err = action(), None
        except Exception as e:
            out, err = None, e
        fingerprint_is(txn, expected, what)          # checked whether or not the action succeeded
        if err is not None:
            raise SleepError(f"{what} failed: {err}") from err
        return out

    while True:
        txn = copy.deepcopy(state.pending)
        ph = state.phase
        if ph == "commit":
            try:
                seen = check_sha256(backend.shared_checkpoint_hash(), "shared-checkpoint hash")
            except Exception as e:
                backend.restore_shared_candidate(txn)
                backend.verify_committed_candidate(txn)
                raise SleepError(f"fingerprinting the committed candidate failed ({e}); immutable candidate was restored")
            state.record_dream_evidence(shared_checkpoint_hash=seen)
            state.transition("dream_generation")
        elif ph == "dream_generation":
            state.reserve_rng("dream_generation", 0, config.candidate_count)
            progress.persist(state)
            txn = copy.deepcopy(state.pending)
            manifest, dreams = guarded(txn, "dream generation", lambda: backend.generate_from_wake_contexts(txn, config.candidate_count, True))
            validate_generated_dreams(dreams, config.candidate_count)
            state.record_generated_manifest(manifest)
            state.transition("dream_ranking")
        elif ph == "dream_ranking":
            receipt = state.reserve_rng("dream_selection", 0)
            progress.persist(state)
            txn = copy.deepcopy(state.pending)
            dreams = guarded(txn, "loading generated dreams", lambda: backend.load_generated_dreams(txn, txn.generated_manifest))
            validate_generated_dreams(dreams, config.candidate_count)
            ref = guarded(txn, "dream reference-gradient evaluation", lambda: backend.reference_gradient(txn, config.reference_set_hash))
            _need(0 < len(ref) <= MAX_GRADIENT_DIMENSIONS and all(math.isfinite(x) for x in ref),
                  "dream reference gradient is empty, non-finite, or exceeds the operational dimension limit")
            # the diversity keys are re-keyed by the selection receipt, so the random quota depends on persisted state only
            salt = (receipt.start * 0x9E3779B97F4A7C15) & U64_MAX
            salt = ((salt << 17) | (salt >> 47)) & U64_MAX
            scores = [(d.id, gradient_cosine(d.gradient, ref), d.diversity_key ^ salt) for d in dreams]
            selected = select_dreams(scores, config.retain_top, config.retain_random)
            progress.metric("dream_selection", {
                "transaction_id": f"sleep-{txn.id}", "selector_version": config.selector_version, "reference_set_hash": config.reference_set_hash,
                "candidates_generated": config.candidate_count, "selected_by_alignment": config.retain_top, "selected_random": config.retain_random,
                "random_quota": config.retain_random, "gradient_cosine_mean": sum(s[1] for s in scores) / len(scores),
                "gradient_cosine_max": max(s[1] for s in scores), "selected_manifest_hash": txn.generated_manifest})
            state.record_dream_evidence(selected=selected)
            state.transition("dream_trials")
        elif ph == "dream_trials":
            dreams = guarded(txn, "loading dreams for isolated trials", lambda: backend.load_generated_dreams(txn, txn.generated_manifest))
            validate_generated_dreams(dreams, config.candidate_count)
            done = {t.candidate_id for t in txn.dream_trials}
            for cid in txn.dream_selected:
                if cid in done:
                    continue
                dream = next((d for d in dreams if d.id == cid), None)
                _need(dream is not None, f"selected dream `{cid}` disappeared")
                state.reserve_rng("dream_trial", 0, candidate_id=cid)
                progress.persist(state)
                cur = copy.deepcopy(state.pending)
                trial = guarded(cur, f"isolated dream trial `{cid}`", lambda: backend.isolated_lora_trial(cur, dream, config.lora_rank, config.lora_alpha))
                _need(trial.candidate_id == cid and math.isfinite(trial.independent_task_improvement), f"dream trial `{cid}` returned incomplete or invalid evidence")
                check_sha256(trial.adapter_hash, "dream trial adapter hash")
                _need(check_sha256(trial.evaluator_hash, "dream trial evaluator hash") == config.trial_evaluator_hash,
                      f"dream trial `{cid}` used an evaluator other than the frozen configured artifact")
                progress.metric("dream_trial", {
                    "transaction_id": f"sleep-{txn.id}", "candidate_hash": dream.artifact_hash, "adapter_hash": trial.adapter_hash,
                    "evaluator_hash": trial.evaluator_hash, "lora_rank": config.lora_rank, "lora_alpha": float(config.lora_alpha),
                    "independent_task_delta": trial.independent_task_improvement, "reward": trial.independent_task_improvement,
                    "elapsed_seconds": 0.0, "accepted": trial.independent_task_improvement > 0.0, "isolated": True, "shared_checkpoint_unchanged": True})
                state.record_dream_evidence(trial=trial)
                progress.persist(state)
            state.transition("dream_policy_update")
        elif ph == "dream_policy_update":
            if txn.dream_policy_receipt is None:
                accepted = [t for t in txn.dream_trials if t.independent_task_improvement > 0.0]
                receipt = guarded(txn, "policy update", lambda: backend.restem_update(txn, accepted, config.restem_iterations))
                state.record_dream_evidence(policy_receipt=receipt)
                progress.persist(state)
            state.transition("candidate")
        elif ph == "candidate":
            fingerprint_is(txn, txn.dream_shared_checkpoint_hash, "finalizing the dream candidate")
            return [t for t in txn.dream_trials if t.independent_task_improvement > 0.0]
        else:
            raise SleepError(f"dreaming cannot resume from sub-phase {ph}")
        progress.persist(state)
