"""In-model sleep: tier schedule, consolidation transactions, imitation reward, tier optimizers.

Memory tiers run fast -> slow with periods that divide one another. At every boundary the due
sender tiers are consolidated into their receivers by a `ConsolidationTxn`, a persisted state
machine (`sleep.rs:78-158,178-298`):

    ProspectiveUpdate -> KnowledgeSeeding -> Imitation -> RetentionValidation -> Commit
        [-> DreamGeneration -> DreamRanking -> DreamTrials -> DreamPolicyUpdate] -> Candidate

The transaction state is written after every transition, so a crash resumes at the phase that
was running; a failed or rejected phase restores the teacher weights and rolls the transaction
back (`sleep.rs:2369-2386,3184-3284`). The tensor work of each phase is supplied by the caller
as a handler (`phase -> callable(ctx) -> PhaseResult`), which keeps this module independent of
the model code (the forward-KL seeding and GRPO-style imitation losses live in `posttrain`).
The wake-side pieces are
`partition_gradients` (wake scope + one scope per tier; dormant slots must carry no gradient)
and `TierOptimizerBank` (one AdamW state and clock per tier, `tier_optimizer.rs:164-419`).
"""
from __future__ import annotations

import json
import os
from dataclasses import asdict, dataclass, field
from typing import Callable, Dict, List, Optional, Sequence

import torch

PHASES = ["prospective_update", "knowledge_seeding", "imitation", "retention_validation", "commit",
          "dream_generation", "dream_ranking", "dream_trials", "dream_policy_update", "candidate"]
DREAM_PHASES = PHASES[5:9]


class SleepError(RuntimeError):
    pass


# ---------------------------------------------------------------------------- schedule
class TierSchedule:
    """`periods[i]` = wake steps between consolidations of tier i into tier i+1; every period
    must divide the next one (fast -> slow)."""

    def __init__(self, periods: Sequence[int]):
        if not periods:
            raise SleepError("at least one tier period is required")
        for i, p in enumerate(periods):
            if p <= 0:
                raise SleepError("tier periods must be positive")
            if i and p % periods[i - 1]:
                raise SleepError(f"tier period {p} is not a multiple of the faster period {periods[i - 1]}")
        self.periods = list(periods)

    def due_senders(self, clock: int) -> List[int]:
        """Tiers whose boundary falls on wake step `clock` (> 0), fastest first."""
        if clock <= 0:
            return []
        return [i for i, p in enumerate(self.periods) if clock % p == 0]

    def next_boundary(self, clock: int) -> int:
        p = self.periods[0]
        return (clock // p + 1) * p


# ---------------------------------------------------------------------------- transaction
@dataclass
class PhaseResult:
    accepted: bool = True
    metrics: Dict[str, float] = field(default_factory=dict)
    reason: str = ""


@dataclass
class TxnState:
    clock: int
    sender: int
    receiver: int
    dreaming: bool
    phase_index: int = 0
    status: str = "running"            # running | committed | rolled_back
    history: List[dict] = field(default_factory=list)


class ConsolidationTxn:
    def __init__(self, path: str, clock: int, sender: int, receiver: int, dreaming: bool = False):
        self.path = path
        if os.path.exists(path):
            with open(path) as f:
                self.state = TxnState(**json.load(f))
            if (self.state.clock, self.state.sender, self.state.receiver) != (clock, sender, receiver):
                raise SleepError("persisted consolidation belongs to another boundary")
        else:
            self.state = TxnState(clock, sender, receiver, dreaming)
            self._persist()

    def _persist(self):
        tmp = self.path + ".tmp"
        with open(tmp, "w") as f:
            json.dump(asdict(self.state), f, sort_keys=True)
            f.flush()
            os.fsync(f.fileno())
        os.replace(tmp, self.path)

    def phases(self) -> List[str]:
        return [p for p in PHASES if self.state.dreaming or p not in DREAM_PHASES]

    @property
    def current_phase(self) -> Optional[str]:
        ph = self.phases()
        return ph[self.state.phase_index] if self.state.status == "running" and self.state.phase_index < len(ph) else None

    def run(self, handlers: Dict[str, Callable[[dict], PhaseResult]], restore_teacher: Callable[[], None],
            ctx: Optional[dict] = None) -> TxnState:
        """Drives the remaining phases. A phase without a handler is a no-op that accepts."""
        ctx = ctx if ctx is not None else {}
        while self.current_phase is not None:
            name = self.current_phase
            try:
                res = handlers.get(name, lambda c: PhaseResult())(ctx)
            except Exception as e:                                   # failure = rejection with the error as reason
                res = PhaseResult(False, {}, f"{type(e).__name__}: {e}")
            self.state.history.append({"phase": name, "accepted": res.accepted, "metrics": res.metrics,
                                       "reason": res.reason})
            if not res.accepted:
                restore_teacher()
                self.state.status = "rolled_back"
                self._persist()
                return self.state
            self.state.phase_index += 1
            self._persist()
        self.state.status = "committed"
        self._persist()
        return self.state


class SleepDriver:
    """Periodic boundary driver: at each due boundary runs one transaction per sender tier."""

    def __init__(self, schedule: TierSchedule, state_dir: str, dreaming_from_tier: Optional[int] = None):
        self.schedule, self.state_dir = schedule, state_dir
        self.dreaming_from_tier = dreaming_from_tier
        os.makedirs(state_dir, exist_ok=True)

    def run_boundary(self, clock: int, handlers_for: Callable[[int], Dict[str, Callable]],
                     restore_teacher: Callable[[int], None], only: Optional[Sequence[int]] = None) -> List[TxnState]:
        """`only`: restrict to these sender tiers (the slowest tier has no receiver)."""
        out = []
        for sender in self.schedule.due_senders(clock):
            if only is not None and sender not in only:
                continue
            receiver = sender + 1
            dreaming = self.dreaming_from_tier is not None and sender >= self.dreaming_from_tier
            path = os.path.join(self.state_dir, f"txn-{clock:012d}-tier{sender}.json")
            txn = ConsolidationTxn(path, clock, sender, receiver, dreaming)
            if txn.state.status == "running":
                txn.run(handlers_for(sender), lambda s=sender: restore_teacher(s), {"clock": clock, "sender": sender})
            out.append(txn.state)
        return out


# ---------------------------------------------------------------------------- imitation reward
def levenshtein(a: Sequence, b: Sequence) -> int:
    if len(a) < len(b):
        a, b = b, a
    prev = list(range(len(b) + 1))
    for i, x in enumerate(a, 1):
        cur = [i]
        for j, y in enumerate(b, 1):
            cur.append(min(prev[j] + 1, cur[j - 1] + 1, prev[j - 1] + (x != y)))
        prev = cur
    return prev[-1]


def imitation_reward(student: Sequence[int], teacher: Sequence[int], semantic: float, gamma: float,
                     threshold: float = 0.0) -> float:
    """`gamma * semantic + (1 - gamma) * edit`, edit = 1 - normalised Levenshtein distance over
    token ids, zeroed below `threshold`."""
    if not (0.0 <= gamma <= 1.0):
        raise SleepError("gamma must be in [0, 1]")
    n = max(len(student), len(teacher), 1)
    edit = 1.0 - levenshtein(list(student), list(teacher)) / n
    r = gamma * semantic + (1.0 - gamma) * edit
    return r if r >= threshold else 0.0


# ---------------------------------------------------------------------------- wake side
def tier_of_parameter(name: str) -> Optional[int]:
    """Tier index of a memory-chain parameter (`...memory.tiers.<i>....`), None for wake parameters."""
    parts = name.split(".")
    for i, p in enumerate(parts[:-1]):
        if p == "tiers" and parts[i + 1].isdigit():
            return int(parts[i + 1])
    return None


def partition_gradients(named_params, dormant: Sequence[str] = ()) -> Dict[str, List[str]]:
    """Scopes: "wake" plus "tier<i>". Parameters listed in `dormant` must not carry gradients."""
    scopes: Dict[str, List[str]] = {"wake": []}
    dormant = set(dormant)
    for name, p in named_params:
        g = getattr(p, "grad", None)
        if name in dormant:
            if g is not None and bool(torch.count_nonzero(g)):
                raise SleepError(f"dormant slot `{name}` received a gradient")
            continue
        t = tier_of_parameter(name)
        scopes.setdefault("wake" if t is None else f"tier{t}", []).append(name)
    return scopes


class TierOptimizerBank:
    """One AdamW state per tier, each with its own step clock: a tier's optimizer only advances
    when that tier's accumulated gradient is applied (at its boundary, or directly in the
    `wake_only` ablation)."""

    def __init__(self, named_params, lr: float = 3e-4, betas=(0.9, 0.95), eps: float = 1e-8, weight_decay: float = 0.0):
        self.lr, self.betas, self.eps, self.wd = lr, betas, eps, weight_decay
        self.params: Dict[int, List] = {}
        for name, p in named_params:
            t = tier_of_parameter(name)
            if t is not None and p.requires_grad:
                self.params.setdefault(t, []).append((name, p))
        # "w": fp32 masters (the parameters themselves may be bf16 compute copies); "count": micro-batches
        # accumulated since the last apply
        self.state = {t: {"step": 0, "count": 0, "m": [torch.zeros_like(p, dtype=torch.float32) for _, p in ps],
                          "v": [torch.zeros_like(p, dtype=torch.float32) for _, p in ps],
                          "acc": [torch.zeros_like(p, dtype=torch.float32) for _, p in ps],
                          "w": [p.detach().float().clone() for _, p in ps]}
                      for t, ps in self.params.items()}

    def accumulate(self, tier: int, reduce=None, staged: bool = False) -> None:
        """Adds the current `.grad` of the tier's parameters into its accumulator and clears them.
        `reduce(tensor)`: in-place mean over data-parallel ranks. `staged`: the gradients wait in a window buffer until
        `commit_window(coefficient)` scales them by the optimizer window's clip coefficient (the trainer's route: one
        global norm covers the wake and the tier scopes)."""
        seen = False
        if staged and "win" not in self.state[tier]:
            self.state[tier]["win"] = [torch.zeros_like(a) for a in self.state[tier]["acc"]]
        into = self.state[tier]["win"] if staged else self.state[tier]["acc"]
        for (name, p), acc in zip(self.params.get(tier, []), into):
            if p.grad is not None:
                g = p.grad.float()
                if reduce is not None:
                    reduce(g)
                acc.add_(g)
                p.grad = None
                seen = True
        if seen:
            self.state[tier]["count"] += 1

    def window_sumsq(self) -> Optional[torch.Tensor]:
        """Squared L2 norm of every tier's staged window gradients (a device scalar), None when nothing is staged."""
        parts = [w.pow(2).sum() for st in self.state.values() for w in st.get("win", [])]
        return torch.stack(parts).sum() if parts else None

    @torch.no_grad()
    def commit_window(self, coefficient: float = 1.0) -> None:
        """Moves the staged window into the accumulators, scaled by the window's clip coefficient."""
        for st in self.state.values():
            for acc, win in zip(st["acc"], st.get("win", [])):
                acc.add_(win, alpha=float(coefficient))
                win.zero_()

    def resync(self, tier: Optional[int] = None) -> None:
        """Masters := current parameter values (after weights were loaded or restored)."""
        with torch.no_grad():
            for t in ([tier] if tier is not None else list(self.params)):
                for (name, p), w in zip(self.params[t], self.state[t]["w"]):
                    w.copy_(p.detach().float())

    def state_tensors(self) -> Dict[str, torch.Tensor]:
        out = {}
        for t, st in self.state.items():
            out[f"tier{t}.clock"] = torch.tensor([st["step"], st["count"]], dtype=torch.int64)
            for i, (name, _) in enumerate(self.params[t]):
                for k in ("m", "v", "acc", "w"):
                    out[f"tier{t}.{k}.{name}"] = st[k][i]
        return out

    def load_state_tensors(self, tensors: Dict[str, torch.Tensor]) -> None:
        with torch.no_grad():
            for t, st in self.state.items():
                c = tensors.get(f"tier{t}.clock")
                if c is not None:
                    st["step"], st["count"] = int(c[0]), int(c[1])
                for i, (name, p) in enumerate(self.params[t]):
                    for k in ("m", "v", "acc", "w"):
                        v = tensors.get(f"tier{t}.{k}.{name}")
                        if v is not None:
                            st[k][i].copy_(v.to(st[k][i].device))
                    if f"tier{t}.w.{name}" in tensors:
                        p.copy_(st["w"][i].to(p.dtype))

    @torch.no_grad()
    def apply(self, tier: int, scale: Optional[float] = None) -> int:
        """One AdamW step of the tier from its accumulator (`scale` defaults to 1 / accumulated
        micro-batches: the tier sees the mean gradient of its period)."""
        st = self.state[tier]
        if scale is None:
            scale = 1.0 / max(st["count"], 1)
        st["step"] += 1
        st["count"] = 0
        b1, b2 = self.betas
        bc1, bc2 = 1 - b1 ** st["step"], 1 - b2 ** st["step"]
        for (name, p), m, v, acc, w in zip(self.params[tier], st["m"], st["v"], st["acc"], st["w"]):
            g = acc * scale
            m.mul_(b1).add_(g, alpha=1 - b1)
            v.mul_(b2).addcmul_(g, g, value=1 - b2)
            upd = (m / bc1) / ((v / bc2).sqrt() + self.eps)
            w.mul_(1 - self.lr * self.wd).add_(upd, alpha=-self.lr)
            p.copy_(w.to(p.dtype))
            acc.zero_()
        return st["step"]

    def clocks(self) -> Dict[int, int]:
        return {t: s["step"] for t, s in self.state.items()}

    # ---- durable form (`summa-train/src/tier_optimizer.rs:422-446,1609-1760`): byte-identical snapshots of identical
    # state, and one immutable content-addressed bundle per tier that a checkpoint's optimizer scopes refer to
    def _tier_tensors(self, tier: int) -> Dict[str, torch.Tensor]:
        prefix = f"tier{tier}."
        return {k: v for k, v in self.state_tensors().items() if k.startswith(prefix)}

    def _hyper(self) -> Dict[str, float]:
        return {"learning_rate": self.lr, "beta_1": self.betas[0], "beta_2": self.betas[1], "epsilon": self.eps, "weight_decay": self.wd}

    def snapshot_bytes(self, tier: Optional[int] = None) -> bytes:
        from .checkpoint import pack_tensors
        tensors = self.state_tensors() if tier is None else self._tier_tensors(tier)
        return pack_tensors(tensors, self._hyper(), {"kind": "tier-optimizer-bank" if tier is None else f"tier-optimizer:{tier}"})

    def restore_bytes(self, data: bytes, tier: Optional[int] = None) -> None:
        """All or nothing: names, shapes and hyper-parameters are checked before the first tensor moves."""
        from .checkpoint import unpack_tensors
        tensors, scalars, meta = unpack_tensors(data)
        want = self.state_tensors() if tier is None else self._tier_tensors(tier)
        if meta.get("kind") != ("tier-optimizer-bank" if tier is None else f"tier-optimizer:{tier}"):
            raise ValueError(f"tier optimizer snapshot is a `{meta.get('kind')}`")
        if set(tensors) != set(want) or any(tuple(tensors[k].shape) != tuple(want[k].shape) or tensors[k].dtype != want[k].dtype for k in want):
            raise ValueError("tier optimizer snapshot belongs to another parameter topology")
        if any(abs(float(scalars.get(k, float("nan"))) - float(v)) > 0 for k, v in self._hyper().items()):
            raise ValueError("tier optimizer snapshot was taken under other optimizer settings")
        self.load_state_tensors(tensors)

    def publish_checkpoint_scopes(self, root: str, identity=None) -> Dict[str, object]:
        """Seals the optimizer and pending-gradient state of every tier under `root/generations/sha256-<hash>.bpk` (write
        once, content addressed; no clock advances) and returns the scope view a checkpoint stores."""
        import hashlib
        identity = identity or (lambda name: int.from_bytes(hashlib.sha256(name.encode()).digest()[:8], "big"))
        gens = os.path.join(root, "generations")
        os.makedirs(gens, exist_ok=True)
        tiers = []
        for t in sorted(self.params):
            body = self.snapshot_bytes(t)
            digest = hashlib.sha256(body).hexdigest()
            path = os.path.join(gens, f"sha256-{digest}.bpk")
            if not os.path.exists(path):
                tmp = f"{path}.{os.getpid()}.partial"
                with open(tmp, "wb") as f:
                    f.write(body)
                    f.flush()
                    os.fsync(f.fileno())
                os.replace(tmp, path)
            st = self.state[t]
            tiers.append({"tier": t, "parameter_ids": sorted(identity(n) for n, _ in self.params[t]), "update_clock": st["step"],
                          "accumulated_micro_steps": st["count"],
                          "artifact": {"path": os.path.join("generations", f"sha256-{digest}.bpk"), "sha256": "sha256:" + digest, "bytes": len(body)}})
        return {"tiers": tiers}

    def restore_scopes(self, root: str, scopes: Dict[str, object], identity=None) -> None:
        """Restores every tier from the bundles a checkpoint's scopes name; a failure leaves the bank as it was."""
        import hashlib
        identity = identity or (lambda name: int.from_bytes(hashlib.sha256(name.encode()).digest()[:8], "big"))
        before = self.snapshot_bytes()
        try:
            tiers = scopes["tiers"]
            if [t["tier"] for t in tiers] != sorted(self.params):
                raise ValueError("checkpoint optimizer scopes differ from tier optimizer bank")
            for sc in tiers:
                t = sc["tier"]
                if sc["parameter_ids"] != sorted(identity(n) for n, _ in self.params[t]):
                    raise ValueError("checkpoint optimizer tier topology differs from bank")
                art = sc.get("artifact")
                if art is None:
                    if sc["update_clock"] or sc["accumulated_micro_steps"]:
                        raise ValueError("checkpoint tier has clocks but no durable optimizer artifact")
                    continue
                rel = art["path"]
                if os.path.isabs(rel) or ".." in rel.split(os.sep):
                    raise ValueError("tier optimizer artifact path leaves its store")
                with open(os.path.join(root, rel), "rb") as f:
                    body = f.read()
                if len(body) != art["bytes"] or "sha256:" + hashlib.sha256(body).hexdigest() != art["sha256"]:
                    raise ValueError(f"tier optimizer artifact {rel} does not match its recorded identity")
                self.restore_bytes(body, t)
                if self.state[t]["step"] != sc["update_clock"] or self.state[t]["count"] != sc["accumulated_micro_steps"]:
                    raise ValueError("checkpoint optimizer tier clocks differ from immutable bundle")
        except Exception:
            self.restore_bytes(before)
            raise
