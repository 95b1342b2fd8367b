"""Post-training objectives: DPO, forward-KL distillation and GRPO.

Each objective exists twice, as in the reference (`summa-train/src/posttrain.rs:415-518`
DPO, `:657-691` forward KL, `:720-1029` GRPO): a float64 scalar oracle that also returns the
analytic gradients (used by tests and for validating the device path), and a tensor loss
that keeps the autograd graph of the policy/student and validates its inputs with a single
device read. `sequence_log_probs` turns model logits into the per-sequence continuation
log-probabilities the DPO/GRPO losses consume, `ExactAnswerVerifier` is the built-in reward
(`posttrain.rs:4743`), and `PostTrainingExecutor` is the resumable update loop whose
prepared-update records are byte-stable under retry (`posttrain.rs:3028-3340`).
"""
from __future__ import annotations

import hashlib
import json
import math
import os
from dataclasses import asdict, dataclass, field
from typing import Callable, Dict, List, Optional, Sequence

import torch

MAX_LOG_RATIO = 80.0
MAX_EXAMPLES_PER_UPDATE = 65_536
MAX_ROLLOUT_TOKENS = 8 * 1024 * 1024
MAX_ROLLOUTS_PER_PROMPT = 4_096


class PostTrainError(ValueError):
    pass


def _finite(values, what):
    for v in values:
        if not math.isfinite(v):
            raise PostTrainError(f"{what} contain a non-finite value")


def _softplus(x: float) -> float:
    return max(x, 0.0) + math.log1p(math.exp(-abs(x)))


def _sigmoid(x: float) -> float:
    if x >= 0:
        return 1.0 / (1.0 + math.exp(-x))
    e = math.exp(x)
    return e / (1.0 + e)


# ---------------------------------------------------------------------------- DPO
@dataclass
class DpoLoss:
    loss: float
    policy_margin: float
    reference_margin: float
    implicit_reward_margin: float
    preference_correct: bool
    d_policy_chosen: float
    d_policy_rejected: float


def _check_dpo_hparams(beta, label_smoothing):
    if not (math.isfinite(beta) and beta > 0.0):
        raise PostTrainError("DPO beta must be finite and positive")
    if not (math.isfinite(label_smoothing) and 0.0 <= label_smoothing < 0.5):
        raise PostTrainError("DPO label_smoothing must be finite and in [0, 0.5)")


def dpo_loss(policy_chosen: float, policy_rejected: float, reference_chosen: float, reference_rejected: float,
             beta: float, label_smoothing: float = 0.0) -> DpoLoss:
    """`(1-s) softplus(-z) + s softplus(z)` with `z = beta((pi_c-pi_r) - (ref_c-ref_r))`."""
    _finite([policy_chosen, policy_rejected, reference_chosen, reference_rejected], "DPO log probabilities")
    _check_dpo_hparams(beta, label_smoothing)
    pm = policy_chosen - policy_rejected
    rm = reference_chosen - reference_rejected
    z = beta * (pm - rm)
    loss = (1.0 - label_smoothing) * _softplus(-z) + label_smoothing * _softplus(z)
    dz = _sigmoid(z) - (1.0 - label_smoothing)
    out = DpoLoss(loss, pm, rm, z, pm > rm, beta * dz, -beta * dz)
    _finite([out.loss, out.implicit_reward_margin, out.d_policy_chosen], "derived DPO objective values")
    return out


def dpo_loss_tensor(policy_chosen: torch.Tensor, policy_rejected: torch.Tensor, reference_chosen: torch.Tensor,
                    reference_rejected: torch.Tensor, beta: float, label_smoothing: float = 0.0) -> torch.Tensor:
    """Batch-mean DPO loss over `[B]` sequence log-probs; reference scores are detached."""
    n = policy_chosen.shape[0] if policy_chosen.dim() == 1 else -1
    if n <= 0:
        raise PostTrainError("DPO tensor batch is empty")
    for t in (policy_rejected, reference_chosen, reference_rejected):
        if tuple(t.shape) != (n,):
            raise PostTrainError(f"DPO tensor score shapes must all be [{n}]")
    _check_dpo_hparams(beta, label_smoothing)
    z = beta * ((policy_chosen - policy_rejected) - (reference_chosen.detach() - reference_rejected.detach()))
    ls = torch.nn.functional.logsigmoid
    return (-(1.0 - label_smoothing) * ls(z) - label_smoothing * ls(-z)).mean()


def reduce_sequence_log_probs(values: Sequence[float], reduction: str = "sum") -> float:
    if len(values) == 0:
        raise PostTrainError("sequence log probabilities are empty")
    _finite(values, "sequence log probabilities")
    s = float(sum(values))
    if reduction == "sum":
        return s
    if reduction == "mean":
        return s / len(values)
    raise PostTrainError(f"unknown sequence reduction `{reduction}`")


def token_log_probs(logits: torch.Tensor, tokens: torch.Tensor) -> torch.Tensor:
    """log p(tokens[:, t+1] | prefix) for every position, `[B, S-1]`, fp32 statistics."""
    lp = torch.log_softmax(logits[:, :-1].float(), dim=-1)
    return lp.gather(-1, tokens[:, 1:].unsqueeze(-1)).squeeze(-1)


def sequence_log_probs(logits: torch.Tensor, tokens: torch.Tensor, continuation_mask: torch.Tensor,
                       reduction: str = "sum") -> torch.Tensor:
    """Per-sequence log-probability of the continuation tokens. `continuation_mask[b, t]`
    is 1 where `tokens[b, t]` is a continuation token (position 0 can never be one)."""
    tlp = token_log_probs(logits, tokens)
    m = continuation_mask[:, 1:].to(tlp.dtype)
    if bool((m.sum(dim=1) == 0).any()):
        raise PostTrainError("every sequence needs at least one continuation token")
    s = (tlp * m).sum(dim=1)
    return s if reduction == "sum" else s / m.sum(dim=1)


# ---------------------------------------------------------------------------- forward KL
@dataclass
class DistillationLoss:
    loss: float
    mean_forward_kl: float
    teacher_entropy: float
    top1_agreement: float


def _log_softmax_row(row: Sequence[float], temperature: float) -> List[float]:
    scaled = [v / temperature for v in row]
    m = max(scaled)
    lse = m + math.log(sum(math.exp(v - m) for v in scaled))
    return [v - lse for v in scaled]


def forward_kl_distillation(teacher_rows: Sequence[Sequence[float]], student_rows: Sequence[Sequence[float]],
                            temperature: float = 1.0, scale_by_temperature_squared: bool = False) -> DistillationLoss:
    """Mean over rows of `sum_v p_T (log p_T - log p_S)` at `temperature`."""
    if len(teacher_rows) == 0:
        raise PostTrainError("distillation batch is empty")
    if len(teacher_rows) != len(student_rows):
        raise PostTrainError("distillation teacher/student row counts differ")
    if not (math.isfinite(temperature) and temperature > 0.0):
        raise PostTrainError("distillation temperature must be finite and positive")
    total_kl = total_h = 0.0
    agree = 0
    for t, s in zip(teacher_rows, student_rows):
        if len(t) < 2 or len(t) != len(s):
            raise PostTrainError("distillation rows need matching vocabularies of at least two logits")
        _finite(t, "teacher logits")
        _finite(s, "student logits")
        lt, ls_ = _log_softmax_row(t, temperature), _log_softmax_row(s, temperature)
        total_kl += sum(math.exp(a) * (a - b) for a, b in zip(lt, ls_))
        total_h += -sum(math.exp(a) * a for a in lt)
        agree += int(max(range(len(t)), key=lambda i: (t[i], -i)) == max(range(len(s)), key=lambda i: (s[i], -i)))
    n = len(teacher_rows)
    kl = total_kl / n
    loss = kl * temperature * temperature if scale_by_temperature_squared else kl
    return DistillationLoss(loss, kl, total_h / n, agree / n)


def forward_kl_distillation_tensor(teacher_logits: torch.Tensor, student_logits: torch.Tensor, temperature: float = 1.0,
                                   scale_by_temperature_squared: bool = False) -> torch.Tensor:
    """Tensor forward KL over already-selected `[tokens, vocab]` rows; the teacher is detached."""
    if teacher_logits.dim() != 2 or teacher_logits.shape[0] == 0:
        raise PostTrainError("distillation tensor batch is empty")
    if teacher_logits.shape[1] < 2:
        raise PostTrainError("distillation tensor vocabulary must contain at least two logits")
    if teacher_logits.shape != student_logits.shape:
        raise PostTrainError("distillation teacher/student tensor shapes differ")
    if not (math.isfinite(temperature) and temperature > 0.0):
        raise PostTrainError("distillation temperature must be finite and positive")
    lt = torch.log_softmax(teacher_logits.detach().float() / temperature, dim=1)
    ls_ = torch.log_softmax(student_logits.float() / temperature, dim=1)
    kl = (lt.exp() * (lt - ls_)).sum(dim=1).mean()
    return kl * (temperature * temperature) if scale_by_temperature_squared else kl


# ---------------------------------------------------------------------------- GRPO
@dataclass
class GrpoRollout:
    reward: float
    current_token_log_probs: Sequence[float]
    behavior_token_log_probs: Sequence[float]
    reference_token_log_probs: Optional[Sequence[float]] = None


@dataclass
class GrpoLoss:
    loss: float
    mean_reward: float
    reward_stddev: float
    mean_kl: float
    clipped_fraction: float
    advantages: List[float]
    current_log_prob_gradients: List[List[float]]


def _check_grpo_hparams(clip_epsilon, advantage_epsilon, kl_coefficient):
    if not (math.isfinite(clip_epsilon) and 0.0 < clip_epsilon < 1.0):
        raise PostTrainError("GRPO clip_epsilon must be finite and in (0, 1)")
    if not (math.isfinite(advantage_epsilon) and advantage_epsilon > 0.0):
        raise PostTrainError("GRPO advantage_epsilon must be finite and positive")
    if not (math.isfinite(kl_coefficient) and kl_coefficient >= 0.0):
        raise PostTrainError("GRPO kl_coefficient must be finite and non-negative")


def grpo_loss(rollouts: Sequence[GrpoRollout], clip_epsilon: float = 0.2, advantage_epsilon: float = 1e-6,
              kl_coefficient: float = 0.0) -> GrpoLoss:
    """Group-relative policy optimisation for the rollouts of ONE prompt."""
    if len(rollouts) < 2:
        raise PostTrainError("GRPO requires at least two rollouts per prompt")
    _check_grpo_hparams(clip_epsilon, advantage_epsilon, kl_coefficient)
    rewards = [r.reward for r in rollouts]
    _finite(rewards, "GRPO rewards")
    g = len(rollouts)
    mean = sum(rewards) / g
    std = math.sqrt(sum((r - mean) ** 2 for r in rewards) / g)
    den = max(std, advantage_epsilon)
    adv = [(r - mean) / den for r in rewards]
    lo, hi = 1.0 - clip_epsilon, 1.0 + clip_epsilon
    objective = total_kl = 0.0
    clipped = count = 0
    grads: List[List[float]] = []
    for ri, (ro, a) in enumerate(zip(rollouts, adv)):
        n = len(ro.current_token_log_probs)
        if n == 0:
            raise PostTrainError(f"GRPO rollout {ri} has no generated tokens")
        if len(ro.behavior_token_log_probs) != n:
            raise PostTrainError(f"GRPO rollout {ri} current/behavior token counts differ")
        if kl_coefficient > 0.0 and ro.reference_token_log_probs is None:
            raise PostTrainError(f"GRPO rollout {ri} needs reference log-probs for positive KL coefficient")
        if ro.reference_token_log_probs is not None and len(ro.reference_token_log_probs) != n:
            raise PostTrainError(f"GRPO rollout {ri} current/reference token counts differ")
        _finite(ro.current_token_log_probs, "GRPO current log probabilities")
        _finite(ro.behavior_token_log_probs, "GRPO behavior log probabilities")
        scale = 1.0 / g / n
        row = []
        for ti in range(n):
            cur = ro.current_token_log_probs[ti]
            lr = cur - ro.behavior_token_log_probs[ti]
            if not (math.isfinite(lr) and lr <= MAX_LOG_RATIO):
                raise PostTrainError(f"GRPO rollout {ri} token {ti} has an unsafe importance ratio")
            ratio = math.exp(lr)
            cr = min(max(ratio, lo), hi)
            sur = min(ratio * a, cr * a)
            clipped += int(sur == cr * a and ratio != cr)
            count += 1
            kl = dkl = 0.0
            if ro.reference_token_log_probs is not None:
                d = ro.reference_token_log_probs[ti] - cur
                if not (math.isfinite(d) and d <= MAX_LOG_RATIO):
                    raise PostTrainError(f"GRPO rollout {ri} token {ti} has an unsafe KL ratio")
                e = math.exp(d)
                kl, dkl = e - d - 1.0, 1.0 - e
            objective += scale * (sur - kl_coefficient * kl)
            total_kl += scale * kl
            active = (a >= 0.0 and ratio <= hi) or (a < 0.0 and ratio >= lo)
            row.append(scale * (-(ratio * a if active else 0.0) + kl_coefficient * dkl))
        grads.append(row)
    if not (math.isfinite(objective) and math.isfinite(total_kl)):
        raise PostTrainError("GRPO objective overflowed")
    return GrpoLoss(-objective, mean, std, total_kl, clipped / count, adv, grads)


def grpo_loss_tensor(rewards: torch.Tensor, current: torch.Tensor, behavior: torch.Tensor,
                     reference: Optional[torch.Tensor], active_mask: torch.Tensor, clip_epsilon: float = 0.2,
                     advantage_epsilon: float = 1e-6, kl_coefficient: float = 0.0) -> torch.Tensor:
    """GRPO over one prompt group: `[G]` rewards, `[G, T]` token log-probs and a 0/1 mask.
    Only `current` carries gradient. All input checks collapse into one device read."""
    if current.dim() != 2 or current.shape[0] < 2:
        raise PostTrainError("GRPO tensor group must contain at least two rollouts")
    G, T = current.shape
    if T == 0:
        raise PostTrainError("GRPO tensor rollouts have no token columns")
    if tuple(rewards.shape) != (G,):
        raise PostTrainError(f"GRPO rewards must have shape [{G}]")
    for name, t in (("behavior", behavior), ("active_mask", active_mask)):
        if tuple(t.shape) != (G, T):
            raise PostTrainError(f"GRPO {name} tensor must have shape [{G}, {T}]")
    if reference is None and kl_coefficient != 0.0:
        raise PostTrainError("GRPO tensor objective needs reference log-probs for positive KL coefficient")
    if reference is not None and tuple(reference.shape) != (G, T):
        raise PostTrainError(f"GRPO reference tensor must have shape [{G}, {T}]")
    _check_grpo_hparams(clip_epsilon, advantage_epsilon, kl_coefficient)
    rewards = rewards.detach().float()
    behavior = behavior.detach().float()
    mask = active_mask.detach().float()
    cur = current.float()
    mean = rewards.mean()
    centred = rewards - mean
    var = centred.pow(2).mean()
    std = var.sqrt().clamp_min(advantage_epsilon)
    adv = (centred / std).reshape(G, 1)
    ratio = (cur - behavior).exp()
    sur = torch.minimum(ratio * adv, ratio.clamp(1.0 - clip_epsilon, 1.0 + clip_epsilon) * adv)
    if reference is not None:
        d = reference.detach().float() - cur
        sur = sur - kl_coefficient * (d.exp() - d - 1.0)
    per_seq = (sur * mask).sum(dim=1) / mask.sum(dim=1)
    loss = -per_seq.mean()
    log_ratio = cur.detach() - behavior
    checks = [
        ("GRPO rewards contain a non-finite value", rewards.isfinite().all()),
        ("GRPO current log probabilities contain a non-finite value", cur.detach().isfinite().all()),
        ("GRPO behavior log probabilities contain a non-finite value", behavior.isfinite().all()),
        ("GRPO active_mask must contain only binary zero/one values", ((mask == 0) | (mask == 1)).all()),
        ("GRPO active_mask must contain at least one active token in every rollout", (mask.sum(dim=1) > 0).all()),
        ("GRPO importance log-ratio exceeds the safe exponential domain",
         (log_ratio.isfinite() & (log_ratio <= MAX_LOG_RATIO)).all()),
        ("GRPO reward normalization overflowed", var.isfinite()),
        ("GRPO tensor objective overflowed", loss.detach().isfinite()),
    ]
    if reference is not None:
        dr = reference.detach().float() - cur.detach()
        checks.append(("GRPO reference log-ratio exceeds the safe exponential domain",
                       (dr.isfinite() & (dr <= MAX_LOG_RATIO)).all()))
    flags = torch.stack([c.reshape(()) for _, c in checks]).tolist()     # the single device read
    for ok, (msg, _) in zip(flags, checks):
        if not ok:
            raise PostTrainError(msg)
    return loss


# ---------------------------------------------------------------------------- verifier
@dataclass
class Verification:
    reward: float
    passed: bool
    components: Dict[str, float] = field(default_factory=dict)


class ExactAnswerVerifier:
    """Reward 1 when the completion equals the reference answer after optional trimming
    (default on) and case folding (default off). Unknown parameters are rejected."""
    adapter_name = "exact_answer"

    def identity(self) -> str:
        return "sha256:" + hashlib.sha256(b"summa_b200.exact_answer.v1").hexdigest()

    def verify(self, parameters: Dict[str, object], completion: str, reference_answer: Optional[str]) -> Verification:
        unknown = set(parameters) - {"case_fold", "trim"}
        if unknown:
            raise PostTrainError(f"invalid exact_answer verifier parameters: unknown {sorted(unknown)}")
        if reference_answer is None:
            raise PostTrainError("exact_answer verifier requires `reference_answer`")
        trim = bool(parameters.get("trim", True))
        fold = bool(parameters.get("case_fold", False))

        def norm(s: str) -> str:
            s = s.strip() if trim else s
            return s.lower() if fold else s

        ok = norm(completion) == norm(reference_answer)
        return Verification(float(ok), ok, {"exact_match": float(ok)})


# ---------------------------------------------------------------------------- resumable executor
@dataclass
class PreparedUpdate:
    """What one optimizer update of a post-training phase consumed and produced. A retried
    window must rebuild a byte-identical record (`canonical_bytes`)."""
    phase_hash: str
    receipt_chain: str
    step: int
    data_begin: int
    data_end: int
    rng_begin: int
    rng_end: int
    batch_sha256: str
    summary: Dict[str, float]

    def canonical_bytes(self) -> bytes:
        return json.dumps(asdict(self), sort_keys=True, separators=(",", ":")).encode()

    def digest(self) -> str:
        return hashlib.sha256(self.canonical_bytes()).hexdigest()


class PostTrainingExecutor:
    """Drives `update_fn(examples, rng_cursor) -> (summary, rng_used)` over a list of examples
    in windows of `examples_per_update`, persisting `pending` (prepared, not yet applied) and
    `committed` cursors in `state_path` so that a crash between prepare and commit replays
    the same window and checks that it prepares the same bytes."""

    def __init__(self, phase_hash: str, state_path: str, examples_per_update: int, publisher: Callable[[PreparedUpdate], None]):
        if not (0 < examples_per_update <= MAX_EXAMPLES_PER_UPDATE):
            raise PostTrainError(f"examples_per_update must be in [1, {MAX_EXAMPLES_PER_UPDATE}]")
        self.phase_hash, self.state_path = phase_hash, state_path
        self.examples_per_update = examples_per_update
        self.publisher = publisher
        self.state = {"step": 0, "data_pos": 0, "rng_pos": 0, "receipt_chain": hashlib.sha256(phase_hash.encode()).hexdigest(),
                      "pending": None}
        if os.path.exists(state_path):
            with open(state_path) as f:
                saved = json.load(f)
            if saved.get("phase_hash") != phase_hash:
                raise PostTrainError("post-training state belongs to a different phase")
            self.state = saved["state"]

    def _persist(self):
        tmp = self.state_path + ".tmp"
        with open(tmp, "w") as f:
            json.dump({"phase_hash": self.phase_hash, "state": self.state}, f, sort_keys=True)
            f.flush()
            os.fsync(f.fileno())
        os.replace(tmp, self.state_path)

    def run(self, examples: Sequence[object], update_fn, max_updates: Optional[int] = None) -> int:
        done = 0
        while self.state["data_pos"] < len(examples) and (max_updates is None or done < max_updates):
            st = self.state
            begin = st["data_pos"]
            end = min(len(examples), begin + self.examples_per_update)
            window = list(examples[begin:end])
            batch_hash = hashlib.sha256(json.dumps(window, sort_keys=True, default=str).encode()).hexdigest()
            summary, rng_used = update_fn(window, st["rng_pos"])
            prepared = PreparedUpdate(self.phase_hash, st["receipt_chain"], st["step"], begin, end, st["rng_pos"],
                                      st["rng_pos"] + int(rng_used), batch_hash,
                                      {k: float(v) for k, v in sorted(summary.items())})
            if st["pending"] is not None and st["pending"] != prepared.digest():
                raise PostTrainError("a retried post-training window prepared a different update")
            st["pending"] = prepared.digest()
            self._persist()                       # prepared boundary
            self.publisher(prepared)              # must be idempotent per (step, digest)
            st["receipt_chain"] = hashlib.sha256((st["receipt_chain"] + prepared.digest()).encode()).hexdigest()
            st["step"] += 1
            st["data_pos"] = end
            st["rng_pos"] = prepared.rng_end
            st["pending"] = None
            self._persist()                       # commit boundary
            done += 1
        return done

    @property
    def complete_for(self):
        return lambda examples: self.state["data_pos"] >= len(examples)
