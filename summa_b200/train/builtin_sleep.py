"""Built-in tensor work of a consolidation transaction on a memory-chain model.

A boundary moves what a fast (sender) tier has learnt into the next slower (receiver) tier
(`summa-train/src/tensor_sleep.rs` header, `summa-train/src/sleep.rs:3287-3312`):

  prospective_update    the sender's accumulated gradient is applied to a COPY of the model (the
                        teacher of this transaction): what the model would become if the fast
                        tier simply kept its update
  knowledge_seeding     student = the current weights + one newly activated low-rank reserve slot
                        in the receiver tier (in every memory block) - and WITHOUT the sender tier's
                        own active reserve slots, which are reclaimed here: what they held reaches
                        the receiver's new slot through the teacher, and the sender can receive
                        again. Only the new slot is trained, with the forward KL from the teacher's
                        next-token distributions on the replay windows, in chunks
  imitation             GRPO-style: for each replay prompt the student samples a group of
                        continuations, each scored against the teacher's greedy continuation
                        with `gamma * semantic + (1 - gamma) * edit` (`sleep.imitation_reward`);
                        group-normalised advantages weight the sequence log-likelihoods
  retention_validation  gates: the KL to the teacher must have dropped by `min_incorporation_gain`
                        of its pre-seeding value (the slot did absorb the update) and the KL
                        from the pre-consolidation model on the anchor windows must stay below
                        `max_anchor_kl` (nothing else was forgotten); a rejected transaction rolls back
  commit                the sender's accumulator is cleared; the student's weights stay

`restore_teacher` puts the pre-consolidation weights back (slot dormant again). The handlers
plug into `sleep.ConsolidationTxn.run`; `BuiltinDreaming` below supplies the dream phases.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Sequence

import torch
import torch.nn.functional as F

from . import sleep as S
from .objectives import forward_kl


@dataclass
class ConsolidationConfig:
    seeding_steps: int = 20
    seeding_lr: float = 5e-3
    kl_chunk_rows: int = 2048
    imitation_steps: int = 2
    imitation_group: int = 4
    imitation_new_tokens: int = 8
    imitation_lr: float = 1e-3
    imitation_temperature: float = 1.0
    gamma: float = 0.5
    reward_threshold: float = 0.0
    min_incorporation_gain: float = 0.05
    max_anchor_kl: float = 0.5
    seed: int = 0


def _memory_blocks(model):
    return [blk.memory for blk in model.layers if getattr(blk, "memory", None) is not None]


def _chunked_kl(student, teacher_logits: List[torch.Tensor], batches: Sequence[torch.Tensor], chunk_rows: int,
                backward: bool) -> float:
    """Mean forward KL(teacher || student) over all rows of `batches`; with `backward` the gradient is
    accumulated chunk by chunk so that no more than `chunk_rows` rows of logits are alive."""
    total_rows = sum(b.numel() for b in batches)
    total = 0.0
    for tok, tl in zip(batches, teacher_logits):
        B = tok.shape[0]
        per = max(1, chunk_rows // max(tok.shape[1], 1))
        for lo in range(0, B, per):
            sl = student(tok[lo:lo + per])
            rows = sl.shape[0] * sl.shape[1]
            kl = forward_kl(sl.reshape(rows, -1), tl[lo:lo + per].reshape(rows, -1)) * (rows / total_rows)
            if backward:
                kl.backward()
            total += float(kl.detach())
    return total


class BuiltinConsolidation:
    """Handlers of one transaction (one sender tier of one boundary)."""

    def __init__(self, model, bank: S.TierOptimizerBank, sender: int, receiver: int,
                 replay: Sequence[torch.Tensor], anchors: Sequence[torch.Tensor],
                 cfg: Optional[ConsolidationConfig] = None):
        """`replay` / `anchors`: lists of `[B, S]` token tensors (recent wake windows to incorporate /
        held-out windows whose behaviour must be retained)."""
        self.model, self.bank, self.sender, self.receiver = model, bank, sender, receiver
        self.replay, self.anchors = list(replay), list(anchors)
        self.cfg = cfg or ConsolidationConfig()
        self.snapshot: Optional[Dict[str, torch.Tensor]] = None
        self.teacher = None
        self.teacher_logits: List[torch.Tensor] = []
        self.anchor_logits: List[torch.Tensor] = []
        self.slots: List = []
        self.kl_before: Optional[float] = None
        self.reclaimed: List[int] = []
        if not _memory_blocks(model):
            raise S.SleepError("the model has no memory chain")
        for mem in _memory_blocks(model):
            if receiver >= len(mem.tiers):
                raise S.SleepError(f"receiver tier {receiver} does not exist")

    # ------------------------------------------------------------------ helpers
    def _slot_params(self):
        ps = []
        for s in self.slots:
            ps += [s.router.weight, s.a, s.b]
        return ps

    def restore_teacher(self) -> None:
        """Pre-consolidation weights back in place (activated slots dormant again)."""
        if self.snapshot is not None:
            with torch.no_grad():
                for n, p in self.model.named_parameters():
                    p.copy_(self.snapshot[n])
        self.slots = []

    # ------------------------------------------------------------------ phases
    @torch.no_grad()
    def prospective_update(self, ctx: dict) -> S.PhaseResult:
        m = self.model
        self.snapshot = {n: p.detach().clone() for n, p in m.named_parameters()}
        m.eval()
        self.anchor_logits = [m(t).float() for t in self.anchors]
        # the teacher = a copy of the model whose sender tier takes its accumulated update
        acc_norm = sum(float(a.norm()) for a in self.bank.state[self.sender]["acc"]) if self.sender in self.bank.state else 0.0
        if self.sender in self.bank.params:
            acc_saved = [a.clone() for a in self.bank.state[self.sender]["acc"]]
            st_saved = copy.deepcopy({k: v for k, v in self.bank.state[self.sender].items() if k != "acc"})
            self.bank.apply(self.sender)
            self.teacher = copy.deepcopy(m).eval()
            # the live model keeps its pre-update weights; the bank keeps the accumulator until commit
            for n, p in m.named_parameters():
                p.copy_(self.snapshot[n])
            for a, s in zip(self.bank.state[self.sender]["acc"], acc_saved):
                a.copy_(s)
            self.bank.state[self.sender].update(st_saved)
        else:
            self.teacher = copy.deepcopy(m).eval()
        for p in self.teacher.parameters():
            p.requires_grad_(False)
        self.teacher_logits = [self.teacher(t).float() for t in self.replay]
        return S.PhaseResult(True, {"accumulated_gradient_norm": acc_norm, "replay_windows": float(len(self.replay))})

    def knowledge_seeding(self, ctx: dict) -> S.PhaseResult:
        c = self.cfg
        self.slots = []
        for mem in _memory_blocks(self.model):
            reserve = mem.tiers[self.receiver].reserve
            dormant = [i for i in range(len(reserve.slots)) if i not in reserve.active_slots()]
            if not dormant:
                return S.PhaseResult(False, {}, f"receiver tier {self.receiver} has no dormant reserve slot")
            slot = ctx.get("receiver_slot", dormant[0])          # the state machine's transaction names the slot
            if slot not in dormant:
                return S.PhaseResult(False, {}, f"receiver slot {slot} of tier {self.receiver} is not dormant")
            reserve.activate(slot)
            self.slots.append(reserve.slots[slot])
            sender_reserve = mem.tiers[self.sender].reserve
            reclaim = ctx.get("sender_slots_to_reset")
            reclaim = list(sender_reserve.active_slots()) if reclaim is None else list(reclaim)
            if sorted(reclaim) != sorted(sender_reserve.active_slots()):
                return S.PhaseResult(False, {}, f"sender reset plan {sorted(reclaim)} is not the active-slot set of tier {self.sender}")
            for i in reclaim:
                sender_reserve.deactivate(i)
            self.reclaimed = sorted(reclaim)
        self.model.eval()                       # no dropout in the distillation forward
        with torch.no_grad():
            self.kl_before = _chunked_kl(self.model, self.teacher_logits, self.replay, c.kl_chunk_rows, False)
        opt = torch.optim.AdamW(self._slot_params(), lr=c.seeding_lr, weight_decay=0.0)
        kl = self.kl_before
        for _ in range(c.seeding_steps):
            opt.zero_grad(set_to_none=True)
            kl = _chunked_kl(self.model, self.teacher_logits, self.replay, c.kl_chunk_rows, True)
            opt.step()
        self.model.zero_grad(set_to_none=True)
        return S.PhaseResult(True, {"kl_before": self.kl_before, "kl_after": kl, "activated_slots": float(len(self.slots))})

    def imitation(self, ctx: dict) -> S.PhaseResult:
        c = self.cfg
        if c.imitation_steps <= 0 or not self.replay:
            return S.PhaseResult(True, {"reward_mean": 0.0})
        # rollouts draw from the transaction's reserved range of the persisted stream when there is one
        gen = torch.Generator(device="cpu").manual_seed(c.seed + 7919 * int(ctx.get("rng_start", ctx.get("clock", 0))))
        opt = torch.optim.AdamW(self._slot_params(), lr=c.imitation_lr, weight_decay=0.0)
        rewards_seen: List[float] = []
        for step in range(c.imitation_steps):
            tok = self.replay[step % len(self.replay)]
            half = max(1, tok.shape[1] // 2)
            prompts = tok[:, :half]
            with torch.no_grad():
                target = _continue(self.teacher, prompts, c.imitation_new_tokens, 0.0, None)
                t_emb = _mean_embedding(self.teacher, target)
            opt.zero_grad(set_to_none=True)
            loss_total = 0.0
            for b in range(prompts.shape[0]):
                group_lp, group_r = [], []
                for _ in range(c.imitation_group):
                    with torch.no_grad():
                        cont = _continue(self.model, prompts[b:b + 1], c.imitation_new_tokens, c.imitation_temperature, gen)
                        sem = float(F.cosine_similarity(_mean_embedding(self.teacher, cont), t_emb[b:b + 1]).clamp(min=0.0))
                    r = S.imitation_reward(cont[0].tolist(), target[b].tolist(), sem, c.gamma, c.reward_threshold)
                    group_r.append(r)
                    group_lp.append(_sequence_logprob(self.model, prompts[b:b + 1], cont))
                r = torch.tensor(group_r)
                adv = (r - r.mean()) / (r.std(unbiased=False) + 1e-6)
                loss = -(torch.stack(group_lp) * adv.to(group_lp[0].device)).mean() / prompts.shape[0]
                if bool(adv.abs().sum() > 0):
                    loss.backward()
                loss_total += float(loss.detach())
                rewards_seen += group_r
            opt.step()
        self.model.zero_grad(set_to_none=True)
        return S.PhaseResult(True, {"reward_mean": sum(rewards_seen) / max(len(rewards_seen), 1),
                                    "rollouts": float(len(rewards_seen))})

    @torch.no_grad()
    def retention_validation(self, ctx: dict) -> S.PhaseResult:
        c = self.cfg
        self.model.eval()
        kl_after = _chunked_kl(self.model, self.teacher_logits, self.replay, c.kl_chunk_rows, False)
        anchor_kl = _chunked_kl(self.model, self.anchor_logits, self.anchors, c.kl_chunk_rows, False) if self.anchors else 0.0
        before = self.kl_before if self.kl_before is not None else kl_after
        gain = 0.0 if before <= 0 else (before - kl_after) / before
        metrics = {"kl_to_teacher": kl_after, "incorporation_gain": gain, "anchor_kl": anchor_kl}
        if before > 1e-9 and gain < c.min_incorporation_gain:
            return S.PhaseResult(False, metrics, f"incorporation gain {gain:.3f} below {c.min_incorporation_gain}")
        if anchor_kl > c.max_anchor_kl:
            return S.PhaseResult(False, metrics, f"anchor KL {anchor_kl:.3f} above {c.max_anchor_kl}")
        return S.PhaseResult(True, metrics)

    @torch.no_grad()
    def commit(self, ctx: dict) -> S.PhaseResult:
        if self.sender in self.bank.state:
            for a in self.bank.state[self.sender]["acc"]:
                a.zero_()
            self.bank.state[self.sender]["count"] = 0
        if self.receiver in self.bank.state:
            self.bank.resync(self.receiver)          # the trained slot's values become the receiver's masters
        if self.reclaimed and self.sender in self.bank.state:
            # the reclaimed sender slots start over: masters from the zeroed weights, moments cleared
            self.bank.resync(self.sender)
            st = self.bank.state[self.sender]
            for i, (name, _) in enumerate(self.bank.params[self.sender]):
                if any(f".reserve.slots.{k}." in name for k in self.reclaimed):
                    st["m"][i].zero_()
                    st["v"][i].zero_()
        self.teacher, self.teacher_logits, self.anchor_logits, self.snapshot = None, [], [], None
        return S.PhaseResult(True, {"committed_slots": float(len(self.slots))})

    def handlers(self) -> Dict[str, Callable[[dict], S.PhaseResult]]:
        return {"prospective_update": self.prospective_update, "knowledge_seeding": self.knowledge_seeding,
                "imitation": self.imitation, "retention_validation": self.retention_validation, "commit": self.commit}


class StateMachineConsolidation:
    """`BuiltinConsolidation` behind the backend contract of `sleep_state.run_consolidation`
    (`summa-train/src/sleep.rs:2369-2386`): the durable state machine owns ids, slots, RNG receipts and the
    commit / roll-back bookkeeping, this object does the tensor work of each sub-phase. `publish(txn, model)`
    returns the (location, `sha256:` digest) of the committed candidate; the default fingerprints the parameters
    in memory."""

    def __init__(self, inner: BuiltinConsolidation, publish: Optional[Callable] = None):
        self.inner, self.publish, self.metrics = inner, publish, {}

    def _run(self, name: str, fn, ctx: dict) -> S.PhaseResult:
        res = fn(ctx)
        self.metrics[name] = res.metrics
        if not res.accepted:
            raise S.SleepError(f"{name} refused: {res.reason}")
        return res

    def knowledge_rng_count(self) -> int:
        return max(1, self.inner.cfg.seeding_steps)

    def imitation_rng_count(self) -> int:
        c = self.inner.cfg
        rows = sum(int(t.shape[0]) for t in self.inner.replay[:max(c.imitation_steps, 0)]) if self.inner.replay else 0
        return max(1, rows * max(c.imitation_group, 1))

    def compute_prospective_update(self, txn) -> None:
        if (txn.sender, txn.receiver) != (self.inner.sender, self.inner.receiver):
            raise S.SleepError("the transaction is for another pair of tiers than this backend was built for")
        self._run("prospective_update", self.inner.prospective_update, {"clock": txn.trigger_clock})

    def stage_student(self, txn) -> None:
        pass                                    # the live model is the student; the teacher is the detached copy

    def knowledge_seed(self, txn) -> None:
        self._run("knowledge_seeding", self.inner.knowledge_seeding, {"clock": txn.trigger_clock, "receiver_slot": txn.receiver_slot,
                                                                      "sender_slots_to_reset": txn.sender_slots_to_reset})

    def learn_to_imitate(self, txn) -> None:
        self._run("imitation", self.inner.imitation, {"clock": txn.trigger_clock, "rng_start": txn.imitation_rng.start})

    def retention_passes(self, txn) -> bool:
        res = self.inner.retention_validation({"clock": txn.trigger_clock})
        self.metrics["retention_validation"] = dict(res.metrics, reason=res.reason)
        return res.accepted

    def commit(self, txn):
        self._run("commit", self.inner.commit, {"clock": txn.trigger_clock})
        if self.publish is not None:
            return self.publish(txn, self.inner.model)
        return f"memory://sleep-candidate-{txn.id}", parameter_fingerprint(self.inner.model)

    def restore_teacher(self, txn) -> None:
        self.inner.restore_teacher()


def validate_model_memory_state(model, state) -> None:
    """The transaction metadata against the masks and generations stored in every memory block: a logical reserve
    slot moves together in all layers, and each (active, generation) pair equals the sleep state's
    (`summa-train/src/sleep.rs:2253-2365`). Called after a load and after every retired transaction."""
    for layer, mem in enumerate(_memory_blocks(model)):
        if len(mem.tiers) != len(state.tiers):
            raise S.SleepError(f"memory block {layer} has {len(mem.tiers)} tiers, the sleep state {len(state.tiers)}")
        for t, (tier, meta) in enumerate(zip(mem.tiers, state.tiers)):
            seen = tier.reserve.slot_states()
            want = [(s.active, s.generation) for s in meta.slots]
            if seen != want:
                raise S.SleepError(f"memory block {layer}, tier `{meta.id}`: slot masks / generations {seen} differ from the sleep state's {want}")


def parameter_fingerprint(model) -> str:
    """`sha256:` digest over the names, shapes and contents of every parameter, in name order. Host tensors are
    hashed byte for byte; device tensors through two 64-bit checksums computed on the device (a plain and a
    position-weighted sum of the raw words), which is enough to notice any accidental write and avoids copying
    the model to the host around every guarded operation."""
    import hashlib
    h = hashlib.sha256()
    for name, p in sorted(model.named_parameters(), key=lambda kv: kv[0]):
        t = p.detach().contiguous()
        h.update(name.encode() + b"\0" + str(tuple(t.shape)).encode() + str(t.dtype).encode())
        words = t.view(torch.int16 if t.element_size() == 2 else (torch.int32 if t.element_size() == 4 else torch.uint8)).reshape(-1)
        if t.device.type == "cpu":
            h.update(words.numpy().tobytes())
        else:
            w64 = words.to(torch.int64)
            weights = (torch.arange(w64.numel(), device=t.device, dtype=torch.int64) % 65521) + 1
            h.update(f"{int(w64.sum())}:{int((w64 * weights).sum())}".encode())
    return "sha256:" + h.hexdigest()


# ---------------------------------------------------------------------------- rollouts
@torch.no_grad()
def _continue(model, prompts: torch.Tensor, new_tokens: int, temperature: float, gen) -> torch.Tensor:
    """`[B, new_tokens]` continuation (greedy when temperature <= 0)."""
    seq = prompts
    out = []
    for _ in range(new_tokens):
        logits = model(seq)[:, -1].float()
        if temperature <= 0:
            nxt = logits.argmax(dim=-1, keepdim=True)
        else:
            p = torch.softmax(logits / temperature, dim=-1).cpu()
            nxt = torch.multinomial(p, 1, generator=gen).to(seq.device)
        out.append(nxt)
        seq = torch.cat([seq, nxt], dim=1)
    return torch.cat(out, dim=1)


def _sequence_logprob(model, prompt: torch.Tensor, cont: torch.Tensor) -> torch.Tensor:
    seq = torch.cat([prompt, cont], dim=1)
    logits = model(seq[:, :-1]).float()
    lp = torch.log_softmax(logits[:, prompt.shape[1] - 1:], dim=-1)
    return lp.gather(2, cont.unsqueeze(-1)).sum()


@torch.no_grad()
def _mean_embedding(model, tokens: torch.Tensor) -> torch.Tensor:
    """Semantic proxy of a continuation: the mean of its token embeddings."""
    return model.embed(tokens).float().mean(dim=1)


# ---------------------------------------------------------------------------- dreaming
@dataclass
class DreamConfig:
    candidates_per_prompt: int = 3
    new_tokens: int = 8
    temperature: float = 1.0
    keep: int = 4                      # candidates that go to trials after ranking
    lora_rank: int = 8                 # the reference runs rank 64 / alpha 128 on its 100M+ models
    lora_alpha: float = 16.0
    trial_steps: int = 4
    trial_lr: float = 5e-2
    policy_steps: int = 4
    policy_lr: float = 5e-3
    seed: int = 0


class BuiltinDreaming:
    """Dream phases after a committed consolidation (`summa-train/src/builtin_dreaming.rs` header,
    `summa-train/src/sleep.rs:2551-2587,3335-3429`):

      dream_generation     continuations of wake-context prompts sampled with dream routing (one extra
                           random expert per token in MoE tiers), so the candidates leave the wake policy
      dream_ranking        each candidate's loss gradient w.r.t. the output projection is compared by
                           cosine with the gradient of the reference set; the best `keep` survive
      dream_trials         per candidate an isolated low-rank adapter on the LM head is trained on it and
                           judged by the reference-set loss it would give (the model itself is untouched)
      dream_policy_update  ReST-EM step: the accepted candidates become training data for the trainable
                           parameters given (by default the receiver tier's active reserve slots)
    """

    def __init__(self, model, prompts: Sequence[torch.Tensor], reference: Sequence[torch.Tensor], trainable=None,
                 cfg: Optional[DreamConfig] = None):
        self.model, self.prompts, self.reference = model, list(prompts), list(reference)
        self.cfg = cfg or DreamConfig()
        self.trainable = list(trainable) if trainable is not None else None
        self.candidates: List[torch.Tensor] = []       # full sequences [1, S]
        self.ranked: List[int] = []
        self.accepted: List[int] = []

    # ---- pieces
    def _head_grad(self, seq: torch.Tensor) -> torch.Tensor:
        """d(loss)/d(output projection) for one sequence, flattened; the hidden states are detached,
        so one forward and one small GEMM give the gradient."""
        m = self.model
        with torch.no_grad():
            h, _ = m.forward_hidden(seq[:, :-1])
        h = h.reshape(-1, h.shape[-1]).float()
        w = m.output_weight().detach().float()[:, :m.cfg.vocab_size]
        logits = h @ w
        p = torch.softmax(logits, dim=-1)
        p[torch.arange(p.shape[0]), seq[0, 1:]] -= 1.0
        return (h.t() @ p / p.shape[0]).reshape(-1)

    @torch.no_grad()
    def _reference_loss(self, delta: Optional[torch.Tensor] = None) -> float:
        m, total, rows = self.model, 0.0, 0
        w = m.output_weight().detach().float()[:, :m.cfg.vocab_size]
        if delta is not None:
            w = w + delta
        for t in self.reference:
            h, _ = m.forward_hidden(t[:, :-1])
            logits = h.reshape(-1, h.shape[-1]).float() @ w
            total += float(F.cross_entropy(logits, t[:, 1:].reshape(-1), reduction="sum"))
            rows += t[:, 1:].numel()
        return total / max(rows, 1)

    # ---- phases
    @torch.no_grad()
    def dream_generation(self, ctx: dict) -> S.PhaseResult:
        c = self.cfg
        gen = torch.Generator(device="cpu").manual_seed(c.seed + 104729 * int(ctx.get("clock", 0)))
        self.model.eval()
        self.candidates = []
        for pi, prompt in enumerate(self.prompts):
            for k in range(c.candidates_per_prompt):
                seq = prompt[:1]
                for step in range(c.new_tokens):
                    h, _ = self.model.forward_hidden(seq, dream_seed=c.seed * 7919 + pi * 131 + k * 17 + step + 1)
                    logits = self.model.project_logits(h[:, -1:])[:, -1, :self.model.cfg.vocab_size].float()
                    p = torch.softmax(logits / max(c.temperature, 1e-3), dim=-1).cpu()
                    nxt = torch.multinomial(p, 1, generator=gen).to(seq.device)
                    seq = torch.cat([seq, nxt], dim=1)
                self.candidates.append(seq)
        return S.PhaseResult(bool(self.candidates), {"candidates": float(len(self.candidates))},
                             "" if self.candidates else "no wake-context prompts to dream from")

    def dream_ranking(self, ctx: dict) -> S.PhaseResult:
        ref = None
        for t in self.reference:
            for b in range(t.shape[0]):
                g = self._head_grad(t[b:b + 1])
                ref = g if ref is None else ref + g
        scores = [float(F.cosine_similarity(self._head_grad(s), ref, dim=0)) for s in self.candidates]
        order = sorted(range(len(scores)), key=lambda i: (-scores[i], i))
        self.ranked = order[:self.cfg.keep]
        return S.PhaseResult(True, {"best_cosine": scores[order[0]], "kept": float(len(self.ranked)),
                                    "mean_cosine": sum(scores) / len(scores)})

    def dream_trials(self, ctx: dict) -> S.PhaseResult:
        c, m = self.cfg, self.model
        base = self._reference_loss()
        H, V = m.cfg.hidden_size, m.cfg.vocab_size
        self.accepted = []
        gains = []
        for i in self.ranked:
            seq = self.candidates[i]
            torch.manual_seed(c.seed + i)
            A = (torch.randn(H, c.lora_rank) / H ** 0.5).requires_grad_(True)
            B = torch.zeros(c.lora_rank, V, requires_grad=True)
            A.data, B.data = A.data.to(seq.device), B.data.to(seq.device)
            with torch.no_grad():
                h, _ = m.forward_hidden(seq[:, :-1])
                h = h.reshape(-1, H).float()
                w = m.output_weight().detach().float()[:, :V]
            opt = torch.optim.SGD([A, B], lr=c.trial_lr)
            for _ in range(c.trial_steps):
                opt.zero_grad()
                logits = h @ (w + (c.lora_alpha / c.lora_rank) * (A @ B))
                F.cross_entropy(logits, seq[0, 1:]).backward()
                opt.step()
            delta = ((c.lora_alpha / c.lora_rank) * (A @ B)).detach()
            gain = base - self._reference_loss(delta)
            gains.append(gain)
            if gain > 0:
                self.accepted.append(i)
        return S.PhaseResult(True, {"reference_loss": base, "accepted": float(len(self.accepted)),
                                    "best_gain": max(gains) if gains else 0.0})

    def dream_policy_update(self, ctx: dict) -> S.PhaseResult:
        c, m = self.cfg, self.model
        if not self.accepted:
            return S.PhaseResult(True, {"trained_on": 0.0})
        params = self.trainable
        if params is None:
            params = [p for mem in _memory_blocks(m) for tier in mem.tiers for i in tier.reserve.active_slots()
                      for p in (tier.reserve.slots[i].router.weight, tier.reserve.slots[i].a, tier.reserve.slots[i].b)]
        if not params:
            return S.PhaseResult(True, {"trained_on": 0.0})
        before = self._reference_loss()
        opt = torch.optim.AdamW(params, lr=c.policy_lr, weight_decay=0.0)
        m.eval()
        for _ in range(c.policy_steps):
            opt.zero_grad(set_to_none=True)
            for i in self.accepted:
                seq = self.candidates[i]
                (m.forward_loss(seq[:, :-1], seq[:, 1:]) / len(self.accepted)).backward()
            opt.step()
        m.zero_grad(set_to_none=True)
        return S.PhaseResult(True, {"trained_on": float(len(self.accepted)), "reference_loss_before": before,
                                    "reference_loss_after": self._reference_loss()})

    def handlers(self) -> Dict[str, Callable[[dict], S.PhaseResult]]:
        return {"dream_generation": self.dream_generation, "dream_ranking": self.dream_ranking,
                "dream_trials": self.dream_trials, "dream_policy_update": self.dream_policy_update}


class TerminalConsolidation:
    """The slowest tier's boundary as a state-machine backend (`distill_into_base_v1`): the tier takes its own
    accumulated update, then its active reserves are distilled into its base FFN; the retention gate is the
    distillation's own acceptance. A rejection puts back every weight, the tier's optimizer moments and its
    accumulated gradient, so the boundary can be retried."""

    def __init__(self, model, bank: S.TierOptimizerBank, tier: int, batches: Sequence[torch.Tensor], publish: Optional[Callable] = None):
        self.model, self.bank, self.tier, self.batches, self.publish = model, bank, tier, list(batches), publish
        self.saved = None
        self.metrics: Dict[str, Dict[str, float]] = {}

    def knowledge_rng_count(self) -> int:
        return 1

    def imitation_rng_count(self) -> int:
        return 1

    def compute_prospective_update(self, txn) -> None:
        if not txn.terminal or txn.sender != self.tier:
            raise S.SleepError("the transaction is not this tier's terminal boundary")
        weights = {n: p.detach().clone() for n, p in self.model.named_parameters()}     # slot masks and generations included
        bank = copy.deepcopy(self.bank.state[self.tier]) if self.tier in self.bank.state else None
        self.saved = (weights, bank)
        if self.tier in self.bank.params:
            self.bank.apply(self.tier)

    def stage_student(self, txn) -> None:
        pass

    def knowledge_seed(self, txn) -> None:
        pass

    def learn_to_imitate(self, txn) -> None:
        pass

    def retention_passes(self, txn) -> bool:
        if not txn.sender_slots_to_reset:
            return True                                  # no reserve is awake: the tier's own update is the whole boundary
        if not self.batches:
            self.metrics["distillation"] = {"reason": "no replay windows to distil the reserves with"}
            return False
        res = distill_into_base(self.model, self.tier, self.batches)
        self.metrics["distillation"] = dict(res.metrics)
        return res.accepted

    def commit(self, txn):
        if self.tier in self.bank.params:
            self.bank.resync(self.tier)
        self.saved = None
        if self.publish is not None:
            return self.publish(txn, self.model)
        return f"memory://sleep-candidate-{txn.id}", parameter_fingerprint(self.model)

    def restore_teacher(self, txn) -> None:
        if self.saved is None:
            return
        weights, bank = self.saved
        with torch.no_grad():
            for n, p in self.model.named_parameters():
                p.copy_(weights[n])
        if bank is not None:
            self.bank.state[self.tier] = bank
        self.saved = None


class StateMachineDreaming:
    """`BuiltinDreaming`'s tensor work behind the backend contract of `sleep_state.run_dreaming`
    (`summa-train/src/sleep.rs:2683-2728`). What the contract adds to the compact handler form:

      * the shared candidate is never written: generation and ranking run without gradients, every trial trains an
        isolated low-rank adapter, and the policy step trains CLONES of the trainable tensors; their new values are
        the content-addressed policy state (`policy_state`), which the caller installs after the transaction is
        retired. `shared_checkpoint_hash` is the parameter fingerprint, so the driver notices any stray write and
        `restore_shared_candidate` puts the sealed copy back;
      * candidates carry a gradient sketch instead of a full gradient: d(loss)/d(output projection) with the
        vocabulary hashed into as many buckets as keep the sketch within 4096 numbers; the reference gradient is
        the same sketch of the reference set;
      * generation is keyed by the transaction's reserved RNG range, so a resumed run that lost its in-memory
        candidates regenerates the same ones and checks them against the recorded manifest."""

    def __init__(self, inner: "BuiltinDreaming", evaluator_hash: str, fingerprint: Optional[Callable[[], str]] = None):
        """`fingerprint()` is the identity the consolidation commit published for the candidate (default: every
        parameter of the model)."""
        self.inner, self.evaluator_hash = inner, evaluator_hash
        self.fingerprint = fingerprint or (lambda: parameter_fingerprint(inner.model))
        self.sealed: Optional[Dict[str, torch.Tensor]] = None
        self.sealed_hash: Optional[str] = None
        self.generated: Dict[str, list] = {}
        self.tokens: Dict[str, torch.Tensor] = {}
        self.receipts: Dict[int, str] = {}
        self.policy_state: Optional[Dict[int, torch.Tensor]] = None
        self.sketch_dimensions = 4096                 # upper bound of a gradient sketch's length (the runtime's `gradient_dimensions`)

    # ---- candidate identity
    def verify_committed_candidate(self, txn) -> None:
        seen = self.fingerprint()
        if txn.candidate_hash != seen:
            raise S.SleepError("the live model is not the committed candidate")
        if self.sealed is None:
            self.sealed = {n: p.detach().clone() for n, p in self.inner.model.named_parameters()}
            self.sealed_hash = seen

    def shared_checkpoint_hash(self) -> str:
        return self.fingerprint()

    def restore_shared_candidate(self, txn) -> None:
        if self.sealed is None:
            raise S.SleepError("no sealed candidate to restore")
        with torch.no_grad():
            for n, p in self.inner.model.named_parameters():
                p.copy_(self.sealed[n])

    # ---- gradient sketches
    def _sketch(self, seq: torch.Tensor) -> List[float]:
        m = self.inner.model
        H, V = m.cfg.hidden_size, m.cfg.vocab_size
        buckets = max(1, min(4096, self.sketch_dimensions) // H)
        g = self.inner._head_grad(seq).reshape(H, V)
        idx = (torch.arange(V, device=g.device) * 2654435761 % 4294967296 % buckets)
        out = torch.zeros(H, buckets, device=g.device, dtype=g.dtype).index_add_(1, idx, g)
        return [float(x) for x in out.reshape(-1).cpu()]

    def _generate(self, txn, count: int):
        import hashlib
        inner, c = self.inner, self.inner.cfg
        if not inner.prompts:
            raise S.SleepError("no wake-context prompts to dream from")
        start = txn.dream_generation_rng.start
        gen = torch.Generator(device="cpu").manual_seed(c.seed + 104729 * int(start) + 1)
        inner.model.eval()
        dreams, tokens = [], {}
        from . import sleep_state as SS
        with torch.no_grad():
            for k in range(count):
                prompt = inner.prompts[k % len(inner.prompts)]
                seq = prompt[:1]
                for step in range(c.new_tokens):
                    h, _ = inner.model.forward_hidden(seq, dream_seed=(c.seed * 7919 + int(start) * 131 + k * 17 + step + 1) & 0x7FFFFFFF)
                    logits = inner.model.project_logits(h[:, -1:])[:, -1, :inner.model.cfg.vocab_size].float()
                    p = torch.softmax(logits / max(c.temperature, 1e-3), dim=-1).cpu()
                    seq = torch.cat([seq, torch.multinomial(p, 1, generator=gen).to(seq.device)], dim=1)
                digest = hashlib.sha256(f"{k}:".encode() + seq.cpu().numpy().tobytes()).hexdigest()
                cid = f"dream-{txn.id}-{k:04d}"
                tokens[cid] = seq
                dreams.append(SS.GeneratedDream(cid, "sha256:" + digest, self._sketch(seq), int(digest[:16], 16)))
        manifest = "sha256:" + hashlib.sha256("".join(d.artifact_hash for d in dreams).encode()).hexdigest()
        return manifest, dreams, tokens

    def generate_from_wake_contexts(self, txn, count: int, random_extra_expert: bool):
        manifest, dreams, tokens = self._generate(txn, count)
        self.generated[manifest] = dreams
        self.tokens.update(tokens)
        return manifest, list(dreams)

    def load_generated_dreams(self, txn, manifest: str):
        if manifest not in self.generated:                   # resumed without the in-memory candidates
            again, dreams, tokens = self._generate(txn, int(txn.dream_generation_rng.count))
            if again != manifest:
                raise S.SleepError("regenerated dreams do not match the recorded manifest")
            self.generated[manifest] = dreams
            self.tokens.update(tokens)
        return list(self.generated[manifest])

    def reference_gradient(self, txn, reference_set_hash: str) -> List[float]:
        total = None
        for t in self.inner.reference:
            for b in range(t.shape[0]):
                g = torch.tensor(self._sketch(t[b:b + 1]))
                total = g if total is None else total + g
        if total is None:
            raise S.SleepError("the reference set is empty")
        return [float(x) for x in total]

    # ---- isolated trial and policy step
    def isolated_lora_trial(self, txn, dream, rank: int, alpha: int):
        import hashlib
        from . import sleep_state as SS
        inner, c, m = self.inner, self.inner.cfg, self.inner.model
        H, V = m.cfg.hidden_size, m.cfg.vocab_size
        rank = max(1, min(rank, H, V))
        seq = self.tokens[dream.id]
        seed = c.seed + int(next(r.start for cid, r in txn.dream_trial_rngs if cid == dream.id))
        g = torch.Generator(device="cpu").manual_seed(seed)
        A = (torch.randn(H, rank, generator=g) / H ** 0.5).to(seq.device).requires_grad_(True)
        B = torch.zeros(rank, V, device=seq.device, requires_grad=True)
        with torch.no_grad():
            h, _ = m.forward_hidden(seq[:, :-1])
            h = h.reshape(-1, H).float()
            w = m.output_weight().detach().float()[:, :V]
        base = inner._reference_loss()
        opt = torch.optim.SGD([A, B], lr=c.trial_lr)
        scale = float(alpha) / rank
        for _ in range(c.trial_steps):
            opt.zero_grad()
            F.cross_entropy(h @ (w + scale * (A @ B)), seq[0, 1:]).backward()
            opt.step()
        delta = (scale * (A @ B)).detach()
        gain = base - inner._reference_loss(delta)
        adapter = "sha256:" + hashlib.sha256(delta.cpu().contiguous().numpy().tobytes()).hexdigest()
        return SS.DreamTrial(dream.id, adapter, self.evaluator_hash, float(gain))

    def restem_update(self, txn, accepted, iterations: int) -> str:
        import hashlib
        if txn.id in self.receipts:
            return self.receipts[txn.id]
        inner, c, m = self.inner, self.inner.cfg, self.inner.model
        params = inner.trainable
        if params is None:
            params = [p for mem in _memory_blocks(m) for tier in mem.tiers for i in tier.reserve.active_slots()
                      for p in (tier.reserve.slots[i].router.weight, tier.reserve.slots[i].a, tier.reserve.slots[i].b)]
        state: Dict[int, torch.Tensor] = {}
        if accepted and params:
            saved = [p.detach().clone() for p in params]
            opt = torch.optim.AdamW(params, lr=c.policy_lr, weight_decay=0.0)
            m.eval()
            try:
                for _ in range(max(1, iterations) * c.policy_steps):
                    opt.zero_grad(set_to_none=True)
                    for trial in accepted:
                        seq = self.tokens[trial.candidate_id]
                        (m.forward_loss(seq[:, :-1], seq[:, 1:]) / len(accepted)).backward()
                    opt.step()
                state = {i: p.detach().clone() for i, p in enumerate(params)}
            finally:                                         # the shared candidate keeps its sealed values
                with torch.no_grad():
                    for p, old in zip(params, saved):
                        p.copy_(old)
                m.zero_grad(set_to_none=True)
        h = hashlib.sha256(f"restem:{txn.id}:{len(accepted)}".encode())
        for i in sorted(state):
            h.update(state[i].cpu().contiguous().view(torch.uint8).numpy().tobytes())
        self.policy_state = {"params": params, "values": state}
        self.receipts[txn.id] = "sha256:" + h.hexdigest()
        return self.receipts[txn.id]

    def install_policy_state(self) -> int:
        """After the transaction is retired: the policy step's values become the live weights."""
        if not self.policy_state or not self.policy_state["values"]:
            return 0
        with torch.no_grad():
            for i, p in enumerate(self.policy_state["params"]):
                p.copy_(self.policy_state["values"][i])
        return len(self.policy_state["values"])


def tier_fingerprint(model) -> str:
    """Fingerprint of the memory tiers' parameters: the part of the model a boundary can change."""
    class _Tiers:
        def named_parameters(self_inner):
            return [(n, p) for n, p in model.named_parameters() if S.tier_of_parameter(n) is not None]
    return parameter_fingerprint(_Tiers())


def drain_due_boundaries(model, bank: S.TierOptimizerBank, state, replay_windows: Sequence[torch.Tensor], consolidation: "ConsolidationConfig", *,
                         terminal_distil: bool = True, dreaming: Optional[dict] = None, runtime=None, progress=None,
                         location: str = "memory://boundary", write_reports: bool = True) -> List[Dict[str, object]]:
    """Runs every boundary queued in `state` (a `sleep_state.SleepState`), fastest tier first (a retried terminal
    boundary first), each as one transaction: ordinary tiers consolidate into the next slower tier, then dream when
    `dreaming` (the workflow's dreaming block) is given; the terminal tier takes its own update and distils its
    reserves into its base. A rejected transaction leaves the weights and the accumulated gradient as they were.
    `runtime` (a `sleep_runtime.SleepRuntimeConfig`) supplies the dreaming runtime settings and the rejection-report
    directory. Returns one record per boundary: sender, trigger, ok, transaction id, receiver slot / generation,
    the backend's metrics and the rejection reason."""
    import hashlib
    from . import sleep_state as SS
    last = len(state.tiers) - 1
    windows = list(replay_windows)
    replay = windows[:-1] or windows
    anchors = windows[-1:] if len(windows) > 1 else []
    fingerprint = lambda: tier_fingerprint(model)
    publish = lambda t, m: (f"{location}/txn-{t.id}", fingerprint())
    out: List[Dict[str, object]] = []
    while state.next_due() is not None:
        sender, trigger = state.next_due()
        fp = fingerprint()
        acc = sum(float(a.norm()) for a in bank.state[sender]["acc"]) if sender in bank.state else 0.0
        plan = "sha256:" + hashlib.sha256(f"{trigger}:{sender}:{acc!r}".encode()).hexdigest()
        txn = state.begin(sender, f"{location}/step-{trigger}", fp, f"{location}/step-{trigger}", fp, plan)
        if sender < last:
            backend = StateMachineConsolidation(BuiltinConsolidation(model, bank, sender, sender + 1, replay, anchors, consolidation), publish=publish)
        else:
            backend = TerminalConsolidation(model, bank, last, replay if (terminal_distil and replay) else [], publish=publish)
        ok = SS.run_consolidation(state, backend, progress)
        slot = generation = None
        reason = ""
        if ok:
            dream = None
            if sender < last and dreaming and replay:
                dcfg = SS.DreamingConfig(**{k: v for k, v in dreaming.items() if k in SS.DreamingConfig.__dataclass_fields__})
                dc = DreamConfig()
                rd = runtime.dreaming if runtime is not None else None
                if rd is not None:
                    dc.new_tokens, dc.temperature = rd.max_new_tokens, rd.generation_temperature
                    dc.trial_steps, dc.trial_lr, dc.policy_lr = rd.lora_steps, rd.lora_learning_rate, rd.restem_learning_rate
                dream = StateMachineDreaming(BuiltinDreaming(model, [r[:1, :max(2, r.shape[1] // 2)] for r in replay], anchors or replay, cfg=dc),
                                             dcfg.trial_evaluator_hash, fingerprint=fingerprint)
                if rd is not None:
                    dream.sketch_dimensions = rd.gradient_dimensions
                SS.run_dreaming(state, dcfg, dream, progress)
            else:
                state.transition("candidate")
            done = state.finish_candidate()
            if dream is not None:
                dream.install_policy_state()
            if not done.terminal:
                slot, generation = done.receiver_slot, state.tiers[done.receiver].slots[done.receiver_slot].generation
            validate_model_memory_state(model, state)          # masks and generations moved together in every layer
        else:
            reason = str((backend.metrics.get("retention_validation") or backend.metrics.get("distillation") or {}).get("reason", "retention gate"))
            if runtime is not None and write_reports:
                from .sleep_runtime import write_rejection_report
                write_rejection_report(runtime.directories["rejection_report_directory"], txn, reason,
                                       {k: v for k, v in backend.metrics.items() if isinstance(v, dict)})
        if progress is not None:
            progress.persist(state)
        out.append({"sender": sender, "trigger": trigger, "ok": ok, "transaction_id": txn.id, "slot": slot, "generation": generation,
                    "metrics": dict(backend.metrics), "reason": reason})
    return out


# ---------------------------------------------------------------------------- terminal tier
def distill_into_base(model, tier: int, batches: Sequence[torch.Tensor], steps: int = 30, lr: float = 2e-3,
                      max_kl: float = 0.05, chunk_rows: int = 2048) -> S.PhaseResult:
    """The slowest tier has no receiver: its active reserve slots are folded into its own base FFN
    (`distill_into_base_v1`, `summa-train/src/sleep.rs:3287-3312`). Teacher = the model as it is;
    student = the same model with that tier's slots dormant and only the tier's base FFN trainable,
    trained with the forward KL on `batches`. Accepted (slots stay dormant, freed for reuse) when the
    remaining KL is at most `max_kl`; otherwise every weight and slot flag is put back."""
    mems = _memory_blocks(model)
    if not mems or tier >= len(mems[0].tiers):
        raise S.SleepError(f"tier {tier} does not exist")
    snapshot = {n: p.detach().clone() for n, p in model.named_parameters()}
    model.eval()
    with torch.no_grad():
        teacher_logits = [model(t).float() for t in batches]
    freed = 0
    params = []
    with torch.no_grad():
        for mem in mems:
            t = mem.tiers[tier]
            for i in t.reserve.active_slots():
                t.reserve.deactivate(i)              # dormant, generation raised, product zeroed
                freed += 1
            params += [p for p in t.feed_forward.parameters() if p.requires_grad]
    if freed == 0:
        return S.PhaseResult(True, {"freed_slots": 0.0, "kl": 0.0})
    with torch.no_grad():
        kl0 = _chunked_kl(model, teacher_logits, batches, chunk_rows, False)
    opt = torch.optim.AdamW(params, lr=lr, weight_decay=0.0)
    kl = kl0
    for _ in range(steps):
        opt.zero_grad(set_to_none=True)
        kl = _chunked_kl(model, teacher_logits, batches, chunk_rows, True)
        opt.step()
    model.zero_grad(set_to_none=True)
    with torch.no_grad():
        kl = _chunked_kl(model, teacher_logits, batches, chunk_rows, False)
    metrics = {"freed_slots": float(freed), "kl_before": kl0, "kl": kl}
    if kl > max_kl:
        with torch.no_grad():
            for n, p in model.named_parameters():
                p.copy_(snapshot[n])
        return S.PhaseResult(False, metrics, f"distillation KL {kl:.4f} above {max_kl}")
    return S.PhaseResult(True, metrics)
