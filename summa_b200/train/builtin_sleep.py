"""Built-in tensor work of a consolidation transaction on a memory-chain model.

A boundary moves what a fast (sender) tier has learnt into the next slower (receiver) tier
(`summa-train/src/tensor_sleep.rs` header, `summa-train/src/sleep.rs:3287-3312`):

  prospective_update    the sender's accumulated gradient is applied to a COPY of the model (the
                        teacher of this transaction): what the model would become if the fast
                        tier simply kept its update
  knowledge_seeding     student = the current weights + one newly activated low-rank reserve slot
                        in the receiver tier (in every memory block); only that slot is trained,
                        with the forward KL from the teacher's next-token distributions on the
                        replay windows, in chunks
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
plug into `sleep.ConsolidationTxn.run`; the dream phases stay caller-supplied.
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
            reserve.activate(dormant[0])
            self.slots.append(reserve.slots[dormant[0]])
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
        gen = torch.Generator(device="cpu").manual_seed(c.seed + 7919 * int(ctx.get("clock", 0)))
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
        self.teacher, self.teacher_logits, self.anchor_logits, self.snapshot = None, [], [], None
        return S.PhaseResult(True, {"committed_slots": float(len(self.slots))})

    def handlers(self) -> Dict[str, Callable[[dict], S.PhaseResult]]:
        return {"prospective_update": self.prospective_update, "knowledge_seeding": self.knowledge_seeding,
                "imitation": self.imitation, "retention_validation": self.retention_validation, "commit": self.commit}


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
