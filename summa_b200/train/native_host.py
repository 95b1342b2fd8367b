"""Embedded workflow host: routes WorkflowV2 phases to in-process executors.

`run-workflow` alone can only hand a phase to an external worker process. This host is the other
half of the reference's lifecycle runtime (`summa-train/src/native_host.rs:82-330`,
`summa-train/src/posttrain.rs:1251-1306,3028-3340`): it resolves EVERY phase of a workflow to an
execution surface before any state file is created (fail-closed), hashes that routing together with
the adapters' identities into a dispatch identity that pins the run-state file, and then drives the
ordinary phase state machine of `runtime.py` with executors that live in this process:

    phase kind / fields                  route                    executor
    ----------------------------------  -----------------------  ------------------------------------------
    sleep                                native_sleep             NativeSleepPhaseExecutor (built-in consolidation)
    promotion                            (rejected)
    any kind with `post_training`        native_post_training     NativePostTrainingPhaseExecutor (DPO / forward-KL / GRPO)
    any kind with `periodic_sleep`       native_periodic_wake     a registered NativePeriodicWakeExecutor
    everything else                      external_worker          the pinned ExternalPhaseExecutor

The device work of post-training sits behind batch-runtime objects (`DpoDeviceBatchRuntime`,
`ForwardKlDeviceBatchRuntime`, `GrpoDeviceBatchRuntime`): each call takes a whole window of examples and
runs the trainable policy and the frozen teacher / reference as batched forward passes on the device;
the host never sees per-example scores, only the update's summary. `TorchPostTrainingFactory` is the
first-party factory over this package's `Transformer`; deployments with other model stores register
their own factory behind the same three runtime interfaces.
"""
from __future__ import annotations

import hashlib
import json
import math
import os
from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import torch

from . import posttrain as PT
from .metrics import MetricWriter
from .runtime import (AtomicRuntimeCheckpoint, Checkpoint, ExecutorRegistry, ExternalPhaseExecutor, PhaseExecutor,
                      ProgressSink, RuntimeError_, WorkflowRuntime)
from .workflow import PHASE_KINDS, Phase, Workflow

NATIVE_HOST_DISPATCH_VERSION = 2
DISPATCH_ROUTES = ("external_worker", "native_post_training", "native_periodic_wake", "native_sleep")


class NativeHostError(RuntimeError_):
    pass


def _validate_identity(identity: str, what: str) -> None:
    if not isinstance(identity, str) or not identity.strip() or any(c in identity for c in "\n\r"):
        raise NativeHostError(f"{what} identity must be a non-empty single-line string")


# ---------------------------------------------------------------------------- device-batch runtimes
def _pad_batch(seqs: Sequence[Sequence[int]], pad: int, device) -> torch.Tensor:
    n = max(len(s) for s in seqs)
    out = torch.full((len(seqs), n), pad, dtype=torch.int64)
    for i, s in enumerate(seqs):
        out[i, :len(s)] = torch.tensor(list(s), dtype=torch.int64)
    return out.to(device)


def _continuation_mask(prompt_lens: Sequence[int], total_lens: Sequence[int], width: int, device) -> torch.Tensor:
    m = torch.zeros(len(prompt_lens), width)
    for i, (p, t) in enumerate(zip(prompt_lens, total_lens)):
        m[i, p:t] = 1.0
    return m.to(device)


class _TorchRuntimeBase:
    """Shared plumbing of the first-party runtimes: tokenisation, batched forwards, one optimizer."""

    def __init__(self, policy, frozen, tokenizer, optimizer, sequence_length: int, eos_id: int):
        self.policy, self.frozen, self.tok, self.opt = policy, frozen, tokenizer, optimizer
        self.seq, self.eos = sequence_length, eos_id
        self.device = next(policy.parameters()).device

    def _encode_pair(self, prompt: str, continuation: str) -> Tuple[List[int], int]:
        p = self.tok.encode(prompt)
        c = self.tok.encode(continuation) + [self.eos]
        room = self.seq - len(c)
        if room < 1:
            raise PT.PostTrainError("continuation does not fit the phase's sequence_length")
        p = p[-room:]
        return p + c, len(p)

    def _step(self, loss: torch.Tensor) -> None:
        self.opt.zero_grad(set_to_none=True)
        loss.backward()
        torch.nn.utils.clip_grad_norm_([p for p in self.policy.parameters() if p.requires_grad], 1.0)
        self.opt.step()


class DpoDeviceBatchRuntime(_TorchRuntimeBase):
    """One DPO update over a window of `{prompt, chosen, rejected}` records: chosen and rejected rows of
    the whole window go through the policy in ONE batch and through the frozen reference in ONE batch."""

    def update(self, records: Sequence[Dict[str, Any]], cfg: Dict[str, Any], rng_cursor: int):
        rows, plens = [], []
        for r in records:
            for key in ("chosen", "rejected"):
                ids, pl = self._encode_pair(r["prompt"], r[key])
                rows.append(ids)
                plens.append(pl)
        toks = _pad_batch(rows, self.eos, self.device)
        mask = _continuation_mask(plens, [len(x) for x in rows], toks.shape[1], self.device)
        pol = PT.sequence_log_probs(self.policy(toks), toks, mask, cfg["sequence_reduction"])
        with torch.no_grad():
            ref = PT.sequence_log_probs(self.frozen(toks), toks, mask, cfg["sequence_reduction"])
        pc, pr, rc, rr = pol[0::2], pol[1::2], ref[0::2], ref[1::2]
        loss = PT.dpo_loss_tensor(pc, pr, rc, rr, cfg["beta"], cfg["label_smoothing"])
        self._step(loss)
        margin = cfg["beta"] * ((pc - pr) - (rc - rr)).detach()
        summary = {"loss": float(loss.detach()), "preference_accuracy": float((margin > 0).float().mean()),
                   "implicit_reward_margin": float(margin.mean())}
        return summary, 2 * len(records)          # two model RNG substreams per record


class ForwardKlDeviceBatchRuntime(_TorchRuntimeBase):
    """One distillation update: student and frozen teacher see the same padded window of framed records."""

    def update(self, records: Sequence[Dict[str, Any]], cfg: Dict[str, Any], rng_cursor: int):
        rows, plens = [], []
        for r in records:
            prompt = r.get("prompt") or r.get("instruction") or r.get("text") or ""
            cont = r.get("response") or r.get("completion") or ""
            if not cont:                                   # plain autoregressive text: every token is supervised
                ids = (self.tok.encode(prompt) + [self.eos])[:self.seq]
                rows.append(ids)
                plens.append(1)
            else:
                ids, pl = self._encode_pair(prompt, cont)
                rows.append(ids)
                plens.append(pl)
        toks = _pad_batch(rows, self.eos, self.device)
        mask = _continuation_mask(plens, [len(x) for x in rows], toks.shape[1], self.device)[:, 1:].bool()
        student = self.policy(toks)[:, :-1][mask]
        with torch.no_grad():
            teacher = self.frozen(toks)[:, :-1][mask]
        loss = PT.forward_kl_distillation_tensor(teacher, student, cfg["temperature"], cfg["scale_by_temperature_squared"])
        self._step(loss)
        with torch.no_grad():
            t = cfg["temperature"]
            lt = torch.log_softmax(teacher.float() / t, -1)
            ls = torch.log_softmax(student.detach().float() / t, -1)
            kl = (lt.exp() * (lt - ls)).sum(-1).mean()
            ent = -(lt.exp() * lt).sum(-1).mean()
            agree = (teacher.argmax(-1) == student.argmax(-1)).float().mean()
        summary = {"loss": max(float(loss.detach()), 0.0), "forward_kl": max(float(kl), 0.0), "teacher_entropy": max(float(ent), 0.0),
                   "top1_agreement": float(agree)}
        return summary, len(records)


class GrpoDeviceBatchRuntime(_TorchRuntimeBase):
    """One GRPO update: `group_size` sampled continuations per prompt (temperature / nucleus sampling with
    a counter-based seed per rollout), verifier rewards, then one batched forward of policy and reference
    over all rollouts of the window."""

    def __init__(self, *a, verifier=None, **k):
        super().__init__(*a, **k)
        self.verifier = verifier or PT.ExactAnswerVerifier()

    @torch.no_grad()
    def _sample(self, prompt_ids: List[int], sampling: Dict[str, Any], seed: int) -> Tuple[List[int], List[float]]:
        gen = torch.Generator(device="cpu").manual_seed(seed & 0x7FFFFFFF)
        ids, lps = list(prompt_ids), []
        for _ in range(sampling["max_new_tokens"]):
            if len(ids) >= self.seq:
                break
            logits = self.policy(torch.tensor([ids], device=self.device))[0, -1].float()
            lp = torch.log_softmax(logits / sampling["temperature"], -1).cpu()
            probs = lp.exp()
            if sampling["top_p"] < 1.0:
                sp, si = probs.sort(descending=True)
                keep = (sp.cumsum(0) - sp) < sampling["top_p"]
                mask = torch.zeros_like(probs, dtype=torch.bool)
                mask[si[keep]] = True
                probs = torch.where(mask, probs, torch.zeros_like(probs))
                probs = probs / probs.sum()
            nxt = int(torch.multinomial(probs, 1, generator=gen))
            ids.append(nxt)
            lps.append(float(torch.log_softmax(logits, -1)[nxt]))
            if nxt == self.eos:
                break
        return ids[len(prompt_ids):], lps

    def update(self, records: Sequence[Dict[str, Any]], cfg: Dict[str, Any], rng_cursor: int):
        G, sampling = cfg["group_size"], cfg["sampling"]
        self.policy.eval()
        groups = []
        for ri, r in enumerate(records):
            p = self.tok.encode(r["prompt"])[-max(1, self.seq - sampling["max_new_tokens"]):]
            rolls = []
            for g in range(G):
                cont, beh = self._sample(p, sampling, rng_cursor + ri * G + g)
                text = self.tok.decode([t for t in cont if t != self.eos])
                params = dict(r.get("verifier_payload") or {}) if isinstance(r.get("verifier_payload"), dict) else {}
                ref_answer = r.get("reference_answer", params.pop("reference_answer", None))
                reward = self.verifier.verify(params, text, ref_answer).reward
                rolls.append((p, cont, beh, float(reward)))
            groups.append(rolls)
        self.policy.train()
        total, stats = None, {"reward": [], "kl": [], "clipped": 0.0, "tokens": 0.0}
        for rolls in groups:
            rows = [list(p) + list(c) for p, c, _, _ in rolls]
            toks = _pad_batch(rows, self.eos, self.device)
            width = toks.shape[1] - 1
            mask = _continuation_mask([len(p) for p, _, _, _ in rolls], [len(x) for x in rows], toks.shape[1],
                                      self.device)[:, 1:]
            if float(mask.sum(dim=1).min()) == 0:
                continue                                      # a rollout that produced no token carries no gradient
            cur = PT.token_log_probs(self.policy(toks), toks)
            beh = torch.zeros(len(rolls), width, device=self.device)
            for i, (p, c, b, _) in enumerate(rolls):
                beh[i, len(p) - 1:len(p) - 1 + len(b)] = torch.tensor(b, device=self.device)
            beh = torch.where(mask.bool(), beh, cur.detach())
            ref = None
            if self.frozen is not None and cfg["kl_coefficient"] > 0:
                with torch.no_grad():
                    ref = PT.token_log_probs(self.frozen(toks), toks)
                ref = torch.where(mask.bool(), ref, cur.detach())
            rewards = torch.tensor([r for _, _, _, r in rolls], device=self.device)
            loss = PT.grpo_loss_tensor(rewards, cur, beh, ref, mask, cfg["clip_epsilon"], cfg["advantage_epsilon"],
                                       cfg["kl_coefficient"])
            total = loss if total is None else total + loss
            with torch.no_grad():
                ratio = (cur.detach() - beh).exp()
                stats["clipped"] += float((((ratio < 1 - cfg["clip_epsilon"]) | (ratio > 1 + cfg["clip_epsilon"])) * mask).sum())
                stats["tokens"] += float(mask.sum())
                stats["reward"] += [r for _, _, _, r in rolls]
                if ref is not None:
                    d = ref - cur.detach()
                    stats["kl"].append(float((((d.exp() - d - 1.0) * mask).sum(1) / mask.sum(1)).mean()))
        if total is None:
            raise PT.PostTrainError("GRPO window produced no rollout with tokens")
        total = total / len(groups)
        self._step(total)
        rw = torch.tensor(stats["reward"])
        summary = {"loss": float(total.detach()), "mean_reward": float(rw.mean()),
                   "reward_stddev": float(rw.std(unbiased=False)), "mean_kl": max(0.0, sum(stats["kl"]) / max(len(stats["kl"]), 1)),
                   "clipped_fraction": stats["clipped"] / max(stats["tokens"], 1.0)}
        return summary, len(records) * G


RUNTIME_BY_ALGORITHM = {"dpo": DpoDeviceBatchRuntime, "forward_kl": ForwardKlDeviceBatchRuntime,
                        "grpo": GrpoDeviceBatchRuntime}


# ---------------------------------------------------------------------------- post-training context + factory
@dataclass
class PostTrainingExecutionContext:
    """What a factory lends to the executor for one phase: the device runtime, the idempotent publisher
    of prepared updates and the identities that are hashed into every prepared update."""
    runtime: Any
    publish: Callable[[PT.PreparedUpdate], Dict[str, str]]      # -> {"checkpoint_sha256", "optimizer_sha256", "uri"}
    device_runtime_identity: str
    publisher_identity: str
    records: List[Dict[str, Any]]
    examples_per_update: int


class TorchPostTrainingFactory:
    """First-party factory: loads this package's `Transformer` from the phase's input checkpoint, the frozen
    teacher / reference from the artifact the workflow pins (sha256 verified before it is loaded), and
    publishes every applied update as `<out>/<phase>/update-<step>-<digest>.safetensors` (+ optimizer
    state), which makes the publication idempotent: a retried window finds its own files."""

    def __init__(self, model_def, tokenizer, out_dir: str, device: str = "cpu", lr: float = 1e-5):
        self.model_def, self.tok, self.out, self.device, self.lr = model_def, tokenizer, out_dir, torch.device(device), lr

    def identity(self) -> str:
        blob = json.dumps({"factory": "torch-post-training-v1", "model": self.model_def.to_json(), "lr": self.lr},
                          sort_keys=True)
        return "sha256:" + hashlib.sha256(blob.encode()).hexdigest()

    def periodic_sleep_identity(self) -> Optional[str]:
        return None

    def _load(self, path: str):
        from ..models import Transformer
        from ..models import weights as W
        m = Transformer(self.model_def)
        W.load_safetensors(m, path)
        return m.to(self.device)

    @staticmethod
    def _frozen_path(spec: Dict[str, Any]) -> str:
        """`summa_checkpoint` adapter: the artifact is either a weights file or a JSON pointer
        `{"weights": "<path>"}` next to it; its bytes must hash to the pinned identity."""
        path = spec.get("artifact")
        if not path:
            raise NativeHostError("frozen model has no local artifact to load")
        data = open(path, "rb").read()
        if "sha256:" + hashlib.sha256(data).hexdigest() != spec["sha256"]:
            raise NativeHostError(f"frozen model artifact {path} sha256 mismatch")
        if path.endswith(".json"):
            w = json.loads(data)["weights"]
            return w if os.path.isabs(w) else os.path.join(os.path.dirname(path), w)
        return path

    def with_context(self, request: Dict[str, Any], operation: Callable[[PostTrainingExecutionContext], None]) -> None:
        phase = request["phase"]
        cfg = phase["post_training"]
        if not request.get("input_checkpoint"):
            raise NativeHostError("post-training needs an input checkpoint")
        policy = self._load(request["input_checkpoint"]["uri"])
        policy.train()
        spec = cfg.get("reference") or cfg.get("teacher")
        frozen = None
        if spec is not None:
            frozen = self._load(self._frozen_path(spec)).eval()
            for p in frozen.parameters():
                p.requires_grad_(False)
        opt = torch.optim.AdamW(policy.parameters(), lr=self.lr * phase.get("learning_rate_scale", 1.0),
                                betas=(0.9, 0.95), weight_decay=0.0)
        phase_dir = os.path.join(self.out, f"{request['phase_index']:03d}-{phase['name']}")
        os.makedirs(phase_dir, exist_ok=True)
        # resume: the newest published update of this phase carries policy and optimizer state
        resume = request.get("resume_state") or {}
        if resume.get("published"):
            from ..models import weights as W
            W.load_safetensors(policy, resume["published"]["uri"])
            opt.load_state_dict(torch.load(resume["published"]["optimizer"], weights_only=False))
        eos = self.tok.eos_id()
        runtime = RUNTIME_BY_ALGORITHM[cfg["algorithm"]](policy, frozen, self.tok, opt, phase["sequence_length"], eos)
        records = [json.loads(l) for l in open(phase["data"]) if l.strip()]

        def publish(prepared: PT.PreparedUpdate) -> Dict[str, str]:
            from ..models import weights as W
            stem = os.path.join(phase_dir, f"update-{prepared.step:08d}-{prepared.digest()[:16]}")
            wpath, opath = stem + ".safetensors", stem + ".optimizer.pt"
            if not (os.path.exists(wpath) and os.path.exists(opath)):
                W.save_safetensors(policy, wpath + ".tmp")
                os.replace(wpath + ".tmp", wpath)
                torch.save(opt.state_dict(), opath + ".tmp")
                os.replace(opath + ".tmp", opath)
            return {"uri": wpath, "optimizer": opath,
                    "checkpoint_sha256": "sha256:" + hashlib.sha256(open(wpath, "rb").read()).hexdigest(),
                    "optimizer_sha256": "sha256:" + hashlib.sha256(open(opath, "rb").read()).hexdigest()}

        operation(PostTrainingExecutionContext(
            runtime=runtime, publish=publish, device_runtime_identity=self.identity(),
            publisher_identity="local-safetensors-publisher-v1", records=records,
            examples_per_update=phase["batch_size"] * phase.get("gradient_accumulation", 1)))


class NativePostTrainingPhaseExecutor(PhaseExecutor):
    """Resumable driver of a typed post-training phase (`posttrain.rs:3028-3340`): windows of
    `examples_per_update` records, each prepared (hash of phase, receipt chain, step, data and RNG ranges,
    batch, summary), persisted as pending through the runtime's progress sink, published, then committed.
    `update_budget` bounds the updates per call; an unfinished phase yields its cursor."""

    def __init__(self, workflow_signature: str, host: "NativeWorkflowHost", update_budget: Optional[int] = None):
        self.sig, self.host, self.budget = workflow_signature, host, update_budget

    def execute(self, request: Dict[str, Any], sink: ProgressSink):
        factory = self.host.adapters.post_training
        result: Dict[str, Any] = {}

        def operation(ctx: PostTrainingExecutionContext) -> None:
            phase = request["phase"]
            cfg = phase["post_training"]
            phase_hash = hashlib.sha256(json.dumps({"sig": self.sig, "phase": phase, "runtime": ctx.device_runtime_identity,
                                                    "publisher": ctx.publisher_identity}, sort_keys=True).encode()).hexdigest()
            st = dict(request.get("resume_state") or {})
            cursor = st.get("cursor") or {"step": 0, "data_pos": 0, "rng_pos": 0, "epoch": 0,
                                          "receipt_chain": hashlib.sha256(phase_hash.encode()).hexdigest()}
            steps_wanted = phase.get("steps")
            n = len(ctx.records)
            if n == 0:
                raise NativeHostError(f"phase `{phase['name']}` has no records")
            done_now = 0
            published = st.get("published")
            while True:
                if steps_wanted is not None and cursor["step"] >= steps_wanted:
                    break
                if cursor["data_pos"] >= n:
                    if steps_wanted is None and cursor["epoch"] + 1 >= phase.get("epochs", 1):
                        break
                    cursor["epoch"] += 1
                    cursor["data_pos"] = 0
                if self.budget is not None and done_now >= self.budget:
                    result["yield"] = {"cursor": cursor, "published": published}
                    return
                begin = cursor["data_pos"]
                end = min(n, begin + ctx.examples_per_update)
                window = ctx.records[begin:end]
                batch_hash = hashlib.sha256(json.dumps(window, sort_keys=True).encode()).hexdigest()
                summary, rng_used = ctx.runtime.update(window, cfg, cursor["rng_pos"])
                prepared = PT.PreparedUpdate(phase_hash, cursor["receipt_chain"], cursor["step"], begin, end,
                                             cursor["rng_pos"], cursor["rng_pos"] + int(rng_used), batch_hash,
                                             {k: float(v) for k, v in sorted(summary.items())})
                pending = st.pop("pending", None)
                if pending is not None and pending != prepared.digest():
                    raise NativeHostError("a retried post-training window prepared a different update than the one "
                                          "that was persisted as pending")
                sink.checkpoint({"cursor": cursor, "published": published, "pending": prepared.digest()})
                receipt = ctx.publish(prepared)
                published = {"uri": receipt["uri"], "optimizer": receipt["optimizer"]}
                self.host.emit_metric(request, "post_training_update", {
                    "transaction_id": "sha256:" + prepared.digest(), "algorithm": cfg["algorithm"], "epoch": cursor["epoch"],
                    "first_record": begin, "records": end - begin, "optimizer_step": cursor["step"] + 1,
                    "rng_counter_start": prepared.rng_begin, "rng_counter_end": prepared.rng_end,
                    "checkpoint_sha256": receipt["checkpoint_sha256"], "optimizer_sha256": receipt["optimizer_sha256"],
                    **{k: v for k, v in summary.items()}})
                cursor = {"step": cursor["step"] + 1, "data_pos": end, "rng_pos": prepared.rng_end, "epoch": cursor["epoch"],
                          "receipt_chain": hashlib.sha256((cursor["receipt_chain"] + prepared.digest()).encode()).hexdigest()}
                sink.checkpoint({"cursor": cursor, "published": published})
                done_now += 1
            if published is None:
                raise NativeHostError(f"phase `{phase['name']}` finished without applying an update")
            result["product"] = {"type": "model_candidate", "checkpoint": {
                "uri": published["uri"], "sha256": hashlib.sha256(open(published["uri"], "rb").read()).hexdigest()}}

        factory.with_context(request, operation)
        if "yield" in result:
            return "yielded", result["yield"]
        return "complete", result["product"]


# ---------------------------------------------------------------------------- native sleep
class TorchSleepFactory:
    """First-party context of a standalone `sleep` phase: the model of the input checkpoint, the replay / anchor
    windows, and the output directory of the candidate. The windows come either from the operator's sleep-runtime
    file (standalone shape: its pinned wake-context journal, which must have been collected under the phase's input
    checkpoint) or, for small set-ups, from a JSONL of `{"tokens": [...]}` rows."""

    def __init__(self, model_def, replay_path: Optional[str], out_dir: str, device: str = "cpu", runtime=None):
        if (replay_path is None) == (runtime is None):
            raise NativeHostError("a sleep factory takes either a replay JSONL or a standalone sleep-runtime file")
        self.model_def, self.replay_path, self.out, self.device, self.runtime = model_def, replay_path, out_dir, torch.device(device), runtime

    def identity(self) -> str:
        source = self.runtime.identity if self.runtime is not None else hashlib.sha256(open(self.replay_path, "rb").read()).hexdigest()
        return "sha256:" + hashlib.sha256(json.dumps({"factory": "torch-sleep-v2", "model": self.model_def.to_json(), "replay": source},
                                                    sort_keys=True).encode()).hexdigest()

    def load(self, request):
        from ..models import Transformer
        from ..models import weights as W
        m = Transformer(self.model_def)
        W.load_safetensors(m, request["input_checkpoint"]["uri"])
        if self.runtime is not None:
            from .sleep_runtime import WakeContextJournal
            journal = WakeContextJournal.load(self.runtime.pins["wake_context_journal"])
            have = request["input_checkpoint"].get("sha256")
            if have and journal.source_checkpoint_sha256 != ("sha256:" + have.replace("sha256:", "")):
                raise NativeHostError("the wake-context journal was collected under another checkpoint than this phase's input")
            keep = self.runtime.rollouts.max_context_tokens
            rows = [r["token_ids"][:keep] for r in journal.records[-self.runtime.max_wake_context_records:]]
        else:
            rows = [json.loads(l)["tokens"] for l in open(self.replay_path) if l.strip()]
        batches = [torch.tensor([r], dtype=torch.int64, device=self.device) for r in rows]
        return m.to(self.device), batches


class NativeSleepPhaseExecutor(PhaseExecutor):
    """Standalone sleep on the durable state machine: the sleep state starts one step before
    `standalone_trigger_clock` with every tier's previous boundary behind it, the clock advance queues the tiers that
    are due, and `builtin_sleep.drain_due_boundaries` runs each as one transaction (consolidation into the next slower
    tier, dreaming when the phase configures it, terminal distillation). The state is persisted beside the candidate
    after every sub-phase. All transactions rejected -> `mutation_rejected` (the input checkpoint stays current)."""

    def __init__(self, workflow_signature: str, host: "NativeWorkflowHost"):
        self.sig, self.host = workflow_signature, host

    def execute(self, request: Dict[str, Any], sink: ProgressSink):
        from . import sleep as S
        from . import sleep_state as SS
        from ..models import weights as W
        from .builtin_sleep import ConsolidationConfig, drain_due_boundaries
        from .metrics import tier_name
        factory = self.host.adapters.sleep
        runtime = getattr(factory, "runtime", None)
        phase = request["phase"]
        cfg = phase["sleep"]
        model, batches = factory.load(request)
        if len(batches) < 2:
            raise NativeHostError("sleep needs at least two replay rows (replay + anchor)")
        schedule = SS.SleepSchedule.from_json(cfg["schedule"])
        periods = [t.update_period for t in schedule.tiers]
        clock = cfg["standalone_trigger_clock"]
        topt = runtime.tier_optimizer if runtime is not None else None
        bank = S.TierOptimizerBank(model.named_parameters(), lr=topt.learning_rate if topt else cfg["receiver_learning_rate"],
                                   betas=(topt.beta_1, topt.beta_2) if topt else (0.9, 0.95), eps=topt.epsilon if topt else 1e-8,
                                   weight_decay=topt.weight_decay if topt else cfg["receiver_weight_decay"])
        # the tiers' prospective updates come from the replay journal (one accumulation pass)
        model.train()
        for b in batches[:-1]:
            loss, aux = model.forward_loss(b[:, :-1], b[:, 1:], with_router=True)
            (loss + (aux if aux is not None else 0)).backward()
            for t in bank.params:
                bank.accumulate(t)
        cc = ConsolidationConfig()
        cc.kl_chunk_rows = cfg["knowledge_seeding"]["chunk_tokens"]
        cc.seeding_steps = cfg["knowledge_seeding"]["teacher_rollouts"]
        cc.seeding_lr = cc.imitation_lr = cfg["receiver_learning_rate"]
        cc.imitation_group = cfg["imitation"]["grpo_group_size"]
        cc.gamma = cfg["imitation"]["semantic_weight"]
        cc.max_anchor_kl = cfg["retention"]["max_anchor_forward_kl"]
        cc.min_incorporation_gain = cfg["retention"]["min_incorporation_gain"]
        if runtime is not None:
            cc.imitation_new_tokens, cc.imitation_temperature = runtime.rollouts.continuation_tokens, runtime.rollouts.temperature
        phase_dir = os.path.join(factory.out, f"{request['phase_index']:03d}-{phase['name']}")
        state_dir = os.path.join(phase_dir, "sleep")
        os.makedirs(state_dir, exist_ok=True)
        state = SS.SleepState(schedule, runtime.rng_streams if runtime is not None else 1)
        for t, period in zip(state.tiers, periods):                 # the phase starts at its trigger: earlier boundaries are history
            t.last_boundary_clock = t.last_update_clock = ((clock - 1) // period) * period
        state.clock = max(clock - 1, 0)
        state.advance_clock(schedule, clock)

        class Progress:
            def persist(self_inner, st):
                tmp = os.path.join(state_dir, "state.json.tmp")
                with open(tmp, "w") as f:
                    json.dump(st.to_json(), f, sort_keys=True)
                    f.flush()
                    os.fsync(f.fileno())
                os.replace(tmp, os.path.join(state_dir, "state.json"))

            def metric(self_inner, kind, fields):
                self.host.emit_metric(request, kind, fields)

        last = len(periods) - 1
        outcomes = drain_due_boundaries(model, bank, state, batches, cc, terminal_distil=True, dreaming=cfg.get("dreaming"), runtime=runtime,
                                        progress=Progress(), location=f"sleep://{phase['name']}")
        for b in outcomes:
            t = b["sender"]
            self.host.emit_metric(request, "tier_update", {
                "transaction_id": f"sleep-{b['transaction_id']}", "tier": tier_name(t, len(periods)),
                "receiver_tier": tier_name(t + 1, len(periods)) if t < last else None, "tier_clock": clock,
                "update_period": periods[t], "accumulated_micro_steps": len(batches) - 1,
                "outcome": "committed" if b["ok"] else "rolled_back", "reserve_slot": b["slot"], "reserve_generation": b["generation"],
                "optimizer_state_reset": False})
        if not any(b["ok"] for b in outcomes):
            return "complete", {"type": "mutation_rejected", "report": {"clock": clock, "outcomes": [
                (b["sender"], "rolled_back", b["reason"]) for b in outcomes]}}
        out = os.path.join(phase_dir, "candidate.safetensors")
        W.save_safetensors(model, out)
        return "complete", {"type": "model_candidate", "checkpoint": {
            "uri": out, "sha256": hashlib.sha256(open(out, "rb").read()).hexdigest()}}


# ---------------------------------------------------------------------------- periodic wake
class TrainerPeriodicWakeExecutor:
    """First-party periodic-wake executor: the phase runs in THIS process through the wake trainer, whose
    memory policy drives the sleep boundary at every due optimizer step before the next step starts; the
    phase's final sealed generation is the candidate."""

    def __init__(self, model_path: str, tokenizer_path: str, out_dir: str, device: str = "cpu", lr: float = 3e-4,
                 warmup: int = 1, optimizer: str = "adamw"):
        self.model_path, self.tokenizer_path, self.out = model_path, tokenizer_path, out_dir
        self.device, self.lr, self.warmup, self.optimizer = device, lr, warmup, optimizer

    def identity(self) -> str:
        return "sha256:" + hashlib.sha256(json.dumps({
            "executor": "trainer-periodic-wake-v1", "model": open(self.model_path).read(),
            "tokenizer": hashlib.sha256(open(self.tokenizer_path, "rb").read()).hexdigest(), "lr": self.lr,
            "warmup": self.warmup, "optimizer": self.optimizer}, sort_keys=True).encode()).hexdigest()

    def execute_periodic_wake(self, request: Dict[str, Any], sink: ProgressSink):
        from .trainer import TrainArgs, train
        phase = request["phase"]
        run_dir = os.path.join(self.out, f"{request['phase_index']:03d}-{phase['name']}")
        os.makedirs(run_dir, exist_ok=True)
        wf_path = os.path.join(run_dir, "phase-workflow.json")
        with open(wf_path, "w") as f:
            json.dump({"version": 2, "phases": [phase]}, f)
        inp = request.get("input_checkpoint")
        resume = os.path.exists(os.path.join(run_dir, "train", "current.json"))
        res = train(TrainArgs(model=self.model_path, tokenizer=self.tokenizer_path, workflow=wf_path,
                              output=os.path.join(run_dir, "train"), lr=self.lr, warmup_steps=self.warmup,
                              checkpoint=inp["uri"] if inp else None, resume=resume, optimizer=self.optimizer,
                              device=self.device, gpu_metrics_interval_ms=0))
        gen = res["generation"]
        weights = os.path.join(run_dir, "train", "generations", gen, "weights.safetensors")
        return "complete", {"type": "model_candidate", "checkpoint": {
            "uri": weights, "sha256": hashlib.sha256(open(weights, "rb").read()).hexdigest()}}


# ---------------------------------------------------------------------------- adapters + host
class NativeWorkflowAdapters:
    """Explicit adapter registrations. Registering an adapter twice is rejected; a phase whose route has no
    adapter fails in `dispatch_plan`, i.e. before any run state exists."""

    def __init__(self):
        self.external: Optional[ExternalPhaseExecutor] = None
        self.sleep = None
        self.post_training = None
        self.periodic_wake = None

    def register_external(self, executor: ExternalPhaseExecutor) -> None:
        if self.external is not None:
            raise NativeHostError("an external phase worker is already registered")
        self.external = executor

    def register_sleep_factory(self, factory) -> None:
        _validate_identity(factory.identity(), "native sleep factory")
        if self.sleep is not None:
            raise NativeHostError("a native sleep factory is already registered")
        self.sleep = factory

    def register_post_training_factory(self, factory) -> None:
        _validate_identity(factory.identity(), "native post-training factory")
        if factory.periodic_sleep_identity() is not None:
            _validate_identity(factory.periodic_sleep_identity(), "native post-training periodic-sleep controller")
        if self.post_training is not None:
            raise NativeHostError("a native post-training context factory is already registered")
        self.post_training = factory

    def register_periodic_wake_executor(self, executor) -> None:
        _validate_identity(executor.identity(), "native periodic-wake executor")
        if self.periodic_wake is not None:
            raise NativeHostError("a native periodic-wake executor is already registered")
        self.periodic_wake = executor

    def dispatch_plan(self, wf: Workflow) -> List[Dict[str, Any]]:
        plan = []
        for i, p in enumerate(wf.phases):
            if p.kind == "sleep":
                if self.sleep is None:
                    raise NativeHostError(f"sleep phase `{p.name}` requires a registered native sleep factory")
                route = "native_sleep"
            elif p.kind == "promotion":
                raise NativeHostError("built-in promotion is not supported")
            elif p.post_training is not None:
                validate_resumable_phase(p)
                if self.post_training is None:
                    raise NativeHostError(f"phase `{p.name}` has typed post_training and requires a registered native "
                                          "post-training context factory")
                if p.periodic_sleep is not None and self.post_training.periodic_sleep_identity() is None:
                    raise NativeHostError(f"phase `{p.name}` has periodic post_training and requires a registered native "
                                          "post-training periodic-sleep controller")
                route = "native_post_training"
            elif p.periodic_sleep is not None:
                if self.periodic_wake is None:
                    raise NativeHostError(f"phase `{p.name}` has periodic_sleep and requires a registered in-process "
                                          "native periodic-wake executor")
                route = "native_periodic_wake"
            else:
                if self.external is None:
                    raise NativeHostError(f"phase `{p.name}` ({p.kind}) has no registered native route or pinned "
                                          "external worker")
                route = "external_worker"
            plan.append({"phase_index": i, "phase_name": p.name, "phase_kind": p.kind, "dispatch": route})
        return plan

    def dispatch_identity(self, wf: Workflow) -> str:
        """sha256 over: a domain tag, the dispatch version, the workflow signature, every phase's route and
        every adapter's identity (`none` for an absent one), each part length-prefixed."""
        h = hashlib.sha256()

        def part(b: bytes) -> None:
            h.update(len(b).to_bytes(8, "little"))
            h.update(b)
        part(b"summa-native-workflow-host")
        part(NATIVE_HOST_DISPATCH_VERSION.to_bytes(4, "little"))
        part(wf.signature().encode())
        for route in self.dispatch_plan(wf):
            part(json.dumps(route, separators=(",", ":")).encode())
        for ident in (self.external.identity() if self.external else None,
                      self.sleep.identity() if self.sleep else None,
                      self.post_training.identity() if self.post_training else None,
                      self.post_training.periodic_sleep_identity() if self.post_training else None,
                      self.periodic_wake.identity() if self.periodic_wake else None):
            part((ident or "none").encode())
        return "sha256:" + h.hexdigest()


def validate_resumable_phase(p: Phase) -> None:
    """What the native post-training executor can resume exactly: a data file, a batch geometry and either
    an exact step count or whole epochs (`posttrain.rs` `validate_resumable_phase`)."""
    if p.post_training is None:
        raise NativeHostError(f"phase `{p.name}` has no typed post_training settings")
    if not p.data or not p.batch_size or not p.sequence_length:
        raise NativeHostError(f"phase `{p.name}` is incompatible with the native post-training executor: it needs data, "
                              "batch_size and sequence_length")
    if p.max_steps is not None:
        raise NativeHostError(f"phase `{p.name}` is incompatible with the native post-training executor: max_steps")
    per_update = p.batch_size * p.grad_accum_or_default()
    if per_update > PT.MAX_EXAMPLES_PER_UPDATE:
        raise NativeHostError(f"phase `{p.name}` update of {per_update} examples exceeds {PT.MAX_EXAMPLES_PER_UPDATE}")
    if p.post_training["algorithm"] == "grpo" and p.post_training["group_size"] > PT.MAX_ROLLOUTS_PER_PROMPT:
        raise NativeHostError(f"phase `{p.name}` exceeds {PT.MAX_ROLLOUTS_PER_PROMPT} rollouts per prompt")


class _Routed(PhaseExecutor):
    """One executor object registered for every non-sleep kind; it looks the phase's route up in the plan."""

    def __init__(self, host: "NativeWorkflowHost"):
        self.host = host

    def execute(self, request, sink):
        route = self.host.plan[request["phase_index"]]["dispatch"]
        if route == "native_post_training":
            return self.host.post_training_executor.execute(request, sink)
        if route == "native_periodic_wake":
            return self.host.adapters.periodic_wake.execute_periodic_wake(request, sink)
        if route == "external_worker":
            return self.host.adapters.external.execute(request, sink)
        raise NativeHostError(f"phase {request['phase_index']} has no executor for route `{route}`")


class NativeWorkflowHost:
    """`start` / `resume` validate the complete routing first; nothing is created when it is incomplete.
    An executor failure marks the host as needing recovery: the metric journal may hold records of the
    failed attempt, so the only way on is `resume`, which cuts the journal back to the committed prefix."""

    def __init__(self, wf: Workflow, adapters: NativeWorkflowAdapters, state_path: str,
                 metrics: Optional[Tuple[str, str]] = None, initial_checkpoint: Optional[Checkpoint] = None,
                 update_budget: Optional[int] = None, _resume: bool = False):
        self.wf, self.adapters = wf, adapters
        self.plan = adapters.dispatch_plan(wf)                    # raises before anything is written
        self.dispatch_sha256 = adapters.dispatch_identity(wf)
        self.recovery_required = False
        exists = os.path.exists(state_path)
        if _resume and not exists:
            raise NativeHostError(f"{state_path} does not exist: nothing to resume")
        if not _resume and exists:
            raise NativeHostError(f"{state_path} already exists: resume it or choose a fresh state path")
        self.metrics_spec = metrics
        self.writer: Optional[MetricWriter] = None
        self.post_training_executor = NativePostTrainingPhaseExecutor(wf.signature(), self, update_budget)
        registry = ExecutorRegistry()
        routed = _Routed(self)
        for kind in PHASE_KINDS:
            if kind == "sleep":
                registry.register(kind, NativeSleepPhaseExecutor(wf.signature(), self))
            elif kind != "promotion":
                registry.register(kind, routed)
        self.runtime = WorkflowRuntime(wf, registry, AtomicRuntimeCheckpoint(state_path, self.dispatch_sha256),
                                       initial_checkpoint)
        if metrics is not None:
            path, run_id = metrics
            committed = int((self.runtime.state.active or {}).get("metric_records", 0)) if _resume else 0
            committed = max(committed, self._committed_records())
            self.writer = (MetricWriter.resume_from_checkpoint(path, run_id, committed) if _resume
                           else MetricWriter.create(path, run_id))

    @staticmethod
    def start(wf, adapters, state_path, metrics=None, initial_checkpoint=None, update_budget=None):
        return NativeWorkflowHost(wf, adapters, state_path, metrics, initial_checkpoint, update_budget, _resume=False)

    @staticmethod
    def resume(wf, adapters, state_path, metrics=None, update_budget=None):
        return NativeWorkflowHost(wf, adapters, state_path, metrics, None, update_budget, _resume=True)

    def _committed_records(self) -> int:
        done = self.runtime.state.completed
        return int(done[-1].get("metric_records", 0)) if done else 0

    def emit_metric(self, request: Dict[str, Any], event_type: str, values: Dict[str, Any]) -> None:
        if self.writer is None:
            return
        phase = request["phase"]
        self.writer.set_context(self.writer.global_step, request["phase_index"], phase["name"], phase["type"])
        self.writer.emit(event_type, values)

    def run_until_yield_or_complete(self) -> str:
        if self.recovery_required:
            raise NativeHostError("a phase executor failed: reopen the run with NativeWorkflowHost.resume")
        try:
            while not self.runtime.done():
                outcome = self.runtime.run_next_phase()
                if self.writer is not None:
                    self.writer.flush()
                    # the journal length is part of the durable boundary that was just stored
                    st = self.runtime.state
                    if outcome == "committed" and st.completed:
                        st.completed[-1]["metric_records"] = self.writer.sequence
                    elif st.active is not None:
                        st.active["metric_records"] = self.writer.sequence
                    self.runtime.store.store(st)
                if outcome == "yielded":
                    return "yielded"
            return "complete"
        except BaseException:
            self.recovery_required = True
            raise

    def close(self) -> None:
        if self.writer is not None:
            self.writer.close()
