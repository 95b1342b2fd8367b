"""Wake trainer: streams packed samples, accumulates micro-batches, clips, steps the
optimizers, journals metrics, seals checkpoints, resumes exactly.

Loop structure follows `summa-train/src/trainer.rs:1028-2358`: a reader thread feeds a
bounded queue; the main thread builds fixed-shape batches, runs forward/backward per
micro-batch, steps once per accumulation window, emits `optimization` + `throughput`
events, and checkpoints every `checkpoint_every` steps and at phase ends. The LR
schedule is linear warmup then WSD (flat, cosine over the last 10 % down to 0.1·lr) or
cosine (`summa-train/src/main.rs:715-730`); each phase scales it by
`learning_rate_scale`. Non-finite loss or gradient norm aborts the run.
"""
from __future__ import annotations

import fcntl
import hashlib
import json
import math
import os
import queue
import threading
import time
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

import torch

from .. import mal
from ..models import Transformer
from ..models import weights as W
from ..ops import reference as ops_reference
from ..tokenizer import Tokenizer
from . import checkpoint as C
from . import data as D
from .engine import FlatTrainEngine, OptimConfig, checked_norm
from .metrics import MetricWriter, run_id_from_signature, tier_name
from .objectives import objective_loss
from .workflow import Phase, Workflow, fnv1a64, load_workflow, planned_steps, run_signature, wake_plan


@dataclass
class TrainArgs:
    model: str
    tokenizer: str
    workflow: str
    output: str
    lr: float = 3e-4
    weight_decay: float = 0.1
    max_grad_norm: float = 1.0
    warmup_steps: int = 1000
    schedule: str = "wsd"                  # wsd | cosine
    checkpoint_every: int = 500
    seed: int = 42
    checkpoint: Optional[str] = None       # initial weights.safetensors
    resume: bool = False
    optimizer: str = "muon"                # muon (Muon on the block matrices + AdamW on the rest: the reference recipe,
                                           # `summa-train/src/trainer.rs:1118-1129`) | adamw (AdamW on everything)
    device: Optional[str] = None
    init_std: Optional[float] = None
    max_steps_override: Optional[int] = None
    print_run_signature: bool = False
    layer_metrics_every: int = 0                    # per-layer pre-clip gradient norms in every N-th optimization record
    gpu_metrics_interval_ms: Optional[int] = None   # nvidia-smi sampling period; None = 1000 on CUDA, off elsewhere; 0 = off
    gpu_physical_device: str = "0"                  # physical index, GPU UUID or PCI bus id handed to nvidia-smi
    token_cache: bool = True                        # causal phases tokenise once into <output>/.token-cache/ and replay it
    sleep_runtime: Optional[str] = None             # sleep-runtime JSON (periodic shape) for a memory-enabled model ...
    sleep_runtime_sha256: Optional[str] = None      # ... and the `sha256:` identity of its bytes; both or neither


def lr_at(step: int, total: int, base: float, warmup: int, schedule: str) -> float:
    """Learning rate for optimizer step `step` (0-based) of `total`."""
    if warmup > 0 and step < warmup:
        return base * (step + 1) / warmup
    if schedule == "cosine":
        span = max(1, total - warmup)
        prog = min(1.0, (step - warmup) / span)
        return base * (0.1 + 0.9 * 0.5 * (1.0 + math.cos(math.pi * prog)))
    decay_start = int(total * 0.9)
    if step < decay_start:
        return base
    prog = min(1.0, (step - decay_start) / max(1, total - decay_start))
    return base * (0.1 + 0.9 * 0.5 * (1.0 + math.cos(math.pi * prog)))


class OutputLock:
    """Single-writer lock on the output directory (flock on `.trainer.lock`)."""

    def __init__(self, out_dir: str):
        os.makedirs(out_dir, exist_ok=True)
        self.f = open(os.path.join(out_dir, ".trainer.lock"), "w")
        try:
            fcntl.flock(self.f, fcntl.LOCK_EX | fcntl.LOCK_NB)
        except OSError:
            raise RuntimeError(f"{out_dir} is locked by another trainer")

    def release(self):
        fcntl.flock(self.f, fcntl.LOCK_UN)
        self.f.close()


def splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & 0xFFFFFFFFFFFFFFFF
    z = x
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & 0xFFFFFFFFFFFFFFFF
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & 0xFFFFFFFFFFFFFFFF
    return z ^ (z >> 31)


class _NullWriter:
    """Metric writer of the ranks that do not own the journal."""
    sequence = 0

    def set_context(self, *a): pass
    def emit(self, *a, **k): pass
    def phase_timing(self, *a, **k): pass
    def flush(self): pass
    def close(self): pass


class _DistContext:
    """Data-parallel launch (`torch.distributed.run` sets WORLD_SIZE / RANK / LOCAL_RANK): one
    process per GPU over NCCL, or gloo ranks on CPU. Rank 0 owns the output directory (lock,
    metrics journal, checkpoints); every micro-batch of `batch_size` samples is cut into equal
    per-rank slices, so the recipe's global batch and its losses do not depend on the rank count."""

    def __init__(self, rank=0, world=1, device=None, dp=None):
        self.rank, self.world, self.device, self.dp = rank, world, device, dp
        self.heartbeat = None

    def start_heartbeat(self, out_dir: str) -> None:
        """Per-rank pulse files under the output directory (one node, shared file system). The step loop
        calls `guard` before each optimizer step, so a rank that has gone away is noticed on the host and
        no kernel is launched that would wait for its flags."""
        if self.world <= 1 or os.environ.get("SUMMA_HEARTBEAT", "1") != "1":
            return
        from ..parallel.health import Heartbeat
        timeout = float(os.environ.get("SUMMA_HEARTBEAT_TIMEOUT", "30"))
        self.heartbeat = Heartbeat(self.rank, self.world, directory=os.path.join(out_dir, ".heartbeat"),
                                   interval=min(1.0, timeout / 10), timeout=timeout).start()
        self.barrier()           # every rank has overwritten what an earlier run left in its pulse file

    def guard(self, step: int) -> None:
        if self.heartbeat is not None:
            self.heartbeat.guard(step)

    @staticmethod
    def from_env(device_arg) -> "_DistContext":
        world = int(os.environ.get("WORLD_SIZE", "1"))
        if world <= 1:
            return _DistContext(device=torch.device(device_arg or ("cuda" if torch.cuda.is_available() else "cpu")))
        import torch.distributed as dist
        from ..parallel.dp import DataParallelGroup
        local = int(os.environ.get("LOCAL_RANK", "0"))
        use_cuda = (device_arg or "cuda").startswith("cuda") and torch.cuda.is_available()
        if use_cuda:
            torch.cuda.set_device(local)
            device = torch.device("cuda", local)
        else:
            device = torch.device("cpu")
        if not dist.is_initialized():
            dist.init_process_group("nccl" if use_cuda else "gloo", device_id=device if use_cuda else None)
        return _DistContext(dist.get_rank(), dist.get_world_size(), device, DataParallelGroup(dist.group.WORLD, device))

    def mean(self, value: float) -> float:
        if self.world == 1:
            return value
        import torch.distributed as dist
        t = torch.tensor([value], dtype=torch.float64 if self.device.type == "cpu" else torch.float32,
                         device=self.device)
        dist.all_reduce(t)
        return float(t) / self.world

    def barrier(self) -> None:
        if self.world > 1:
            self.dp.barrier()

    def close(self) -> None:
        if self.heartbeat is not None:
            self.heartbeat.leave()
        if self.world > 1:
            import torch.distributed as dist
            if dist.is_initialized():
                dist.destroy_process_group()


class _MemoryPolicy:
    """Update policy of a memory-chain model (`summa-train/src/trainer.rs:1861-1883,1965-1995`,
    `summa-train/src/tier_optimizer.rs:263-404`): the tiers' parameters stay out of the wake optimizer;
    their gradients accumulate per tier in a `TierOptimizerBank` and are used at the tier's boundary
    (global step divisible by its `update_period`):

      memory_update_mode {type: wake_only}   the due tier takes its own averaged update directly
      periodic_sleep                         the due tier is consolidated into the next slower one by a
                                             persisted `ConsolidationTxn` with the built-in handlers
                                             (a rejected transaction leaves the update pending); the
                                             slowest tier takes its update directly and, when the schedule
                                             asks for it, folds its reserve slots into its base FFN
    """

    def __init__(self, model, spec: Dict[str, Any], mode: str, out_dir: str, dctx, runtime=None):
        """`runtime`: the operator's sleep-runtime file (`sleep_runtime.SleepRuntimeConfig`, periodic shape). It
        overrides the tier optimizer's hyper-parameters, the rollout and dreaming settings, the size of the wake-context
        ring and the number of RNG streams, and names the directories of the boundary state and rejection reports."""
        from . import sleep as S
        self.S, self.model, self.mode, self.dctx, self.out_dir = S, model, mode, dctx, out_dir
        self.runtime = runtime if mode == "sleep" else None
        sched = spec["schedule"]
        self.periods = [int(t["update_period"]) for t in sched["tiers"]]
        self.schedule = S.TierSchedule(self.periods)
        self.terminal = sched.get("terminal_consolidation")
        topt = spec.get("tier_optimizer") or {}
        if self.runtime is not None:
            t = self.runtime.tier_optimizer
            topt = {"learning_rate": t.learning_rate, "beta_1": t.beta_1, "beta_2": t.beta_2, "epsilon": t.epsilon, "weight_decay": t.weight_decay}
        lr = float(topt.get("learning_rate", spec.get("receiver_learning_rate", 3e-4)))
        self.bank = S.TierOptimizerBank(model.named_parameters(), lr=lr,
                                        betas=(float(topt.get("beta_1", 0.9)), float(topt.get("beta_2", 0.95))),
                                        eps=float(topt.get("epsilon", 1e-8)),
                                        weight_decay=float(topt.get("weight_decay", spec.get("receiver_weight_decay", 0.0))))
        if sorted(self.bank.params) != list(range(len(self.periods))):
            raise RuntimeError(f"the schedule names {len(self.periods)} memory tiers, the model has {len(self.bank.params)}")
        self.spec = spec
        self.replay: List[torch.Tensor] = []
        self.state_dir = os.path.join(out_dir, "sleep")
        self.replay_capacity = self.runtime.max_wake_context_records if self.runtime is not None else 6
        self.sleep_state = None
        if mode == "sleep":
            self._init_sleep_state()

    @staticmethod
    def owns(name: str) -> bool:
        from .sleep import tier_of_parameter
        return tier_of_parameter(name) is not None

    def verify_optimizer_scopes(self, state) -> None:
        """The tier bundles a wake-only checkpoint names must exist, hash to their identity and hold exactly the tier state
        the generation's optimizer container restored."""
        scopes = (state.memory_update or {}).get("optimizer_scopes") if isinstance(state.memory_update, dict) else None
        for sc in (scopes or {}).get("tiers", []):
            art = sc.get("artifact")
            if not art:
                continue
            path = os.path.join(self.out_dir, "tier-optimizers", art["path"])
            if not os.path.isfile(path):
                raise RuntimeError(f"tier optimizer bundle {art['path']} named by the checkpoint is missing")
            with open(path, "rb") as f:
                body = f.read()
            if "sha256:" + hashlib.sha256(body).hexdigest() != art["sha256"]:
                raise RuntimeError(f"tier optimizer bundle {art['path']} does not match its recorded identity")
            if body != self.bank.snapshot_bytes(sc["tier"]):
                raise RuntimeError(f"tier {sc['tier']}: the optimizer container and the tier bundle of the checkpoint disagree")

    def stamp_training_state(self, state) -> None:
        """Checkpoint-bound memory strategy (`summa-train/src/checkpoint.rs:255-267`) and one optimizer scope per tier
        with its own clock; the tier moments, masters and pending accumulators travel inside `adamw-state.bpk`."""
        ident = lambda name: int.from_bytes(hashlib.sha256(name.encode()).digest()[:8], "big")
        if self.dctx.rank == 0:                 # one immutable bundle per tier beside the generations; the scopes name them
            tiers = self.bank.publish_checkpoint_scopes(os.path.join(self.out_dir, "tier-optimizers"), ident)["tiers"]
        else:
            clocks = self.bank.clocks()
            tiers = [{"tier": t, "parameter_ids": sorted(ident(n) for n, _ in self.bank.params[t]), "update_clock": clocks[t],
                      "accumulated_micro_steps": self.bank.state[t]["count"], "artifact": None} for t in sorted(self.bank.params)]
        if self.mode == "wake_only":
            owned = {i for t in tiers for i in t["parameter_ids"]}
            wake = sorted(ident(n) for n, _ in self.model.named_parameters() if ident(n) not in owned)
            state.memory_update = {"type": "wake_only", "config": json.loads(json.dumps(self.spec)),
                                   "optimizer_scopes": {"wake_parameter_ids": wake, "tiers": tiers}}
        else:
            state.memory_update = {"type": "periodic_sleep"}
        state.optimizer_states = [r for r in state.optimizer_states if not r.get("scope", "").startswith("tier")] + [
            {"scope": f"tier{t['tier']}", "adamw": "adamw-state.bpk", "muon": "muon-state.bpk",
             "gradient_accumulator": (t["artifact"] or {}).get("path", "adamw-state.bpk"), "update_clock": t["update_clock"]} for t in tiers]

    def after_backward(self) -> None:
        reduce = None
        if self.dctx.world > 1:
            import torch.distributed as dist
            world = self.dctx.world

            def reduce(g):
                dist.all_reduce(g)
                g.div_(world)
        for t in self.bank.params:
            self.bank.accumulate(t, reduce, staged=True)

    def before_step(self, engine) -> None:
        """The tier scopes join the step's ONE global gradient norm: their staged window, in the flat buffers' units
        (summed over ranks; the tier gradients are already rank means)."""
        sq = self.bank.window_sumsq()
        engine.extra_sumsq = None if sq is None else sq * float(self.dctx.world) ** 2

    def commit_window(self, norm: float, max_grad_norm: float) -> None:
        coefficient = min(1.0, max_grad_norm / (norm + 1e-6)) if max_grad_norm > 0 else 1.0
        self.bank.commit_window(coefficient)

    def remember(self, tokens: torch.Tensor) -> None:
        if self.runtime is not None:
            tokens = tokens[:, :self.runtime.rollouts.max_context_tokens]
        self.replay.append(tokens.detach())
        del self.replay[:-self.replay_capacity]

    def consolidation_config(self):
        from .builtin_sleep import ConsolidationConfig
        sp, c = self.spec, ConsolidationConfig()
        ks, im, rt = sp.get("knowledge_seeding") or {}, sp.get("imitation") or {}, sp.get("retention") or {}
        c.kl_chunk_rows = int(ks.get("chunk_tokens", c.kl_chunk_rows))
        c.seeding_steps = int(ks.get("teacher_rollouts", c.seeding_steps))
        c.seeding_lr = float(sp.get("receiver_learning_rate", c.seeding_lr))
        c.imitation_lr = float(sp.get("receiver_learning_rate", c.imitation_lr))
        c.imitation_group = int(im.get("grpo_group_size", c.imitation_group))
        c.gamma = float(im.get("semantic_weight", c.gamma))
        c.imitation_temperature = float(ks.get("temperature", c.imitation_temperature))
        c.max_anchor_kl = float(rt.get("max_anchor_forward_kl", c.max_anchor_kl))
        c.min_incorporation_gain = float(rt.get("min_incorporation_gain", c.min_incorporation_gain))
        if self.runtime is not None:
            r = self.runtime.rollouts
            c.imitation_new_tokens = r.continuation_tokens
            c.imitation_temperature = r.temperature
            c.imitation_steps = max(c.imitation_steps, r.imitation_groups)
        return c

    # ------------------------------------------------------------------ periodic sleep on the durable state machine
    def _init_sleep_state(self) -> None:
        from . import sleep_state as SS
        self.SS = SS
        self.sleep_schedule = SS.SleepSchedule.from_json(self.spec["schedule"])
        for blk in self.model.layers:
            mem = getattr(blk, "memory", None)
            if mem is None:
                continue
            for t, tier in enumerate(self.sleep_schedule.tiers):
                have = len(mem.tiers[t].reserve.slots) if mem.tiers[t].reserve is not None else 0
                if have != tier.reserve_slots:
                    raise RuntimeError(f"memory tier `{tier.id}` schedules {tier.reserve_slots} reserve slots, the model has {have}")
        self.sleep_state = SS.SleepState(self.sleep_schedule, self.runtime.rng_streams if self.runtime is not None else 1)

    def sleep_state_json(self) -> Optional[Dict[str, Any]]:
        return self.sleep_state.to_json() if self.sleep_state is not None else None

    def load_sleep_state(self, data: Optional[Dict[str, Any]]) -> None:
        if self.sleep_state is None or not data:
            return
        st = self.SS.SleepState.from_json(data)
        if [t.id for t in st.tiers] != [t.id for t in self.sleep_schedule.tiers]:
            raise RuntimeError("the checkpoint's sleep state names other memory tiers than the workflow's schedule")
        if st.pending is not None:
            # checkpoints are sealed between steps, so a pending transaction is foreign; its tensors are gone and the
            # checkpoint's weights ARE its teacher: retire the attempt (the id stays consumed)
            if st.pending.committed:
                raise RuntimeError("the checkpoint's sleep state holds a committed but unfinished transaction")
            st.rollback()
        from .builtin_sleep import validate_model_memory_state
        validate_model_memory_state(self.model, st)
        self.sleep_state = st

    def _persist_sleep_state(self, state) -> None:
        if self.dctx.rank != 0:
            return
        os.makedirs(self.state_dir, exist_ok=True)
        tmp = os.path.join(self.state_dir, "state.json.tmp")
        with open(tmp, "w") as f:
            json.dump(state.to_json(), f, sort_keys=True)
            f.flush()
            os.fsync(f.fileno())
        os.replace(tmp, os.path.join(self.state_dir, "state.json"))

    def _drain_sleep(self, writer, emit) -> None:
        """Every queued boundary as one transaction of the durable state machine (`builtin_sleep.drain_due_boundaries`);
        the sleep state is persisted after each step and every boundary emits its `tier_update`."""
        from .builtin_sleep import drain_due_boundaries
        policy = self

        class Progress:
            def persist(self, state):
                policy._persist_sleep_state(state)

            def metric(self, kind, fields):
                writer.emit(kind, fields)

        distil = bool(self.terminal) and str(self.terminal).lower() not in ("none", "disabled", "off")
        for b in drain_due_boundaries(self.model, self.bank, self.sleep_state, self.replay, self.consolidation_config(),
                                      terminal_distil=distil, dreaming=self.spec.get("dreaming"),
                                      runtime=self.runtime, progress=Progress(), location="memory://wake", write_reports=self.dctx.rank == 0):
            emit(b["sender"], b["trigger"], "committed" if b["ok"] else "rolled_back", f"sleep-{b['transaction_id']}", b["slot"], b["generation"])
        self.model.train()

    def after_step(self, clock: int, writer) -> None:
        last = len(self.periods) - 1
        n_tiers = len(self.periods)

        def emit(t, tier_clock, outcome, txn_id, slot=None, generation=None):
            consolidated = self.mode != "wake_only" and t < last
            writer.emit("tier_update", {
                "transaction_id": txn_id, "tier": tier_name(t, n_tiers),
                "receiver_tier": tier_name(t + 1, n_tiers) if consolidated else None,
                "tier_clock": tier_clock, "update_period": self.periods[t], "accumulated_micro_steps": self.periods[t],
                "outcome": outcome, "reserve_slot": slot, "reserve_generation": generation, "optimizer_state_reset": False})

        if self.mode == "wake_only":
            for t in self.schedule.due_senders(clock):
                self.bank.apply(t)
                emit(t, clock, "committed", f"clock-{clock}-tier-{t}-applied")
            return
        st = self.sleep_state
        if st.clock > clock:
            raise RuntimeError(f"the sleep state is at clock {st.clock}, ahead of the training clock {clock}")
        self._drain_sleep(writer, emit)                    # boundaries left over from before a resume
        scheduled = self.sleep_schedule.due_senders(clock) if clock > st.clock else []
        st.advance_clock(self.sleep_schedule, clock)
        queued = {s for _, s in st.due}
        for t in scheduled:
            if t not in queued:                            # held back behind a rejected terminal boundary
                emit(t, clock, "skipped", f"clock-{clock}-tier-{t}-held-back")
        self._drain_sleep(writer, emit)


def train(args: TrainArgs) -> Dict[str, Any]:
    wf = load_workflow(args.workflow)
    phases = wake_plan(wf)
    tok = Tokenizer.from_file(args.tokenizer)
    cfg = mal.load_model_def(args.model)
    cfg.vocab_size = tok.vocab_size()           # the tokenizer defines the vocabulary
    eos = tok.eos_id()
    if eos is None:
        raise RuntimeError("tokenizer has no end-of-sequence token")
    from .workflow import WorkflowError, validate_against_model
    validate_against_model(wf, cfg)             # the workflow and the exact MAL topology form one executable recipe
    args._phase_steps = [_select_phase_steps(p, tok, cfg.vocab_size, eos, args.seed) for p in phases]
    first_step = 0
    for p, n in zip(phases, args._phase_steps): # quantization phases must reach their target codec inside their own window
        if p.kind == "quantization" and p.quantization is not None:
            try:
                p.quantization.validate_phase_window(first_step, n)
            except WorkflowError as e:
                raise WorkflowError(f"workflow quantization phase `{p.name}` never trains its target format: {e}")
        first_step += n
    tok_sha = D.file_sha256(args.tokenizer)
    data_ids = [D.file_sha256(p.data) for p in phases]
    # Everything that changes what the run writes is part of its identity: the optimizer, the initial checkpoint's
    # bytes (a fine-tune resumes only from the same starting point) and explicit telemetry settings (they decide which
    # metric records exist); the output location is not.
    extra: Dict[str, Any] = {"optimizer": args.optimizer}
    if args.checkpoint:
        extra["initial_checkpoint_sha256"] = D.file_sha256(args.checkpoint)
    if args.gpu_metrics_interval_ms is not None and 0 < args.gpu_metrics_interval_ms < 100:
        raise RuntimeError("--gpu-metrics-interval-ms must be 0 (disabled) or at least 100")
    if args.gpu_metrics_interval_ms is not None or args.gpu_physical_device != "0":
        extra["device_telemetry"] = {"interval_ms": args.gpu_metrics_interval_ms, "physical_device": args.gpu_physical_device}
    if args.layer_metrics_every > 0:
        extra["layer_metrics_every"] = args.layer_metrics_every
    signature = run_signature(wf, cfg.to_json(), tok_sha, data_ids, args.seed, args.lr, args.weight_decay,
                              args.max_grad_norm, args.warmup_steps, args.schedule, 20.0, extra)
    if args.print_run_signature:
        print(signature)
        return {"run_signature": signature}
    if (args.sleep_runtime is None) != (args.sleep_runtime_sha256 is None):
        raise RuntimeError("--sleep-runtime and --sleep-runtime-sha256 go together")
    args._sleep_runtime = None
    if args.sleep_runtime is not None:
        # the runtime file is bound to THIS run: its workflow_signature is what --print-run-signature prints
        from .sleep_runtime import load_sleep_runtime
        rt = load_sleep_runtime(args.sleep_runtime, args.sleep_runtime_sha256, "periodic")
        if rt.workflow_signature != "sha256:" + signature:
            raise RuntimeError(f"sleep runtime {args.sleep_runtime} is bound to workflow signature {rt.workflow_signature}, "
                               f"this run's is sha256:{signature}")
        if not any(p.periodic_sleep for p in phases):
            raise RuntimeError("--sleep-runtime was given but no phase of the workflow configures periodic sleep")
        model_bytes = rt.pins["model_mal"].verify_bytes()
        if hashlib.sha256(model_bytes).hexdigest() != D.file_sha256(args.model):
            raise RuntimeError("the sleep runtime pins another model file than --model")
        args._sleep_runtime = rt
    args._cache_identities = {"data": data_ids, "tokenizer": tok_sha}
    dctx = _DistContext.from_env(args.device)
    lock = OutputLock(args.output) if dctx.rank == 0 else None
    try:
        return _train_locked(args, wf, phases, tok, cfg, eos, signature, data_ids, dctx)
    finally:
        if lock is not None:
            lock.release()
        dctx.close()


def _train_locked(args, wf: Workflow, phases: List[Phase], tok, cfg, eos, signature, data_ids, dctx=None):
    out = args.output
    dctx = dctx or _DistContext(device=torch.device(args.device or ("cuda" if torch.cuda.is_available() else "cpu")))
    device = dctx.device
    for ph in phases:
        if dctx.world > 1 and ph.batch_size and ph.batch_size % dctx.world:
            raise RuntimeError(f"phase `{ph.name}`: batch_size {ph.batch_size} is not divisible by {dctx.world} ranks")
    torch.manual_seed(args.seed)
    model = Transformer(cfg, init_std=args.init_std)
    if args.checkpoint:
        W.load_safetensors(model, args.checkpoint)
    model = model.to(device)
    use_bf16 = device.type == "cuda"
    if use_bf16:
        model.stream_dtype = torch.bfloat16
    ocfg = OptimConfig(lr=args.lr, weight_decay=args.weight_decay, max_grad_norm=args.max_grad_norm)
    mem_policy = None
    if any(getattr(blk, "memory", None) is not None for blk in model.layers):
        spec = next(((p.periodic_sleep, "sleep") for p in phases if p.periodic_sleep), None) or \
            next(((p.memory_update_mode, "wake_only") for p in phases if p.memory_update_mode), None)
        if spec is not None:
            mem_policy = _MemoryPolicy(model, spec[0], spec[1], out, dctx, runtime=getattr(args, "_sleep_runtime", None))
    engine = FlatTrainEngine(model, ocfg, dp=dctx.dp, param_dtype=torch.bfloat16 if use_bf16 else torch.float32,
                             muon=(args.optimizer == "muon"),
                             exclude=_MemoryPolicy.owns if mem_policy is not None else None)
    engine.dctx = dctx
    dctx.start_heartbeat(out)
    # read-only nvidia-smi telemetry child of the journal's owner (`summa-train/src/main.rs:1245-1318`): fail-soft
    interval_ms = args.gpu_metrics_interval_ms
    if interval_ms is None:
        interval_ms = 1000 if device.type == "cuda" else 0
    engine.device_sampler = None
    if interval_ms > 0 and dctx.rank == 0 and device.type == "cuda":
        from .device_sampler import NvidiaSmiSampler
        engine.device_sampler = NvidiaSmiSampler(interval_ms / 1000.0, args.gpu_physical_device)
        engine.device_sampler_window = interval_ms / 1000.0
    engine.mem_policy = mem_policy
    if mem_policy is not None:
        engine.extra_state = mem_policy.bank.state_tensors
    run_id = run_id_from_signature(signature)
    if dctx.rank == 0:
        with open(os.path.join(out, "config.json"), "w") as f:
            f.write(cfg.to_json_str())
        with open(os.path.join(out, "resolved-workflow.json"), "w") as f:
            json.dump(wf.to_json(), f, indent=2)

    state = C.TrainingState(workflow_signature=signature, data_manifest_hash=data_ids[0] if data_ids else None)
    metrics_path = os.path.join(out, "metrics.jsonl")
    if args.resume and C.read_current(out) is not None:
        state, adamw_bytes, muon_bytes, gen = C.load_training_state(out, model)
        if state.workflow_signature != signature:
            raise RuntimeError("run signature differs from the checkpoint's: refusing to resume; a run started from `--checkpoint` "
                               "must repeat the same `--checkpoint` when resuming, because the initial checkpoint identity is "
                               "part of the run signature")
        engine.load_packed(adamw_bytes, muon_bytes)
        engine.resync_from_model()
        _authenticate_candidates(state, cfg)
        if mem_policy is not None:
            mem_policy.bank.resync()
            mem_policy.bank.load_state_tensors(engine.loaded_extra)
            mem_policy.verify_optimizer_scopes(state)
            mem_policy.load_sleep_state(state.sleep)
        dctx.barrier()                       # every rank has read the generation before rank 0 appends to the journal
        writer = (MetricWriter.resume_from_checkpoint(metrics_path, run_id, state.metric_records)
                  if dctx.rank == 0 else _NullWriter())
        writer.set_context(state.global_step, min(state.phase, len(phases) - 1),
                           phases[min(state.phase, len(phases) - 1)].name, phases[min(state.phase, len(phases) - 1)].kind)
    else:
        writer = MetricWriter.create(metrics_path, run_id) if dctx.rank == 0 else _NullWriter()

    total_steps = sum(args._phase_steps)
    last_loss = None
    t_run = time.time()
    for pi, phase in enumerate(phases):
        if pi < state.phase:
            continue
        steps_full = args._phase_steps[pi]
        steps_planned = steps_full
        if args.max_steps_override is not None:
            steps_planned = min(steps_full, args.max_steps_override)
        seq, bs, ga = phase.sequence_length, phase.batch_size, phase.grad_accum_or_default()
        writer.set_context(state.global_step, pi, phase.name, phase.kind)
        state.phase_id, state.phase_kind = phase.name, phase.kind
        t_phase = time.time()
        if state.steps_in_phase == 0:
            writer.phase_timing("started", 0.0)
        epoch = state.epoch
        while state.steps_in_phase < steps_planned and epoch < phase.epochs_or_default():
            last_loss = _run_epoch(args, model, engine, writer, state, phase, pi, epoch, tok, cfg, eos, device,
                                   steps_planned, total_steps, out)
            if state.steps_in_phase < steps_planned:
                epoch += 1
                state.epoch = epoch
                state.records_in_phase = 0
        if steps_planned < steps_full:
            # stopped early on request (as a preempted run would be): keep the phase open
            _checkpoint(out, model, engine, state, writer, t_run)
            writer.close()
            return {"global_step": state.global_step, "tokens_seen": state.tokens_seen, "final_loss": last_loss,
                    "run_signature": signature, "generation": C.read_current(out), "stopped_early": True}
        writer.phase_timing("completed", time.time() - t_phase)
        if phase.kind == "quantization" and dctx.rank == 0:
            pub = _publish_qat_candidate(out, model, cfg, phase, pi, state)
            q, m = phase.quantization, pub.metrics
            writer.emit("quantization", {
                "stage": "export", "format": q.format, "group_size": q.group_size, "progress_fraction": 1.0,
                "tensors_quantized": int(m["quantized_tensors"]), "weights_quantized": int(m["quantized_elements"]),
                "average_bits_per_weight": float(m["average_bits_per_weight"]), "packed_bytes": int(m["packed_bytes"]),
                "mean_squared_error": float(m["weighted_mean_squared_error"]), "max_absolute_error": float(m["maximum_absolute_error"]),
                "embeddings_quantized": bool(q.embeddings), "lm_head_quantized": bool(q.lm_head)})
            # the sealed generation names the candidate it produced: a resume authenticates it instead of replaying the phase
            state.quantization = {"format": q.format, "fake_quant_active": False, "calibration_step": state.global_step,
                                  "manifest": pub.candidate_manifest_path, "candidate_weights_sha256": pub.weights_sha256,
                                  "teacher_hash": (q.training or {}).get("teacher_sha256")}
            state.artifacts = [a for a in state.artifacts if a.get("manifest") != pub.candidate_manifest_path] + [
                {"kind": "hquant_candidate", "manifest": pub.candidate_manifest_path, "hash": pub.candidate_manifest_sha256}]
        state.phase = pi + 1
        state.phase_id = phase.name
        state.epoch = 0
        state.records_in_phase = 0
        state.steps_in_phase = 0
        _checkpoint(out, model, engine, state, writer, t_run)
    if getattr(engine, "device_sampler", None) is not None:
        _drain_device_sampler(engine, writer)
        engine.device_sampler.close()
    writer.close()
    return {"global_step": state.global_step, "tokens_seen": state.tokens_seen, "final_loss": last_loss,
            "run_signature": signature, "generation": C.read_current(out)}


def _drain_device_sampler(engine, writer) -> None:
    """Queued nvidia-smi samples become `device_utilization` records; a sampler problem is a warning, never
    a training failure."""
    sampler = getattr(engine, "device_sampler", None)
    if sampler is None:
        return
    drained = sampler.drain()
    for msg in drained.diagnostics:
        print(f"warning: GPU utilization sampler: {msg}", flush=True)
    now_ms = int(time.time() * 1000)
    for smp in drained.samples:
        values = smp.as_metric(0, engine.device_sampler_window)
        values["sampled_at_unix_ms"] = min(values["sampled_at_unix_ms"], now_ms)
        if values["memory_used_bytes"] > values["memory_total_bytes"]:
            continue
        try:
            writer.emit("device_utilization", values)
        except ValueError as e:
            print(f"warning: GPU utilization sample dropped: {e}", flush=True)


def _checkpoint(out, model, engine, state, writer, t_run):
    if getattr(engine, "mem_policy", None) is not None:
        engine.mem_policy.stamp_training_state(state)
    if getattr(engine, "mem_policy", None) is not None and engine.mem_policy.sleep_state is not None:
        state.sleep = engine.mem_policy.sleep_state_json()       # the durable sleep state travels inside the sealed generation
    writer.flush()
    state.metric_records = writer.sequence
    adamw, muon = engine.pack_state()            # collective under data parallelism
    dctx = getattr(engine, "dctx", None)
    if dctx is not None and dctx.rank != 0:
        dctx.barrier()                           # rank 0 publishes the generation
        return None
    gen = _write_checkpoint(out, model, state, adamw, muon, writer, t_run)
    if dctx is not None:
        dctx.barrier()
    return gen


def _write_checkpoint(out, model, state, adamw, muon, writer, t_run):
    stored, active = model.parameter_accounting()
    t_save = time.time()
    gen = C.save_training_checkpoint(out, model, state, adamw, muon,
                                     {"training_gpu_hours": (time.time() - t_run) / 3600.0, "parameters": stored,
                                      "routed_active_parameters": active})
    # a sealed generation is a progress boundary of the phase; the record carries the generation's identity
    dt_save = time.time() - t_save
    writer.phase_timing("progress", dt_save, checkpoint=dt_save, checkpoint_hash=gen.replace("sha256-", "sha256:", 1))
    writer.flush()
    state.metric_records = writer.sequence
    return gen


_NVTX = os.environ.get("SUMMA_NVTX", "0") == "1"


def _nvtx_push(name: str) -> None:
    """NVTX ranges around micro-batches and optimizer steps (SUMMA_NVTX=1) for external profilers."""
    if _NVTX and torch.cuda.is_available():
        torch.cuda.nvtx.range_push(name)


def _nvtx_pop() -> None:
    if _NVTX and torch.cuda.is_available():
        torch.cuda.nvtx.range_pop()


def _authenticate_candidates(state, cfg) -> None:
    """Every sealed candidate a checkpoint names must still be the one it named: receipt, weights, archive and the
    manifest's own hash (`summa-train/tests/trainer_lifecycle.rs:563-690`)."""
    from . import qat_candidate as QC
    for art in state.artifacts:
        if art.get("kind") != "hquant_candidate":
            continue
        pub = QC.open_candidate(os.path.dirname(art["manifest"]), lambda: Transformer(cfg))
        if pub.candidate_manifest_sha256 != art["hash"]:
            raise RuntimeError(f"quantization candidate {art['manifest']} is not the one the checkpoint sealed")
    q = state.quantization
    if q and q.get("manifest") and not any(a.get("manifest") == q["manifest"] for a in state.artifacts):
        raise RuntimeError("the checkpoint's quantization state names a candidate that its artifact list does not")


def _publish_qat_candidate(out, model, cfg, phase, pi, state):
    """The weights a quantisation phase ends with, sealed with their archive as a write-once
    candidate under `<out>/quantized-candidates/` (a resumed run that reaches this point again adopts
    the existing candidate)."""
    from . import qat_candidate as QC
    key = f"{phase.name}.step-{state.global_step}"
    try:
        QC.validate_candidate_key(key)
    except QC.CandidateError:
        key = f"phase-{pi}.step-{state.global_step}"
    q = phase.quantization
    return QC.publish(model, os.path.join(out, "quantized-candidates"), key, QC.Recipe(q.format, q.embeddings, q.lm_head),
                      lambda: Transformer(cfg))


def _load_quantization_teacher(training, cfg, device, student):
    """Frozen full-precision teacher of a quantisation-distillation phase; its file must hash to
    the recorded identity."""
    import hashlib
    path = training["teacher_checkpoint"]
    if os.path.islink(path) or not os.path.isfile(path):
        raise RuntimeError(f"quantization teacher {path} must be a regular file (symbolic links are refused)")
    with open(path, "rb") as f:
        digest = hashlib.sha256(f.read()).hexdigest()
    if training.get("teacher_sha256") and digest != training["teacher_sha256"].removeprefix("sha256:"):
        raise RuntimeError(f"quantization teacher {path} hashes to {digest}, expected {training['teacher_sha256']}")
    teacher = Transformer(cfg)
    W.load_safetensors(teacher, path)
    teacher = teacher.to(device).eval()
    teacher.stream_dtype = student.stream_dtype
    for p in teacher.parameters():
        p.requires_grad_(False)
    return teacher


def _distilled_loss(model, teacher, training, phase, samples, device):
    """(task loss, router aux, tokens, forward KL to the teacher at temperature T, scaled by T^2):
    the student's logits come from the same forward that produced the task loss
    (`summa-train/src/trainer.rs:1779-1845`)."""
    from .objectives import forward_kl
    if phase.task.type != "causal_lm":
        raise RuntimeError("quantization distillation supports causal_lm phases")
    x = torch.tensor(samples, dtype=torch.int64, device=device)
    inp, tgt = x[:, :-1], x[:, 1:]
    hidden, aux = model.forward_hidden(inp)
    flat = hidden.reshape(-1, hidden.shape[-1])
    loss, logits = ops_reference.linear_cross_entropy(flat, model.output_weight(), model.output_bias(),
                                                     tgt.reshape(-1), model.cfg.vocab_size, 4, return_logits=True)
    with torch.no_grad():
        t_logits = teacher(inp).reshape(-1, logits.shape[-1])
    kl = forward_kl(logits, t_logits, training["temperature"], scale_by_t2=True)
    return loss, (aux if aux is not None else loss.new_zeros(())), inp.numel(), kl


def _run_epoch(args, model, engine, writer, state, phase, pi, epoch, tok, cfg, eos, device, steps_planned,
               total_steps, out):
    seq, bs, ga = phase.sequence_length, phase.batch_size, phase.grad_accum_or_default()
    dctx = getattr(engine, "dctx", None) or _DistContext(device=device)
    seed = D.shuffle_seed(args.seed, pi, epoch)
    q: "queue.Queue" = queue.Queue(maxsize=min(4096, 2 * bs))
    stop = threading.Event()

    # causal phases tokenise their source once into `<output>/.token-cache/` and replay it on later epochs and resumes
    # (`summa-train/src/trainer.rs:1088-1098,1628-1650`)
    token_cache = None
    ids = getattr(args, "_cache_identities", None)
    if ids is not None and phase.task.type == "causal_lm" and getattr(args, "token_cache", True):
        from .token_cache import token_cache_path
        token_cache = token_cache_path(os.path.join(out, ".token-cache"), ids["data"][pi], phase.data, ids["tokenizer"],
                                       cfg.vocab_size, dctx.rank, dctx.world)

    def reader():
        try:
            for s in objective_sample_stream(phase, tok, cfg.vocab_size, seq, eos, seed, state.records_in_phase, token_cache):
                if stop.is_set():
                    return
                q.put(s)
        except BaseException as e:      # surfaced on the main thread
            q.put(e)
        q.put(None)

    th = threading.Thread(target=reader, daemon=True)
    th.start()
    qplan = phase.quantization if phase.kind == "quantization" else None
    qnames, teacher, window_fmt, window_count = [], None, None, 0
    if qplan is not None:
        from . import quantization as Q
        qnames = Q.qat_parameter_names(model, qplan.embeddings, qplan.lm_head)
        if qplan.training["type"] == "distillation":
            teacher = _load_quantization_teacher(qplan.training, cfg, device, model)
    model.train()
    micro: List[Any] = []
    window_loss, window_aux, micro_done = 0.0, 0.0, 0
    window_supervised = 0
    qweights = 0
    if qplan is not None:
        named = dict(model.named_parameters())
        qweights = sum(named[n].numel() for n in qnames)
    last = None
    t_step = time.time()
    input_wait = gpu_busy = 0.0
    engine.zero_grad()
    try:
        while state.steps_in_phase < steps_planned:
            t0 = time.time()
            item = q.get()
            input_wait += time.time() - t0
            if item is None:
                break
            if isinstance(item, BaseException):
                raise item
            micro.append(item)
            state.records_in_phase += 1
            if len(micro) < bs:
                continue
            if dctx.world > 1:                   # this rank's slice of the global micro-batch
                per = bs // dctx.world
                micro = micro[dctx.rank * per:(dctx.rank + 1) * per]
            # dropout determinism: seed from a checkpointed counter
            torch.manual_seed(splitmix64(args.seed ^ (state.global_step * 1000003 + micro_done)) & 0x7FFFFFFF)
            if qplan is not None and micro_done == 0:
                # one fake-quantised set of compute weights per accumulation window
                window_fmt = qplan.format_at(state.global_step)
                window_count = engine.begin_quantized_window(window_fmt, qnames) if window_fmt else 0
            t_busy0 = time.time()
            _nvtx_push("micro_batch")
            if micro_done == ga - 1:
                engine.arm_overlap()             # this backward pass feeds the reduce-scatter bucket by bucket
            micro_tokens = micro
            if teacher is not None:
                loss, aux, ntok, kl = _distilled_loss(model, teacher, qplan.training, phase, micro, device)
                aux = aux + kl * qplan.training["loss_weight"]
            else:
                loss, aux, ntok = objective_loss(model, phase, micro, device)
            micro = []
            w = phase.loss_weight_or_default()
            ((loss + aux) * w).backward()
            if engine.mem_policy is not None:
                engine.mem_policy.after_backward()
                if phase.task.type == "causal_lm":
                    engine.mem_policy.remember(torch.tensor(micro_tokens, dtype=torch.int64, device=device)[:, :-1])
            window_loss += float(loss.detach())
            window_aux += float(aux.detach()) if torch.is_tensor(aux) else float(aux)
            _nvtx_pop()
            gpu_busy += time.time() - t_busy0
            micro_done += 1
            state.tokens_seen += ntok * dctx.world
            window_supervised += int(ntok)
            if micro_done < ga:
                continue
            lr = lr_at(state.global_step, max(total_steps, 1), args.lr, args.warmup_steps, args.schedule) \
                * phase.learning_rate_scale_or_default()
            if qplan is not None:
                engine.end_quantized_window()
            t_busy0 = time.time()
            _nvtx_push("optimizer_step")
            dctx.guard(state.global_step)        # a peer that left is noticed before anything waits on it
            layer_norms = None
            if args.layer_metrics_every > 0 and (state.global_step + 1) % args.layer_metrics_every == 0:
                # root of the rank-mean of the squared per-layer norms of the rank-local gradients
                local = engine.layer_gradient_norms(cfg.num_layers, grad_scale=1.0 / ga)
                layer_norms = [math.sqrt(dctx.mean(v * v)) for v in local]
            if getattr(engine, "mem_policy", None) is not None:
                engine.mem_policy.before_step(engine)
            norm = checked_norm(engine, engine.step(lr, grad_scale=1.0 / ga))
            if getattr(engine, "mem_policy", None) is not None:
                engine.mem_policy.commit_window(norm, args.max_grad_norm)
            _nvtx_pop()
            gpu_busy += time.time() - t_busy0
            mean_loss = dctx.mean(window_loss / ga)
            window_aux = dctx.mean(window_aux)
            if not math.isfinite(mean_loss) or not math.isfinite(norm):
                raise RuntimeError(f"non-finite loss ({mean_loss}) or gradient norm ({norm}) at step {state.global_step}")
            state.global_step += 1
            state.steps_in_phase += 1
            if engine.mem_policy is not None:
                engine.mem_policy.after_step(state.global_step, writer)
            dt = time.time() - t_step
            writer.set_context(state.global_step, pi, phase.name, phase.kind)
            examples = bs * ga
            compute_tokens = bs * seq * ga
            writer.emit("optimization", {
                "objective": phase.task.type, "loss": mean_loss, "optimized_loss": mean_loss + window_aux / ga,
                "weighted_loss": (mean_loss + window_aux / ga) * w, "router_aux_loss": window_aux / ga,
                "learning_rate": lr, "muon_learning_rate": lr * 20.0, "gradient_norm": norm, "sequence_length": seq,
                "batch_size": bs, "gradient_accumulation": ga, "compute_tokens": compute_tokens,
                "supervised_tokens": min(window_supervised * dctx.world, compute_tokens), "examples": examples,
                "truncated_tokens": 0, "retrieval_candidates": 0, **({"layer_gradient_norms": layer_norms} if layer_norms else {})})
            if qplan is not None and window_fmt in ("binary_g128", "ternary_g128", "ternary_entropy_g128"):
                writer.emit("quantization", {
                    "stage": "fake_quantization", "format": window_fmt, "group_size": qplan.group_size,
                    "progress_fraction": min(1.0, state.steps_in_phase / max(steps_planned, 1)),
                    "tensors_quantized": window_count, "weights_quantized": qweights,
                    "embeddings_quantized": bool(qplan.embeddings), "lm_head_quantized": bool(qplan.lm_head)})
            dt = max(dt, 1e-9)
            writer.emit("throughput", {
                "optimizer_steps": 1, "compute_tokens": compute_tokens,
                "supervised_tokens": min(window_supervised * dctx.world, compute_tokens), "examples": examples,
                "elapsed_seconds": dt, "tokens_per_second": compute_tokens / dt, "examples_per_second": examples / dt,
                "input_wait_seconds": min(input_wait, dt), "host_to_device_seconds": 0.0,
                "gpu_busy_seconds": min(gpu_busy, dt)})
            _drain_device_sampler(engine, writer)
            if dctx.rank == 0:
                print(f"step {state.global_step} phase {phase.name} loss {mean_loss:.4f} gnorm {norm:.3f} "
                      f"lr {lr:.3e} tok/s {bs * seq * ga / max(dt, 1e-9):.0f}", flush=True)
            last = mean_loss
            window_loss, window_aux, micro_done, input_wait, gpu_busy = 0.0, 0.0, 0, 0.0, 0.0
            window_supervised = 0
            t_step = time.time()
            engine.zero_grad()
            if args.checkpoint_every and state.global_step % args.checkpoint_every == 0:
                _checkpoint(out, model, engine, state, writer, t_step)
    finally:
        stop.set()
        while th.is_alive():
            try:
                q.get_nowait()
            except queue.Empty:
                time.sleep(0.01)
    if (micro or micro_done) and dctx.rank == 0:
        # incomplete batches and accumulation windows are dropped and logged (`summa-train/src/trainer.rs:2229-2262`)
        print(f"phase {phase.name}: dropped {len(micro) + micro_done * bs} samples of an incomplete batch or "
              "accumulation window", flush=True)
    return last


def _select_phase_steps(phase: Phase, tok, vocab, eos, seed) -> int:
    """Optimizer steps a phase runs (`summa-train/src/main.rs`, `select_phase_steps`): an exact `steps`, else the natural
    epoch count floor(floor(samples / batch) / accumulation) * epochs from one counting pass over the phase's data, capped
    by `max_steps` (a cap above the natural count is not an exact request: the data wins). Zero steps is an error."""
    if phase.steps is not None:
        return phase.steps
    samples = sum(1 for _ in objective_sample_stream(phase, tok, vocab, phase.sequence_length, eos, seed, 0))
    n = planned_steps(phase, samples)
    if n <= 0:
        raise RuntimeError(f"workflow phase `{phase.name}` produces zero complete optimizer steps "
                           f"({samples} samples at batch {phase.batch_size} x accumulation {phase.grad_accum_or_default()})")
    return n


def objective_sample_stream(phase: Phase, tok, vocab, seq, eos, seed, skip, token_cache=None):
    """Samples of a phase in training order, after `skip` already-consumed records."""
    from .objectives import structured_samples
    t = phase.task.type
    if t == "causal_lm":
        yield from D.iter_samples(phase.data, tok, vocab, seq, eos, phase.shuffle_buffer_or_default(), seed, skip, token_cache)
    else:
        yield from structured_samples(phase, tok, seq, eos, seed, skip)
