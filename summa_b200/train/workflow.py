"""WorkflowV2: the training-recipe JSON (strict schema, bounds, path resolution,
phase-kind / task compatibility, run and workflow signatures).

Schema and rules follow `summa-train/src/workflow.rs:20-32,48-128,371-422,441-726,
774-843,1059-1075`: the integer `version` must be 2 before anything else is parsed,
unknown fields are errors everywhere, paths resolve relative to the workflow file,
`steps` (exact) and `max_steps` (cap on natural epoch steps) are exclusive.
The subset of phases `train` executes directly follows `summa-train/src/wake.rs:18-134`.
"""
from __future__ import annotations

import hashlib
import json
import os
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from . import workflow_config as WC
from .task import TaskConfig, TaskError

WORKFLOW_VERSION = 2
MAX_WORKFLOW_JSON_BYTES = 16 * 1024 * 1024
MAX_PHASES = 4096
MAX_NAME_BYTES = 1024
MAX_PHASE_NAME_BYTES = 256
MAX_BATCH = 65536
MAX_GRAD_ACCUM = 1048576
MAX_SHUFFLE_SAMPLES = 262144
MAX_BATCH_TOKENS = 8 * 1024 * 1024
MAX_SHUFFLE_TOKENS = 256 * 1024 * 1024

PHASE_KINDS = ["pretrain", "continued_pretrain", "sft", "preference", "rl", "distillation", "sleep",
               "quantization", "evaluation", "promotion"]
OPTIMIZATION = {"pretrain", "continued_pretrain", "sft", "preference", "rl", "distillation"}
MODEL_MUTATION = {"sleep", "quantization"}
WAKE_KINDS = {"pretrain", "continued_pretrain", "sft", "quantization"}
WAKE_TASKS = {"causal_lm", "summarization", "retrieval_representation", "retrieval_planning",
              "instruction_tuning", "qa_reasoning"}
QUANT_FORMATS = {"binary_g128", "ternary_g128", "ternary_entropy_g128", "int4_g128"}

PHASE_FIELDS = {"name", "type", "task", "data", "sequence_length", "batch_size", "gradient_accumulation",
                "epochs", "shuffle_buffer", "steps", "max_steps", "loss_weight", "learning_rate_scale",
                "post_training", "sleep", "periodic_sleep", "memory_update_mode", "quantization", "parameters"}


class WorkflowError(ValueError):
    pass


def phase_class(kind: str) -> str:
    if kind in OPTIMIZATION:
        return "optimization"
    if kind in MODEL_MUTATION:
        return "model_mutation"
    return "assessment" if kind == "evaluation" else "release"


def uses_optimizer(kind: str) -> bool:
    return kind in OPTIMIZATION or kind == "quantization"


@dataclass
class QuantizationConfig:
    format: str
    training: Dict[str, Any]
    warmup_format: Optional[str] = None
    group_size: int = 128
    start_step: int = 0
    end_step: Optional[int] = None
    embeddings: bool = True
    lm_head: bool = True

    @staticmethod
    def from_json(d: Dict[str, Any], phase: str) -> "QuantizationConfig":
        allowed = {"format", "warmup_format", "group_size", "start_step", "end_step", "embeddings", "lm_head", "training"}
        _no_unknown(d, allowed, f"quantization of phase `{phase}`")
        if d.get("format") not in QUANT_FORMATS:
            raise WorkflowError(f"phase `{phase}`: unknown quantization format {d.get('format')!r}")
        tr = d.get("training")
        if not isinstance(tr, dict) or tr.get("type") not in ("qat", "distillation"):
            raise WorkflowError(f"phase `{phase}`: quantization.training.type must be qat|distillation")
        if tr["type"] == "qat":
            _no_unknown(tr, {"type", "warmup_steps", "straight_through"}, "quantization.training")
            tr = {"type": "qat", "warmup_steps": int(tr.get("warmup_steps", 0)),
                  "straight_through": bool(tr.get("straight_through", True))}
        else:
            _no_unknown(tr, {"type", "teacher_checkpoint", "teacher_sha256", "temperature", "loss_weight"},
                        "quantization.training")
            if not tr.get("teacher_checkpoint"):
                raise WorkflowError(f"phase `{phase}`: quantization distillation requires teacher_checkpoint")
            _sha256(tr.get("teacher_sha256", ""), "quantization teacher identity")
            t = float(tr.get("temperature", 1.0))
            w = float(tr.get("loss_weight", 1.0))
            if not (t > 0) or not (w >= 0):
                raise WorkflowError(f"phase `{phase}`: invalid distillation temperature / loss_weight")
            tr = dict(tr, temperature=t, loss_weight=w)
        q = QuantizationConfig(d["format"], tr, d.get("warmup_format"), int(d.get("group_size", 128)),
                               int(d.get("start_step", 0)), d.get("end_step"), bool(d.get("embeddings", True)),
                               bool(d.get("lm_head", True)))
        if q.group_size != 128:
            raise WorkflowError(f"workflow phase `{phase}` quantization group_size must be 128 for a *_g128 format")
        if q.end_step is not None and q.end_step <= q.start_step:
            raise WorkflowError(f"workflow phase `{phase}` quantization end_step must be greater than start_step")
        return q

    def validate_phase_window(self, phase_start: int, phase_steps: int) -> None:
        """The phase's optimizer window [start, start + steps) must hold at least one step trained in the TARGET
        format: a warm-up (or a late `start_step`) must not consume the whole phase before its archive is published
        (`summa-train/src/quantization.rs:320-345`)."""
        if phase_steps <= 0:
            raise WorkflowError("quantization phase has no optimizer steps")
        phase_end = phase_start + phase_steps
        target_start = self.start_step + int(self.training.get("warmup_steps", 0))
        target_end = self.end_step if self.end_step is not None else float("inf")
        if not max(phase_start, target_start) < min(phase_end, target_end):
            raise WorkflowError(f"quantization phase optimizer window [{phase_start}, {phase_end}) contains no target-format "
                                f"{self.format} step from configured interval [{target_start}, "
                                f"{'unbounded' if self.end_step is None else self.end_step})")

    def format_at(self, step: int) -> Optional[str]:
        """Codec of the forward pass at an absolute optimizer step; None = full precision (before
        `start_step`, from `end_step` on, or during a warm-up without a warm-up codec)
        (`summa-train/src/quantization.rs:308-319`)."""
        if step < self.start_step or (self.end_step is not None and step >= self.end_step):
            return None
        if step - self.start_step < int(self.training.get("warmup_steps", 0)):
            return self.warmup_format
        return self.format

    def to_json(self):
        d = {"format": self.format, "group_size": self.group_size, "start_step": self.start_step,
             "embeddings": self.embeddings, "lm_head": self.lm_head, "training": self.training}
        if self.warmup_format is not None:
            d["warmup_format"] = self.warmup_format
        if self.end_step is not None:
            d["end_step"] = self.end_step
        return d


@dataclass
class Phase:
    name: str
    kind: str
    task: Optional[TaskConfig] = None
    data: Optional[str] = None
    sequence_length: Optional[int] = None
    batch_size: Optional[int] = None
    gradient_accumulation: Optional[int] = None
    epochs: Optional[int] = None
    shuffle_buffer: Optional[int] = None
    steps: Optional[int] = None
    max_steps: Optional[int] = None
    loss_weight: Optional[float] = None
    learning_rate_scale: Optional[float] = None
    post_training: Optional[Dict[str, Any]] = None
    sleep: Optional[Dict[str, Any]] = None
    periodic_sleep: Optional[Dict[str, Any]] = None
    memory_update_mode: Optional[Dict[str, Any]] = None
    quantization: Optional[QuantizationConfig] = None
    parameters: Dict[str, Any] = field(default_factory=dict)

    def epochs_or_default(self) -> int:
        return self.epochs if self.epochs is not None else 1

    def shuffle_buffer_or_default(self) -> int:
        return self.shuffle_buffer if self.shuffle_buffer is not None else 8192

    def loss_weight_or_default(self) -> float:
        return self.loss_weight if self.loss_weight is not None else 1.0

    def learning_rate_scale_or_default(self) -> float:
        return self.learning_rate_scale if self.learning_rate_scale is not None else 1.0

    def grad_accum_or_default(self) -> int:
        return self.gradient_accumulation if self.gradient_accumulation is not None else 1

    def to_json(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"name": self.name, "type": self.kind}
        if self.task is not None:
            d["task"] = self.task.to_json()
        for k in ("data", "sequence_length", "batch_size", "gradient_accumulation", "epochs", "shuffle_buffer",
                  "steps", "max_steps", "loss_weight", "learning_rate_scale", "post_training", "sleep",
                  "periodic_sleep", "memory_update_mode"):
            v = getattr(self, k)
            if v is not None:
                d[k] = v
        if self.quantization is not None:
            d["quantization"] = self.quantization.to_json()
        if self.parameters:
            d["parameters"] = dict(sorted(self.parameters.items()))
        return d


@dataclass
class Workflow:
    version: int
    phases: List[Phase]
    name: Optional[str] = None

    def to_json(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"version": self.version}
        if self.name is not None:
            d["name"] = self.name
        d["phases"] = [p.to_json() for p in self.phases]
        return d

    def signature(self) -> str:
        """sha256 of the canonical JSON of the RESOLVED workflow."""
        return hashlib.sha256(json.dumps(self.to_json(), sort_keys=True, separators=(",", ":")).encode()).hexdigest()


def _no_unknown(d: Dict[str, Any], allowed, where: str) -> None:
    extra = set(d) - set(allowed)
    if extra:
        raise WorkflowError(f"unknown field(s) {sorted(extra)} in {where}")


def _sha256(s: str, what: str) -> None:
    """Accepts the identity form `sha256:<64 lowercase hex>` (`summa-train/src/artifact_io.rs:42-76`) or the bare digest."""
    if isinstance(s, str) and s.startswith("sha256:"):
        s = s[len("sha256:"):]
    if not (isinstance(s, str) and len(s) == 64 and all(c in "0123456789abcdef" for c in s)):
        raise WorkflowError(f"{what} must be `sha256:` + 64 lowercase hex characters")


def _pos_int(v, name, phase, hi=None):
    if not isinstance(v, int) or isinstance(v, bool) or v < 1 or (hi is not None and v > hi):
        raise WorkflowError(f"workflow phase `{phase}` {name} must be an integer in [1, {hi or 'inf'}]")
    return v


def parse_phase(d: Dict[str, Any]) -> Phase:
    if not isinstance(d, dict):
        raise WorkflowError("phase must be an object")
    _no_unknown(d, PHASE_FIELDS, f"phase `{d.get('name', '?')}`")
    name = d.get("name")
    if not isinstance(name, str) or not name or len(name.encode()) > MAX_PHASE_NAME_BYTES:
        raise WorkflowError("phase needs a non-empty name of at most 256 bytes")
    kind = d.get("type")
    if kind not in PHASE_KINDS:
        raise WorkflowError(f"workflow phase `{name}` has unknown type {kind!r}")
    try:
        task = TaskConfig.from_json(d["task"]) if d.get("task") is not None else None
    except TaskError as e:
        raise WorkflowError(f"workflow phase `{name}`: {e}")
    try:
        post = WC.decode_post_training(d["post_training"]) if d.get("post_training") is not None else None
        sleep = WC.decode_in_model_sleep(d["sleep"], name, "sleep") if d.get("sleep") is not None else None
        periodic = (WC.decode_in_model_sleep(d["periodic_sleep"], name, "periodic_sleep")
                    if d.get("periodic_sleep") is not None else None)
        mode = (WC.decode_memory_update_mode(d["memory_update_mode"], name)
                if d.get("memory_update_mode") is not None else None)
    except WC.ConfigError as e:
        raise WorkflowError(f"workflow phase `{name}`: {e}")
    data = d.get("data")
    if data is not None and not isinstance(data, str):
        raise WorkflowError(f"workflow phase `{name}` data must be a path string")
    params = d.get("parameters")
    if params is not None and not isinstance(params, dict):
        raise WorkflowError(f"workflow phase `{name}` parameters must be an object")
    p = Phase(name=name, kind=kind, task=task, data=data, post_training=post, sleep=sleep, periodic_sleep=periodic,
              memory_update_mode=mode, parameters=dict(params or {}))
    for key, hi in (("sequence_length", None), ("batch_size", MAX_BATCH), ("gradient_accumulation", MAX_GRAD_ACCUM),
                    ("epochs", None), ("steps", None), ("max_steps", None)):
        if d.get(key) is not None:
            setattr(p, key, _pos_int(d[key], key, name, hi))
    if d.get("shuffle_buffer") is not None:
        sb = d["shuffle_buffer"]
        if not isinstance(sb, int) or sb < 0 or sb > MAX_SHUFFLE_SAMPLES:
            raise WorkflowError(f"workflow phase `{name}` shuffle_buffer must be in [0, {MAX_SHUFFLE_SAMPLES}]")
        p.shuffle_buffer = sb
    for key in ("loss_weight", "learning_rate_scale"):
        if d.get(key) is not None:
            v = float(d[key])
            if not (v > 0) or v != v or v == float("inf"):
                raise WorkflowError(f"workflow phase `{name}` {key} must be finite and positive")
            setattr(p, key, v)
    if d.get("quantization") is not None:
        p.quantization = QuantizationConfig.from_json(d["quantization"], name)
    _validate_phase(p)
    return p


SUPERVISED_GENERATION = ("summarization", "retrieval_planning", "instruction_tuning", "qa_reasoning")


def _sequences_per_example(task: TaskConfig) -> int:
    """Model sequences one example can expand to (`summa-train/src/task.rs` `maximum_model_sequences_per_example`):
    a retrieval record carries its query plus up to 32 documents, a preference pair two continuations."""
    if task.type == "retrieval_representation":
        return 33
    if task.type == "pairwise_preference":
        return 2
    return 1


def _validate_phase(p: Phase) -> None:
    """Cross-field rules of one phase, in the order of `summa-train/src/workflow.rs:441-711`."""
    n, kind = p.name, p.kind
    if p.steps is not None and p.max_steps is not None:
        raise WorkflowError(f"workflow phase `{n}` cannot set both steps and max_steps")
    if p.max_steps is not None and kind not in ("pretrain", "continued_pretrain", "sft", "quantization"):
        raise WorkflowError(f"workflow phase `{n}` ({kind}) cannot set max_steps because its executor does not "
                            "implement adaptive data-derived step caps")
    if kind not in ("sleep", "promotion"):
        if p.task is None:
            raise WorkflowError(f"workflow phase `{n}` ({kind}) requires a task")
        if not p.data:
            raise WorkflowError(f"workflow phase `{n}` ({kind}) requires a data path")
        if p.sequence_length is None:
            raise WorkflowError(f"workflow phase `{n}` ({kind}) requires sequence_length")
        if p.batch_size is None:
            raise WorkflowError(f"workflow phase `{n}` ({kind}) requires batch_size")
        per = _sequences_per_example(p.task)
        if p.sequence_length * p.batch_size * per > MAX_BATCH_TOKENS:
            raise WorkflowError(f"workflow phase `{n}` batch geometry exceeds the {MAX_BATCH_TOKENS}-token "
                                "materialization limit")
        if p.sequence_length * p.shuffle_buffer_or_default() * per > MAX_SHUFFLE_TOKENS:
            raise WorkflowError(f"workflow phase `{n}` shuffle geometry exceeds the {MAX_SHUFFLE_TOKENS}-token buffer limit")
    elif p.task is not None or p.data is not None:
        raise WorkflowError(f"workflow phase `{n}` ({kind}) must not read task data")
    if uses_optimizer(kind):
        if p.gradient_accumulation is None:
            raise WorkflowError(f"workflow phase `{n}` ({kind}) requires gradient_accumulation")
    elif kind == "evaluation":
        if p.gradient_accumulation is not None:
            raise WorkflowError(f"workflow phase `{n}` (evaluation) must not set gradient_accumulation")
        if p.loss_weight is not None or p.learning_rate_scale is not None:
            raise WorkflowError(f"workflow phase `{n}` (evaluation) must not set optimizer weights")
    else:
        for k in ("sequence_length", "batch_size", "gradient_accumulation", "epochs", "shuffle_buffer", "steps",
                  "max_steps", "loss_weight", "learning_rate_scale"):
            if getattr(p, k) is not None:
                raise WorkflowError(f"workflow phase `{n}` ({kind}) must not set task execution or optimizer geometry")
    t = p.task.type if p.task else None
    if kind == "sft" and t not in SUPERVISED_GENERATION:
        raise WorkflowError(f"workflow phase `{n}` (sft) requires a supervised-generation task")
    if kind == "distillation" and t not in ("causal_lm",) + SUPERVISED_GENERATION:
        raise WorkflowError(f"workflow phase `{n}` (distillation) requires an autoregressive or supervised-generation task")
    if kind == "preference" and t != "pairwise_preference":
        raise WorkflowError(f"workflow phase `{n}` (preference) requires a pairwise-preference task")
    if kind == "rl" and t != "verifiable_rl":
        raise WorkflowError(f"workflow phase `{n}` (rl) requires a verifiable-reward task")
    wanted = {"preference": ("dpo", "a DPO"), "distillation": ("forward_kl", "a forward-KL"), "rl": ("grpo", "a GRPO")}
    if kind in wanted:
        if p.post_training is None:
            raise WorkflowError(f"workflow phase `{n}` ({kind}) requires typed post_training settings")
        if p.post_training["algorithm"] != wanted[kind][0]:
            raise WorkflowError(f"workflow phase `{n}` ({kind}) requires {wanted[kind][1]} post-training algorithm")
    elif p.post_training is not None:
        raise WorkflowError(f"workflow phase `{n}` ({kind}) must not set post_training settings")
    if p.post_training is not None and p.post_training["algorithm"] == "grpo":
        if p.post_training["sampling"]["max_new_tokens"] > (p.sequence_length or 0):
            raise WorkflowError(f"workflow phase `{n}` GRPO max_new_tokens must not exceed sequence_length")
    if kind == "quantization" and p.quantization is None:
        raise WorkflowError(f"workflow phase `{n}` (quantization) requires quantization settings")
    if kind != "quantization" and p.quantization is not None:
        raise WorkflowError(f"workflow phase `{n}` ({kind}) must not set quantization settings")
    if kind == "sleep":
        if p.sleep is None:
            raise WorkflowError(f"workflow phase `{n}` (sleep) requires typed sleep settings")
        if not p.sleep.get("standalone_trigger_clock"):
            raise WorkflowError(f"workflow phase `{n}` (sleep) requires a positive standalone_trigger_clock")
    elif p.sleep is not None:
        raise WorkflowError(f"workflow phase `{n}` ({kind}) must not set sleep settings")
    if p.periodic_sleep is not None:
        if not uses_optimizer(kind):
            raise WorkflowError(f"workflow phase `{n}` ({kind}) cannot install a periodic sleep hook")
        if p.periodic_sleep.get("standalone_trigger_clock") is not None:
            raise WorkflowError(f"workflow phase `{n}` periodic_sleep must not set standalone_trigger_clock")
    if p.memory_update_mode is not None:
        if not uses_optimizer(kind):
            raise WorkflowError(f"workflow phase `{n}` ({kind}) cannot set memory_update_mode")
        if p.periodic_sleep is not None:
            raise WorkflowError(f"workflow phase `{n}` cannot combine memory_update_mode with periodic_sleep")


def parse_workflow(text: str, base_dir: Optional[str] = None) -> Workflow:
    if len(text.encode()) > MAX_WORKFLOW_JSON_BYTES:
        raise WorkflowError("workflow JSON exceeds 16 MiB")
    try:
        raw = json.loads(text)
    except json.JSONDecodeError as e:
        raise WorkflowError(f"invalid workflow JSON: {e}")
    if not isinstance(raw, dict):
        raise WorkflowError("workflow must be a JSON object")
    v = raw.get("version")
    if not isinstance(v, int) or isinstance(v, bool):
        raise WorkflowError("workflow `version` must be an integer")
    if v != WORKFLOW_VERSION:
        raise WorkflowError(f"unsupported workflow version {v} (expected {WORKFLOW_VERSION})")
    _no_unknown(raw, {"version", "name", "phases"}, "workflow")
    name = raw.get("name")
    if name is not None and (not isinstance(name, str) or len(name.encode()) > MAX_NAME_BYTES):
        raise WorkflowError("workflow name must be a string of at most 1024 bytes")
    phases = raw.get("phases")
    if not isinstance(phases, list) or not phases:
        raise WorkflowError("workflow needs at least one phase")
    if len(phases) > MAX_PHASES:
        raise WorkflowError(f"workflow has more than {MAX_PHASES} phases")
    parsed = [parse_phase(p) for p in phases]
    seen = set()
    for p in parsed:
        if p.name in seen:
            raise WorkflowError(f"duplicate phase name `{p.name}`")
        seen.add(p.name)
    if base_dir is not None:
        for p in parsed:
            if p.data is not None and not os.path.isabs(p.data):
                p.data = os.path.normpath(os.path.join(base_dir, p.data))
            if p.quantization and p.quantization.training.get("teacher_checkpoint"):
                tc = p.quantization.training["teacher_checkpoint"]
                if not os.path.isabs(tc):
                    p.quantization.training["teacher_checkpoint"] = os.path.normpath(os.path.join(base_dir, tc))
            if p.post_training is not None:
                WC.resolve_post_training_paths(p.post_training, base_dir)
            for cfg in (p.sleep, p.periodic_sleep):
                if cfg is not None:
                    WC.resolve_sleep_paths(cfg, base_dir)
    return Workflow(v, parsed, name)


def load_workflow(path: str) -> Workflow:
    if os.path.getsize(path) > MAX_WORKFLOW_JSON_BYTES:
        raise WorkflowError("workflow JSON exceeds 16 MiB")
    with open(path, "r", encoding="utf-8") as f:
        return parse_workflow(f.read(), os.path.dirname(os.path.abspath(path)))


def validate_retrieval_layer(layer: int, model, context: str) -> None:
    """Retrieval embeddings are read after `layer` (one-based): it must exist and at least one
    full-attention layer must sit at or before it (`summa-train/src/workflow.rs:851-869`)."""
    if not (0 < layer <= model.num_layers):
        raise WorkflowError(f"{context} requests retrieval layer {layer}, model has {model.num_layers} layers")
    for i in range(layer):
        b = model.block_for_layer(i)
        if not b.is_ssm() and b.attention.window_size is None:
            return
    raise WorkflowError(f"{context} retrieval layer {layer} has no full-attention layer at or before it")


def _validate_schedule_for_model(model, schedule: Dict[str, Any], phase_name: str) -> None:
    tiers = schedule["tiers"]
    for layer in range(model.num_layers):
        memory = model.block_for_layer(layer).memory
        if memory is None:
            raise WorkflowError(f"workflow phase `{phase_name}` enables sleep, but model layer {layer} has no memory hierarchy")
        if len(memory.tiers) != len(tiers):
            raise WorkflowError(f"workflow phase `{phase_name}` declares {len(tiers)} memory tiers, but model layer "
                                f"{layer} defines {len(memory.tiers)}")
        for i, (conf, defined) in enumerate(zip(tiers, memory.tiers)):
            if conf["id"] != defined.name:
                raise WorkflowError(f"workflow phase `{phase_name}` tier {i} is `{conf['id']}`, but model layer {layer} "
                                    f"defines `{defined.name}`")
            if conf["reserve_slots"] != defined.reserve_experts.capacity:
                raise WorkflowError(f"workflow phase `{phase_name}` tier `{conf['id']}` reserves {conf['reserve_slots']} "
                                    f"slots, but model layer {layer} preallocates {defined.reserve_experts.capacity}")


def _validate_dreaming_topology(model, sleep: Dict[str, Any], phase_name: str) -> None:
    if sleep.get("dreaming") is None:
        return
    for layer in range(model.num_layers):
        memory = model.block_for_layer(layer).memory
        if memory is not None and any(t.ffn.moe is not None and t.ffn.moe.experts > t.ffn.moe.top_k for t in memory.tiers):
            return
    raise WorkflowError(f"workflow phase `{phase_name}` enables Dreaming, but the MAL memory hierarchy has no persistent "
                        "FFN MoE with an expert outside ordinary top-k")


def validate_against_model(wf: Workflow, model) -> None:
    """A workflow and the exact MAL topology it will train must form one executable recipe
    (`summa-train/src/workflow.rs:871-985`): sequence lengths within `max_seq_len`, retrieval read-out layers
    that exist, and, for memory models, ONE identical update policy (periodic_sleep or wake_only) on every
    optimizer-bearing phase whose tier ids and reserve capacities equal the model's memory tiers in every layer."""
    if model.num_layers <= 0:
        raise WorkflowError("model contains no layers")
    for p in wf.phases:
        if p.sequence_length is not None and p.sequence_length > model.max_seq_len:
            raise WorkflowError(f"workflow phase `{p.name}` sequence_length {p.sequence_length} exceeds model max_seq_len "
                                f"{model.max_seq_len}")
        if p.task is not None and p.task.is_retrieval() and p.task.params.get("layer") is not None:
            validate_retrieval_layer(p.task.params["layer"], model, f"workflow phase `{p.name}`")
    memory_layers = sum(1 for i in range(model.num_layers) if model.block_for_layer(i).memory is not None)
    if memory_layers not in (0, model.num_layers):
        raise WorkflowError(f"model mixes {memory_layers} memory layers with {model.num_layers - memory_layers} "
                            "ordinary-FFN layers; in-model sleep requires an explicit memory hierarchy in every layer")
    opt = [p for p in wf.phases if uses_optimizer(p.kind)]
    standalone = [p for p in wf.phases if p.sleep is not None]
    if memory_layers == 0:
        if any(p.periodic_sleep is not None or p.memory_update_mode is not None for p in opt) or standalone:
            raise WorkflowError("memory update modes and in-model sleep require a MAL model with an explicit memory "
                                "hierarchy; no implicit topology upgrade is performed")
        return
    if opt:
        periodic = sum(1 for p in opt if p.periodic_sleep is not None)
        wake_only = sum(1 for p in opt if p.memory_update_mode is not None)
        if periodic != len(opt) and wake_only != len(opt):
            raise WorkflowError("memory MAL models require one identical update policy on every optimizer-bearing phase: "
                                "periodic_sleep or memory_update_mode wake_only, including QAT")
        if periodic == len(opt):
            ref = opt[0].periodic_sleep
            if any(p.periodic_sleep != ref for p in opt):
                raise WorkflowError("all optimizer-bearing phases in one memory-model workflow must use an identical "
                                    "periodic_sleep configuration")
            _validate_schedule_for_model(model, ref["schedule"], opt[0].name)
            _validate_dreaming_topology(model, ref, opt[0].name)
        else:
            if standalone:
                raise WorkflowError("memory_update_mode wake_only is a no-sleep ablation and cannot be combined with "
                                    "standalone sleep phases")
            ref = opt[0].memory_update_mode
            if any(p.memory_update_mode != ref for p in opt):
                raise WorkflowError("all optimizer-bearing phases in one memory-model workflow must use an identical "
                                    "memory_update_mode configuration")
            _validate_schedule_for_model(model, ref["schedule"], opt[0].name)
    for p in standalone:
        _validate_schedule_for_model(model, p.sleep["schedule"], p.name)
        _validate_dreaming_topology(model, p.sleep, p.name)


def wake_plan(wf: Workflow) -> List[Phase]:
    """Phases the `train` command executes itself; anything else needs `run-workflow`."""
    out = []
    for p in wf.phases:
        if p.kind not in WAKE_KINDS:
            raise WorkflowError(f"phase `{p.name}` of type {p.kind} must run through run-workflow")
        if p.task is None or p.task.type not in WAKE_TASKS:
            raise WorkflowError(f"phase `{p.name}`: task is not executable by train")
        if p.parameters:
            raise WorkflowError(f"phase `{p.name}`: raw `parameters` are not accepted by train")
        if not p.sequence_length or not p.batch_size:
            raise WorkflowError(f"phase `{p.name}` needs sequence_length and batch_size")
        out.append(p)
    return out


def planned_steps(p: Phase, samples: Optional[int]) -> int:
    """`steps`, or min(floor(floor(samples / batch) / ga) * epochs, max_steps)."""
    if p.steps is not None:
        return p.steps
    if samples is None:
        raise WorkflowError(f"phase `{p.name}` needs `steps` when the sample count is unknown")
    natural = (samples // p.batch_size) // p.grad_accum_or_default() * p.epochs_or_default()
    return min(natural, p.max_steps) if p.max_steps is not None else natural


def run_signature(workflow: Workflow, model_json: Dict[str, Any], tokenizer_sha256: str, data_ids: List[str],
                  seed: int, lr: float, weight_decay: float, clip: float, warmup: int, schedule: str,
                  muon_lr_scale: float, extra: Optional[Dict[str, Any]] = None) -> str:
    """Everything training-semantic, hashed (`summa-train/src/main.rs:1329-1376`)."""
    blob = {"workflow": workflow.to_json(), "model": model_json, "tokenizer_sha256": tokenizer_sha256,
            "data": data_ids, "seed": seed, "learning_rate": lr, "weight_decay": weight_decay,
            "max_grad_norm": clip, "warmup_steps": warmup, "schedule": schedule, "muon_lr_scale": muon_lr_scale}
    if extra:
        blob["extra"] = extra
    return hashlib.sha256(json.dumps(blob, sort_keys=True, separators=(",", ":")).encode()).hexdigest()


def fnv1a64(data: bytes) -> int:
    h = 0xCBF29CE484222325
    for b in data:
        h ^= b
        h = (h * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
    return h
