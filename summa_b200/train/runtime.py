"""Workflow lifecycle runtime: a crash-consistent phase state machine plus the external
phase-worker protocol.

State machine (`summa-train/src/runtime.rs:20-36,215-226,391-489,599-674,786-920`):
every boundary is persisted BEFORE the in-memory transition —
`started → progress* → (yielded | prepared → committed)`. A run that died after `prepared`
commits without re-running the executor. Product legality by phase class: optimization
and model-mutation phases must return a NEW candidate (different uri and content),
model-mutation may instead return `mutation_rejected`, assessment returns a report, release
must republish exactly its input candidate. Every kind except `pretrain` needs an input
checkpoint. The full history is validated on every load (receipts chain checkpoints).

Worker protocol v2 (`summa-train/src/worker.rs:41-149`): the worker is spawned with a
cleared environment in its own process group, receives one JSON request line on stdin and
answers with JSON lines `metric | progress | yielded | complete`; a timeout kills the
whole process group.
"""
from __future__ import annotations

import hashlib
import json
import os
import select
import signal
import subprocess
import tempfile
import time
from dataclasses import asdict, dataclass, field
from typing import Any, Callable, Dict, List, Optional

from .workflow import Phase, Workflow, load_workflow, phase_class

STATE_VERSION = 2
PROTOCOL_VERSION = 2


class RuntimeError_(RuntimeError):
    pass


@dataclass
class Checkpoint:
    uri: str
    sha256: str

    def to_json(self):
        return {"uri": self.uri, "sha256": self.sha256}


def _ckpt(d) -> Optional[Checkpoint]:
    return Checkpoint(d["uri"], d["sha256"]) if d else None


@dataclass
class Receipt:
    phase_index: int
    phase_name: str
    kind: str
    input: Optional[Dict[str, str]]
    product: Dict[str, Any]


@dataclass
class RunState:
    version: int
    workflow_signature: str
    initial_checkpoint: Optional[Dict[str, str]]
    current_checkpoint: Optional[Dict[str, str]]
    next_phase: int = 0
    completed: List[Dict[str, Any]] = field(default_factory=list)
    active: Optional[Dict[str, Any]] = None      # {phase_index, boundary, resume_state, prepared_product, metrics}

    def to_json(self) -> str:
        return json.dumps(asdict(self), indent=2, sort_keys=True)


class AtomicRuntimeCheckpoint:
    """The run state file, replaced atomically (temp file + fsync + rename)."""

    def __init__(self, path: str, dispatch_identity: str):
        self.path = path
        self.identity = dispatch_identity

    def load(self) -> Optional[RunState]:
        if not os.path.exists(self.path):
            return None
        raw = json.load(open(self.path))
        if raw.get("dispatch_identity") != self.identity:
            raise RuntimeError_("run state belongs to a different executor configuration")
        st = raw["state"]
        if st.get("version") != STATE_VERSION:
            raise RuntimeError_(f"unsupported run state version {st.get('version')}")
        return RunState(**st)

    def store(self, state: RunState) -> None:
        d = os.path.dirname(os.path.abspath(self.path))
        os.makedirs(d, exist_ok=True)
        fd, tmp = tempfile.mkstemp(prefix=".runstate-", dir=d)
        with os.fdopen(fd, "w") as f:
            json.dump({"dispatch_identity": self.identity, "state": asdict(state)}, f, indent=2, sort_keys=True)
            f.flush()
            os.fsync(f.fileno())
        os.replace(tmp, self.path)


def validate_product(phase: Phase, inp: Optional[Checkpoint], product: Dict[str, Any]) -> None:
    cls = phase_class(phase.kind)
    t = product.get("type")
    if cls in ("optimization", "model_mutation"):
        if t == "mutation_rejected" and cls == "model_mutation":
            if "report" not in product:
                raise RuntimeError_("mutation_rejected needs a report")
            return
        if t != "model_candidate":
            raise RuntimeError_(f"phase `{phase.name}` must return a model_candidate")
        c = product.get("checkpoint") or {}
        if not c.get("uri") or not c.get("sha256"):
            raise RuntimeError_("model_candidate needs checkpoint {uri, sha256}")
        if inp is not None and (c["uri"] == inp.uri or c["sha256"] == inp.sha256):
            raise RuntimeError_(f"phase `{phase.name}` must return a NEW candidate (different uri and content)")
    elif cls == "assessment":
        if t != "assessment" or "report" not in product:
            raise RuntimeError_(f"phase `{phase.name}` must return an assessment report")
    else:
        c = (product.get("candidate") or {})
        if t != "release" or inp is None or c.get("uri") != inp.uri or c.get("sha256") != inp.sha256:
            raise RuntimeError_(f"phase `{phase.name}` must republish exactly its input candidate")


def validate_history(wf: Workflow, st: RunState) -> None:
    cur = _ckpt(st.initial_checkpoint)
    if len(st.completed) != st.next_phase:
        raise RuntimeError_("run state: completed receipts do not match next_phase")
    for i, r in enumerate(st.completed):
        if r["phase_index"] != i or r["phase_name"] != wf.phases[i].name:
            raise RuntimeError_(f"run state: receipt {i} does not match the workflow")
        rin = _ckpt(r.get("input"))
        if (rin is None) != (cur is None) or (rin and (rin.uri != cur.uri or rin.sha256 != cur.sha256)):
            raise RuntimeError_(f"run state: receipt {i} does not chain from the previous checkpoint")
        p = r["product"]
        if p.get("type") == "model_candidate":
            cur = _ckpt(p["checkpoint"])
    now = _ckpt(st.current_checkpoint)
    if (now is None) != (cur is None) or (now and (now.uri != cur.uri or now.sha256 != cur.sha256)):
        raise RuntimeError_("run state: current checkpoint does not follow from the receipts")


class ProgressSink:
    def __init__(self, runtime: "WorkflowRuntime"):
        self.rt = runtime

    def checkpoint(self, resume_state: Any) -> None:
        st = self.rt.state
        st.active["resume_state"] = resume_state
        st.active["boundary"] = "progress"
        self.rt.store.store(st)

    def metric(self, record: Dict[str, Any]) -> None:
        if record.get("phase_index", self.rt.state.active["phase_index"]) != self.rt.state.active["phase_index"]:
            raise RuntimeError_("metric context does not match the active phase")
        self.rt.metrics.append(record)


class PhaseExecutor:
    """execute(request, sink) → ("yielded", resume_state) | ("complete", product)."""

    def execute(self, request: Dict[str, Any], sink: ProgressSink):
        raise NotImplementedError


class ExecutorRegistry:
    def __init__(self):
        self._by_kind: Dict[str, PhaseExecutor] = {}

    def register(self, kind: str, ex: PhaseExecutor) -> None:
        if kind in self._by_kind:
            raise RuntimeError_(f"executor for `{kind}` already registered")
        self._by_kind[kind] = ex

    def get(self, kind: str) -> PhaseExecutor:
        if kind not in self._by_kind:
            raise RuntimeError_(f"no executor registered for phase kind `{kind}`")
        return self._by_kind[kind]


class WorkflowRuntime:
    def __init__(self, wf: Workflow, registry: ExecutorRegistry, store: AtomicRuntimeCheckpoint,
                 initial_checkpoint: Optional[Checkpoint] = None):
        self.wf, self.registry, self.store = wf, registry, store
        self.metrics: List[Dict[str, Any]] = []
        sig = wf.signature()
        st = store.load()
        if st is None:
            st = RunState(STATE_VERSION, sig, initial_checkpoint.to_json() if initial_checkpoint else None,
                          initial_checkpoint.to_json() if initial_checkpoint else None)
            store.store(st)
        else:
            if st.workflow_signature != sig:
                raise RuntimeError_("run state was produced by a different workflow")
            validate_history(wf, st)
        self.state = st

    def done(self) -> bool:
        return self.state.next_phase >= len(self.wf.phases)

    def run_next_phase(self) -> str:
        """Runs (or finishes) one phase. Returns "committed" or "yielded"."""
        st = self.state
        i = st.next_phase
        phase = self.wf.phases[i]
        inp = _ckpt(st.current_checkpoint)
        if phase.kind != "pretrain" and inp is None:
            raise RuntimeError_(f"phase `{phase.name}` of type {phase.kind} needs an input checkpoint")
        if st.active is not None and st.active.get("boundary") == "prepared":
            product = st.active["prepared_product"]       # died between prepare and commit
        else:
            if st.active is None or st.active.get("phase_index") != i:
                st.active = {"phase_index": i, "boundary": "started", "resume_state": None, "prepared_product": None}
                self.store.store(st)
            request = {"protocol_version": PROTOCOL_VERSION, "workflow_signature": st.workflow_signature,
                       "phase_index": i, "phase": phase.to_json(),
                       "input_checkpoint": inp.to_json() if inp else None,
                       "resume_state": st.active.get("resume_state")}
            kind, payload = self.registry.get(phase.kind).execute(request, ProgressSink(self))
            if kind == "yielded":
                st.active["boundary"] = "yielded"
                st.active["resume_state"] = payload
                self.store.store(st)
                return "yielded"
            product = payload
            validate_product(phase, inp, product)
            st.active["boundary"] = "prepared"
            st.active["prepared_product"] = product
            self.store.store(st)
        st.completed.append(asdict(Receipt(i, phase.name, phase.kind, inp.to_json() if inp else None, product)))
        if product.get("type") == "model_candidate":
            st.current_checkpoint = dict(product["checkpoint"])
        st.next_phase = i + 1
        st.active = None
        self.store.store(st)
        return "committed"

    def run_until_yield_or_complete(self) -> str:
        while not self.done():
            if self.run_next_phase() == "yielded":
                return "yielded"
        return "complete"


class ExternalPhaseExecutor(PhaseExecutor):
    """Runs a phase in a subprocess speaking the JSON-lines worker protocol."""

    def __init__(self, argv: List[str], timeout_s: float = 3600.0):
        self.argv, self.timeout = argv, timeout_s

    def identity(self) -> str:
        return hashlib.sha256(json.dumps({"argv": self.argv, "timeout": self.timeout}).encode()).hexdigest()

    def execute(self, request, sink: ProgressSink):
        proc = subprocess.Popen(self.argv, stdin=subprocess.PIPE, stdout=subprocess.PIPE, stderr=subprocess.DEVNULL,
                                env={"PATH": os.environ.get("PATH", "/usr/bin:/bin")}, cwd="/",
                                start_new_session=True, text=True)
        deadline = time.time() + self.timeout
        try:
            proc.stdin.write(json.dumps(request) + "\n")
            proc.stdin.flush()
            proc.stdin.close()
            while True:
                left = deadline - time.time()
                if left <= 0:
                    raise RuntimeError_("phase worker timed out")
                ready, _, _ = select.select([proc.stdout], [], [], min(left, 1.0))
                if not ready:
                    if proc.poll() is not None:
                        raise RuntimeError_(f"phase worker exited with {proc.returncode} before completing")
                    continue
                line = proc.stdout.readline()
                if not line:
                    raise RuntimeError_(f"phase worker closed its output (exit {proc.poll()})")
                msg = json.loads(line)
                t = msg.get("type")
                if t == "metric":
                    sink.metric(msg.get("record", {}))
                elif t == "progress":
                    sink.checkpoint(msg.get("resume_state"))
                elif t == "yielded":
                    proc.wait(timeout=10)
                    return "yielded", msg.get("resume_state")
                elif t == "complete":
                    proc.wait(timeout=10)
                    return "complete", msg["product"]
                else:
                    raise RuntimeError_(f"unknown worker message type {t!r}")
        finally:
            if proc.poll() is None:
                try:
                    os.killpg(proc.pid, signal.SIGKILL)      # the worker's own process group only
                except ProcessLookupError:
                    pass
                proc.wait()


def run_workflow_command(args) -> Dict[str, Any]:
    wf = load_workflow(args.workflow)
    initial = None
    if args.initial_checkpoint:
        h = hashlib.sha256(open(args.initial_checkpoint, "rb").read()).hexdigest()
        initial = Checkpoint(os.path.abspath(args.initial_checkpoint), h)
    if getattr(args, "native", False):
        return _run_workflow_native(args, wf, initial)
    if not args.worker:
        raise RuntimeError_("run-workflow needs --worker (or --native with the first-party adapters)")
    ex = ExternalPhaseExecutor(list(args.worker), args.timeout)
    reg = ExecutorRegistry()
    for kind in {p.kind for p in wf.phases}:
        reg.register(kind, ex)
    rt = WorkflowRuntime(wf, reg, AtomicRuntimeCheckpoint(args.state, ex.identity()), initial)
    outcome = rt.run_until_yield_or_complete()
    return {"outcome": outcome, "next_phase": rt.state.next_phase, "current_checkpoint": rt.state.current_checkpoint}


def _run_workflow_native(args, wf, initial) -> Dict[str, Any]:
    """`run-workflow --native`: the embedded host of `native_host.py` with this package's first-party adapters
    (reference: `summa-train/src/native_host.rs:163-230`, the adapters a binary registers before `start`).
    Only adapters whose inputs were given are registered, so a workflow that needs a missing one is refused by
    the routing check, before the state file exists."""
    from .. import mal
    from ..tokenizer import Tokenizer
    from . import native_host as NH
    if not args.model or not args.output:
        raise RuntimeError_("run-workflow --native needs --model and --output")
    model_def = mal.parse_mal_file(args.model)
    tok = Tokenizer.from_file(args.tokenizer) if args.tokenizer else Tokenizer.byte_level()
    if not model_def.vocab_size:
        model_def.vocab_size = tok.vocab_size()
    adapters = NH.NativeWorkflowAdapters()
    adapters.register_post_training_factory(
        NH.TorchPostTrainingFactory(model_def, tok, args.output, device=args.device, lr=args.lr))
    rt_path, rt_sha = getattr(args, "sleep_runtime", None), getattr(args, "sleep_runtime_sha256", None)
    if (rt_path is None) != (rt_sha is None):
        raise RuntimeError_("--sleep-runtime and --sleep-runtime-sha256 go together")
    if rt_path is not None:
        if args.replay:
            raise RuntimeError_("--replay and --sleep-runtime are alternatives")
        from .sleep_runtime import load_sleep_runtime
        rt = load_sleep_runtime(rt_path, rt_sha, "standalone")
        if rt.workflow_signature != "sha256:" + wf.signature():
            raise RuntimeError_(f"sleep runtime {rt_path} is bound to workflow signature {rt.workflow_signature}, this workflow's is "
                                f"sha256:{wf.signature()}")
        adapters.register_sleep_factory(NH.TorchSleepFactory(model_def, None, args.output, device=args.device, runtime=rt))
    elif args.replay:
        adapters.register_sleep_factory(NH.TorchSleepFactory(model_def, args.replay, args.output, device=args.device))
    if args.tokenizer:
        adapters.register_periodic_wake_executor(
            NH.TrainerPeriodicWakeExecutor(args.model, args.tokenizer, args.output, device=args.device))
    if args.worker:
        adapters.register_external(ExternalPhaseExecutor(list(args.worker), args.timeout))
    metrics = None
    if args.metrics:
        from .metrics import run_id_from_signature
        metrics = (args.metrics, getattr(args, "run_id", None) or run_id_from_signature(wf.signature()))
    if args.resume:
        host = NH.NativeWorkflowHost.resume(wf, adapters, args.state, metrics, update_budget=args.update_budget)
    else:
        host = NH.NativeWorkflowHost.start(wf, adapters, args.state, metrics, initial, update_budget=args.update_budget)
    try:
        outcome = host.run_until_yield_or_complete()
    finally:
        host.close()
    st = host.runtime.state
    return {"outcome": outcome, "next_phase": st.next_phase, "current_checkpoint": st.current_checkpoint,
            "dispatch_sha256": host.dispatch_sha256, "routes": [r["dispatch"] for r in host.plan]}
