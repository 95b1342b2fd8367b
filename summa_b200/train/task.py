"""Task configs, prompt framing and record validation.

The nine task types, their default instruction / prefix strings and the prompt
segmentation (`prefix ⧺ source ⧺ suffix ⧺ target`, where only `source` may be
truncated) follow `summa-train/src/task.rs:246-292,373-475`; the framing into token
windows follows `summa-train/src/data/structured.rs:131-292`.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

DEFAULTS = {
    "temperature": 0.05,
    "summarization": "Summarize the document faithfully and concisely.",
    "retrieval_planning": "Create a concise retrieval plan as an ordered action trace.",
    "instruction_tuning": "Follow the instruction and provide the requested response.",
    "qa_reasoning": "Solve the problem carefully and provide the final answer.",
    "query_prefix": "Represent this query for retrieval:\n",
    "document_prefix": "Represent this document for retrieval:\n",
}
MAX_RETRIEVAL_DOCUMENTS = 32

TASK_FIELDS = {
    "causal_lm": set(),
    "summarization": {"instruction"},
    "retrieval_representation": {"temperature", "layer", "query_prefix", "document_prefix"},
    "retrieval_ranking": {"temperature", "layer", "query_prefix", "document_prefix"},
    "retrieval_planning": {"instruction"},
    "instruction_tuning": {"instruction"},
    "qa_reasoning": {"instruction", "require_reasoning"},
    "pairwise_preference": set(),
    "verifiable_rl": {"verifier"},
}
SUPERVISED = ("summarization", "retrieval_planning", "instruction_tuning", "qa_reasoning")
RETRIEVAL = ("retrieval_representation", "retrieval_ranking")


class TaskError(ValueError):
    pass


@dataclass
class TaskConfig:
    type: str
    params: Dict[str, Any] = field(default_factory=dict)

    @staticmethod
    def from_json(d: Dict[str, Any]) -> "TaskConfig":
        if not isinstance(d, dict) or "type" not in d:
            raise TaskError("task needs a `type`")
        t = d["type"]
        if t not in TASK_FIELDS:
            raise TaskError(f"unknown task type `{t}`")
        extra = set(d) - {"type"} - TASK_FIELDS[t]
        if extra:
            raise TaskError(f"unknown field(s) {sorted(extra)} for task `{t}`")
        p = {k: v for k, v in d.items() if k != "type"}
        for key in ("instruction", "query_prefix", "document_prefix"):
            if key in p and not isinstance(p[key], str):
                raise TaskError(f"`{key}` of task `{t}` must be a string")
        if t in SUPERVISED:
            p.setdefault("instruction", DEFAULTS[t])
            if not p["instruction"].strip():
                raise TaskError(f"{t} instruction must not be empty")
        if t == "qa_reasoning":
            p.setdefault("require_reasoning", False)
            if not isinstance(p["require_reasoning"], bool):
                raise TaskError("`require_reasoning` must be a boolean")
        if t in RETRIEVAL:
            p.setdefault("temperature", DEFAULTS["temperature"])
            p.setdefault("query_prefix", DEFAULTS["query_prefix"])
            p.setdefault("document_prefix", DEFAULTS["document_prefix"])
            temp = p["temperature"]
            if isinstance(temp, bool) or not isinstance(temp, (int, float)) or not (temp > 0) or temp == float("inf"):
                raise TaskError(f"{t} temperature must be finite and positive")
            layer = p.get("layer")
            if layer is not None and (isinstance(layer, bool) or not isinstance(layer, int) or layer < 1):
                raise TaskError(f"{t} layer is one-based and must be positive")
            if not p["query_prefix"] or not p["document_prefix"]:
                raise TaskError(f"{t} query and document prefixes must not be empty")
        if t == "verifiable_rl":
            # `VerifierSpec {adapter, parameters}` (`summa-train/src/task.rs:763-777`): a verifier the RL
            # executor resolves by name; `exact_answer` is the built-in one
            v = p.get("verifier")
            if not isinstance(v, dict):
                raise TaskError("verifiable_rl requires `verifier` {adapter, parameters?}")
            extra = set(v) - {"adapter", "parameters"}
            if extra:
                raise TaskError(f"unknown field `{sorted(extra)[0]}` in `verifier`")
            if not isinstance(v.get("adapter"), str) or not v["adapter"].strip():
                raise TaskError("`verifier.adapter` must be a non-empty string")
            params = v.get("parameters")
            if params is not None and not isinstance(params, dict):
                raise TaskError("`verifier.parameters` must be an object")
            spec = {"adapter": v["adapter"]}
            if params:
                spec["parameters"] = dict(sorted(params.items()))
            p["verifier"] = spec
        return TaskConfig(t, p)

    def to_json(self) -> Dict[str, Any]:
        d = {"type": self.type}
        d.update({k: v for k, v in self.params.items() if v is not None})
        return d

    def is_supervised_generation(self) -> bool:
        return self.type in SUPERVISED

    def is_retrieval(self) -> bool:
        return self.type in RETRIEVAL


def _need(rec: Dict[str, Any], key: str) -> str:
    v = rec.get(key)
    if not isinstance(v, str) or not v:
        raise TaskError(f"`{key}` must be a non-empty string")
    return v


def _opt(rec: Dict[str, Any], key: str) -> Optional[str]:
    v = rec.get(key)
    if v is None:
        return None
    if not isinstance(v, str) or not v:
        raise TaskError(f"`{key}` must be a non-empty string when present")
    return v


@dataclass
class PromptSegments:
    prefix: str
    source: str
    suffix: str
    target: str
    source_required: bool


def supervised_prompt(task: TaskConfig, rec: Dict[str, Any]) -> PromptSegments:
    ins = task.params.get("instruction", "")
    if task.type == "summarization":
        return PromptSegments(f"{ins}\n\nDocument:\n", _need(rec, "document"), "\n\nSummary:\n",
                              _need(rec, "summary"), True)
    if task.type == "retrieval_planning":
        req, plan, ctx = _need(rec, "request"), _need(rec, "plan"), _opt(rec, "context")
        if ctx is not None:
            return PromptSegments(f"{ins}\n\nRequest:\n{req}\n\nContext:\n", ctx, "\nPlan:\n", plan, True)
        return PromptSegments(f"{ins}\n\nRequest:\n{req}\n", "", "Plan:\n", plan, False)
    if task.type == "instruction_tuning":
        prefix = ""
        system = _opt(rec, "system")
        if system is not None:
            prefix += f"System:\n{system}\n\n"
        prefix += f"{ins}\n\nInstruction:\n{_need(rec, 'instruction')}"
        inp = _opt(rec, "input")
        if inp is not None:
            return PromptSegments(prefix + "\n\nInput:\n", inp, "\n\nResponse:\n", _need(rec, "response"), True)
        return PromptSegments(prefix, "", "\n\nResponse:\n", _need(rec, "response"), False)
    if task.type == "qa_reasoning":
        q, a, r = _need(rec, "question"), _need(rec, "answer"), _opt(rec, "reasoning")
        if task.params.get("require_reasoning") and r is None:
            raise TaskError("`reasoning` is required by this task")
        target = f"Reasoning:\n{r}\n\nAnswer:\n{a}" if r is not None else a
        return PromptSegments(f"{ins}\n\nQuestion:\n", q, "\n\nResponse:\n", target, True)
    raise TaskError(f"task `{task.type}` is not a supervised-generation task")


class OversizedRecord(TaskError):
    pass


def frame_supervised(task: TaskConfig, rec: Dict[str, Any], tokenizer, seq_len: int, eos_id: int, stats: Optional[Dict[str, int]] = None):
    """Tokens `prefix ⧺ source[:kept] ⧺ suffix ⧺ target ⧺ EOS`, padded with EOS to
    `seq_len + 1`; each segment is tokenised on its own and only `source` truncates.
    Returns (tokens, loss_positions) with loss positions `prompt_len-1 .. prompt_len+target_len-1`
    (the EOS is supervised)."""
    seg = supervised_prompt(task, rec)
    pre, src = tokenizer.encode(seg.prefix), tokenizer.encode(seg.source)
    suf, tgt = tokenizer.encode(seg.suffix), tokenizer.encode(seg.target)
    fixed = len(pre) + len(suf) + len(tgt) + 1
    room = seq_len + 1 - fixed
    if room < 0 or (seg.source_required and room < 1):
        raise OversizedRecord(f"record needs {fixed} fixed tokens, window is {seq_len + 1}")
    if stats is not None:
        stats["truncated_tokens"] = stats.get("truncated_tokens", 0) + max(0, len(src) - room)
    src = src[:room]
    prompt_len = len(pre) + len(src) + len(suf)
    toks = pre + src + suf + tgt + [eos_id]
    toks += [eos_id] * (seq_len + 1 - len(toks))
    positions = list(range(prompt_len - 1, prompt_len + len(tgt)))
    return toks, positions


def frame_retrieval_text(prefix: str, text: str, tokenizer, seq_len: int, eos_id: int,
                         stats: Optional[Dict[str, int]] = None) -> Tuple[List[int], int]:
    """`prefix ⧺ text[:kept] ⧺ EOS` padded with EOS to `seq_len`; returns (tokens, end_position)."""
    pre, body = tokenizer.encode(prefix), tokenizer.encode(text)
    room = seq_len - len(pre) - 1
    if room < 1:
        raise OversizedRecord("retrieval prefix leaves no room for text")
    if stats is not None:
        stats["truncated_tokens"] = stats.get("truncated_tokens", 0) + max(0, len(body) - room)
    body = body[:room]
    toks = pre + body + [eos_id]
    end = len(toks) - 1
    toks += [eos_id] * (seq_len - len(toks))
    return toks, end


def retrieval_record(task: TaskConfig, rec: Dict[str, Any]) -> Tuple[str, List[str], int]:
    """(query, documents, index of the positive)."""
    if task.type == "retrieval_representation":
        q, pos = _need(rec, "query"), _need(rec, "positive")
        negs = rec.get("negatives", []) or []
        docs = [pos] + [n for n in negs]
        if len(set(docs)) != len(docs):
            raise TaskError("negatives must be distinct from each other and from the positive")
        if len(docs) > MAX_RETRIEVAL_DOCUMENTS:
            raise TaskError(f"at most {MAX_RETRIEVAL_DOCUMENTS} documents per record")
        return q, docs, 0
    if task.type == "retrieval_ranking":
        q = _need(rec, "query")
        docs = rec.get("documents") or []
        if not (2 <= len(docs) <= MAX_RETRIEVAL_DOCUMENTS):
            raise TaskError("`documents` must contain 2..32 candidates")
        texts = [_need(d, "text") for d in docs]
        rel = [float(d.get("relevance", 0.0)) for d in docs]
        best = max(range(len(rel)), key=lambda i: (rel[i], -i))
        return q, texts, best
    raise TaskError(f"task `{task.type}` is not a retrieval task")


def exact_answer_verifier(completion: str, answer: str) -> float:
    """1.0 when the completion's final non-empty line equals the expected answer
    (whitespace-trimmed, case-sensitive), else 0.0."""
    lines = [l.strip() for l in completion.strip().splitlines() if l.strip()]
    return 1.0 if lines and lines[-1] == answer.strip() else 0.0
