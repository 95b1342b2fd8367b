"""Training objectives: causal LM, the four supervised-generation tasks (masked
positions), contrastive retrieval with in-batch and explicit negatives, optional QAT
teacher KL (`summa-train/src/main.rs:1447-1628`, `summa-train/src/data/batch.rs:124-339`).
"""
from __future__ import annotations

import json
from typing import Any, Dict, Iterator, List, Tuple

import torch
import torch.nn.functional as F

from . import data as D
from . import task as T


def structured_samples(phase, tok, seq, eos, seed, skip) -> Iterator[Dict[str, Any]]:
    """Framed records of a supervised or retrieval phase, shuffled like causal samples.
    Oversized records abort training (evaluation skips and counts them instead)."""
    buf = D.ShuffleBuffer(phase.shuffle_buffer_or_default(), seed)
    emitted = 0

    def rows():
        with D._open_text(phase.data) as f:
            for n, line in enumerate(f, 1):
                line = line.strip()
                if not line:
                    continue
                try:
                    rec = json.loads(line)
                except json.JSONDecodeError as e:
                    raise D.DataError(f"{phase.data}:{n}: invalid JSON: {e}")
                yield frame_record(phase.task, rec, tok, seq, eos)

    for item in rows():
        got = buf.push(item)
        if got is not None:
            emitted += 1
            if emitted > skip:
                yield got
    for got in buf.drain():
        emitted += 1
        if emitted > skip:
            yield got


def frame_record(task: T.TaskConfig, rec: Dict[str, Any], tok, seq: int, eos: int, stats=None) -> Dict[str, Any]:
    """`stats` (a dict) accumulates `truncated_tokens`: source / text tokens cut to make the record fit."""
    if task.is_supervised_generation():
        toks, pos = T.frame_supervised(task, rec, tok, seq, eos, stats)
        return {"tokens": toks, "positions": pos}
    if task.is_retrieval():
        q, docs, positive = T.retrieval_record(task, rec)
        qt, qe = T.frame_retrieval_text(task.params["query_prefix"], q, tok, seq, eos, stats)
        framed = [T.frame_retrieval_text(task.params["document_prefix"], d, tok, seq, eos, stats) for d in docs]
        return {"query": qt, "query_end": qe, "docs": [f[0] for f in framed], "doc_ends": [f[1] for f in framed],
                "positive": positive}
    raise T.TaskError(f"task `{task.type}` has no wake-trainer framing")


def objective_loss(model, phase, samples: List[Any], device) -> Tuple[torch.Tensor, torch.Tensor, int]:
    """(loss, router aux loss, compute tokens) for one micro-batch of framed samples."""
    t = phase.task.type
    if t == "causal_lm":
        x = torch.tensor(samples, dtype=torch.int64, device=device)
        loss, aux = model.forward_loss(x[:, :-1], x[:, 1:], with_router=True)
        return loss, aux, x[:, :-1].numel()
    if phase.task.is_supervised_generation():
        x = torch.tensor([s["tokens"] for s in samples], dtype=torch.int64, device=device)
        S = x.shape[1] - 1
        flat = [b * S + p for b, s in enumerate(samples) for p in s["positions"]]
        pos = torch.tensor(flat, dtype=torch.int64, device=device)
        loss, aux = model.forward_masked_loss(x[:, :-1], x[:, 1:], pos, with_router=True)
        return loss, aux, x[:, :-1].numel()
    if phase.task.is_retrieval():
        return _retrieval_loss(model, phase.task, samples, device)
    raise T.TaskError(f"task `{t}` is not trainable by the wake trainer")


def _retrieval_loss(model, task, samples, device):
    """Queries against every document in the batch: own positive is the label, own
    explicit negatives and all other queries' documents are negatives."""
    q = torch.tensor([s["query"] for s in samples], dtype=torch.int64, device=device)
    qe = torch.tensor([s["query_end"] for s in samples], dtype=torch.int64, device=device)
    docs, ends, labels = [], [], []
    for s in samples:
        labels.append(len(docs) + s["positive"])
        docs.extend(s["docs"])
        ends.extend(s["doc_ends"])
    d = torch.tensor(docs, dtype=torch.int64, device=device)
    de = torch.tensor(ends, dtype=torch.int64, device=device)
    layer = task.params.get("layer")
    qv = model.forward_embeddings(q, qe, layer)
    dv = model.forward_embeddings(d, de, layer)
    logits = qv @ dv.t() / task.params["temperature"]
    y = torch.tensor(labels, dtype=torch.int64, device=device)
    loss = F.cross_entropy(logits, y)
    return loss, loss.new_zeros(()), q.numel() + d.numel()


def retrieval_accuracy(logits: torch.Tensor, labels: torch.Tensor) -> float:
    return float((logits.argmax(dim=-1) == labels).float().mean())


def forward_kl(student_logits: torch.Tensor, teacher_logits: torch.Tensor, temperature: float = 1.0,
               scale_by_t2: bool = False) -> torch.Tensor:
    """mean_rows Σ_v p_T (log p_T − log p_S) at temperature T (`posttrain.rs:657-691`)."""
    ls = F.log_softmax(student_logits.float() / temperature, dim=-1)
    lt = F.log_softmax(teacher_logits.float() / temperature, dim=-1)
    kl = (lt.exp() * (lt - ls)).sum(dim=-1).mean()
    return kl * temperature * temperature if scale_by_t2 else kl
