"""Evaluation commands: `eval` (token-weighted CE / perplexity; in-batch retrieval
top-1 / MRR / recall@k), `retrieval-pool-eval` (global pool ranks with nDCG@10) and
`generate-eval` (greedy decode quality metrics).

Reports are deterministic JSON without timing; rank ties break toward the lower index
(`summa-train/src/eval.rs:87-105,145-194`, `docs/generation-eval.md:22-36`,
`docs/retrieval-pool-eval.md`).
"""
from __future__ import annotations

import json
import math
import sys
from collections import Counter
from typing import Any, Dict, List

import torch

from .. import mal
from ..models import Transformer
from ..models import weights as W
from ..models.generate import SamplingConfig, TextGenerator
from ..tokenizer import Tokenizer
from . import data as D
from . import task as T
from .objectives import frame_record


def _load(args):
    tok = Tokenizer.from_file(args.tokenizer)
    cfg = mal.load_model_def(args.model)
    cfg.vocab_size = tok.vocab_size()
    model = Transformer(cfg)
    W.load_safetensors(model, args.checkpoint)
    dev = torch.device(args.device or ("cuda" if torch.cuda.is_available() else "cpu"))
    model = model.to(dev).eval()
    if dev.type == "cuda":
        model.prepare_inference(torch.bfloat16)
    return model, tok, cfg, dev


def rank_of(scores: torch.Tensor, label: int) -> int:
    """1-based rank of `label`; ties resolve toward the lower index."""
    s = scores[label]
    better = int((scores > s).sum())
    ties_before = int((scores[:label] == s).sum())
    return better + ties_before + 1


def retrieval_metrics(ranks: List[int], ks=(1, 5, 10)) -> Dict[str, float]:
    n = max(len(ranks), 1)
    out = {"top1": sum(r == 1 for r in ranks) / n, "mrr": sum(1.0 / r for r in ranks) / n,
           "ndcg@10": sum((1.0 / math.log2(r + 1)) if r <= 10 else 0.0 for r in ranks) / n}
    for k in ks:
        out[f"recall@{k}"] = sum(r <= k for r in ranks) / n
    return out


EVAL_REPORT_VERSION = 3
OBJECTIVE_TASKS = {"causal_lm": "causal_lm", "contrastive_retrieval": "retrieval_representation", "summarization": "summarization",
                   "instruction_tuning": "instruction_tuning", "qa_reasoning": "qa_reasoning", "retrieval_planning": "retrieval_planning"}


class _WeightedMean:
    def __init__(self):
        self.total, self.weight = 0.0, 0

    def push(self, value: float, weight: int) -> None:
        if not math.isfinite(value):
            raise T.TaskError("evaluation produced a non-finite value; check that the configuration and the checkpoint match")
        self.total += value * weight
        self.weight += weight

    def mean(self):
        return self.total / self.weight if self.weight else None


def eval_task_config(args) -> T.TaskConfig:
    """The task a held-out evaluation frames its prompts with: `--objective` plus the few fields the command line
    exposes over the trainer's defaults (`summa-train/src/eval.rs:385-460`); `--task` (a task JSON) is the long
    form of the same thing."""
    objective = getattr(args, "objective", None)
    if objective is None:
        return T.TaskConfig.from_json(json.loads(getattr(args, "task", None) or '{"type": "causal_lm"}'))
    if objective not in OBJECTIVE_TASKS:
        raise T.TaskError(f"unknown objective `{objective}`")
    layer, temp = getattr(args, "retrieval_layer", None), getattr(args, "temperature", None)
    instruction, reasoning = getattr(args, "instruction", None), bool(getattr(args, "require_reasoning", False))
    if objective != "contrastive_retrieval" and (layer is not None or temp is not None):
        raise T.TaskError("--retrieval-layer and --temperature only apply to --objective contrastive_retrieval")
    supervised = objective in ("summarization", "instruction_tuning", "qa_reasoning", "retrieval_planning")
    if not supervised and instruction is not None:
        raise T.TaskError("--instruction only applies to a supervised-generation objective")
    if reasoning and objective != "qa_reasoning":
        raise T.TaskError("--require-reasoning only applies to --objective qa_reasoning")
    spec: Dict[str, Any] = {"type": OBJECTIVE_TASKS[objective]}
    if temp is not None:
        spec["temperature"] = temp
    if layer is not None:
        spec["layer"] = layer
    if instruction is not None:
        spec["instruction"] = instruction
    if objective == "qa_reasoning":
        spec["require_reasoning"] = reasoning
    return T.TaskConfig.from_json(spec)


def _held_out_samples(path: str, task: T.TaskConfig, tok, vocab: int, seq: int, eos: int, shuffle: int, seed: int, oversized: List[int], stats=None):
    """Framed samples of one held-out shard in evaluation order. Supervised records that do not fit the sequence
    length are skipped and counted (training aborts on them; one long record must not void an evaluation)."""
    if task.type == "causal_lm":
        yield from D.iter_samples(path, tok, vocab, seq, eos, shuffle, seed)
        return
    base = path[:-4] if path.endswith(".zst") else path
    if not base.endswith(".jsonl"):
        raise D.DataError(f"{path}: structured objectives need .jsonl or .jsonl.zst data")
    buf = D.ShuffleBuffer(shuffle, seed)
    with D._open_text(path) as f:
        for n, line in enumerate(f, 1):
            if not line.strip():
                continue
            try:
                rec = json.loads(line)
            except json.JSONDecodeError as e:
                raise D.DataError(f"{path}:{n}: invalid JSON: {e}")
            try:
                item = frame_record(task, rec, tok, seq, eos, stats)
            except T.OversizedRecord:
                if not task.is_supervised_generation():
                    raise
                oversized[0] += 1
                continue
            got = buf.push(item)
            if got is not None:
                yield got
    yield from buf.drain()


@torch.no_grad()
def eval_command(args) -> Dict[str, Any]:
    """Held-out evaluation with the trainer's own objective forward pass. The report has the reference's shape
    (`summa-train/src/eval.rs:145-194,493-693`, version 3): identities of configuration / tokenizer / checkpoint
    / every shard, the complete task, counters, warnings, and one metrics object per objective family; it holds no
    timing and no host name, so equal inputs give byte-identical JSON. Language losses are weighted by supervised
    tokens (a short last batch is scored); contrastive losses by queries (a short last batch is dropped, because
    in-batch negatives make accuracy a function of the pool size)."""
    task = eval_task_config(args)
    seq, bs = args.sequence_length, args.batch_size
    recall_k = int(getattr(args, "recall_k", 10) or 10)
    max_batches = getattr(args, "max_batches", None)
    shuffle, seed = int(getattr(args, "shuffle_buffer", 0) or 0), int(getattr(args, "seed", 0) or 0)
    if seq <= 0 or bs <= 0 or recall_k <= 0 or (max_batches is not None and max_batches <= 0):
        raise T.TaskError("--sequence-length, --batch-size, --recall-k and --max-batches must be positive")
    warnings: List[str] = []
    if shuffle == 0 and seed != 0:
        warnings.append(f"--seed {seed} has no effect with --shuffle-buffer 0; held-out shards are read in source order")
    model_path = getattr(args, "config", None) or args.model
    tok = Tokenizer.from_file(args.tokenizer)
    cfg = mal.load_model_def(model_path)
    if cfg.vocab_size != tok.vocab_size():
        warnings.append(f"model config vocab_size {cfg.vocab_size} differs from tokenizer vocab_size {tok.vocab_size()}; "
                        "evaluating with the tokenizer vocabulary exactly as `train` does")
        cfg.vocab_size = tok.vocab_size()
    if seq > cfg.max_seq_len:
        raise T.TaskError(f"--sequence-length {seq} exceeds model max_seq_len {cfg.max_seq_len}")
    if task.is_retrieval() and task.params.get("layer") is not None and task.params["layer"] > cfg.num_layers:
        raise T.TaskError(f"retrieval layer {task.params['layer']} exceeds the model's {cfg.num_layers} layers")
    dev = torch.device(args.device or ("cuda" if torch.cuda.is_available() else "cpu"))
    model = Transformer(cfg)
    W.load_safetensors(model, args.checkpoint)
    # the training forward in evaluation mode: no inference-time weight casts, so the numbers compare with training metrics
    model = model.to(dev).eval()
    if dev.type == "cuda":
        model = model.to(torch.bfloat16)
        model.stream_dtype = torch.bfloat16
    eos = tok.eos_id()
    if eos is None:
        raise T.TaskError("tokenizer has no end-of-sequence token")
    retrieval = task.is_retrieval()
    stats = {"examples": 0, "compute_tokens": 0, "supervised_tokens": 0, "truncated_tokens": 0, "retrieval_candidates": 0}
    language, router, r_loss, r_top1, r_rr, r_recall = (_WeightedMean() for _ in range(6))
    cand_range: List[int] = []
    batches = 0

    def score(samples) -> None:
        nonlocal batches
        batches += 1
        if task.type == "causal_lm":
            x = torch.tensor(samples, dtype=torch.int64, device=dev)
            loss, aux = model.forward_loss(x[:, :-1], x[:, 1:], with_router=True)
            n = x[:, 1:].numel()
            stats["examples"] += x.shape[0]
            stats["compute_tokens"] += n
            stats["supervised_tokens"] += n
            language.push(float(loss), n)
            weight = n
        elif task.is_supervised_generation():
            x = torch.tensor([c["tokens"] for c in samples], dtype=torch.int64, device=dev)
            S = x.shape[1] - 1
            pos = torch.tensor([b * S + p for b, c in enumerate(samples) for p in c["positions"]], dtype=torch.int64, device=dev)
            loss, aux = model.forward_masked_loss(x[:, :-1], x[:, 1:], pos, with_router=True)
            stats["examples"] += x.shape[0]
            stats["compute_tokens"] += x[:, :-1].numel()
            stats["supervised_tokens"] += pos.numel()
            language.push(float(loss), pos.numel())
            weight = pos.numel()
        else:
            q = torch.tensor([c["query"] for c in samples], dtype=torch.int64, device=dev)
            qe = torch.tensor([c["query_end"] for c in samples], dtype=torch.int64, device=dev)
            docs, ends, labels = [], [], []
            for c in samples:
                labels.append(len(docs) + c["positive"])
                docs.extend(c["docs"])
                ends.extend(c["doc_ends"])
            d = torch.tensor(docs, dtype=torch.int64, device=dev)
            de = torch.tensor(ends, dtype=torch.int64, device=dev)
            layer = task.params.get("layer")
            sim = (model.forward_embeddings(q, qe, layer) @ model.forward_embeddings(d, de, layer).t()).float()
            y = torch.tensor(labels, dtype=torch.int64, device=dev)
            loss = torch.nn.functional.cross_entropy(sim / task.params["temperature"], y)
            aux = None
            nq = len(samples)
            stats["examples"] += nq
            stats["compute_tokens"] += q.numel() + d.numel()
            stats["retrieval_candidates"] += len(docs)
            cand_range[:] = [min(cand_range[0], len(docs)), max(cand_range[1], len(docs))] if cand_range else [len(docs), len(docs)]
            r_loss.push(float(loss), nq)
            r_top1.push(float((sim.argmax(dim=1) == y).float().mean()), nq)
            for row, lab in zip(sim.cpu(), labels):          # ranking does not depend on the positive temperature scale
                rank = rank_of(row, lab)
                r_rr.push(1.0 / rank, 1)
                r_recall.push(1.0 if rank <= recall_k else 0.0, 1)
            weight = nq
        if aux is not None and model_has_router:
            router.push(float(aux), weight)

    model_has_router = any(getattr(getattr(blk, "feed_forward", None), "moe", None) is not None for blk in model.layers) or \
        any(getattr(blk, "memory", None) is not None for blk in model.layers)
    paths = args.data if isinstance(args.data, (list, tuple)) else [args.data]
    sources, pending, done = [], [], False
    oversized_total = 0
    for index, path in enumerate(paths):
        if done:
            break
        oversized = [0]
        read = 0
        for sample in _held_out_samples(path, task, tok, cfg.vocab_size, seq, eos, shuffle, D.shuffle_seed(seed, index, 0), oversized, stats):
            read += 1
            pending.append(sample)
            if len(pending) < bs:
                continue
            score(pending)
            pending = []
            if max_batches is not None and batches >= max_batches:
                done = True
                break
        sources.append({"path": path, "identity": "sha256:" + D.file_sha256(path), "samples_read": read, "oversized_records": oversized[0]})
        oversized_total += oversized[0]
    if oversized_total:
        warnings.append(f"skipped {oversized_total} held-out record(s) whose prompt, complete target, and EOS exceed --sequence-length {seq}; "
                        "they are excluded from every reported number")
    dropped = 0
    if pending:
        if retrieval or done:
            dropped = len(pending)
            warnings.append(f"dropped {dropped} held-out sample(s) that could not fill --batch-size {bs}")
        else:
            score(pending)
    if batches == 0:
        raise T.TaskError(f"held-out data produced no complete batch of --batch-size {bs}; {dropped} sample(s) were read and "
                          f"{oversized_total} record(s) did not fit --sequence-length {seq}")
    report: Dict[str, Any] = {
        "version": EVAL_REPORT_VERSION, "objective": task.type, "task": task.to_json(),
        "config": model_path, "config_sha256": D.file_sha256(model_path), "tokenizer": args.tokenizer,
        "tokenizer_sha256": D.file_sha256(args.tokenizer), "checkpoint": args.checkpoint,
        "checkpoint_sha256": D.file_sha256(args.checkpoint), "device": str(dev), "sequence_length": seq, "batch_size": bs,
        "shuffle_buffer": shuffle, "seed": seed, "max_batches": max_batches, "data": sources, "batches": batches,
        "examples": stats["examples"], "compute_tokens": stats["compute_tokens"], "supervised_tokens": stats["supervised_tokens"],
        "truncated_tokens": stats["truncated_tokens"], "dropped_samples": dropped, "oversized_records": oversized_total,
        "warnings": warnings}
    if router.mean() is not None:
        report["router_loss"] = router.mean()
    lang = language.mean()
    if lang is not None:
        ppl = math.exp(lang) if lang < 700 else float("inf")
        if not math.isfinite(ppl):
            raise T.TaskError(f"mean held-out loss {lang} overflows perplexity; check that the configuration and the checkpoint match")
        report["supervised_generation" if task.is_supervised_generation() else "causal_lm"] = {"loss": lang, "perplexity": ppl}
    if r_loss.mean() is not None:
        report["retrieval"] = {"loss": r_loss.mean(), "top1_accuracy": r_top1.mean(), "mrr": r_rr.mean(), "recall_at_k": r_recall.mean(),
                               "k": recall_k, "candidates": {"total": stats["retrieval_candidates"], "min_per_batch": cand_range[0],
                                                              "max_per_batch": cand_range[1]}}
    for w in warnings:
        print(f"warning: {w}", file=sys.stderr)
    out = getattr(args, "output", None)
    if out:
        import os
        body = (json.dumps(report, indent=2) + "\n").encode()
        tmp = f"{out}.{os.getpid()}.tmp"
        with open(tmp, "wb") as f:
            f.write(body)
            f.flush()
            os.fsync(f.fileno())
        os.replace(tmp, out)
    return report


@torch.no_grad()
def retrieval_pool_eval(model, tok, task: T.TaskConfig, rows: List[Dict[str, Any]], seq: int, dev,
                        batch_size: int = 32) -> Dict[str, Any]:
    """Every query is ranked against the GLOBAL pool of distinct documents (report v3)."""
    eos = tok.eos_id()
    pool: Dict[str, int] = {}
    queries, labels = [], []
    for r in rows:
        q, docs, positive = T.retrieval_record(task, r)
        for dtext in docs:
            pool.setdefault(dtext, len(pool))
        queries.append(q)
        labels.append(pool[docs[positive]])
    layer = task.params.get("layer")

    def embed(texts, prefix):
        out = []
        for i in range(0, len(texts), batch_size):
            fr = [T.frame_retrieval_text(prefix, t, tok, seq, eos) for t in texts[i:i + batch_size]]
            x = torch.tensor([f[0] for f in fr], dtype=torch.int64, device=dev)
            e = torch.tensor([f[1] for f in fr], dtype=torch.int64, device=dev)
            out.append(model.forward_embeddings(x, e, layer).float().cpu())
        return torch.cat(out)
    dv = embed(list(pool), task.params["document_prefix"])
    qv = embed(queries, task.params["query_prefix"])
    sim = qv @ dv.t()
    ranks = [rank_of(row, lab) for row, lab in zip(sim, labels)]
    out = {"version": 3, "queries": len(ranks), "pool_size": len(pool),
           "rank_distribution": dict(sorted(Counter(min(r, 101) for r in ranks).items()))}
    out.update(retrieval_metrics(ranks, ks=(1, 5, 10, 100)))
    return out


def retrieval_pool_command(args) -> Dict[str, Any]:
    """`retrieval-pool-eval`: global-pool ranking report for a contrastive-retrieval task."""
    model, tok, cfg, dev = _load(args)
    task = T.TaskConfig.from_json(json.loads(args.task))
    rows = []
    with open(args.data) as f:
        for line in f:
            if line.strip():
                rows.append(json.loads(line))
    return retrieval_pool_eval(model, tok, task, rows, args.sequence_length, dev, args.batch_size)


def _ngrams(tokens: List[str], n: int):
    return [tuple(tokens[i:i + n]) for i in range(len(tokens) - n + 1)]


def generation_metrics(outputs: List[Dict[str, Any]]) -> Dict[str, float]:
    """Aggregate over records `{generated, target, source, stopped_at_eos, tokens}`."""
    n = max(len(outputs), 1)
    tri_rates, contain, overlap, words, toks = [], [], [], [], []
    for o in outputs:
        w = o["generated"].split()
        tri = _ngrams(w, 3)
        rate = 1.0 - len(set(tri)) / len(tri) if tri else 0.0
        tri_rates.append(rate)
        contain.append(1.0 if o.get("target") and o["target"].strip() and o["target"].strip() in o["generated"] else 0.0)
        src4 = set(_ngrams(o.get("source", "").split(), 4))
        gen4 = _ngrams(w, 4)
        overlap.append(sum(g in src4 for g in gen4) / len(gen4) if gen4 else 0.0)
        words.append(len(w))
        toks.append(o.get("tokens", 0))
    return {
        "records": len(outputs),
        "repeated_trigram_rate": sum(tri_rates) / n,
        "degenerate_fraction": sum(r > 0.10 for r in tri_rates) / n,
        "target_containment": sum(contain) / n,
        "source_overlap": sum(overlap) / n,
        "stopped_at_eos": sum(1.0 for o in outputs if o.get("stopped_at_eos")) / n,
        "empty_fraction": sum(1.0 for o in outputs if not o["generated"].strip()) / n,
        "mean_tokens": sum(toks) / n,
        "mean_words": sum(words) / n,
    }


@torch.no_grad()
def generate_eval_command(args) -> Dict[str, Any]:
    model, tok, cfg, dev = _load(args)
    task = T.TaskConfig.from_json(json.loads(args.task))
    gen = TextGenerator(model, tok)
    eos = tok.eos_id()
    outs = []
    with D._open_text(args.data) as f:
        for i, line in enumerate(l for l in f if l.strip()):
            if i >= args.limit:
                break
            rec = json.loads(line)
            seg = T.supervised_prompt(task, rec)
            pre, suf = tok.encode(seg.prefix), tok.encode(seg.suffix)
            room = args.sequence_length - len(pre) - len(suf)
            src = tok.encode(seg.source)[:max(room, 0)]
            ids = gen.generate_ids(pre + src + suf, SamplingConfig(max_new_tokens=args.max_new_tokens))
            stopped = bool(ids) and ids[-1] == eos
            text = tok.decode(ids[:-1] if stopped else ids)
            outs.append({"generated": text, "target": seg.target, "source": tok.decode(src),
                         "stopped_at_eos": stopped, "tokens": len(ids)})
    rep = generation_metrics(outs)
    rep["task"] = task.type
    return rep
