"""Evaluation commands: `eval` (token-weighted CE / perplexity; in-batch retrieval top-1 / MRR / recall@k),
`retrieval-pool-eval` (global pool ranks with nDCG@10 and the rank tail) and `generate-eval` (decode-quality text
statistics). Each writes the reference's report for that command (`summa-train/src/eval.rs:145-194`, version 3;
`retrieval_pool.rs:127-150`, version 3; `generate_eval.rs:86-121`, version 1) with the same flags.

Reports are deterministic JSON without timing or host name; rank ties break toward the lower index
(`summa-train/src/eval.rs:87-105`).
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


RETRIEVAL_POOL_REPORT_VERSION = 3


def rank_distribution(ranks: List[int]) -> Dict[str, Any]:
    """Where the positives landed: mean, nearest-rank median / p90 / p99 (always an observed rank), the worst rank and
    the number of queries beyond rank 100 (`summa-train/src/retrieval_pool.rs:88-125`)."""
    if not ranks:
        raise T.TaskError("rank distribution needs at least one query")
    r = sorted(ranks)
    q = lambda f: r[min(max(math.ceil(f * len(r)) - 1, 0), len(r) - 1)]
    return {"mean": sum(r) / len(r), "median": q(0.5), "p90": q(0.9), "p99": q(0.99), "worst": r[-1], "beyond_100": sum(x > 100 for x in r)}


class _Pool:
    """Deduplicated document pool keyed by `document_id`, plus the queries asked against it."""

    def __init__(self):
        self.documents: List = []          # (tokens, end position)
        self.index: Dict[str, int] = {}
        self.queries: List = []            # ((tokens, end position), pool index of the positive)
        self.stats = {"truncated_tokens": 0}

    def intern(self, doc_id: str, framed, truncated: int):
        at = self.index.get(doc_id)
        if at is not None:
            if self.documents[at] != framed:      # the same id must carry the same model-visible text
                raise T.TaskError(f"document_id `{doc_id}` maps to different model-visible text")
            return at
        self.index[doc_id] = len(self.documents)
        self.documents.append(framed)
        self.stats["truncated_tokens"] += truncated
        return len(self.documents) - 1

    def absorb(self, task: T.TaskConfig, rec: Dict[str, Any], tok, seq: int, eos: int, collect_queries: bool) -> None:
        query, docs, positive = T.retrieval_record(task, rec)
        if positive != 0:
            raise T.TaskError(f"retrieval adapter placed the positive at index {positive}; this command assumes index 0")
        pid = rec.get("document_id")
        if not isinstance(pid, str):
            raise T.TaskError("retrieval record has no string `document_id`; the pool is keyed by it")
        nids = rec.get("negative_document_ids", [])
        if not isinstance(nids, list) or not all(isinstance(i, str) for i in nids):
            raise T.TaskError("`negative_document_ids` must be an array of strings")
        if len(nids) != len(docs) - 1:
            raise T.TaskError(f"record has {len(docs) - 1} negative document(s) but {len(nids)} negative id(s); the pool cannot be keyed reliably")
        where = None
        for offset, text in enumerate(docs):
            st = {"truncated_tokens": 0}
            framed = T.frame_retrieval_text(task.params["document_prefix"], text, tok, seq, eos, st)
            at = self.intern(pid if offset == 0 else nids[offset - 1], framed, st["truncated_tokens"])
            if offset == 0:
                where = at
        if collect_queries:
            self.queries.append((T.frame_retrieval_text(task.params["query_prefix"], query, tok, seq, eos, self.stats), where))


@torch.no_grad()
def retrieval_pool_eval(model, tok, task: T.TaskConfig, pool: "_Pool", seq: int, dev, batch_size: int, recall_k: int) -> Dict[str, Any]:
    """Ranks every query against the whole pool; returns the `retrieval` block of the report."""
    layer = task.params.get("layer")

    def embed(framed):
        out = []
        for i in range(0, len(framed), batch_size):
            chunk = framed[i:i + batch_size]
            x = torch.tensor([f[0] for f in chunk], dtype=torch.int64, device=dev)
            e = torch.tensor([f[1] for f in chunk], dtype=torch.int64, device=dev)
            out.append(model.forward_embeddings(x, e, layer).float())
        return torch.cat(out)

    dv = embed(pool.documents).t().contiguous()            # embeddings are L2-normalised: the product is the cosine
    ranks = []
    for i in range(0, len(pool.queries), batch_size):
        chunk = pool.queries[i:i + batch_size]
        sim = (embed([q for q, _ in chunk]) @ dv).cpu()
        ranks += [rank_of(row, positive) for row, (_, positive) in zip(sim, chunk)]
    n = len(ranks)
    return {"top1_accuracy": sum(r == 1 for r in ranks) / n, "mrr": sum(1.0 / r for r in ranks) / n,
            "recall_at_k": sum(r <= recall_k for r in ranks) / n, "k": recall_k,
            "ndcg_at_10": sum(1.0 / math.log2(r + 1) for r in ranks if r <= 10) / n, "ranks": rank_distribution(ranks)}


def retrieval_pool_command(args) -> Dict[str, Any]:
    """`retrieval-pool-eval` (`summa-train/src/retrieval_pool.rs:127-150,326-560`, report version 3): every query of
    the `--data` shards is ranked against the pool of ALL distinct documents (by `document_id`) of those shards plus
    the `--distractors` shards, which only enlarge the pool. Query shards are pooled first, so the report can say
    how many documents came from distractors."""
    seq, bs = args.sequence_length, args.batch_size
    recall_k = int(getattr(args, "recall_k", 10) or 10)
    if seq <= 0 or bs <= 0 or recall_k <= 0:
        raise T.TaskError("--sequence-length, --batch-size and --recall-k must be positive")
    spec: Dict[str, Any] = {"type": "retrieval_representation"}
    if getattr(args, "task", None):
        spec = json.loads(args.task)
    layer = getattr(args, "retrieval_layer", None)
    if layer is not None:
        spec["layer"] = layer
    task = T.TaskConfig.from_json(spec)
    if task.type != "retrieval_representation":
        raise T.TaskError("retrieval-pool-eval scores the retrieval_representation objective")
    warnings: List[str] = []
    model_path = getattr(args, "config", None) or args.model
    tok = Tokenizer.from_file(args.tokenizer)
    cfg = mal.load_model_def(model_path)
    if cfg.vocab_size != tok.vocab_size():
        warnings.append(f"model config vocab_size {cfg.vocab_size} differs from tokenizer vocab_size {tok.vocab_size()}; "
                        "evaluating with the tokenizer vocabulary exactly as `train` does")
        cfg.vocab_size = tok.vocab_size()
    if seq > cfg.max_seq_len:
        raise T.TaskError(f"--sequence-length {seq} exceeds model max_seq_len {cfg.max_seq_len}")
    if task.params.get("layer") is not None and task.params["layer"] > cfg.num_layers:
        raise T.TaskError(f"retrieval layer {task.params['layer']} exceeds the model's {cfg.num_layers} layers")
    dev = torch.device(args.device or ("cuda" if torch.cuda.is_available() else "cpu"))
    model = Transformer(cfg)
    W.load_safetensors(model, args.checkpoint)
    model = model.to(dev).eval()
    if dev.type == "cuda":
        model = model.to(torch.bfloat16)
        model.stream_dtype = torch.bfloat16
    eos = tok.eos_id()
    pool = _Pool()
    sources = []
    data = args.data if isinstance(args.data, (list, tuple)) else [args.data]
    distractors = list(getattr(args, "distractors", None) or [])
    from_queries = 0
    for path, collect in [(p, True) for p in data] + [(p, False) for p in distractors]:
        docs0, q0, read = len(pool.documents), len(pool.queries), 0
        with D._open_text(path) as f:
            for line in f:
                if len(line) > MAX_EVAL_RECORD_BYTES:
                    raise D.DataError(f"record {read + 1} in {path} exceeds the {MAX_EVAL_RECORD_BYTES}-byte limit")
                if not line.strip():
                    continue
                read += 1
                try:
                    rec = json.loads(line)
                except json.JSONDecodeError as e:
                    raise D.DataError(f"cannot parse {path}:{read} as JSON: {e}")
                try:
                    pool.absorb(task, rec, tok, seq, eos, collect)
                except T.TaskError as e:
                    raise T.TaskError(f"cannot pool {path}:{read}: {e}")
        if collect:
            from_queries = len(pool.documents)
        sources.append({"path": path, "identity": "sha256:" + D.file_sha256(path), "records_read": read,
                        "queries": len(pool.queries) - q0, "documents_added": len(pool.documents) - docs0})
    if not pool.queries:
        raise T.TaskError("--data produced no retrieval queries")
    if len(pool.documents) < 2:
        raise T.TaskError(f"the candidate pool holds {len(pool.documents)} document(s); ranking needs at least two")
    if len(pool.documents) <= bs:
        warnings.append(f"pool holds only {len(pool.documents)} document(s), no more than --batch-size {bs}; this is no harder than the "
                        "in-batch `eval` metric")
    metrics = retrieval_pool_eval(model, tok, task, pool, seq, dev, bs, recall_k)
    sequences = len(pool.documents) + len(pool.queries)
    report = {"version": RETRIEVAL_POOL_REPORT_VERSION, "objective": task.type, "task": task.to_json(), "config": model_path,
              "config_sha256": D.file_sha256(model_path), "tokenizer": args.tokenizer, "tokenizer_sha256": D.file_sha256(args.tokenizer),
              "checkpoint": args.checkpoint, "checkpoint_sha256": D.file_sha256(args.checkpoint), "device": str(dev),
              "sequence_length": seq, "batch_size": bs, "retrieval_layer": task.params.get("layer"), "data": sources,
              "pool": {"documents": len(pool.documents), "queries": len(pool.queries), "from_distractors": len(pool.documents) - from_queries},
              "embedded_sequences": sequences, "compute_tokens": sequences * seq, "truncated_tokens": pool.stats["truncated_tokens"],
              "warnings": warnings, "retrieval": metrics}
    for w in warnings:
        print(f"warning: {w}", file=sys.stderr)
    if getattr(args, "output", None):
        _write_json(report, args.output)
    return report


GENERATE_EVAL_REPORT_VERSION = 1
DEGENERATE_TRIGRAM_RATE = 0.10      # most frequent trigram above this share of all trigrams = a degenerate decode
MAX_EVAL_RECORD_BYTES = 64 * 1024 * 1024


def words(text: str) -> List[str]:
    """Lower-case alphanumeric words: the comparison basis of every text metric here."""
    out, cur = [], []
    for ch in text:
        if ch.isalnum():
            cur.append(ch)
        elif cur:
            out.append("".join(cur).lower())
            cur = []
    if cur:
        out.append("".join(cur).lower())
    return out


def repeated_trigram_rate(w: List[str]) -> float:
    """Share of the word trigrams taken by the most frequent one, not counting its first occurrence (unique text
    scores zero; fewer than five words score zero)."""
    if len(w) < 5:
        return 0.0
    counts = Counter(tuple(w[i:i + 3]) for i in range(len(w) - 2))
    return (max(counts.values()) - 1) / (len(w) - 2)


def source_overlap(generated: List[str], source: List[str]) -> float:
    """Share of the generation's word 4-grams that also occur in the source text."""
    if len(generated) < 4:
        return 0.0
    ref = {tuple(source[i:i + 4]) for i in range(len(source) - 3)}
    grams = [tuple(generated[i:i + 4]) for i in range(len(generated) - 3)]
    return sum(g in ref for g in grams) / len(grams)


def contains_word_sequence(generated: List[str], target: List[str]) -> bool:
    n = len(target)
    return 0 < n <= len(generated) and any(generated[i:i + n] == target for i in range(len(generated) - n + 1))


def generation_metrics(outputs: List[Dict[str, Any]]) -> Dict[str, float]:
    """Means over records `{generated, target, source, stopped_at_eos, tokens}` (`generate_eval.rs:59-84,125-170`)."""
    n = len(outputs)
    mean = (lambda xs: sum(xs) / n) if n else (lambda xs: 0.0)
    gen = [words(o["generated"]) for o in outputs]
    rates = [repeated_trigram_rate(g) for g in gen]
    return {
        "repeated_trigram_rate": mean(rates),
        "degenerate_fraction": mean([1.0 if r > DEGENERATE_TRIGRAM_RATE else 0.0 for r in rates]),
        "target_containment": mean([1.0 if contains_word_sequence(g, words(o.get("target", ""))) else 0.0 for g, o in zip(gen, outputs)]),
        "source_overlap": mean([source_overlap(g, words(o.get("source", ""))) for g, o in zip(gen, outputs)]),
        "empty_fraction": mean([1.0 if not o["generated"].strip() else 0.0 for o in outputs]),
        "stopped_at_eos": mean([1.0 if o.get("stopped_at_eos") else 0.0 for o in outputs]),
        "mean_generated_tokens": mean([float(o.get("tokens", 0)) for o in outputs]),
        "mean_generated_words": mean([float(len(g)) for g in gen]),
    }


def _write_json(value, path: str) -> None:
    import os
    tmp = f"{path}.{os.getpid()}.tmp"
    with open(tmp, "wb") as f:
        f.write((json.dumps(value, indent=2) + "\n").encode())
        f.flush()
        os.fsync(f.fileno())
    os.replace(tmp, path)


@torch.no_grad()
def generate_eval_command(args) -> Dict[str, Any]:
    """Decode-quality evaluation of a supervised-generation objective (`summa-train/src/generate_eval.rs:86-121,
    188-488`, report version 1): every held-out record is framed exactly like its training example, the prompt is
    decoded with pinned sampling settings (always seeded), and the report carries means of the text statistics,
    identities of every input, skipped over-long records and warnings. `--samples` writes the verbatim decodes to
    their own file (and keeps them out of the metrics report)."""
    objective = getattr(args, "objective", None)
    if objective is not None:
        if objective not in ("summarization", "instruction_tuning", "qa_reasoning", "retrieval_planning"):
            raise T.TaskError(f"`{objective}` is not a supervised-generation objective")
        spec: Dict[str, Any] = {"type": objective}
        if getattr(args, "instruction", None) is not None:
            spec["instruction"] = args.instruction
        if objective == "qa_reasoning":
            spec["require_reasoning"] = bool(getattr(args, "require_reasoning", False))
        elif getattr(args, "require_reasoning", False):
            raise T.TaskError("--require-reasoning only applies to --objective qa_reasoning")
        task = T.TaskConfig.from_json(spec)
    else:
        task = T.TaskConfig.from_json(json.loads(args.task))
        if not task.is_supervised_generation():
            raise T.TaskError(f"`{task.type}` is not a supervised-generation objective")
    out_path, samples_path = getattr(args, "output", None), getattr(args, "samples", None)
    if out_path and samples_path and out_path == samples_path:
        raise T.TaskError("--output and --samples must name different files")
    seq, max_new = args.sequence_length, args.max_new_tokens
    if seq <= 0 or max_new <= 0:
        raise T.TaskError("--sequence-length and --max-new-tokens must be positive")
    max_records = getattr(args, "max_records", None)
    if max_records is None:
        max_records = getattr(args, "limit", None)
    warnings: List[str] = []
    model_path = getattr(args, "config", None) or args.model
    tok = Tokenizer.from_file(args.tokenizer)
    cfg = mal.load_model_def(model_path)
    if cfg.vocab_size != tok.vocab_size():
        warnings.append(f"model config vocab_size {cfg.vocab_size} differs from tokenizer vocab_size {tok.vocab_size()}; "
                        "decoding with the tokenizer vocabulary exactly as `train` does")
        cfg.vocab_size = tok.vocab_size()
    if seq > cfg.max_seq_len:
        raise T.TaskError(f"--sequence-length {seq} exceeds model max_seq_len {cfg.max_seq_len}")
    dev = torch.device(args.device or ("cuda" if torch.cuda.is_available() else "cpu"))
    model = Transformer(cfg)
    W.load_safetensors(model, args.checkpoint)
    model = model.to(dev).eval()
    if dev.type == "cuda":
        model.prepare_inference(torch.bfloat16)
    eos = tok.eos_id()
    gen = TextGenerator(model, tok)
    temperature, top_k = float(getattr(args, "temperature", 0.0) or 0.0), getattr(args, "top_k", None)
    penalty, seed = float(getattr(args, "repetition_penalty", 1.0) or 1.0), int(getattr(args, "seed", 0) or 0)
    sampling = SamplingConfig(max_new_tokens=max_new, temperature=temperature, top_k=int(top_k or 0), repetition_penalty=penalty, seed=seed)
    outs, samples, sources = [], [], []
    stats = {"truncated_tokens": 0}
    paths = args.data if isinstance(args.data, (list, tuple)) else [args.data]
    for path in paths:
        read = oversized = 0
        with D._open_text(path) as f:
            for line in f:
                if max_records is not None and len(outs) >= max_records:
                    break
                if len(line) > MAX_EVAL_RECORD_BYTES:
                    raise D.DataError(f"record {read + 1} in {path} exceeds the {MAX_EVAL_RECORD_BYTES}-byte limit")
                if not line.strip():
                    continue
                read += 1
                try:
                    rec = json.loads(line)
                except json.JSONDecodeError as e:
                    raise D.DataError(f"cannot parse {path}:{read} as JSON: {e}")
                seg = T.supervised_prompt(task, rec)
                try:
                    toks, positions = T.frame_supervised(task, rec, tok, seq, eos, stats)
                except T.OversizedRecord:
                    oversized += 1
                    continue
                prompt = toks[:positions[0] + 1]                     # everything before the first supervised target token
                pre_len = len(tok.encode(seg.prefix))
                suf_len = len(tok.encode(seg.suffix))
                visible_source = tok.decode(prompt[pre_len:len(prompt) - suf_len])
                new = gen.generate_ids(prompt, sampling)
                stopped = bool(new) and new[-1] == eos
                if stopped:
                    new = new[:-1]
                text = tok.decode(new).strip()
                outs.append({"generated": text, "target": seg.target, "source": visible_source, "stopped_at_eos": stopped, "tokens": len(new)})
                if samples_path:
                    g = words(text)
                    samples.append({"prompt": tok.decode(prompt), "generated": text, "target": seg.target,
                                    "repeated_trigram_rate": repeated_trigram_rate(g),
                                    "contains_target": contains_word_sequence(g, words(seg.target))})
        if oversized:
            warnings.append(f"skipped {oversized} record(s) in {path} whose prompt, complete target, and EOS exceed --sequence-length {seq}")
        sources.append({"path": path, "identity": "sha256:" + D.file_sha256(path), "records_read": read, "oversized_records": oversized})
    if not outs:
        raise T.TaskError("held-out data produced no scorable record")
    report: Dict[str, Any] = {
        "version": GENERATE_EVAL_REPORT_VERSION, "objective": task.type, "task": task.to_json(), "config": model_path,
        "config_sha256": D.file_sha256(model_path), "tokenizer": args.tokenizer, "tokenizer_sha256": D.file_sha256(args.tokenizer),
        "checkpoint": args.checkpoint, "checkpoint_sha256": D.file_sha256(args.checkpoint), "device": str(dev), "sequence_length": seq,
        "max_new_tokens": max_new, "temperature": temperature, "top_k": top_k, "repetition_penalty": penalty, "seed": seed, "data": sources,
        "scored_records": len(outs), "oversized_records": sum(s_["oversized_records"] for s_ in sources),
        "truncated_tokens": stats["truncated_tokens"], "warnings": warnings, "generation": generation_metrics(outs)}
    for w in warnings:
        print(f"warning: {w}", file=sys.stderr)
    if samples_path:
        _write_json(samples, samples_path)
    elif samples:
        report["samples"] = samples
    if out_path:
        _write_json(report, out_path)
    return report
