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


@torch.no_grad()
def eval_command(args) -> Dict[str, Any]:
    model, tok, cfg, dev = _load(args)
    task = T.TaskConfig.from_json(json.loads(args.task))
    eos = tok.eos_id()
    seq, bs = args.sequence_length, args.batch_size
    if task.type == "causal_lm":
        total, count = 0.0, 0
        for batch in D.iter_batches(D.iter_samples(args.data, tok, cfg.vocab_size, seq, eos), bs):
            x = torch.tensor(batch, dtype=torch.int64, device=dev)
            loss = model.forward_loss(x[:, :-1], x[:, 1:])
            n = x[:, 1:].numel()
            total += float(loss) * n
            count += n
        mean = total / max(count, 1)
        return {"task": task.type, "tokens": count, "loss": mean, "perplexity": math.exp(min(mean, 50.0))}
    skipped = 0
    if task.is_supervised_generation():
        total, count = 0.0, 0
        with D._open_text(args.data) as f:
            rows = [json.loads(l) for l in f if l.strip()]
        framed = []
        for r in rows:
            try:
                framed.append(frame_record(task, r, tok, seq, eos))
            except T.OversizedRecord:
                skipped += 1
        for i in range(0, len(framed), bs):
            chunk = framed[i:i + bs]
            x = torch.tensor([c["tokens"] for c in chunk], dtype=torch.int64, device=dev)
            pos = torch.tensor([b * seq + p for b, c in enumerate(chunk) for p in c["positions"]],
                               dtype=torch.int64, device=dev)
            loss = model.forward_masked_loss(x[:, :-1], x[:, 1:], pos)
            total += float(loss) * pos.numel()
            count += pos.numel()
        mean = total / max(count, 1)
        return {"task": task.type, "supervised_tokens": count, "loss": mean,
                "perplexity": math.exp(min(mean, 50.0)), "skipped_oversized": skipped}
    if task.is_retrieval():
        ranks = []
        with D._open_text(args.data) as f:
            rows = [json.loads(l) for l in f if l.strip()]
        framed = []
        for r in rows:
            try:
                framed.append(frame_record(task, r, tok, seq, eos))
            except T.OversizedRecord:
                skipped += 1
        for i in range(0, len(framed), bs):
            chunk = framed[i:i + bs]
            q = torch.tensor([c["query"] for c in chunk], dtype=torch.int64, device=dev)
            qe = torch.tensor([c["query_end"] for c in chunk], dtype=torch.int64, device=dev)
            docs, ends, labels = [], [], []
            for c in chunk:
                labels.append(len(docs) + c["positive"])
                docs.extend(c["docs"]); ends.extend(c["doc_ends"])
            d = torch.tensor(docs, dtype=torch.int64, device=dev)
            de = torch.tensor(ends, dtype=torch.int64, device=dev)
            layer = task.params.get("layer")
            sim = model.forward_embeddings(q, qe, layer) @ model.forward_embeddings(d, de, layer).t()
            for row, lab in zip(sim.float().cpu(), labels):
                ranks.append(rank_of(row, lab))
        out = {"task": task.type, "queries": len(ranks), "skipped_oversized": skipped}
        out.update(retrieval_metrics(ranks))
        return out
    raise T.TaskError(f"task `{task.type}` has no eval implementation")


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
