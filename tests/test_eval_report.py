"""`eval`: the held-out report in the reference's shape (version 3), its counters, warnings and flag rules."""
import argparse
import json

import pytest
import torch

from summa_b200 import mal
from summa_b200.models import Transformer
from summa_b200.models import weights as W
from summa_b200.tokenizer import Tokenizer
from summa_b200.train import task as T
from summa_b200.train.eval import eval_command

MAL = """attention a { num_heads: 2 } ffn f { hidden_dim: 64 }
  block b { attention: a ffn: f norm: rmsnorm { eps: 1e-5 } }
  model t { vocab_size: 257 max_seq_len: 64 hidden_size: 32 num_layers: 2 block: b }"""


@pytest.fixture()
def fixture(tmp_path):
    tok = Tokenizer.byte_level()
    (tmp_path / "tokenizer.json").write_text(tok.to_json())
    (tmp_path / "m.mal").write_text(MAL)
    cfg = mal.parse_mal(MAL)
    torch.manual_seed(0)
    W.save_safetensors(Transformer(cfg), str(tmp_path / "w.safetensors"))

    def args(**kw):
        base = dict(model=str(tmp_path / "m.mal"), tokenizer=str(tmp_path / "tokenizer.json"), checkpoint=str(tmp_path / "w.safetensors"),
                    objective=None, task=None, sequence_length=32, batch_size=4, max_batches=None, shuffle_buffer=0, seed=0, recall_k=2,
                    retrieval_layer=None, temperature=None, instruction=None, require_reasoning=False, output=None, device="cpu")
        base.update(kw)
        return argparse.Namespace(**base)
    return tmp_path, args


def test_causal_report_counts_identities_and_is_deterministic(fixture):
    tmp, args = fixture
    a, b = tmp / "a.jsonl", tmp / "b.jsonl"
    a.write_text("\n".join(json.dumps({"text": "the quick brown fox jumps over the lazy dog " * 3}) for _ in range(6)))
    b.write_text("\n".join(json.dumps({"text": "pack my box with five dozen liquor jugs " * 2}) for _ in range(5)))
    out = tmp / "report.json"
    rep = eval_command(args(objective="causal_lm", data=[str(a), str(b)], output=str(out), seed=5))
    assert rep["version"] == 3 and rep["objective"] == "causal_lm" and rep["task"] == {"type": "causal_lm"}
    assert [d["path"] for d in rep["data"]] == [str(a), str(b)] and all(d["identity"].startswith("sha256:") and d["samples_read"] > 0 for d in rep["data"])
    n = sum(d["samples_read"] for d in rep["data"])
    assert rep["examples"] == n and rep["batches"] == -(-n // 4) and rep["dropped_samples"] == 0          # the short last batch is scored
    assert rep["supervised_tokens"] == rep["compute_tokens"] == n * 32
    assert rep["causal_lm"]["perplexity"] == pytest.approx(pytest.importorskip("math").exp(rep["causal_lm"]["loss"]))
    assert 4.0 < rep["causal_lm"]["loss"] < 7.0 and "retrieval" not in rep and "supervised_generation" not in rep and "router_loss" not in rep
    assert any("--seed 5 has no effect" in w for w in rep["warnings"])
    assert json.loads(out.read_text()) == rep
    assert eval_command(args(objective="causal_lm", data=[str(a), str(b)], seed=5)) == rep                     # no timing, no host name
    capped = eval_command(args(objective="causal_lm", data=[str(a), str(b)], max_batches=2))
    assert capped["batches"] == 2 and capped["examples"] == 8 and len(capped["data"]) == 1
    with pytest.raises(T.TaskError, match="exceeds model max_seq_len"):
        eval_command(args(objective="causal_lm", data=[str(a)], sequence_length=128))


def test_supervised_report_skips_and_counts_oversized_records(fixture):
    tmp, args = fixture
    data = tmp / "s.jsonl"
    rows = [{"document": "short text %d" % i, "summary": "ok"} for i in range(5)] + [{"document": "doc", "summary": "y" * 400}, {"document": "z" * 200, "summary": "cut"}]
    data.write_text("\n".join(json.dumps(r) for r in rows))
    rep = eval_command(args(objective="summarization", data=[str(data)], sequence_length=64, instruction="Summarise:"))
    assert rep["objective"] == "summarization" and rep["task"]["instruction"] == "Summarise:"
    assert rep["oversized_records"] == 1 and rep["data"][0]["oversized_records"] == 1 and rep["examples"] == 6 and rep["batches"] == 2 and rep["truncated_tokens"] > 100
    assert 0 < rep["supervised_tokens"] < rep["compute_tokens"] and "supervised_generation" in rep and "causal_lm" not in rep
    assert any("skipped 1 held-out record" in w for w in rep["warnings"])
    with pytest.raises(T.TaskError, match="only apply to --objective contrastive_retrieval"):
        eval_command(args(objective="summarization", data=[str(data)], temperature=0.1))
    with pytest.raises(T.TaskError, match="--instruction only applies"):
        eval_command(args(objective="causal_lm", data=[str(data)], instruction="x"))
    with pytest.raises(T.TaskError, match="--require-reasoning only applies"):
        eval_command(args(objective="summarization", data=[str(data)], require_reasoning=True))


def test_retrieval_report_ranks_and_drops_the_short_batch(fixture):
    tmp, args = fixture
    data = tmp / "r.jsonl"
    rows = [{"query": f"question {i}", "positive": f"answer {i}", "negatives": [f"wrong {i}"]} for i in range(10)]
    data.write_text("\n".join(json.dumps(r) for r in rows))
    rep = eval_command(args(objective="contrastive_retrieval", data=[str(data)], temperature=0.05, retrieval_layer=1, sequence_length=64))
    r = rep["retrieval"]
    assert rep["objective"] == "retrieval_representation" and rep["task"]["temperature"] == 0.05 and rep["task"]["layer"] == 1
    assert rep["batches"] == 2 and rep["examples"] == 8 and rep["dropped_samples"] == 2 and any("dropped 2" in w for w in rep["warnings"])
    assert r["k"] == 2 and r["candidates"] == {"total": 16, "min_per_batch": 8, "max_per_batch": 8}
    assert 0.0 <= r["top1_accuracy"] <= r["recall_at_k"] <= 1.0 and r["top1_accuracy"] <= r["mrr"] <= 1.0 and r["loss"] > 0
    with pytest.raises(T.TaskError, match="exceeds the model's 2 layers"):
        eval_command(args(objective="contrastive_retrieval", data=[str(data)], retrieval_layer=3, sequence_length=64))
    with pytest.raises(T.TaskError, match="no complete batch"):
        eval_command(args(objective="contrastive_retrieval", data=[str(data)], batch_size=16, sequence_length=64))


def test_generate_eval_report_and_text_statistics(fixture):
    from summa_b200.train import eval as E
    tmp, args = fixture
    assert E.words("Berlin, Berlin! the-End 42") == ["berlin", "berlin", "the", "end", "42"]
    assert E.repeated_trigram_rate(E.words("a b c a b c a b c")) == pytest.approx(2 / 7)
    assert E.repeated_trigram_rate(E.words("one two three four")) == 0.0 and E.repeated_trigram_rate(E.words("a b c d e f")) == 0.0
    assert E.source_overlap(E.words("the quick brown fox jumps"), E.words("x the quick brown fox y")) == 0.5
    assert E.contains_word_sequence(E.words("It is Paris, France."), E.words("paris france"))
    assert not E.contains_word_sequence(E.words("Paris"), E.words("")) and not E.contains_word_sequence(E.words("a"), E.words("a b"))
    m = E.generation_metrics([{"generated": "x x x x x x x", "target": "x", "source": "", "stopped_at_eos": True, "tokens": 7},
                              {"generated": "", "target": "y", "source": "", "stopped_at_eos": False, "tokens": 0}])
    assert m["degenerate_fraction"] == 0.5 and m["empty_fraction"] == 0.5 and m["target_containment"] == 0.5 and m["stopped_at_eos"] == 0.5
    assert m["mean_generated_tokens"] == 3.5 and m["mean_generated_words"] == 3.5

    data = tmp / "g.jsonl"
    rows = [{"document": "alpha beta gamma delta %d" % i, "summary": "alpha"} for i in range(4)] + [{"document": "d", "summary": "s" * 300}]
    data.write_text("\n".join(json.dumps(r) for r in rows))
    out, samples = tmp / "gen.json", tmp / "samples.json"
    base = dict(objective="summarization", instruction="S:", data=[str(data)], sequence_length=64, max_new_tokens=6, temperature=0.0, top_k=None,
                repetition_penalty=1.0, seed=3, max_records=None, samples=str(samples), output=str(out))
    rep = E.generate_eval_command(args(**base))
    assert rep["version"] == 1 and rep["objective"] == "summarization" and rep["scored_records"] == 4 and rep["oversized_records"] == 1
    assert rep["data"][0]["records_read"] == 5 and rep["max_new_tokens"] == 6 and rep["seed"] == 3 and rep["top_k"] is None
    assert set(rep["generation"]) == {"repeated_trigram_rate", "degenerate_fraction", "target_containment", "source_overlap", "empty_fraction",
                                      "stopped_at_eos", "mean_generated_tokens", "mean_generated_words"}
    assert 0 < rep["generation"]["mean_generated_tokens"] <= 6 and "samples" not in rep
    assert json.loads(out.read_text()) == rep
    dumped = json.loads(samples.read_text())
    assert len(dumped) == 4 and dumped[0]["prompt"].endswith("Summary:\n") and "alpha beta gamma delta 0" in dumped[0]["prompt"]
    assert E.generate_eval_command(args(**base)) == rep                                   # greedy and seeded: reproducible
    two = E.generate_eval_command(args(**dict(base, max_records=2, samples=None, output=None)))
    assert two["scored_records"] == 2
    with pytest.raises(T.TaskError, match="different files"):
        E.generate_eval_command(args(**dict(base, samples=str(out))))
    with pytest.raises(T.TaskError, match="not a supervised-generation objective"):
        E.generate_eval_command(args(**dict(base, objective="causal_lm")))


def test_retrieval_pool_report_dedups_by_id_and_describes_the_rank_tail(fixture):
    from summa_b200.train import eval as E
    tmp, args = fixture
    d = E.rank_distribution([1, 1, 2, 3, 5, 8, 13, 21, 150, 300])
    assert d == {"mean": 50.4, "median": 5, "p90": 150, "p99": 300, "worst": 300, "beyond_100": 2}
    with pytest.raises(T.TaskError):
        E.rank_distribution([])
    q, dist = tmp / "q.jsonl", tmp / "dist.jsonl"
    rows = [{"query": f"q{i}", "positive": f"doc text {i}", "document_id": f"d{i}", "negatives": [f"doc text {(i + 1) % 6}"],
             "negative_document_ids": [f"d{(i + 1) % 6}"]} for i in range(6)]
    q.write_text("\n".join(json.dumps(r) for r in rows))
    dist.write_text("\n".join(json.dumps({"query": "unused", "positive": f"other {i}", "document_id": f"x{i}"}) for i in range(4)) + "\n"
                    + json.dumps({"query": "unused", "positive": "doc text 0", "document_id": "d0"}))
    out = tmp / "pool.json"
    base = dict(data=[str(q)], distractors=[str(dist)], sequence_length=64, batch_size=4, recall_k=3, retrieval_layer=None, output=str(out))
    rep = E.retrieval_pool_command(args(**base))
    assert rep["version"] == 3 and rep["objective"] == "retrieval_representation" and rep["retrieval_layer"] is None
    assert rep["pool"] == {"documents": 10, "queries": 6, "from_distractors": 4}                  # d0 of the distractor shard was already pooled
    assert [s["documents_added"] for s in rep["data"]] == [6, 4] and [s["queries"] for s in rep["data"]] == [6, 0]
    assert rep["embedded_sequences"] == 16 and rep["compute_tokens"] == 16 * 64
    r = rep["retrieval"]
    assert r["k"] == 3 and 1 <= r["ranks"]["median"] <= r["ranks"]["worst"] <= 10 and r["ranks"]["beyond_100"] == 0
    assert 0 <= r["top1_accuracy"] <= r["recall_at_k"] <= 1 and r["mrr"] <= 1 and r["ndcg_at_10"] <= 1
    assert json.loads(out.read_text()) == rep and E.retrieval_pool_command(args(**base)) == rep
    small = E.retrieval_pool_command(args(**dict(base, distractors=None, batch_size=8, output=None)))
    assert any("no harder than the in-batch" in w for w in small["warnings"])
    bad = tmp / "bad.jsonl"
    bad.write_text(json.dumps({"query": "q", "positive": "changed text", "document_id": "d0"}))
    with pytest.raises(T.TaskError, match="maps to different model-visible text"):
        E.retrieval_pool_command(args(**dict(base, distractors=[str(bad)], output=None)))
    noid = tmp / "noid.jsonl"
    noid.write_text(json.dumps({"query": "q", "positive": "p"}))
    with pytest.raises(T.TaskError, match="no string `document_id`"):
        E.retrieval_pool_command(args(**dict(base, data=[str(noid)], distractors=None, output=None)))
    miss = tmp / "miss.jsonl"
    miss.write_text(json.dumps({"query": "q", "positive": "p", "document_id": "a", "negatives": ["n"]}))
    with pytest.raises(T.TaskError, match="1 negative document\\(s\\) but 0 negative id"):
        E.retrieval_pool_command(args(**dict(base, data=[str(miss)], distractors=None, output=None)))
