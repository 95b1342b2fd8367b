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
