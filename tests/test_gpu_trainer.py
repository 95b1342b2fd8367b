"""The wake trainer on a GPU through the command line: bf16 flat engine with the native kernels,
a QAT phase (device fake-quant kernel) and a memory-model run under the wake-only tier policy."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

DENSE = """attention a { num_heads: 4 } ffn f { hidden_dim: 512 }
  block b { attention: a ffn: f norm: rmsnorm { eps: 1e-5 } }
  model t { max_seq_len: 256 hidden_size: 256 num_layers: 2 block: b }"""
MEMORY = """attention a { num_heads: 4 } ffn f { hidden_dim: 512 }
  memory mm {
    tier fast { ffn: f reserve_experts { capacity: 2 rank: 8 top_k: 1 } }
    tier slow { ffn: f residual_init: zero reserve_experts { capacity: 2 rank: 8 top_k: 1 } }
  }
  block b { attention: a memory: mm norm: rmsnorm { eps: 1e-5 } }
  model t { max_seq_len: 256 hidden_size: 256 num_layers: 2 block: b }"""


def _cli(*argv):
    return subprocess.run([sys.executable, "-m", "summa_b200.cli.train", *argv], capture_output=True, text=True,
                          cwd=ROOT, timeout=900)


def _fixture(tmp_path, mal_text):
    sys.path.insert(0, ROOT)
    from summa_b200.tokenizer import Tokenizer
    tok = tmp_path / "tokenizer.json"
    tok.write_text(Tokenizer.byte_level().to_json())
    data = tmp_path / "train.jsonl"
    rows = [{"text": ("the quick brown fox %d jumps over the lazy dog. " % i) * 12} for i in range(300)]
    data.write_text("\n".join(json.dumps(r) for r in rows))
    mal = tmp_path / "m.mal"
    mal.write_text(mal_text)
    return str(tok), str(mal)


def _losses(out):
    from summa_b200.train.metrics import read_metrics
    recs = list(read_metrics(os.path.join(out, "metrics.jsonl")))
    return recs, [r["event"]["values"]["loss"] for r in recs if r["event"]["type"] == "optimization"]


def test_gpu_trainer_pretrain_then_qat(tmp_path):
    tok, mal = _fixture(tmp_path, DENSE)
    base = {"task": {"type": "causal_lm"}, "data": "train.jsonl", "sequence_length": 128, "batch_size": 8,
            "gradient_accumulation": 2, "shuffle_buffer": 32}
    wf = tmp_path / "wf.json"
    wf.write_text(json.dumps({"version": 2, "phases": [
        dict(base, name="p0", type="pretrain", steps=6),
        dict(base, name="q", type="quantization", steps=4,
             quantization={"format": "ternary_g128", "start_step": 6, "training": {"type": "qat", "warmup_steps": 0}})]}))
    out = str(tmp_path / "run")
    r = _cli("train", "--model", mal, "--tokenizer", tok, "--workflow", str(wf), "--output", out, "--warmup", "2",
             "--lr", "3e-3", "--device", "cuda", "--optimizer", "muon")
    assert r.returncode == 0, r.stderr[-4000:]
    recs, losses = _losses(out)
    assert len(losses) == 10 and all(l == l for l in losses) and losses[5] < losses[0]
    q = [x["event"]["values"] for x in recs if x["event"]["type"] == "quantization"]
    fake = [v for v in q if v["stage"] == "fake_quantization"]
    assert len(fake) == 4 and all(v["tensors_quantized"] > 0 for v in fake)
    assert [v["stage"] for v in q if v["stage"] != "fake_quantization"] == ["export"] and q[-1]["packed_bytes"] > 0
    assert os.path.isdir(os.path.join(out, "quantized-candidates", "q.step-10"))


def test_gpu_trainer_memory_model_wake_only(tmp_path):
    tok, mal = _fixture(tmp_path, MEMORY)
    sched = {"clock": "optimizer_steps", "terminal_consolidation": "distill_into_base_v1",
             "tiers": [{"id": "fast", "update_period": 2, "reserve_slots": 2},
                       {"id": "slow", "update_period": 4, "reserve_slots": 2}]}
    wf = tmp_path / "wf.json"
    wf.write_text(json.dumps({"version": 2, "phases": [
        {"name": "p0", "type": "pretrain", "task": {"type": "causal_lm"}, "data": "train.jsonl", "sequence_length": 128,
         "batch_size": 8, "gradient_accumulation": 1, "steps": 8, "shuffle_buffer": 32,
         "memory_update_mode": {"type": "wake_only", "schedule": sched, "tier_optimizer": {"learning_rate": 3e-3, "beta_1": 0.9, "beta_2": 0.95, "epsilon": 1e-8,
                                                   "weight_decay": 0.0}}}]}))
    out = str(tmp_path / "run")
    r = _cli("train", "--model", mal, "--tokenizer", tok, "--workflow", str(wf), "--output", out, "--warmup", "2",
             "--lr", "3e-3", "--device", "cuda", "--optimizer", "adamw")
    assert r.returncode == 0, r.stderr[-4000:]
    recs, losses = _losses(out)
    assert len(losses) == 8 and all(l == l for l in losses) and losses[-1] < losses[0]
    ups = [x["event"]["values"] for x in recs if x["event"]["type"] == "tier_update"]
    assert [(u["tier_clock"], u["tier"]) for u in ups] == [(2, "fast"), (4, "fast"), (4, "slow"), (6, "fast"),
                                                            (8, "fast"), (8, "slow")]
    assert all(u["outcome"] == "committed" for u in ups)
