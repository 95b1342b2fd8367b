"""HQUANT codecs, fake-quant, the quantisation plan and the QAT phase of the trainer (CPU)."""
import json
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("fmt", ["binary_g128", "ternary_g128", "ternary_entropy_g128"])
@pytest.mark.parametrize("shape", [(256, 64), (7, 19), (3, 128)])
def test_codec_roundtrip_and_fake_quant_agree(fmt, shape):
    from summa_b200.train import quantization as Q
    torch.manual_seed(0)
    w = torch.randn(*shape) * 0.1
    pt = Q.quantize_tensor(w, fmt)
    back = Q.PackedTensor.from_bytes(pt.to_bytes())
    dec = back.decode()
    assert dec.shape == w.shape
    n = w.numel()
    groups = -(-n // 128)
    assert back.scales.size == groups
    # the decoded tensor takes at most 2 (binary) / 3 (ternary) values per group
    flat = torch.zeros(groups * 128)
    flat[:n] = dec.reshape(-1)
    for g in range(groups):
        vals = flat[g * 128:min((g + 1) * 128, n)].unique()
        assert vals.numel() <= (2 if fmt == "binary_g128" else 3)
    # fake-quant is the same estimator with the scale kept in fp32 (codec scales are fp16)
    fq = Q.fake_quantize(w, fmt)
    if fmt == "binary_g128":
        torch.testing.assert_close(fq, dec, rtol=2e-3, atol=1e-5)
    else:
        # a near-tie between two prefixes may resolve differently in fp32 and fp64: same error, other support
        close = torch.isclose(fq, dec, rtol=2e-3, atol=1e-5)
        assert close.float().mean() > 0.98
        e_fq, e_dec = (fq - w).pow(2).sum(), (dec - w).pow(2).sum()
        assert abs(e_fq - e_dec) < 2e-3 * e_dec
    if fmt == "binary_g128":
        ref_scale = w.reshape(-1)[:min(128, n)].abs().mean()
        assert abs(dec.reshape(-1)[0].abs() - ref_scale) < 1e-3 * ref_scale + 1e-6
    else:
        # the optimal ternary code never has a larger error than sign * mean|w|
        b = Q.quantize_tensor(w, "binary_g128").decode()
        assert (dec - w).pow(2).sum() <= (b - w).pow(2).sum() + 1e-6
    bits = {"binary_g128": 1.0, "ternary_g128": 2.0, "ternary_entropy_g128": 1.625}[fmt]
    assert back.codes.size * 8 == pytest.approx(groups * 128 * bits, rel=0.02)


def test_codec_detects_corruption():
    from summa_b200.train import quantization as Q
    data = bytearray(Q.quantize_tensor(torch.randn(128, 4), "ternary_g128").to_bytes())
    data[-12] ^= 0x40
    with pytest.raises(Q.QuantError):
        Q.PackedTensor.from_bytes(bytes(data))
    with pytest.raises(Q.QuantError):
        Q.quantize_tensor(torch.tensor([[float("nan")]]), "binary_g128")


def test_fake_quant_is_straight_through():
    from summa_b200.train import quantization as Q
    w = torch.randn(4, 128, requires_grad=True)
    q = Q.fake_quantize(w, "ternary_g128")
    (q * torch.arange(512.0).view(4, 128)).sum().backward()
    torch.testing.assert_close(w.grad, torch.arange(512.0).view(4, 128))
    assert q.detach().unique().numel() <= 3 * 4


def test_quantization_plan_format_at():
    from summa_b200.train.workflow import QuantizationConfig
    q = QuantizationConfig.from_json({"format": "binary_g128", "warmup_format": "ternary_g128", "start_step": 10,
                                      "end_step": 20, "training": {"type": "qat", "warmup_steps": 3}}, "p")
    assert [q.format_at(s) for s in (9, 10, 12, 13, 19, 20)] == [None, "ternary_g128", "ternary_g128", "binary_g128",
                                                                   "binary_g128", None]
    q2 = QuantizationConfig.from_json({"format": "ternary_g128", "training": {"type": "qat", "warmup_steps": 2}}, "p")
    assert [q2.format_at(s) for s in (0, 1, 2)] == [None, None, "ternary_g128"]


def test_engine_quantized_window_restores_masters():
    from summa_b200 import mal
    from summa_b200.models import Transformer
    from summa_b200.train import quantization as Q
    from summa_b200.train.engine import FlatTrainEngine, OptimConfig
    cfg = mal.get_builtin_model("bench_tiny")
    torch.manual_seed(1)
    model = Transformer(cfg, init_std=0.05)
    eng = FlatTrainEngine(model, OptimConfig(lr=1e-2), param_dtype=torch.float32)
    names = Q.qat_parameter_names(model)
    before = {n: p.detach().clone() for n, p in model.named_parameters()}
    master0 = eng.master.clone()
    assert eng.begin_quantized_window("ternary_g128", names) == len(names)
    params = dict(model.named_parameters())
    for n in names:
        torch.testing.assert_close(params[n].detach(), Q.fake_quant_values(before[n], "ternary_g128"))
    torch.testing.assert_close(eng.master, master0)          # masters never see the codes
    tok = torch.randint(0, cfg.vocab_size, (2, 17))
    eng.zero_grad()
    model.forward_loss(tok[:, :-1], tok[:, 1:]).backward()
    eng.end_quantized_window()
    eng.step()
    # after the step every compute copy is its (updated) full-precision master again
    moved = 0
    for n in names:
        p = params[n].detach()
        assert p.unique().numel() > 3 * (-(-p.numel() // 128)) or p.numel() < 8
        moved += int(not torch.equal(p, before[n]))
    assert moved > 0


def _cli(*argv):
    return subprocess.run([sys.executable, "-m", "summa_b200.cli.train", *argv], capture_output=True, text=True,
                          cwd=ROOT, timeout=600)


def test_qat_and_distillation_phases_in_the_trainer(tmp_path):
    from summa_b200.tokenizer import Tokenizer
    from summa_b200.train.metrics import read_metrics
    tok = tmp_path / "tokenizer.json"
    tok.write_text(Tokenizer.byte_level().to_json())
    data = tmp_path / "train.jsonl"
    rows = [{"text": ("the quick brown fox %d jumps over the lazy dog. " % i) * 4} for i in range(200)]
    data.write_text("\n".join(json.dumps(r) for r in rows))
    mal = tmp_path / "m.mal"
    mal.write_text("""attention a { num_heads: 2 } ffn f { hidden_dim: 64 }
      block b { attention: a ffn: f norm: rmsnorm { eps: 1e-5 } }
      model t { max_seq_len: 64 hidden_size: 32 num_layers: 2 block: b }""")
    base = {"task": {"type": "causal_lm"}, "data": "train.jsonl", "sequence_length": 32, "batch_size": 4,
            "gradient_accumulation": 2, "shuffle_buffer": 16}
    wf = tmp_path / "workflow.json"
    wf.write_text(json.dumps({"version": 2, "phases": [
        dict(base, name="p0", type="pretrain", steps=3),
        dict(base, name="q", type="quantization", steps=4,
             quantization={"format": "ternary_g128", "start_step": 3,
                           "training": {"type": "qat", "warmup_steps": 1}})]}))
    out = str(tmp_path / "run")
    r = _cli("train", "--model", str(mal), "--tokenizer", str(tok), "--workflow", str(wf), "--output", out,
             "--warmup", "1", "--lr", "3e-3", "--device", "cpu", "--optimizer", "adamw")
    assert r.returncode == 0, r.stderr[-3000:]
    recs = list(read_metrics(os.path.join(out, "metrics.jsonl")))
    q_all = lambda records: [x["event"]["values"] for x in records if x["event"]["type"] == "quantization"]
    q = [v for v in q_all(recs) if v["stage"] == "fake_quantization"]
    # the first optimizer step runs before `start_step`: no fake-quantised window, no record
    assert [v["stage"] for v in q] == ["fake_quantization"] * 3
    assert all(v["format"] == "ternary_g128" and v["tensors_quantized"] > 0 and v["weights_quantized"] > 0
               and v["group_size"] == 128 for v in q)
    losses = [x["event"]["values"]["loss"] for x in recs if x["event"]["type"] == "optimization"]
    assert len(losses) == 7 and all(l == l and l < 7 for l in losses)

    # the phase sealed its final weights and their archive as a candidate
    from summa_b200 import mal as mal_mod
    from summa_b200.models import Transformer
    from summa_b200.train import qat_candidate as QC
    cand = os.path.join(out, "quantized-candidates", "q.step-7")
    cfg = mal_mod.load_model_def(str(mal))
    cfg.vocab_size = 320
    pub = QC.open_candidate(cand, lambda: Transformer(cfg))
    assert pub.metrics["quantized_tensors"] > 0 and pub.metrics["packed_bytes"] < pub.metrics["archive_weight_bytes"]
    # ... reported it as an export record, and the sealed generation names it (`trainer_lifecycle.rs:563-690`)
    export = [v for v in q_all(recs) if v["stage"] == "export"]
    assert len(export) == 1 and export[0]["packed_bytes"] == pub.metrics["packed_bytes"] and export[0]["progress_fraction"] == 1.0
    gen0 = json.load(open(os.path.join(out, "current.json")))["generation"]
    st = json.load(open(os.path.join(out, "generations", gen0, "training-state.json")))
    assert st["quantization"]["manifest"] == pub.candidate_manifest_path and st["quantization"]["candidate_weights_sha256"] == pub.weights_sha256
    assert {"kind": "hquant_candidate", "manifest": pub.candidate_manifest_path, "hash": pub.candidate_manifest_sha256} in st["artifacts"]
    # a completed run resumes idempotently: the candidate is authenticated, not rewritten
    sealed = open(pub.candidate_manifest_path, "rb").read()
    train_cmd = ["train", "--model", str(mal), "--tokenizer", str(tok), "--workflow", str(wf), "--output", out,
                 "--warmup", "1", "--lr", "3e-3", "--device", "cpu", "--optimizer", "adamw"]
    again = _cli(*train_cmd, "--resume")
    assert again.returncode == 0, again.stderr[-3000:]
    assert open(pub.candidate_manifest_path, "rb").read() == sealed and json.load(open(os.path.join(out, "current.json")))["generation"] == gen0

    # export the trained weights as an archive and read one tensor back
    gen = json.load(open(os.path.join(out, "current.json")))["generation"]
    ckpt = os.path.join(out, "generations", gen, "weights.safetensors")
    arch = str(tmp_path / "arch")
    e = _cli("quantize", "--model", str(mal), "--tokenizer", str(tok), "--checkpoint", ckpt, "--format", "ternary_g128",
             "--output", arch)
    assert e.returncode == 0, e.stderr[-3000:]
    man = json.load(open(os.path.join(arch, "archive-manifest.json")))
    assert man["quantized_tensors"] > 0 and 2.0 <= man["bits_per_quantized_weight"] < 3.5
    # the reference's spellings: -o, boolean switches for the embedding and the head, the recorded training recipe
    e2 = _cli("quantize", "--model", str(mal), "--tokenizer", str(tok), "--checkpoint", ckpt, "--format", "ternary-g128", "-o", str(tmp_path / "arch2"),
              "--quantize-embeddings", "false", "--quantize-lm-head", "false", "--ternary-warmup-steps", "3", "--distillation-weight", "0.5")
    assert e2.returncode == 0, e2.stderr[-3000:]
    man2 = json.loads(e2.stdout.strip().splitlines()[-1])
    assert 0 < man2["quantized_tensors"] < man["quantized_tensors"] and man2["training_recipe"] == {"ternary_warmup_steps": 3, "distillation_weight": 0.5}
    # an ordinary checkpoint becomes the memory topology only if it fits the source model it names
    memory = tmp_path / "memory.mal"
    memory.write_text("""attention a { num_heads: 2 } ffn f { hidden_dim: 64 }
      memory mm { tier fast { ffn: f reserve_experts { capacity: 2 rank: 4 top_k: 1 } } }
      block b { attention: a memory: mm norm: rmsnorm { eps: 1e-5 } }
      model t { vocab_size: 320 max_seq_len: 64 hidden_size: 32 num_layers: 2 block: b }""")
    ordinary = tmp_path / "ordinary.mal"
    ordinary.write_text(mal.read_text().replace("model t {", "model t { vocab_size: 320"))
    up = _cli("upgrade-memory-checkpoint", "--source-config", str(ordinary), "--target-config", str(memory), "--checkpoint", ckpt, "-o", str(tmp_path / "up.safetensors"))
    assert up.returncode == 0 and os.path.getsize(tmp_path / "up.safetensors") > 0, up.stderr[-3000:]
    wrong = tmp_path / "wrong.mal"
    wrong.write_text(ordinary.read_text().replace("hidden_dim: 64", "hidden_dim: 96"))
    bad = _cli("upgrade-memory-checkpoint", "--source-config", str(wrong), "--target-config", str(memory), "--checkpoint", ckpt, "-o", str(tmp_path / "bad.safetensors"))
    assert bad.returncode != 0 and not os.path.exists(tmp_path / "bad.safetensors")

    # quantisation by distillation from the full-precision checkpoint
    import hashlib
    sha = hashlib.sha256(open(ckpt, "rb").read()).hexdigest()
    wf2 = tmp_path / "workflow2.json"
    wf2.write_text(json.dumps({"version": 2, "phases": [
        dict(base, name="qd", type="quantization", steps=2,
             quantization={"format": "binary_g128",
                           "training": {"type": "distillation", "teacher_checkpoint": ckpt, "teacher_sha256": sha,
                                        "temperature": 2.0, "loss_weight": 0.5}})]}))
    out2 = str(tmp_path / "run2")
    r2 = _cli("train", "--model", str(mal), "--tokenizer", str(tok), "--workflow", str(wf2), "--output", out2,
              "--checkpoint", ckpt, "--warmup", "1", "--lr", "1e-3", "--device", "cpu", "--optimizer", "adamw")
    assert r2.returncode == 0, r2.stderr[-3000:]
    recs2 = list(read_metrics(os.path.join(out2, "metrics.jsonl")))
    opt = [x["event"]["values"] for x in recs2 if x["event"]["type"] == "optimization"]
    assert len(opt) == 2 and all(v["optimized_loss"] >= v["loss"] for v in opt)

    # a candidate that changed under a sealed checkpoint stops the resume
    with open(pub.weights_path, "r+b") as f:
        f.seek(200)
        f.write(b"\x7f\x7f")
    broken = _cli(*train_cmd, "--resume")
    assert broken.returncode != 0 and "candidate" in broken.stderr.lower()


@pytest.mark.parametrize("fmt", ["binary_g128", "ternary_g128", "ternary_entropy_g128", "int4_g128"])
def test_archive_loads_into_kernel_layers(tmp_path, fmt):
    """export_archive -> load_archive: the swapped-in quantised layers give the logits of a model
    whose dense weights are the decoded tensors; a flipped byte is refused."""
    from summa_b200 import mal
    from summa_b200.models import Transformer
    from summa_b200.models.quantized import HQuantLinear, QuantLinear, load_archive
    from summa_b200.train import quantization as Q
    cfg = mal.parse_mal("""attention a { num_heads: 2 } ffn f { hidden_dim: 256 }
      block b { attention: a ffn: f norm: rmsnorm { eps: 1e-5 } }
      model t { vocab_size: 300 max_seq_len: 64 hidden_size: 128 num_layers: 2 block: b }""")
    torch.manual_seed(0)
    src = Transformer(cfg, init_std=0.05)
    man = Q.export_archive(src, fmt, str(tmp_path / "a"))
    assert man["quantized_tensors"] > 0
    dst = Transformer(cfg, init_std=0.05)
    info = load_archive(dst, str(tmp_path / "a"))
    kinds = {type(m) for m in dst.modules()}
    if fmt == "int4_g128":
        assert QuantLinear in kinds and info["kernel_layers"] > 0
    elif fmt != "ternary_entropy_g128":
        assert HQuantLinear in kinds and info["kernel_layers"] > 0
    else:
        assert info["kernel_layers"] == 0 and info["decoded_tensors"] == man["quantized_tensors"]
    # oracle: the same model with every quantised tensor decoded into a dense weight
    ref = Transformer(cfg, init_std=0.05)
    packed = Q.quantize_model(src, fmt)
    with torch.no_grad():
        for n, p in ref.named_parameters():
            p.copy_(packed[n].decode() if n in packed else dict(src.named_parameters())[n])
    tok = torch.randint(0, 300, (2, 16))
    with torch.no_grad():
        torch.testing.assert_close(dst.eval()(tok), ref.eval()(tok), rtol=2e-3, atol=2e-3)
    victim = os.path.join(str(tmp_path / "a"), man["files"][0]["path"])
    blob = bytearray(open(victim, "rb").read())
    blob[len(blob) // 2] ^= 1
    open(victim, "wb").write(bytes(blob))
    with pytest.raises(Q.QuantError):
        load_archive(Transformer(cfg), str(tmp_path / "a"))


def test_qat_phase_that_never_reaches_its_target_format_is_refused(tmp_path):
    """`summa-train/tests/trainer_lifecycle.rs:513-560`: a warm-up as long as the phase leaves no step in the target codec."""
    from summa_b200.tokenizer import Tokenizer
    from summa_b200.train.workflow import QuantizationConfig, WorkflowError
    q = QuantizationConfig.from_json({"format": "binary_g128", "start_step": 4, "end_step": 9, "training": {"type": "qat", "warmup_steps": 2}}, "p")
    q.validate_phase_window(0, 7)                                                    # steps 6 of [0, 7) is trained in the target codec
    for start, steps in [(0, 6), (9, 4), (0, 0)]:
        with pytest.raises(WorkflowError):
            q.validate_phase_window(start, steps)
    tok = tmp_path / "tokenizer.json"
    tok.write_text(Tokenizer.byte_level().to_json())
    (tmp_path / "train.jsonl").write_text("\n".join(json.dumps({"text": "the quick brown fox " * 8}) for _ in range(20)))
    mal = tmp_path / "m.mal"
    mal.write_text("""attention a { num_heads: 2 } ffn f { hidden_dim: 64 }
      block b { attention: a ffn: f norm: rmsnorm { eps: 1e-5 } }
      model t { max_seq_len: 64 hidden_size: 32 num_layers: 2 block: b }""")
    wf = tmp_path / "inactive-qat.json"
    wf.write_text(json.dumps({"version": 2, "phases": [{
        "name": "inactive-binary-qat", "type": "quantization", "task": {"type": "causal_lm"}, "data": "train.jsonl", "sequence_length": 4,
        "batch_size": 1, "gradient_accumulation": 1, "steps": 2,
        "quantization": {"format": "binary_g128", "group_size": 128, "start_step": 0,
                         "training": {"type": "qat", "warmup_steps": 2, "straight_through": True}}}]}))
    out = tmp_path / "inactive-output"
    r = _cli("train", "--model", str(mal), "--tokenizer", str(tok), "--workflow", str(wf), "--output", str(out), "--device", "cpu")
    assert r.returncode != 0 and "never trains its target format" in r.stderr and "contains no target-format" in r.stderr
    assert not out.exists()
