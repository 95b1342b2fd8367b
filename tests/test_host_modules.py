"""Tokenizer, data packing / shuffle, sealed checkpoints."""
import json
import os

import pytest
import torch

from summa_b200.tokenizer import Tokenizer, TokenizerError
from summa_b200.train import checkpoint as C
from summa_b200.train import data as D


def _bpe_json():
    t = Tokenizer.byte_level()
    vocab = dict(t.vocab)
    vocab["<eos>"] = 256
    merges = [("h", "e"), ("l", "l"), ("he", "ll"), ("Ġ", "w")]
    nid = 257
    for a, b in merges:
        vocab[a + b] = nid
        nid += 1
    cfg = json.loads(t.to_json())
    cfg["model"]["vocab"] = vocab
    cfg["model"]["merges"] = [f"{a} {b}" for a, b in merges]
    cfg["pre_tokenizer"]["use_regex"] = True
    return json.dumps(cfg).encode()


def test_byte_tokenizer_roundtrip_and_eos():
    t = Tokenizer.byte_level()
    assert t.vocab_size() == 257 and t.eos_id() == 256
    s = "héllo wörld\n<eos>"
    ids = t.encode(s)
    assert ids[-1] == 256 and t.decode(ids) == s
    t2 = Tokenizer.from_bytes(t.to_json().encode())
    assert t2.encode(s) == ids


def test_bpe_merges_and_hf_parity():
    data = _bpe_json()
    t = Tokenizer.from_bytes(data)
    ids = t.encode("hello world hell")
    assert t.decode(ids) == "hello world hell"
    assert t.token_to_id("hell") in ids
    try:
        from tokenizers import Tokenizer as HF
    except Exception:
        pytest.skip("HuggingFace tokenizers not installed")
    hf = HF.from_str(data.decode())
    for s in ["hello world", "hell  o\twell", "héllo", "", "a<eos>b"]:
        assert hf.encode(s, add_special_tokens=False).ids == t.encode(s)


def test_tokenizer_rejects_unsupported():
    cfg = json.loads(Tokenizer.byte_level().to_json())
    cfg["model"]["byte_fallback"] = True
    with pytest.raises(TokenizerError):
        Tokenizer.from_bytes(json.dumps(cfg).encode())
    cfg = json.loads(Tokenizer.byte_level().to_json())
    cfg["decoder"] = {"type": "WordPiece"}
    with pytest.raises(TokenizerError):
        Tokenizer.from_bytes(json.dumps(cfg).encode())


def test_packing_windows_and_shuffle(tmp_path):
    p = tmp_path / "d.jsonl"
    rows = [{"tokens": list(range(1, 8))}, {"tokens": list(range(10, 15))}, {"text": "ab"}]
    p.write_text("\n".join(json.dumps(r) for r in rows))
    tok = Tokenizer.byte_level()
    s = list(D.iter_samples(str(p), tok, 257, seq_len=4, eos_id=256))
    flat = list(range(1, 8)) + [256] + list(range(10, 15)) + [256] + [97, 98, 256]
    assert s == [flat[i:i + 5] for i in range(0, len(flat) - 4, 4)]
    a = list(D.iter_samples(str(p), tok, 257, 4, 256, shuffle=3, seed=5))
    b = list(D.iter_samples(str(p), tok, 257, 4, 256, shuffle=3, seed=5))
    assert a == b and sorted(a) == sorted(s)
    assert list(D.iter_samples(str(p), tok, 257, 4, 256, skip=2)) == s[2:]
    bad = tmp_path / "bad.jsonl"
    bad.write_text(json.dumps({"tokens": [999]}))
    with pytest.raises(D.DataError):
        list(D.iter_samples(str(bad), tok, 257, 4, 256))
    x, y = D.make_batch(s[:2])
    assert x.shape == (2, 4) and torch.equal(x[:, 1:], y[:, :-1])
    cache = tmp_path / "c.tokens"
    D.write_token_cache(str(cache), [[1, 2, 3], [], [7]])
    assert list(D.read_token_cache(str(cache))) == [[1, 2, 3], [], [7]]


def test_sealed_checkpoint_roundtrip_and_tamper_detection(tmp_path):
    from summa_b200 import mal
    from summa_b200.models import Transformer
    cfg = mal.get_builtin_model("nano"); cfg.vocab_size = 300
    torch.manual_seed(0)
    m = Transformer(cfg)
    st = C.TrainingState(global_step=7, phase_id="p0", tokens_seen=123, rng_streams=[C.RngStream("data", 1, 2)], workflow_signature="ab" * 32)
    opt = C.pack_tensors({"b": torch.ones(3), "a": torch.arange(4.0)}, {"step": 7.0}, {"k": "v"})
    out = str(tmp_path / "run")
    os.makedirs(out)
    name = C.save_training_checkpoint(out, m, st, adamw_state=opt)
    assert C.read_current(out) == name and name.startswith("sha256-")
    name2 = C.save_training_checkpoint(out, m, st, adamw_state=opt)
    assert name2 == name                                   # identical state -> identical generation
    m2 = Transformer(cfg)
    st2, adam, muon, n = C.load_training_state(out, m2)
    assert st2.global_step == 7 and st2.rng_streams[0].counter == 2 and n == name
    assert st2.workflow_signature == "ab" * 32 and st2.parameter_ids == C.parameter_ids_of(m) and st2.optimizer_states[0]["scope"] == "wake"
    tens, sc, meta = C.unpack_tensors(adam)
    assert torch.equal(tens["a"], torch.arange(4.0)) and sc["step"] == 7.0 and meta["k"] == "v"
    assert torch.equal(m.embedding.weight, m2.embedding.weight)

    def tamper(stage, d):
        if stage == "verified":
            with open(os.path.join(d, "weights.safetensors"), "r+b") as f:
                f.seek(100); f.write(b"\x00\x01\x02")
    with pytest.raises(C.CheckpointError):
        C.load_training_state(out, Transformer(cfg), stage_hook=tamper)
    with pytest.raises(C.CheckpointError):
        C.verify_generation(out, name)


def test_training_state_has_the_reference_container_shapes():
    """A state in the shapes of `summa-train/src/checkpoint.rs:216-307` (arrays, tagged memory mode, `sha256:` identities,
    no defaults) decodes; anything else fails with the field's name."""
    ref = {"version": 2, "global_step": 12, "phase": 1, "phase_id": "sft", "phase_kind": "sft", "epoch": 0, "records_in_phase": 40,
           "steps_in_phase": 2, "tokens_seen": 4096, "metric_records": 30, "workflow_signature": "sha256:" + "0f" * 32,
           "data_manifest_hash": None, "parameter_ids": [1, 2 ** 64 - 1], "memory_update": {"type": "periodic_sleep"}, "sleep": None,
           "optimizer_states": [{"scope": "wake", "adamw": "adamw-state.bpk", "muon": "muon-state.bpk", "gradient_accumulator": None, "update_clock": 12}],
           "artifacts": [{"kind": "quantization_candidate", "manifest": "m.json", "hash": "sha256:" + "00" * 32}], "evaluator_hashes": ["sha256:" + "11" * 32],
           "rng_streams": [{"name": "data", "seed": 7, "counter": 3}], "wake_context_buffer": [{"id": "sft:11:0", "optimizer_step": 11, "token_ids": [1, 2]}],
           "quantization": {"format": "ternary_g128", "fake_quant_active": True, "calibration_step": 5, "manifest": None,
                            "candidate_weights_sha256": None, "teacher_hash": None}}
    st = C.TrainingState.from_json(json.dumps(ref))
    assert st.workflow_signature == "0f" * 32 and st.parameter_ids[1] == 2 ** 64 - 1 and st.rng_streams[0].counter == 3
    assert json.loads(st.to_json()) == ref                                          # and is written back byte-compatibly
    for mutate, field in [(lambda d: d.pop("sleep"), "lacks"), (lambda d: d.update(parameter_ids={"a": "b"}), "parameter_ids"),
                          (lambda d: d.update(memory_update={"type": "wake_only"}), "memory_update"), (lambda d: d.update(extra=1), "unknown"),
                          (lambda d: d["artifacts"][0].pop("hash"), "artifacts"), (lambda d: d.update(workflow_signature="abc"), "workflow_signature"),
                          (lambda d: d["wake_context_buffer"][0].update(optimizer_step="1"), "wake_context_buffer"),
                          (lambda d: d.update(tokens_seen=0), "no token count"), (lambda d: d["quantization"].pop("teacher_hash"), "quantization")]:
        d = json.loads(json.dumps(ref))
        mutate(d)
        with pytest.raises(C.CheckpointError, match=field):
            C.TrainingState.from_json(json.dumps(d))


def test_device_sampler_fail_soft(tmp_path):
    import sys, time
    from summa_b200.train import device_sampler as ds
    s = ds.parse_line("0, 87, 1024, 40960, 245.75, 61, 1965")
    assert s.gpu_utilization == 87.0 and s.power_watts == 245.75 and s.sm_clock_mhz == 1965.0
    assert ds.parse_line("0, 5, 10, 100, [N/A], N/A, [N/A]").power_watts is None
    for bad in ("0, N/A, 1, 2, 3, 4, 5", "0, 120, 1, 2, 3, 4, 5", "0, 5, 10", "0, 5, 200, 100, 1, 1, 1"):
        with pytest.raises(ValueError):
            ds.parse_line(bad)
    with pytest.raises(ds.SamplerConfigError):
        ds.validate_selector("0; rm -rf /")
    with pytest.raises(ds.SamplerConfigError):
        ds.NvidiaSmiSampler(0.0)
    script = tmp_path / "fake_smi.py"
    script.write_text("import sys\nfor i in range(5):\n    print(f'0, {10*i}, 100, 1000, 50.0, 40, 1500', flush=True)\n"
                      "print('garbage', flush=True)\n")
    with ds.NvidiaSmiSampler(0.01, "0", capacity=3, command=[sys.executable, str(script)]) as smp:
        deadline = time.time() + 10
        got = ds.Drain()
        while time.time() < deadline and not any("stopped" in d for d in got.diagnostics):
            d = smp.drain()
            got.samples += d.samples
            got.diagnostics += d.diagnostics
            time.sleep(0.05)
    assert 1 <= len(got.samples) <= 5
    assert any("invalid" in d for d in got.diagnostics) and any("stopped" in d for d in got.diagnostics)
    # a missing binary is a diagnostic, not an exception
    with ds.NvidiaSmiSampler(1.0, "0", command=["/nonexistent/nvidia-smi-binary"]) as smp:
        assert any("stopped" in d for d in smp.drain().diagnostics)


def test_metrics_sidecar_and_relaunch_script(tmp_path):
    import json, os, subprocess, sys
    from summa_b200.train import metrics_sidecar as ms
    p = tmp_path / "metrics.jsonl"
    p.write_text(json.dumps({"event": "optimization", "global_step": 3, "loss": 2.5, "nested": {"lr": 0.1, "tag": "x"}}) + "\n"
                 + '{"event": "partial"')                      # no newline yet: must be left for the next pass
    assert ms.main(["--metrics", str(p), "--once"]) == 0
    rows = (tmp_path / "metrics.sidecar.tsv").read_text().strip().split("\n")
    assert len(rows) == 1 and rows[0].startswith("optimization\t3\t") and '"nested.lr": 0.1' in rows[0]
    script = os.path.join(os.path.dirname(ms.__file__), "..", "cli", "relaunch.sh")
    assert subprocess.run(["bash", "-n", script]).returncode == 0          # syntax check
    r = subprocess.run(["bash", script], capture_output=True, text=True)
    assert r.returncode == 2 and "--output is required" in r.stderr
