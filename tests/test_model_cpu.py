"""Model semantics on CPU: parameter counts, stateful == stateless, MoE oracle, weights I/O."""
import json
import os
import pytest
import torch

from summa_b200 import mal
from summa_b200.models import Transformer
from summa_b200.models import weights as W
from summa_b200.ops import reference


def _small(name, vocab=300, layers=None):
    cfg = mal.get_builtin_model(name)
    cfg.vocab_size = vocab
    if layers:
        cfg.num_layers = layers
    return cfg


@pytest.mark.parametrize("name", ["nano", "hybrid_tiny", "bench_tiny"])
def test_param_count_matches_estimator_and_stateful_equals_stateless(name):
    cfg = _small(name)
    torch.manual_seed(0)
    m = Transformer(cfg).eval()
    assert sum(p.numel() for p in m.parameters() if p.requires_grad) == cfg.estimated_params()
    tok = torch.randint(0, cfg.vocab_size, (2, 20))
    with torch.no_grad():
        full = m(tok)
        st = m.make_state(2, 32)
        parts = [m.forward_with_state(tok[:, :11], st)]
        for t in range(11, 20):
            parts.append(m.forward_with_state(tok[:, t:t + 1], st))
        nxt = m.forward_next_logits_with_state(tok[:, :1], m.make_state(2, 4))
    assert (torch.cat(parts, 1) - full).abs().max() < 1e-4
    assert nxt.shape == (2, cfg.vocab_size)


def test_padded_vocab_rows_are_zero_and_sliced():
    cfg = _small("nano", vocab=300)
    m = Transformer(cfg)
    assert m.embedding.weight.shape[0] == 320 and m.embedding.weight[300:].abs().sum() == 0
    assert m.lm_head.weight[:, 300:].abs().sum() == 0
    assert m(torch.zeros(1, 3, dtype=torch.long)).shape[-1] == 300


def test_moe_sorted_dispatch_matches_masked_dense_oracle():
    from summa_b200 import ops
    torch.manual_seed(0)
    T, H, I, E, k = 50, 32, 48, 6, 2
    x = torch.randn(T, H)
    logits = torch.randn(T, E)
    idx, gates = reference.moe_route(logits, k)
    wi, wd = torch.randn(E, H, 2 * I) * 0.1, torch.randn(E, I, H) * 0.1
    a = ops.moe_experts(x, idx, gates, wi, wd, None, None, "swiglu", True)
    b = reference.moe_experts_dense(x, idx, gates, wi, wd, None, None, "swiglu", True)
    torch.testing.assert_close(a, b, rtol=1e-4, atol=1e-5)
    order, inverse, counts = reference.route_plan(idx, E)
    assert counts.sum() == T * k and torch.equal(order[inverse], torch.arange(T * k))


def test_memory_model_trains_and_upgrade_preserves_logits():
    base = _small("retriever_300m_moe", layers=6)
    mem = _small("retriever_300m_moe_sleep", layers=6)
    torch.manual_seed(0)
    mb = Transformer(base).eval()
    mm = Transformer(mem).eval()
    assert sum(p.numel() for p in mm.parameters() if p.requires_grad) == mem.estimated_params()
    up = W.upgrade_safetensors_to_memory(W.serialize(W.model_tensors(mb)), mm)
    W.load_safetensors_bytes(mm, up)
    tok = torch.randint(0, 300, (1, 12))
    with torch.no_grad():
        assert (mb(tok) - mm(tok)).abs().max() < 1e-4
    mm.train()
    loss, aux = mm.forward_loss(tok[:, :-1], tok[:, 1:], with_router=True)
    (loss + aux).backward()
    # dormant reserve slots receive no gradient
    slot = mm.layers[0].memory.tiers[0].reserve.slots[0]
    assert slot.a.grad is None or slot.a.grad.abs().sum() == 0


def test_weights_canonical_strict_atomic(tmp_path):
    cfg = _small("nano")
    torch.manual_seed(0)
    m = Transformer(cfg)
    p = tmp_path / "w.safetensors"
    h1 = W.save_safetensors(m, str(p))
    b1 = p.read_bytes()
    h2 = W.save_safetensors(m, str(p))
    assert h1 == h2 and p.read_bytes() == b1
    m2 = Transformer(cfg)
    W.load_safetensors(m2, str(p))
    t = W.deserialize(b1)
    t.pop("final_norm.gamma")
    before = m2.embedding.weight.clone()
    with pytest.raises(W.WeightsError):
        W.load_safetensors_bytes(m2, W.serialize(t))
    t2 = W.deserialize(b1); t2["extra.weight"] = torch.zeros(1)
    with pytest.raises(W.WeightsError):
        W.load_safetensors_bytes(m2, W.serialize(t2))
    t3 = W.deserialize(b1); t3["final_norm.gamma"] = torch.zeros(3)
    with pytest.raises(W.WeightsError):
        W.load_safetensors_bytes(m2, W.serialize(t3))
    assert torch.equal(before, m2.embedding.weight)
    assert "_rope" not in "".join(t.keys())


def test_embeddings_are_l2_normalised():
    cfg = _small("nano")
    m = Transformer(cfg).eval()
    tok = torch.randint(0, 300, (3, 10))
    with torch.no_grad():
        e = m.forward_embeddings(tok, torch.tensor([9, 4, 0]), layer=1)
    torch.testing.assert_close(e.norm(dim=-1), torch.ones(3), rtol=1e-5, atol=1e-5)


def test_rope_is_interleaved_pairs():
    cos, sin = reference.rope_table(8, 4, 10000.0)
    x = torch.tensor([1.0, 0.0, 0.0, 1.0]).view(1, 1, 1, 4).repeat(1, 8, 1, 1)
    y = reference.apply_rope(x, cos, sin)
    # pair 0 = (1, 0) rotated by pos * 1.0 ; pair 1 = (0, 1) rotated by pos * 0.01
    torch.testing.assert_close(y[0, 3, 0, 0], torch.cos(torch.tensor(3.0)))
    torch.testing.assert_close(y[0, 3, 0, 1], torch.sin(torch.tensor(3.0)))
    torch.testing.assert_close(y[0, 3, 0, 2], -torch.sin(torch.tensor(0.03)))


def test_lab_server_serves_ui_and_a_trace_the_ui_accepts(tmp_path):
    """`/` serves the shipped browser UI, `/api/trace` returns a bundle that satisfies the rules
    of the UI's validator (`lab_ui/trace-utils.js::validateTrace`, restated here), and paths
    outside the UI directory are not served."""
    import json
    import threading
    import urllib.error
    import urllib.request
    from summa_b200 import mal
    from summa_b200.models import Transformer
    from summa_b200.models.lab import DEFAULT_UI, make_server
    from summa_b200.tokenizer import Tokenizer
    for f in ("model-lab.html", "main.js", "trace-utils.js", "demo-trace.js", "styles.css"):
        assert os.path.isfile(os.path.join(DEFAULT_UI, f))
    tok = Tokenizer.byte_level()
    cfg = mal.get_builtin_model("bench_tiny")
    cfg.vocab_size = tok.vocab_size()
    model = Transformer(cfg, init_std=0.05).eval()
    metrics = tmp_path / "metrics.jsonl"
    metrics.write_text(json.dumps({"schema_version": 2, "sequence": 0, "global_step": 1,
                                   "event": {"type": "optimization", "values": {"loss": 3.0}}}) + "\n")
    srv = make_server(model, tok, metrics_path=str(metrics))
    th = threading.Thread(target=srv.serve_forever, daemon=True)
    th.start()
    base = f"http://127.0.0.1:{srv.server_address[1]}"
    try:
        page = urllib.request.urlopen(base + "/").read().decode()
        assert "<title>summa_b200 model lab</title>" in page and "main.js" in page
        r = urllib.request.urlopen(base + "/trace-utils.js")
        assert r.headers["Content-Type"].startswith("text/javascript") and b"validateTrace" in r.read()
        for bad in ("/../models/lab.py", "/..%2fmodels%2flab.py", "/nope.js"):
            with pytest.raises(urllib.error.HTTPError):
                urllib.request.urlopen(base + bad)
        st = json.load(urllib.request.urlopen(base + "/api/status"))
        assert st["ready"] and st["max_trace_tokens"] == 128
        t = json.load(urllib.request.urlopen(base + "/api/trace?prompt=hello%20lab"))
    finally:
        srv.shutdown()
    # the bundle has the reference's shape and passes the viewer's rules
    from summa_b200.models.trace import validate_bundle
    validate_bundle(t)
    assert t["kind"] == "summa_model_trace" and t["version"] == 1
    assert t["model"]["num_layers"] == len(t["model"]["layers"]) and t["model"]["layers"][0]["index"] == 1
    inf = t["inference"]
    n = len(inf["tokens"])
    assert 0 < n <= 128 and inf["prompt"] == "hello lab" and inf["generated_token_count"] == n - inf["prompt_token_count"] > 0
    assert [x["source"] for x in inf["tokens"]] == ["prompt"] * inf["prompt_token_count"] + ["generated"] * inf["generated_token_count"]
    assert [s["stage"] for s in inf["stages"]] == ["embedding"] + ["block"] * t["model"]["num_layers"] + ["final_norm"]
    assert "token_delta_rms" not in inf["stages"][0] and len(inf["stages"][1]["token_delta_rms"]) == n
    for s in inf["stages"][1:-1]:
        att = s["attention"]
        assert att["captured_heads"] == len(att["heads"]) <= 4 <= att["total_heads"] or att["total_heads"] < 4
        for h in att["heads"]:
            assert h["rows"] == h["cols"] == n and h["value_kind"] == "probability"
            rows = [h["values"][i * n:(i + 1) * n] for i in range(n)]
            assert all(abs(sum(r) - 1.0) < 1e-3 for r in rows)
    assert t["training"]["rows"][0]["event"]["values"]["loss"] == 3.0 and t["capture"]["metrics_total_rows"] == 1
    assert t["capture"]["captured_tokens"] == n and t["capture"]["channels_reduced"] == (model.cfg.hidden_size > 64)


def test_trace_bundle_of_a_hybrid_model_has_mamba_state_and_truncation(tmp_path):
    """`summa-llm/src/trace.rs:272-440`: the LAST `token_limit` tokens are kept, Mamba stages carry the final
    recurrent state binned over channels, metrics rows are sub-sampled evenly with first and last kept."""
    from summa_b200.models import Transformer
    from summa_b200.models.trace import TraceOptions, capture_bundle, selected_rows, validate_bundle
    from summa_b200.tokenizer import Tokenizer
    tok = Tokenizer.byte_level()
    cfg = mal.get_builtin_model("hybrid_tiny")
    cfg.vocab_size = tok.vocab_size()
    torch.manual_seed(0)
    model = Transformer(cfg, init_std=0.05).eval()
    ids = tok.encode("a hybrid of state-space and attention blocks", False)
    metrics = tmp_path / "m.jsonl"
    metrics.write_text("".join(json.dumps({"sequence": i}) + "\n" for i in range(10)))
    b = validate_bundle(capture_bundle(model, tok, "a hybrid", 8, ids, None, str(metrics),
                                       TraceOptions(token_limit=16, channel_limit=8, attention_head_limit=2,
                                                    metrics_row_limit=4)))
    assert b["capture"]["tokens_truncated"] and b["capture"]["dropped_leading_tokens"] == len(ids) - 16
    assert b["inference"]["tokens"][0]["original_index"] == len(ids) - 16 and b["inference"]["token_offset"] == len(ids) - 16
    kinds = [l["mixer"]["kind"] for l in b["model"]["layers"]]
    assert "mamba" in kinds and "attention" in kinds
    for stage, kind in zip(b["inference"]["stages"][1:-1], kinds):
        assert stage["mixer"] == kind and stage["activation"]["cols"] == 8
        if kind == "mamba":
            ms = stage["mamba_state"]
            assert ms["rows"] == ms["original_rows"] and ms["cols"] == 8 and ms["row_labels"][0] == "state 0"
            assert "attention" not in stage
        else:
            assert stage["attention"]["captured_heads"] == 2 and "mamba_state" not in stage
    assert [r["sequence"] for r in b["training"]["rows"]] == selected_rows(10, 4) == [0, 3, 6, 9]
    assert b["training"]["dropped_rows"] == 6 and abs(b["training"]["sampling_stride"] - 3.0) < 1e-9


def test_reserve_routing_with_fixed_width_matches_a_per_token_reference():
    """The reserve evaluates every slot with dormant ones masked on the device; against a plain per-token rule
    (top-1 of the active slots' logits against a zero lane, gate = that slot's softmax weight), for no / one /
    several active slots, and gradients reach active slots only."""
    from summa_b200.models.memory import LowRankExpertReserve
    torch.manual_seed(0)
    res = LowRankExpertReserve(hidden=16, capacity=4, rank=3, top_k=1, seed=5)
    with torch.no_grad():
        for s in res.slots:
            s.b.normal_(0, 0.3)
            s.router.weight.normal_(0, 0.5)
    x = torch.randn(2, 7, 16)

    def reference(active):
        flat = x.reshape(-1, 16)
        out = torch.zeros_like(flat)
        for t in range(flat.shape[0]):
            if not active:
                continue
            logit = torch.stack([flat[t] @ res.slots[i].router.weight[:, 0] for i in active])
            best = int(logit.argmax())
            gate = torch.softmax(torch.cat([logit, torch.zeros(1)]), dim=0)[best]
            s = res.slots[active[best]]
            out[t] = gate * ((flat[t] @ s.a) @ s.b)
        return out.reshape(x.shape)

    assert torch.equal(res(x), torch.zeros_like(x))                       # all dormant: exactly nothing
    for wake in ([2], [0, 2], [0, 1, 2, 3]):
        for i in wake:
            if i not in res.active_slots():
                res.activate(i)
        assert res.active_slots() == wake
        torch.testing.assert_close(res(x), reference(wake), rtol=1e-5, atol=1e-6)
    res2 = LowRankExpertReserve(hidden=16, capacity=3, rank=3, top_k=1, seed=6)
    with torch.no_grad():
        for s in res2.slots:
            s.b.normal_(0, 0.3)
    res2.activate(1)
    res2(x).square().sum().backward()
    assert res2.slots[1].a.grad.abs().sum() > 0 and res2.slots[1].router.weight.grad.abs().sum() > 0
    for i in (0, 2):
        assert res2.slots[i].a.grad is None or float(res2.slots[i].a.grad.abs().sum()) == 0.0
        assert res2.slots[i].router.weight.grad is None or float(res2.slots[i].router.weight.grad.abs().sum()) == 0.0
