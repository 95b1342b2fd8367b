"""Post-training objectives: tensor losses against the float64 scalar oracles, analytic
gradients against autograd, verifier and the resumable executor."""
import json
import math

import pytest
import torch

from summa_b200.train import posttrain as pt


def test_dpo_scalar_tensor_and_gradients():
    torch.manual_seed(0)
    pc, pr, rc, rr = (torch.randn(5, dtype=torch.float64) for _ in range(4))
    pc.requires_grad_(); pr.requires_grad_()
    for beta, s in [(0.1, 0.0), (0.5, 0.2)]:
        loss = pt.dpo_loss_tensor(pc, pr, rc, rr, beta, s)
        oracle = [pt.dpo_loss(float(pc[i]), float(pr[i]), float(rc[i]), float(rr[i]), beta, s) for i in range(5)]
        assert abs(float(loss) - sum(o.loss for o in oracle) / 5) < 1e-12
        gc, gr = torch.autograd.grad(loss, (pc, pr))
        for i, o in enumerate(oracle):
            assert abs(float(gc[i]) * 5 - o.d_policy_chosen) < 1e-12
            assert abs(float(gr[i]) * 5 - o.d_policy_rejected) < 1e-12
            assert o.preference_correct == (o.policy_margin > o.reference_margin)
    with pytest.raises(pt.PostTrainError):
        pt.dpo_loss(0.0, 0.0, 0.0, 0.0, beta=0.0)
    with pytest.raises(pt.PostTrainError):
        pt.dpo_loss(0.0, 0.0, 0.0, 0.0, beta=0.1, label_smoothing=0.5)
    with pytest.raises(pt.PostTrainError):
        pt.dpo_loss(float("nan"), 0.0, 0.0, 0.0, beta=0.1)


def test_forward_kl_matches_oracle():
    torch.manual_seed(1)
    t, s = torch.randn(6, 11, dtype=torch.float64), torch.randn(6, 11, dtype=torch.float64)
    for temp, sq in [(1.0, False), (2.5, True)]:
        o = pt.forward_kl_distillation(t.tolist(), s.tolist(), temp, sq)
        v = pt.forward_kl_distillation_tensor(t, s, temp, sq)
        assert abs(float(v) - o.loss) < 1e-5
        assert o.mean_forward_kl >= 0 and 0 <= o.top1_agreement <= 1
    same = pt.forward_kl_distillation(t.tolist(), t.tolist())
    assert abs(same.loss) < 1e-12 and same.top1_agreement == 1.0


def test_grpo_tensor_matches_oracle_and_gradients():
    torch.manual_seed(2)
    G, T = 4, 7
    lens = [7, 3, 5, 1]
    mask = torch.zeros(G, T, dtype=torch.float64)
    for i, n in enumerate(lens):
        mask[i, :n] = 1
    cur = (torch.randn(G, T, dtype=torch.float64) * 0.3 - 1).requires_grad_()
    beh = cur.detach() + torch.randn(G, T, dtype=torch.float64) * 0.4
    ref = cur.detach() + torch.randn(G, T, dtype=torch.float64) * 0.2
    rewards = torch.tensor([1.0, 0.0, 0.5, 0.0], dtype=torch.float64)
    for kl in (0.0, 0.05):
        loss = pt.grpo_loss_tensor(rewards, cur, beh, ref if kl > 0 else None, mask, 0.2, 1e-6, kl)
        ro = [pt.GrpoRollout(float(rewards[i]), cur[i, :n].tolist(), beh[i, :n].tolist(),
                             ref[i, :n].tolist() if kl > 0 else None) for i, n in enumerate(lens)]
        o = pt.grpo_loss(ro, 0.2, 1e-6, kl)
        assert abs(float(loss) - o.loss) < 1e-6
        (g,) = torch.autograd.grad(loss, cur)
        for i, n in enumerate(lens):
            for j in range(n):
                assert abs(float(g[i, j]) - o.current_log_prob_gradients[i][j]) < 1e-6
            assert float(g[i, n:].abs().sum()) == 0.0
    with pytest.raises(pt.PostTrainError):
        pt.grpo_loss_tensor(rewards, cur, beh - 200.0, None, mask)          # log-ratio guard
    with pytest.raises(pt.PostTrainError):
        pt.grpo_loss_tensor(rewards, cur, beh, None, torch.zeros_like(mask))
    with pytest.raises(pt.PostTrainError):
        pt.grpo_loss([ro[0]], 0.2, 1e-6, 0.0)


def test_sequence_log_probs_and_verifier():
    torch.manual_seed(3)
    logits = torch.randn(2, 6, 13)
    tok = torch.randint(0, 13, (2, 6))
    mask = torch.tensor([[0, 0, 1, 1, 1, 0], [0, 1, 1, 0, 0, 0]])
    s = pt.sequence_log_probs(logits, tok, mask, "sum")
    lp = torch.log_softmax(logits.float(), -1)
    want0 = sum(float(lp[0, t - 1, tok[0, t]]) for t in (2, 3, 4))
    assert abs(float(s[0]) - want0) < 1e-5
    m = pt.sequence_log_probs(logits, tok, mask, "mean")
    assert abs(float(m[0]) - want0 / 3) < 1e-5
    v = pt.ExactAnswerVerifier()
    assert v.verify({}, " 42 \n", "42").passed
    assert not v.verify({"trim": False}, " 42", "42").passed
    assert v.verify({"case_fold": True}, "Paris", "paris").reward == 1.0
    with pytest.raises(pt.PostTrainError):
        v.verify({"fuzzy": True}, "a", "a")
    assert pt.reduce_sequence_log_probs([-1.0, -3.0], "mean") == -2.0


def test_executor_resumes_and_replays_identically(tmp_path):
    examples = [{"id": i, "text": f"ex{i}"} for i in range(10)]
    published = []

    def update(window, rng_pos):
        return {"loss": sum(e["id"] for e in window) / len(window), "n": len(window)}, 2 * len(window)

    state = str(tmp_path / "state.json")
    ex = pt.PostTrainingExecutor("phasehash", state, 4, published.append)
    assert ex.run(examples, update, max_updates=1) == 1
    assert published[0].data_end == 4 and published[0].rng_end == 8
    # simulate a crash after prepare, before commit: pending digest persisted, cursor not advanced
    ex2 = pt.PostTrainingExecutor("phasehash", state, 4, published.append)
    st = ex2.state
    nxt = pt.PreparedUpdate("phasehash", st["receipt_chain"], 1, 4, 8, 8, 16,
                            __import__("hashlib").sha256(json.dumps(examples[4:8], sort_keys=True, default=str).encode()).hexdigest(),
                            {"loss": 5.5, "n": 4.0})
    st["pending"] = nxt.digest()
    ex2._persist()
    ex3 = pt.PostTrainingExecutor("phasehash", state, 4, published.append)
    assert ex3.run(examples, update) == 2          # replays window 1 byte-identically, then the tail
    assert [p.step for p in published] == [0, 1, 2] and published[-1].data_end == 10
    assert ex3.complete_for(examples)
    # a retry that prepares different bytes is refused
    ex3.state.update({"data_pos": 0, "pending": "deadbeef"})
    with pytest.raises(pt.PostTrainError):
        ex3.run(examples, update)
    with pytest.raises(pt.PostTrainError):
        pt.PostTrainingExecutor("other", state, 4, published.append)
