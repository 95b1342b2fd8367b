"""The reference project's own example files are the fixtures: every WorkflowV2 example must load
unchanged (strict decoding, defaults, path resolution) and agree with the MAL preset it is written
for; the typed sub-configurations must re-serialise to what the file says."""
import glob
import json
import os

import pytest

# where the reference project is mounted (its `summa-train` directory); the tests skip when it is absent
REF = os.environ.get("SUMMA_REFERENCE_TREE", os.path.join(os.sep, "root", "reference", "summa-train"))
WORKFLOWS = sorted(glob.glob(os.path.join(REF, "workflow*.example.json")))

pytestmark = pytest.mark.skipif(not WORKFLOWS, reason="reference tree not mounted")


@pytest.mark.parametrize("path", WORKFLOWS, ids=[os.path.basename(p) for p in WORKFLOWS])
def test_reference_workflow_examples_load_unchanged(path):
    from summa_b200.train.workflow import load_workflow
    wf = load_workflow(path)
    raw = json.load(open(path))
    assert wf.version == 2 and wf.name == raw.get("name") and len(wf.phases) == len(raw["phases"])
    base = os.path.dirname(path)
    for ph, rp in zip(wf.phases, raw["phases"]):
        assert ph.name == rp["name"] and ph.kind == rp["type"]
        if rp.get("data"):
            assert ph.data == os.path.normpath(os.path.join(base, rp["data"]))
        out = ph.to_json()
        # every field the file states survives a decode / encode round trip (paths become absolute)
        for key in ("sequence_length", "batch_size", "gradient_accumulation", "steps", "max_steps", "epochs",
                    "shuffle_buffer", "loss_weight", "learning_rate_scale"):
            assert out.get(key) == rp.get(key), (ph.name, key)
        if rp.get("post_training"):
            got, want = out["post_training"], rp["post_training"]
            assert got["algorithm"] == want["algorithm"]
            for k, v in want.items():
                if k in ("reference", "teacher"):
                    assert got[k]["adapter"] == v["adapter"] and got[k]["sha256"] == v["sha256"]
                    assert got[k]["artifact"] == os.path.join(base, v["artifact"])
                else:
                    assert got[k] == v, (ph.name, k)
        for key in ("periodic_sleep", "sleep"):
            if rp.get(key):
                got, want = out[key], rp[key]
                assert got["schedule"] == want["schedule"]
                for k in ("knowledge_seeding", "imitation", "dreaming", "retention"):
                    assert got.get(k) == want.get(k), (ph.name, key, k)
                assert got["retention_suite"] == os.path.join(base, want["retention_suite"])
        if rp.get("memory_update_mode"):
            assert out["memory_update_mode"]["schedule"] == rp["memory_update_mode"]["schedule"]
    assert len(wf.signature()) == 64


def test_education_example_phase_kinds_and_algorithms():
    from summa_b200.train.workflow import load_workflow
    wf = load_workflow(os.path.join(REF, "workflow.education.example.json"))
    algos = {p.kind: p.post_training["algorithm"] for p in wf.phases if p.post_training}
    assert algos == {"distillation": "forward_kl", "preference": "dpo", "rl": "grpo"}
    rl = next(p for p in wf.phases if p.kind == "rl")
    assert rl.task.params["verifier"] == {"adapter": "exact_answer"}
    assert rl.post_training["sampling"] == {"max_new_tokens": 512, "temperature": 0.7, "top_p": 0.95}


def test_memory_workflows_match_the_sleep_preset():
    """`summa-train/src/workflow.rs:898-1057`: tier ids and reserve slots of a phase's schedule must equal the
    MAL memory tiers of every layer; the education and sleep examples are written for the 300M sleep preset."""
    from summa_b200 import mal
    from summa_b200.train.workflow import load_workflow, validate_against_model
    cfg = mal.get_builtin_model("retriever_300m_moe_sleep")
    for name in ("workflow.education.example.json", "workflow.sleep.example.json"):
        validate_against_model(load_workflow(os.path.join(REF, name)), cfg)
    plain = mal.get_builtin_model("retriever_300m_moe")
    with pytest.raises(Exception, match="memory"):
        validate_against_model(load_workflow(os.path.join(REF, "workflow.sleep.example.json")), plain)
