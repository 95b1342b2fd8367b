"""Corpus pipeline: resumable build, dedup, authenticated reads, pagination guard, composition."""
import json
import os

import pytest

from summa_b200.train import corpus as C


class ByteTok:
    def encode(self, text):
        return list(text.encode())


def _setup(n=23):
    recs = {f"k{i}": f"document number {i % 17}\r\nline two \x07 bell   " for i in range(n)}   # some duplicates
    recs["k3"] = ""
    q = {"q1": [f"k{i}" for i in range(0, n, 2)], "q2": [f"k{i}" for i in range(1, n, 2)] + ["missing"]}
    cfg = C.CorpusConfig("demo", ["q1", "q2"], page_size=4, docs_per_shard=5)
    return cfg, C.ListSearchBackend(q), C.DictMaterializer(recs)


def test_pipeline_resume_and_authenticated_open(tmp_path):
    cfg, search, mat = _setup()
    pipe = C.CorpusPipeline(cfg, search, mat, ByteTok(), C.SqliteDeduplicator,
                            classify=lambda k, t: {"parity": "even" if int(k[1:]) % 2 == 0 else "odd"})
    root = str(tmp_path)
    assert pipe.run(root, max_pages=2) is None                     # interrupted
    assert any(n.endswith(".building") for n in os.listdir(root))
    out = pipe.run(root)                                            # resumed
    assert out is not None and not any(n.endswith(".building") for n in os.listdir(root))
    assert pipe.run(root) == out                                    # idempotent
    manifest, docs = C.open_corpus(out)
    st = manifest["stats"]
    assert st["discovered"] == 24 and st["materialised"] == 23 and st["too_short"] == 1
    assert st["kept"] == 17 and st["duplicates"] == 5               # 17 distinct texts among the 22 non-empty records
    got = list(docs())
    assert len(got) == 17 and bytes(got[0]).decode() == "document number 0\nline two  bell"
    assert sum(s["documents"] for s in manifest["shards"]) == 17 and len(manifest["shards"]) == 4
    # a one-shot build of the same inputs is byte-identical
    root2 = str(tmp_path / "again")
    os.makedirs(root2)
    out2 = C.CorpusPipeline(cfg, search, mat, ByteTok(), C.SqliteDeduplicator,
                            classify=lambda k, t: {"parity": "even" if int(k[1:]) % 2 == 0 else "odd"}).run(root2)
    assert open(os.path.join(out, "manifest.json"), "rb").read() == open(os.path.join(out2, "manifest.json"), "rb").read()
    # tampering is caught on read
    shard = os.path.join(out, manifest["shards"][1]["file"])
    b = bytearray(open(shard, "rb").read()); b[-1] ^= 1
    open(shard, "wb").write(bytes(b))
    with pytest.raises(C.CorpusError):
        list(C.open_corpus(out)[1]())


def test_pagination_guard_and_inmemory_dedup(tmp_path):
    class Bad(C.ListSearchBackend):
        def discover(self, q, off, lim):
            keys, total = super().discover(q, off, lim)
            return keys, total - 3                                  # total shrinks under the cursor
    cfg, search, mat = _setup()
    with pytest.raises(C.CorpusError):
        C.CorpusPipeline(cfg, Bad(search.queries), mat, ByteTok(), lambda p: C.InMemoryDeduplicator()).run(str(tmp_path))


def test_compose_stage_interleaves_by_weight():
    recs = [({"topic": "math" if i % 3 == 0 else "code"}, [i] * 10) for i in range(30)]
    strata = [C.Stratum("math", 1.0, lambda l: l["topic"] == "math"), C.Stratum("code", 3.0, lambda l: True)]
    out = C.compose_stage(recs, strata, token_budget=200)
    names = [n for n, _ in out]
    assert len(out) == 20 and names.count("math") == 5 and names.count("code") == 15
    assert out == C.compose_stage(recs, strata, token_budget=200)              # deterministic
    assert names[:4].count("math") >= 1                                        # interleaved, not concatenated
    with pytest.raises(C.CorpusError):
        C.compose_stage(recs, [C.Stratum("x", 0.0, lambda l: True)], 10)
