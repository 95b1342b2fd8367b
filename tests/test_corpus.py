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


# ---------------------------------------------------------------------------------------- remote backends (fakes)
from summa_b200.train import corpus_backends as B


def _search_cfg(**over):
    cfg = {
        "endpoint": "https://search.example/api",
        "request_template": {
            "q": "", "page": {"offset": 0, "limit": 1}, "rev": "", "lang": None,
            "rerank": {"cross": True, "llm": True}, "return_documents": True,
            "fusion": {"kind": "rrf", "sparse": {"text": "", "field": "x"}, "dense": {"text": "", "field": "y"}},
        },
        "request_mapping": {"query_pointer": "/q", "offset_pointer": "/page/offset", "limit_pointer": "/page/limit",
                            "parameter_pointers": {"language": "/lang", "evil": "/fusion/dense"},
                            "disabled_reranker_pointers": ["/rerank/cross", "/rerank/llm"],
                            "return_documents_pointer": "/return_documents"},
        "response_mapping": {"hits_pointer": "/result/hits", "total_hits_pointer": "/result/total",
                             "record_key_pointer": "/id", "score_pointer": "/score", "uris_pointer": "/links",
                             "inline_text_pointer": "/body", "metadata_pointers": {"year": "/meta/year"}},
        "fusion": {"marker_pointer": "/fusion/kind", "marker_value": "rrf",
                   "sparse": {"clause_pointer": "/fusion/sparse", "vector_field_pointer": "/fusion/sparse/field", "vector_field": "bm25"},
                   "dense": {"clause_pointer": "/fusion/dense", "vector_field_pointer": "/fusion/dense/field", "vector_field": "emb_v3"}},
        "snapshot": {"provider": "idx", "revision": "r7", "request_revision_pointer": "/rev",
                     "response_provider_pointer": "/snapshot/provider", "response_revision_pointer": "/snapshot/revision"},
        "page_size": 4,
    }
    cfg.update(over)
    return cfg


class FakeTransport:
    def __init__(self, keys, revision="r7"):
        self.keys, self.revision, self.requests = keys, revision, []

    def post_json(self, endpoint, body):
        self.requests.append((endpoint, body))
        off, lim = body["page"]["offset"], body["page"]["limit"]
        hits = [{"id": k, "score": 1.0 / (1 + i), "links": f"doi:{k}", "body": f"text of {k}", "meta": {"year": 2000 + i}}
                for i, k in enumerate(self.keys)][off:off + lim]
        return {"snapshot": {"provider": "idx", "revision": self.revision}, "result": {"hits": hits, "total": len(self.keys)}}


def test_search_api_request_contract_and_paging():
    tr = FakeTransport([f"k{i}" for i in range(10)])
    api = B.SearchApiClient(_search_cfg(), tr)
    req = api.request_for("graph neural nets", 4, 3, {"language": "en"})
    assert req["q"] == "graph neural nets" and req["page"] == {"offset": 4, "limit": 3} and req["rev"] == "r7" and req["lang"] == "en"
    assert req["rerank"] == {"cross": False, "llm": False} and req["return_documents"] is False
    assert req["fusion"]["sparse"]["field"] == "bm25" and req["fusion"]["dense"]["field"] == "emb_v3"
    assert api.config["request_template"]["q"] == ""                               # the template is never mutated
    with pytest.raises(B.CorpusError, match="exceeds configured page_size"):
        api.request_for("q", 0, 5)
    with pytest.raises(B.CorpusError, match="unmapped"):
        api.request_for("q", 0, 1, {"nope": 1})
    with pytest.raises(B.CorpusError):                                             # a parameter must not knock out a fusion clause
        api.request_for("q", 0, 1, {"evil": None})
    page = api.discover_page("q", 8, 4)
    assert [h.record_key for h in page.hits] == ["k8", "k9"] and page.total_hits == 10
    assert page.hits[0].uris == ["doi:k8"] and page.hits[0].metadata == {"year": 2008} and page.hits[0].inline_text == "text of k8"
    assert api.discover("q", 0, 4) == (["k0", "k1", "k2", "k3"], 10)
    assert api.snapshot() == "idx@r7" and tr.requests[0][0] == "https://search.example/api"
    # the pipeline consumes it directly, materialising from a record store keyed the same way
    recs = {f"k{i}": f"body {i}" for i in range(10)}
    cfg = C.CorpusConfig("remote", ["q"], page_size=4, docs_per_shard=4)
    import tempfile
    with tempfile.TemporaryDirectory() as root:
        out = C.CorpusPipeline(cfg, api, C.DictMaterializer(recs), ByteTok(), C.SqliteDeduplicator).run(root)
        manifest, docs = C.open_corpus(out)
        assert manifest["stats"]["kept"] == 10 and manifest["source_snapshot"] == "idx@r7" and len(list(docs())) == 10


def test_search_api_rejects_bad_responses_and_configs():
    api = B.SearchApiClient(_search_cfg(), FakeTransport(["a"], revision="r8"))
    with pytest.raises(B.CorpusError, match="snapshot mismatch"):
        api.discover_page("q", 0, 1)
    api = B.SearchApiClient(_search_cfg(), FakeTransport(["a"]))
    ok = {"snapshot": {"provider": "idx", "revision": "r7"}, "result": {"hits": [{"id": 5, "score": 1}], "total": 1}}
    assert api.parse_response(ok).hits[0].record_key == "5"                        # scalar keys are stringified
    for mutate, pat in [
        (lambda r: r.pop("snapshot"), "snapshot proof"),
        (lambda r: r["result"].__setitem__("hits", {}), "not an array"),
        (lambda r: r["result"]["hits"][0].__setitem__("id", ""), "record key"),
        (lambda r: r["result"]["hits"][0].__setitem__("id", True), "record key"),
        (lambda r: r["result"]["hits"][0].__setitem__("score", float("nan")), "finite"),
        (lambda r: r["result"]["hits"][0].__setitem__("links", [1]), "uris"),
        (lambda r: r["result"]["hits"][0].__setitem__("body", 3), "inline text"),
        (lambda r: r["result"].__setitem__("total", -1), "total_hits"),
    ]:
        bad = json.loads(json.dumps(ok))
        mutate(bad)
        with pytest.raises(B.CorpusError, match=pat):
            api.parse_response(bad)
    cfg = _search_cfg()
    cfg["request_mapping"]["disabled_reranker_pointers"] = []
    with pytest.raises(B.CorpusError, match="reranker"):
        B.SearchApiClient(cfg, FakeTransport([]))
    cfg = _search_cfg()
    cfg["fusion"]["marker_value"] = "linear"
    with pytest.raises(B.CorpusError, match="fusion marker"):
        B.SearchApiClient(cfg, FakeTransport([]))
    cfg = _search_cfg()
    cfg["fusion"]["dense"]["vector_field_pointer"] = "/q"
    with pytest.raises(B.CorpusError, match="inside its fusion clause"):
        B.SearchApiClient(cfg, FakeTransport([]))
    with pytest.raises(B.CorpusError, match="unknown field"):
        B.SearchApiClient(_search_cfg(api_key="secret"), FakeTransport([]))


def test_search_api_http_transport_retries_bounds_and_secret(monkeypatch):
    import io
    import urllib.error
    cfg = B.validate_search_api_config(_search_cfg(auth={"header": "authorization", "environment": "SB_TEST_SEARCH_KEY", "prefix": "Bearer "},
                                                   max_retries=2, retry_initial_ms=10, retry_max_ms=15, max_response_bytes=64))
    with pytest.raises(B.CorpusError, match="not set"):
        B.UrllibSearchApiTransport(cfg)
    monkeypatch.setenv("SB_TEST_SEARCH_KEY", "s3cr3t")
    assert "s3cr3t" not in json.dumps(B.SearchApiClient(cfg, FakeTransport([])).configuration())

    class Resp(io.BytesIO):
        def __enter__(self):
            return self

        def __exit__(self, *a):
            return False

    calls, sleeps = [], []

    def opener(req, timeout):
        calls.append(req)
        if len(calls) < 3:
            raise urllib.error.HTTPError(req.full_url, 503, "busy", {}, None)
        return Resp(b'{"ok": 1}')

    tr = B.UrllibSearchApiTransport(cfg, opener=opener, sleep=sleeps.append)
    assert tr.post_json("https://search.example/api", {"a": 1}) == {"ok": 1}
    assert len(calls) == 3 and sleeps == [0.01, 0.015] and calls[0].get_header("Authorization") == "Bearer s3cr3t"
    tr = B.UrllibSearchApiTransport(cfg, opener=lambda req, timeout: Resp(b"x" * 100), sleep=sleeps.append)
    with pytest.raises(B.CorpusError, match="exceeds 64 bytes"):
        tr.post_json("https://search.example/api", {})

    def always_404(req, timeout):
        calls.append(req)
        raise urllib.error.HTTPError(req.full_url, 404, "nope", {}, None)

    calls.clear()
    with pytest.raises(B.CorpusError, match="HTTP 404"):
        B.UrllibSearchApiTransport(cfg, opener=always_404, sleep=sleeps.append).post_json("https://search.example/api", {})
    assert len(calls) == 1                                                         # client errors are not retried


class FakeExecutor:
    def __init__(self, rows):
        self.rows, self.calls = rows, []

    def snapshot_revision(self):
        return "lsn:42"

    def fetch(self, statement, columns, keys):
        self.calls.append((statement, dict(columns), list(keys)))
        return [dict(r) for r in self.rows]


def _pg_cfg(**over):
    cfg = {"connection_environment": "SB_TEST_PG_DSN", "statement": "select id, body from docs where id = any($1)",
           "columns": {"record_key": "id", "text": "body", "uris": "links", "metadata": "meta"},
           "snapshot_statement": "select pg_current_snapshot()", "transport_security": {"mode": "verify_full"}}
    cfg.update(over)
    return cfg


def test_postgres_materializer_contract():
    hits = [B.DiscoveryHit("a", 1.0, ["u:a"], {"year": 1999, "src": "hit"}), B.DiscoveryHit("b", 0.5, ["u:b"], {})]
    ex = FakeExecutor([{"record_key": "a", "text": "alpha", "uris": [], "metadata": {"src": "row"}},
                       {"record_key": "b", "text": "beta", "uris": ["pg:b"], "metadata": {}}])
    mat = B.PostgresRecordMaterializer(_pg_cfg(), ex)
    recs = mat.materialize(hits)
    assert [(r.record_key, r.text) for r in recs] == [("a", "alpha"), ("b", "beta")]
    assert recs[0].uris == ["u:a"] and recs[1].uris == ["pg:b"]                    # row uris win, hit uris are the fallback
    assert recs[0].metadata == {"year": 1999, "src": "row"}                        # row metadata overrides hit metadata
    assert ex.calls[0][2] == ["a", "b"] and mat.source_snapshot().revision == "lsn:42"
    assert mat.fetch(["a", "b"]) == {"a": "alpha", "b": "beta"}
    with pytest.raises(B.CorpusError, match="unrequested"):
        B.PostgresRecordMaterializer(_pg_cfg(), FakeExecutor([{"record_key": "z", "text": "?"}])).materialize(hits)
    dup = [{"record_key": "a", "text": "1"}, {"record_key": "a", "text": "2"}]
    with pytest.raises(B.CorpusError, match="duplicate"):
        B.PostgresRecordMaterializer(_pg_cfg(), FakeExecutor(dup)).materialize(hits)
    only_a = [{"record_key": "a", "text": "alpha"}]
    with pytest.raises(B.CorpusError, match="1 of 2"):
        B.PostgresRecordMaterializer(_pg_cfg(), FakeExecutor(only_a)).materialize(hits)
    assert len(B.PostgresRecordMaterializer(_pg_cfg(require_every_record=False), FakeExecutor(only_a)).materialize(hits)) == 1
    with pytest.raises(B.CorpusError, match="unknown field"):
        B.PostgresRecordMaterializer(_pg_cfg(password="x"), ex)
    with pytest.raises(B.CorpusError, match="must not be empty"):
        B.PostgresRecordMaterializer(_pg_cfg(columns={"record_key": "id", "text": " "}), ex)
    inline = B.InlineRecordMaterializer()
    assert inline.materialize([B.DiscoveryHit("k", inline_text="t")])[0].text == "t"
    with pytest.raises(B.CorpusError, match="no inline text"):
        inline.materialize([B.DiscoveryHit("k")])
