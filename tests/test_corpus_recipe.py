"""Version-2 corpus recipe and curriculum composition: configuration decoding, record steps, the resumable build
over fake discovery / materialisation backends, manifest sealing, the training data path over a corpus manifest,
and stratified stage composition."""
import copy
import hashlib
import json
import os

import pytest

from summa_b200.train import corpus_backends as B
from summa_b200.train import corpus_recipe as R
from summa_b200.train.corpus import CorpusError

REF = os.environ.get("SUMMA_REFERENCE_TREE", os.path.join(os.sep, "root", "reference", "summa-train"))


class ByteTok:
    def encode(self, text, *a):
        return list(text.encode())

    def vocab_size(self):
        return 256


class FakeSearch:
    """Pages over a fixed hit list per query text."""

    def __init__(self, hits, page=3):
        self.hits, self.page, self.calls = hits, page, 0

    def name(self):
        return "fake_search"

    def source_snapshot(self):
        return B.SourceSnapshot("fake", "rev-1")

    def page_size(self):
        return self.page

    def discover_page(self, query, offset, limit, parameters=None):
        self.calls += 1
        rows = self.hits[query]
        return B.DiscoveryPage(rows[offset:offset + limit], len(rows), self.source_snapshot())


class FakeMaterializer:
    def __init__(self, texts):
        self.texts = texts

    def materialize(self, hits):
        return [B.MaterializedRecord(h.record_key, self.texts[h.record_key], list(h.uris), dict(h.metadata)) for h in hits if h.record_key in self.texts]


def recipe_json(**over):
    d = {"version": 2, "build_id": "demo", "discovery": {"materialization_batch_size": 4, "queries": [{"name": "q", "text": "Q", "limit": 100}]},
         "normalization": {"minimum_characters": 4},
         "classification": {"topic_rules": [{"label": "stem", "any_terms": ["Math"]}, {"label": "language", "any_terms": ["grammar"]}],
                            "difficulty_rules": [{"label": "school", "priority": 2, "any_terms": ["school"]},
                                                 {"label": "scholarly", "priority": 1, "any_terms": ["proof", "school"]}],
                            "default_topic": "general", "default_difficulty": "unclassified"},
         "transformations": [{"name": "study", "template": "T=${topic} D=${difficulty} K=${metadata.kind} U=${unknown}\n${text}",
                              "when": {"metadata_equals": {"study": True}}}],
         "repetition": {"base_copies": 1, "max_copies_per_record": 3, "topic_copies": {"stem": 2}},
         "token_target": {"minimum": 40, "desired": 200, "maximum": 400}, "sharding": {"max_tokens_per_shard": 90}}
    d.update(over)
    return d


def test_reference_example_files_decode():
    path = os.path.join(REF, "corpus.production.example.json")
    if not os.path.exists(path):
        pytest.skip("reference tree not present")
    doc = json.load(open(path))
    r = R.CorpusRecipe.decode(doc["corpus"])
    assert r.build_id == "retrieval-curriculum-2026-08" and len(r.queries) == 4 and r.materialization_batch_size == 500
    assert r.normalization["minimum_characters"] == 200 and r.transformations[0].name == "controlled-study-view"
    B.SearchApiClient(doc["search_api"], transport=object())
    B.PostgresRecordMaterializer(doc["postgres"], executor=None)
    c = R.CompositionConfig.decode(json.load(open(os.path.join(REF, "curriculum-composition.example.json"))), "/x")
    assert [s.name for s in c.stages][:2] == ["foundation", "school"] or len(c.stages) >= 2
    assert c.source_manifest.startswith("/x/") and c.stages[0].max_fraction_deviation == 0.01
    assert [n for n, _, _ in c.stages[0].strata] == ["language", "stem", "humanities", "general"]


@pytest.mark.parametrize("mutate, message", [
    (lambda d: d.update(version=1), "unsupported corpus schema version"),
    (lambda d: d.update(build_id="a/b"), "safe path component"),
    (lambda d: d["discovery"].update(queries=[]), "queries"),
    (lambda d: d["discovery"]["queries"].append({"name": "q", "text": "x", "limit": 1}), "duplicate discovery query"),
    (lambda d: d["discovery"].update(materialization_batch_size=0), "materialization_batch_size"),
    (lambda d: d.update(deduplication={"by_record_key": False, "by_normalized_text": False}), "deduplication must enable"),
    (lambda d: d["transformations"].append({"name": "source", "template": "${text}"}), "reserved"),
    (lambda d: d["transformations"].append({"name": "x", "template": "no placeholder"}), "must contain"),
    (lambda d: d["repetition"].update(base_copies=4), "max_copies_per_record"),
    (lambda d: d["token_target"].update(desired=10), "minimum <= desired <= maximum"),
    (lambda d: d["classification"]["topic_rules"].append({"label": "empty"}), "has no condition"),
    (lambda d: d.update(surprise=1), "unknown field"),
])
def test_recipe_rejections(mutate, message):
    d = recipe_json()
    mutate(d)
    with pytest.raises(CorpusError, match=message):
        R.CorpusRecipe.decode(d)


def test_record_steps():
    r = R.CorpusRecipe.decode(recipe_json())
    assert R.normalize_text("  a \t b\r\nc\r\r\r\r\rd  ", r.normalization) == "a b\nc\n\n\nd"
    assert R.normalize_text("bad � char", r.normalization) is None and R.normalize_text(" ab ", r.normalization) is None
    # priority wins; on a tie the rule with more matched terms, then the smaller label
    assert R.classify("a school proof", {}, r.difficulty_rules, "d") == "school"
    assert R.classify("nothing", {}, r.difficulty_rules, "d") == "d"
    assert R.classify("MATH".lower(), {}, r.topic_rules, None) == "stem"                  # rule terms are case-folded
    tie = [R.Rule("b", 1, ["x"]), R.Rule("a", 1, ["x"]), R.Rule("c", 1, ["x", "y"])]
    assert R.classify("x y", {}, tie, None) == "c" and R.classify("x", {}, tie, None) == "a"
    # single-pass substitution: a value that looks like a placeholder is not expanded again
    assert R.render_template("${text}|${topic}|${metadata.n}|${nope}|${open", "${topic}", "t", None, {"n": 3}) == "${topic}|t|3|${nope}|${open"
    views, texts = R.render_views(r, "body", "stem", "school", {"study": True, "kind": "book"})
    assert [(v, c) for v, c, _ in views] == [("source", 0), ("source", 1), ("study", 0)] and texts[1].startswith("T=stem D=school K=book U=${unknown}\n")
    views, _ = R.render_views(r, "body", "general", None, {})
    assert views == [("source", 0, 0)]


def _world(n=12):
    hits = {"Q": [B.DiscoveryHit(f"k{i}", uris=[f"doi:{i}"], metadata={"study": i % 3 == 0, "kind": "book"}) for i in range(n)]}
    texts = {f"k{i}": (f"school math lesson number {i:02d} " if i % 2 else f"grammar proof text number {i:02d} ") + "x" * 10 for i in range(n)}
    return hits, texts


def test_build_dedup_resume_and_manifest(tmp_path):
    hits, texts = _world()
    hits["Q"].insert(5, B.DiscoveryHit("k1"))                                           # duplicate key
    hits["Q"].insert(7, B.DiscoveryHit("dup-text"))
    texts["dup-text"] = "  " + texts["k2"].replace(" ", "  ") + "\r\n"                  # same text after normalisation
    hits["Q"].insert(8, B.DiscoveryHit("gone"))                                         # never materialised
    r = R.CorpusRecipe.decode(recipe_json(token_target={"minimum": 40, "desired": 330, "maximum": 400}))
    one = R.build_corpus(r, FakeSearch(hits), FakeMaterializer(texts), ByteTok(), str(tmp_path / "a"))
    # an interrupted build resumed batch by batch publishes the same bytes
    out = None
    while out is None:
        out = R.build_corpus(r, FakeSearch(hits), FakeMaterializer(texts), ByteTok(), str(tmp_path / "b"), max_batches=1)
    m1, m2 = (json.load(open(os.path.join(d, "manifest.json"))) for d in (one, out))
    assert m1 == m2 and sorted(os.listdir(one)) == sorted(os.listdir(out))
    build = m1["build"]
    st = build["stats"]
    assert st["duplicate_records"] == 2 and st["missing_records"] == 1 and st["unique_tokens"] >= 330 == r.token_target.desired
    assert build["desired_token_target_reached"] and st["exposure_tokens"] > st["unique_tokens"] and st["emitted_views"] > st["unique_records"]
    assert build["topic_counts"].keys() <= {"stem", "language", "general"} and all(s["tokens"] <= 90 or s["records"] == 1 for s in build["shards"])
    manifest, rows = R.open_corpus_manifest(os.path.join(one, "manifest.json"))
    rows = list(rows())
    assert len(rows) == st["emitted_views"] and {r_["view"] for r_ in rows} == {"source", "study"}
    stem = [r_ for r_ in rows if r_["record_key"] == "k1"]
    assert [(r_["view"], r_["copy"]) for r_ in stem] == [("source", 0), ("source", 1)] and stem[0]["difficulty"] == "school" and stem[0]["uris"] == ["doi:1"]
    # a published build is immutable: a second call returns it without touching the backends
    s = FakeSearch(hits)
    assert R.build_corpus(r, s, FakeMaterializer(texts), ByteTok(), str(tmp_path / "a")) == one and s.calls == 0
    # tampering with a shard or the manifest is found
    shard = os.path.join(one, build["shards"][0]["path"])
    body = open(shard, "rb").read()
    open(shard, "wb").write(body.replace(b"k0", b"k9", 1))
    with pytest.raises(CorpusError, match="manifest hash"):
        list(R.open_corpus_manifest(os.path.join(one, "manifest.json"))[1]())
    m1["build"]["stats"]["unique_tokens"] += 1
    open(os.path.join(out, "manifest.json"), "w").write(json.dumps(m1))
    with pytest.raises(CorpusError, match="its own hash"):
        R.open_corpus_manifest(os.path.join(out, "manifest.json"))


def test_token_target_bounds(tmp_path):
    hits, texts = _world(4)
    small = recipe_json(token_target={"minimum": 1000, "desired": 2000, "maximum": 3000})
    with pytest.raises(CorpusError, match="outside the target range"):
        R.build_corpus(R.CorpusRecipe.decode(small), FakeSearch(hits), FakeMaterializer(texts), ByteTok(), str(tmp_path / "a"))
    texts["k1"] = "y" * 500
    tight = recipe_json(token_target={"minimum": 60, "desired": 80, "maximum": 90})
    with pytest.raises(CorpusError, match="no legal canonical prefix"):
        R.build_corpus(R.CorpusRecipe.decode(tight), FakeSearch(hits), FakeMaterializer(texts), ByteTok(), str(tmp_path / "b"))
    other = recipe_json(build_id="demo")
    other["normalization"]["minimum_characters"] = 5
    R.build_corpus(R.CorpusRecipe.decode(recipe_json()), FakeSearch(_world()[0]), FakeMaterializer(_world()[1]), ByteTok(), str(tmp_path / "c"), max_batches=1)
    with pytest.raises(CorpusError, match="another recipe"):
        R.build_corpus(R.CorpusRecipe.decode(other), FakeSearch(_world()[0]), FakeMaterializer(_world()[1]), ByteTok(), str(tmp_path / "c"))


def test_corpus_manifest_is_a_training_data_path(tmp_path):
    from summa_b200.train import data as D
    hits, texts = _world()
    out = R.build_corpus(R.CorpusRecipe.decode(recipe_json()), FakeSearch(hits), FakeMaterializer(texts), ByteTok(), str(tmp_path))
    _, rows = R.open_corpus_manifest(os.path.join(out, "manifest.json"))
    docs = list(D.iter_documents(os.path.join(out, "manifest.json"), ByteTok(), 256))
    assert docs == [r["tokens"] for r in rows()]
    with pytest.raises(D.DataError, match="tokens must be integers"):
        list(D.iter_documents(os.path.join(out, "manifest.json"), ByteTok(), 64))


def _composition(source, **stage_over):
    stage = {"name": "school", "when": {"difficulties": ["school", "scholarly"]}, "unmatched": "exclude",
             "token_target": {"minimum": 300, "desired": 400, "maximum": 480}, "sharding": {"max_tokens_per_shard": 150},
             "max_fraction_deviation": 0.15,
             "strata": [{"name": "stem", "weight": 3, "when": {"topics": ["stem"]}}, {"name": "language", "weight": 1, "when": {"topics": ["language"]}}]}
    stage.update(stage_over)
    return {"version": 2, "build_id": "curriculum", "source_manifest": source, "seed": 7, "stages": [stage]}


def test_compose_curriculum(tmp_path):
    hits, texts = _world(40)
    big = recipe_json(token_target={"minimum": 500, "desired": 1400, "maximum": 5000}, repetition={"base_copies": 1, "max_copies_per_record": 1})
    big["discovery"]["queries"][0]["limit"] = 1000
    src = R.build_corpus(R.CorpusRecipe.decode(big), FakeSearch(hits), FakeMaterializer(texts), ByteTok(), str(tmp_path / "corpus"))
    manifest = os.path.join(src, "manifest.json")
    pinned = json.load(open(manifest))["manifest_sha256"]
    cfg = R.CompositionConfig.decode(dict(_composition(manifest), source_manifest_sha256=pinned))
    out = R.compose_curriculum(cfg, str(tmp_path / "out"))
    root = json.load(open(os.path.join(out, "manifest.json")))["build"]
    stage = root["stages"][0]
    assert stage["tokens"] >= 400 and abs(stage["stratum_tokens"]["stem"] / stage["tokens"] - 0.75) <= 0.15
    sm, rows = R.open_corpus_manifest(os.path.join(out, "school", "manifest.json"))
    rows = list(rows())
    assert sm["manifest_sha256"] == stage["manifest_sha256"] and sum(len(r["tokens"]) for r in rows) == stage["tokens"]
    assert sm["build"]["deduplicator"]["type"] == "stratified_curriculum_composition" and not os.path.exists(os.path.join(out, ".spools"))
    # source order is kept inside a stratum, and the draw is a pure function of the configuration
    stem = [r["record_key"] for r in rows if r["topic"] == "stem"]
    assert stem == sorted(stem, key=lambda k: int(k[1:]))
    again = R.compose_curriculum(R.CompositionConfig.decode(dict(_composition(manifest), build_id="again")), str(tmp_path / "out"))
    assert [r["record_key"] for r in R.open_corpus_manifest(os.path.join(again, "school", "manifest.json"))[1]()] == [r["record_key"] for r in rows]
    with pytest.raises(CorpusError, match="already published"):
        R.compose_curriculum(cfg, str(tmp_path / "out"))
    for over, message in [(dict(token_target={"minimum": 3000, "desired": 4000, "maximum": 4800}), "exhausted"),
                          (dict(max_fraction_deviation=0.0), "differs from configured"),
                          (dict(unmatched="error", strata=[{"name": "stem", "weight": 1, "when": {"topics": ["stem"]}}]), "no stratum does")]:
        c = _composition(manifest, **over)
        c["build_id"] = "bad"
        with pytest.raises(CorpusError, match=message):
            R.compose_curriculum(R.CompositionConfig.decode(c), str(tmp_path / "out"))
    with pytest.raises(CorpusError, match="pinned generation"):
        R.compose_curriculum(R.CompositionConfig.decode(dict(_composition(manifest), build_id="p", source_manifest_sha256="0" * 64)), str(tmp_path / "out"))


def test_postgres_plan_and_executor():
    pem = "-----BEGIN CERTIFICATE-----\nAAAA\n-----END CERTIFICATE-----\n"
    cfg = {"connection_environment": "DSN", "statement": "SELECT k, t, u, m FROM d WHERE k = ANY($1::text[]) AND t LIKE '%x'", "columns":
           {"record_key": "k", "text": "t", "uris": "u", "metadata": "m"}, "snapshot_statement": "SELECT rev",
           "transport_security": {"mode": "verified_tls", "server_names": ["db.example"], "trust":
                                  {"source": "pinned_pem", "certificate_pem_environment": "PEM", "certificate_sha256": "sha256:" + hashlib.sha256(pem.encode()).hexdigest()}}}
    plan = B.postgres_connection_plan(cfg, {"DSN": "postgresql://u:p@db.example:5432/x", "PEM": pem})
    assert plan["sslmode"] == "verify-full" and plan["root_pem"] == pem
    for env, message in [({"DSN": "postgresql://u@other.example/x", "PEM": pem}, "exactly match"), ({"DSN": "host=db.example", "PEM": pem + " "}, "digest"),
                         ({"DSN": "host=/var/run/pg", "PEM": pem}, "Unix socket"), ({"PEM": pem}, "not set")]:
        with pytest.raises(CorpusError, match=message):
            B.postgres_connection_plan(cfg, env)
    local = dict(cfg, transport_security={"mode": "plaintext_local_proxy", "acknowledge_plaintext": True})
    assert B.postgres_connection_plan(local, {"DSN": "host=127.0.0.1 dbname=x"})["sslmode"] == "disable"
    with pytest.raises(CorpusError, match="not loopback"):
        B.postgres_connection_plan(local, {"DSN": "host=10.0.0.1"})
    with pytest.raises(CorpusError, match="acknowledge_plaintext"):
        B.postgres_connection_plan(dict(cfg, transport_security={"mode": "plaintext_local_proxy", "acknowledge_plaintext": False}), {"DSN": "host=127.0.0.1"})

    class Cursor:
        def __init__(self, log):
            self.log, self.description, self.rows = log, None, []

        def execute(self, sql, params=None):
            self.log.append((sql, params))
            if sql == "SELECT rev":
                self.description, self.rows = [("rev",)], [("g42",)]
            elif sql.startswith("SELECT k"):
                self.description = [("m",), ("k",), ("t",), ("u",)]
                self.rows = [('{"a":1}', key, "text of " + key, ["doi:" + key]) for key in params[0] if key != "gone"]

        def fetchall(self):
            return self.rows

    class Conn:
        def __init__(self):
            self.log = []

        def cursor(self):
            return Cursor(self.log)

    conn = Conn()
    ex = B.DbApiPostgresExecutor(conn).bind(cfg)
    mat = B.PostgresRecordMaterializer(dict(cfg, require_every_record=False), ex)
    got = mat.materialize([B.DiscoveryHit("a", metadata={"z": 0}), B.DiscoveryHit("gone")])
    assert [(g.record_key, g.text, g.uris, g.metadata) for g in got] == [("a", "text of a", ["doi:a"], {"z": 0, "a": 1})]
    assert mat.source_snapshot().revision == "g42" and conn.log[0][0].startswith("BEGIN TRANSACTION ISOLATION LEVEL REPEATABLE READ READ ONLY")
    assert conn.log[1] == ("SELECT k, t, u, m FROM d WHERE k = ANY(%s::text[]) AND t LIKE '%%x'", (["a", "gone"],))
    with pytest.raises(CorpusError, match="materialized 1 of 2"):
        B.PostgresRecordMaterializer(cfg, ex).materialize([B.DiscoveryHit("a"), B.DiscoveryHit("gone")])


def test_compose_curriculum_command(tmp_path, capsys):
    from summa_b200.cli import train as cli
    hits, texts = _world(40)
    big = recipe_json(token_target={"minimum": 500, "desired": 1400, "maximum": 5000}, repetition={"base_copies": 1, "max_copies_per_record": 1})
    src = R.build_corpus(R.CorpusRecipe.decode(big), FakeSearch(hits), FakeMaterializer(texts), ByteTok(), str(tmp_path / "corpus"))
    cfg = _composition(os.path.relpath(os.path.join(src, "manifest.json"), tmp_path))                     # relative to the config file
    (tmp_path / "composition.json").write_text(json.dumps(cfg))
    assert cli.main(["compose-curriculum", "--config", str(tmp_path / "composition.json"), "-o", str(tmp_path / "out"),
                     "--work-directory", str(tmp_path / "work")]) == 0
    published = json.loads(capsys.readouterr().out.strip().splitlines()[-1])["published"]
    assert os.path.exists(os.path.join(published, "school", "manifest.json")) and os.listdir(tmp_path / "work") == []


def test_prepare_corpus_command_over_a_loopback_search_service(tmp_path, capsys):
    """The production file shape end to end: `corpus` + `search_api` (inline text, no database) against an HTTP service on
    loopback that answers the configured request shape."""
    import http.server
    import threading
    from summa_b200.cli import train as cli
    from tests.test_corpus import _search_cfg
    keys = [f"k{i}" for i in range(30)]
    seen = []

    class Handler(http.server.BaseHTTPRequestHandler):
        def do_POST(self):
            body = json.loads(self.rfile.read(int(self.headers["content-length"])))
            seen.append(body)
            off, lim = body["page"]["offset"], body["page"]["limit"]
            hits = [{"id": k, "score": 1.0, "links": f"doi:{k}", "body": f"school math text number {k} " + "y" * 20, "meta": {"year": 2001}}
                    for k in keys][off:off + lim]
            out = json.dumps({"snapshot": {"provider": "idx", "revision": "r7"}, "result": {"hits": hits, "total": len(keys)}}).encode()
            self.send_response(200)
            self.send_header("content-type", "application/json")
            self.send_header("content-length", str(len(out)))
            self.end_headers()
            self.wfile.write(out)

        def log_message(self, *a):
            pass

    server = http.server.HTTPServer(("127.0.0.1", 0), Handler)
    thread = threading.Thread(target=server.serve_forever, daemon=True)
    thread.start()
    try:
        recipe = {"corpus": recipe_json(token_target={"minimum": 200, "desired": 600, "maximum": 900}),
                  "search_api": _search_cfg(endpoint=f"http://127.0.0.1:{server.server_address[1]}/search")}
        recipe["corpus"]["discovery"]["queries"][0]["parameters"] = {"language": "en"}
        (tmp_path / "recipe.json").write_text(json.dumps(recipe))
        from summa_b200.tokenizer import Tokenizer
        tok_path = tmp_path / "tokenizer.json"
        tok_path.write_text(Tokenizer.byte_level().to_json())
        assert cli.main(["prepare-corpus", "--recipe", str(tmp_path / "recipe.json"), "-t", str(tok_path), "-o", str(tmp_path / "corpus"),
                         "--work-directory", str(tmp_path / "work")]) == 0
    finally:
        server.shutdown()
    published = json.loads(capsys.readouterr().out.strip().splitlines()[-1])["published"]
    manifest, rows = R.open_corpus_manifest(os.path.join(published, "manifest.json"))
    build = manifest["build"]
    assert build["discovery"]["backend"] == "search_api" and build["discovery"]["snapshot"] == "idx@r7" and build["materializer"]["backend"] == "inline"
    assert build["tokenizer"]["snapshot"].startswith("sha256:") and build["stats"]["unique_tokens"] >= 600
    assert all(b["lang"] == "en" and b["rerank"] == {"cross": False, "llm": False} for b in seen) and seen[0]["page"]["limit"] <= 4
    assert [r["topic"] for r in rows()][0] == "stem" and not os.path.exists(tmp_path / "work" / "dedup.sqlite")
