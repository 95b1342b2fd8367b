"""Version-2 corpus recipes and curriculum composition: the configuration files of the reference's corpus tooling
(`summa-train/corpus.production.example.json`, `curriculum-composition.example.json`) and the pipeline behind them.

A recipe (`corpus` block, `summa-train/src/corpus/config.rs:22-420`) names discovery queries (text, per-query hit
limit, backend parameters), text normalisation, deduplication by record key and / or normalised text, rule-based
topic and difficulty classification, transformations that emit extra rendered views of a record, repetition, a
token target over UNIQUE tokens and the shard size. Records flow through `build_corpus` as in
`corpus/pipeline.rs:1840-1955`:

    discover (paged, merged by record key) -> materialise in batches -> normalise -> deduplicate -> tokenise ->
    admit against the token target -> classify -> render views -> JSONL shards -> sealed manifest

The token target counts each unique record once (its canonical text); a build stops at the first record that
reaches `desired`, refuses to pass `maximum`, and is rejected below `minimum`. Shards are JSONL rows
`{record_key, uris, topic, difficulty, view, copy, metadata, tokens}`; the manifest seals every shard's SHA-256 and
carries the build's statistics and source snapshots. A build is resumable at materialisation-batch granularity: the
open shard is closed at every batch commit, so the cursor only names finished shards.

`compose_curriculum` (`corpus/compose.rs:166-260,669-800,1854-2140`) cuts a published corpus into stages: a stage
selects records by predicate, assigns each to its first matching stratum (`unmatched`: error or exclude), then draws
from the stratum whose emitted-tokens / weight ratio is lowest (ties by a seed-derived digest), in source order
inside a stratum, until the stage's desired tokens are reached; exhaustion, overshooting `maximum`, undershooting
`minimum` and a token fraction further than `max_fraction_deviation` from a stratum's weight are errors."""
from __future__ import annotations

import hashlib
import json
import math
import os
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Iterator, List, Optional, Sequence, Tuple

from .corpus import CorpusError, SqliteDeduplicator

CORPUS_SCHEMA_VERSION = 2
MAX_DISCOVERY_QUERIES = 4096
MAX_DISCOVERY_HITS = 1_000_000_000
MAX_DISCOVERY_BATCH_SIZE = 65536
MAX_CLASSIFICATION_RULES = 4096
MAX_CLASSIFICATION_TERMS = 4096
MAX_TRANSFORMATIONS = 1024
MAX_COPIES_PER_RECORD = 4096
MAX_STRATA_PER_STAGE = 1024
MAX_RENDERED_VIEW_TEXT_BYTES = 64 * 1024 * 1024


def _need(cond: bool, message: str) -> None:
    if not cond:
        raise CorpusError(message)


def _obj(v: Any, what: str, allowed: Sequence[str], required: Sequence[str] = ()) -> Dict[str, Any]:
    _need(isinstance(v, dict), f"{what} must be an object")
    unknown = set(v) - set(allowed)
    if unknown:
        raise CorpusError(f"unknown field `{sorted(unknown)[0]}` in {what}")
    for k in required:
        _need(k in v, f"missing field `{k}` in {what}")
    return v


def _uint(v: Any, what: str) -> int:
    _need(isinstance(v, int) and not isinstance(v, bool) and v >= 0, f"{what} must be a non-negative integer")
    return v


def _component(v: Any, what: str) -> str:
    _need(isinstance(v, str) and v.strip() != "", f"{what} must not be empty")
    _need("/" not in v and "\\" not in v and v not in (".", ".."), f"{what} must be one safe path component")
    return v


def _strings(v: Any, what: str) -> List[str]:
    _need(isinstance(v, list) and all(isinstance(x, str) for x in v), f"{what} must be an array of strings")
    return list(v)


# ------------------------------------------------------------------------------------------------ recipe
@dataclass
class TokenTarget:
    minimum: int
    desired: int
    maximum: int

    @staticmethod
    def decode(v: Any, what: str = "`token_target`") -> "TokenTarget":
        d = _obj(v, what, ("minimum", "desired", "maximum"), ("minimum", "desired", "maximum"))
        t = TokenTarget(_uint(d["minimum"], f"{what}.minimum"), _uint(d["desired"], f"{what}.desired"), _uint(d["maximum"], f"{what}.maximum"))
        _need(t.minimum > 0, "minimum token target must be positive")
        _need(t.minimum <= t.desired <= t.maximum, "token targets must satisfy minimum <= desired <= maximum")
        return t

    def accepts(self, tokens: int) -> bool:
        return self.minimum <= tokens <= self.maximum

    def to_json(self) -> Dict[str, int]:
        return {"minimum": self.minimum, "desired": self.desired, "maximum": self.maximum}


@dataclass
class Rule:
    label: str
    priority: int = 0
    any_terms: List[str] = field(default_factory=list)
    all_terms: List[str] = field(default_factory=list)
    none_terms: List[str] = field(default_factory=list)
    metadata_equals: Dict[str, Any] = field(default_factory=dict)

    @staticmethod
    def decode(v: Any, what: str) -> "Rule":
        d = _obj(v, what, ("label", "priority", "any_terms", "all_terms", "none_terms", "metadata_equals"), ("label",))
        r = Rule(d["label"], d.get("priority", 0), _strings(d.get("any_terms", []), f"{what}.any_terms"),
                 _strings(d.get("all_terms", []), f"{what}.all_terms"), _strings(d.get("none_terms", []), f"{what}.none_terms"),
                 dict(d.get("metadata_equals", {})))
        _need(isinstance(r.label, str) and r.label.strip() != "", "classification labels must not be empty")
        _need(isinstance(r.priority, int) and not isinstance(r.priority, bool), f"{what}.priority must be an integer")
        terms = r.any_terms + r.all_terms + r.none_terms
        _need(len(terms) <= MAX_CLASSIFICATION_TERMS, f"classification rule `{r.label}` exceeds the {MAX_CLASSIFICATION_TERMS}-term limit")
        _need(bool(terms) or bool(r.metadata_equals), f"classification rule `{r.label}` has no condition")
        _need(all(t.strip() for t in terms), f"classification rule `{r.label}` contains an empty term")
        return r

    def folded(self) -> Tuple[List[str], List[str], List[str]]:
        return [t.lower() for t in self.any_terms], [t.lower() for t in self.all_terms], [t.lower() for t in self.none_terms]


@dataclass
class Predicate:
    topics: List[str] = field(default_factory=list)
    difficulties: List[str] = field(default_factory=list)
    views: List[str] = field(default_factory=list)
    metadata_equals: Dict[str, Any] = field(default_factory=dict)

    @staticmethod
    def decode(v: Any, what: str, with_views: bool) -> "Predicate":
        allowed = ("topics", "difficulties", "metadata_equals") + (("views",) if with_views else ())
        d = _obj(v if v is not None else {}, what, allowed)
        p = Predicate(_strings(d.get("topics", []), f"{what}.topics"), _strings(d.get("difficulties", []), f"{what}.difficulties"),
                      _strings(d.get("views", []), f"{what}.views") if with_views else [], dict(d.get("metadata_equals", {})))
        _need(all(s.strip() for s in p.topics + p.difficulties + p.views), f"{what} contains an empty selector")
        return p

    def matches(self, topic: Optional[str], difficulty: Optional[str], metadata: Dict[str, Any], view: Optional[str] = None) -> bool:
        return ((not self.topics or topic in self.topics) and (not self.difficulties or difficulty in self.difficulties)
                and (not self.views or view in self.views) and all(metadata.get(k, _ABSENT) == v for k, v in self.metadata_equals.items()))

    def to_json(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"topics": self.topics, "difficulties": self.difficulties, "metadata_equals": self.metadata_equals}
        if self.views:
            out["views"] = self.views
        return out


_ABSENT = object()


@dataclass
class Transformation:
    name: str
    template: str
    copies: int = 1
    when: Predicate = field(default_factory=Predicate)


@dataclass
class CorpusRecipe:
    build_id: str
    queries: List[Dict[str, Any]]
    materialization_batch_size: int
    normalization: Dict[str, Any]
    deduplication: Dict[str, bool]
    topic_rules: List[Rule]
    difficulty_rules: List[Rule]
    default_topic: Optional[str]
    default_difficulty: Optional[str]
    transformations: List[Transformation]
    repetition: Dict[str, Any]
    token_target: TokenTarget
    max_tokens_per_shard: int
    raw: Dict[str, Any] = field(default_factory=dict)

    @staticmethod
    def decode(v: Any) -> "CorpusRecipe":
        d = _obj(v, "the corpus recipe", ("version", "build_id", "discovery", "normalization", "deduplication", "classification",
                                            "transformations", "repetition", "token_target", "sharding"),
                 ("version", "build_id", "discovery", "token_target", "sharding"))
        _need(d["version"] == CORPUS_SCHEMA_VERSION, f"unsupported corpus schema version {d['version']}; expected {CORPUS_SCHEMA_VERSION}")
        build_id = _component(d["build_id"], "corpus build_id")
        disc = _obj(d["discovery"], "`discovery`", ("queries", "materialization_batch_size"), ("queries",))
        _need(isinstance(disc["queries"], list) and 0 < len(disc["queries"]) <= MAX_DISCOVERY_QUERIES,
              f"corpus discovery requires 1..={MAX_DISCOVERY_QUERIES} queries")
        batch = _uint(disc.get("materialization_batch_size", 500), "materialization_batch_size")
        _need(1 <= batch <= MAX_DISCOVERY_BATCH_SIZE, f"materialization_batch_size must be within 1..={MAX_DISCOVERY_BATCH_SIZE}")
        names, total, queries = set(), 0, []
        for q in disc["queries"]:
            q = _obj(q, "a discovery query", ("name", "text", "limit", "parameters"), ("name", "text", "limit"))
            _need(isinstance(q["name"], str) and q["name"].strip() and isinstance(q["text"], str) and q["text"].strip(),
                  "discovery query name and text must not be empty")
            _need(q["name"] not in names, f"duplicate discovery query name `{q['name']}`")
            names.add(q["name"])
            limit = _uint(q["limit"], f"query `{q['name']}` limit")
            _need(1 <= limit <= MAX_DISCOVERY_HITS, f"query `{q['name']}` limit must be within 1..={MAX_DISCOVERY_HITS}")
            total += limit
            _need(total <= MAX_DISCOVERY_HITS, f"aggregate discovery query limit exceeds {MAX_DISCOVERY_HITS} hits")
            _need(isinstance(q.get("parameters", {}), dict), f"query `{q['name']}` parameters must be an object")
            queries.append({"name": q["name"], "text": q["text"], "limit": limit, "parameters": dict(q.get("parameters", {}))})
        norm = {"trim": True, "normalize_newlines": True, "collapse_horizontal_whitespace": True, "max_consecutive_blank_lines": 2,
                "reject_replacement_character": True, "minimum_characters": 1}
        norm.update(_obj(d.get("normalization", {}), "`normalization`", tuple(norm)))
        _need(_uint(norm["minimum_characters"], "minimum_characters") > 0, "normalization minimum_characters must be positive")
        _uint(norm["max_consecutive_blank_lines"], "max_consecutive_blank_lines")
        dedup = {"by_record_key": True, "by_normalized_text": True}
        dedup.update(_obj(d.get("deduplication", {}), "`deduplication`", tuple(dedup)))
        _need(bool(dedup["by_record_key"]) or bool(dedup["by_normalized_text"]), "deduplication must enable record-key or normalized-text matching")
        cls = _obj(d.get("classification", {}), "`classification`", ("topic_rules", "difficulty_rules", "default_topic", "default_difficulty"))
        topic_rules = [Rule.decode(r, "a topic rule") for r in cls.get("topic_rules", [])]
        diff_rules = [Rule.decode(r, "a difficulty rule") for r in cls.get("difficulty_rules", [])]
        _need(len(topic_rules) + len(diff_rules) <= MAX_CLASSIFICATION_RULES, f"classification exceeds the {MAX_CLASSIFICATION_RULES}-rule limit")
        for k in ("default_topic", "default_difficulty"):
            _need(cls.get(k) is None or (isinstance(cls[k], str) and cls[k].strip() != ""), "classification default labels must not be empty")
        transforms, seen = [], set()
        _need(isinstance(d.get("transformations", []), list) and len(d.get("transformations", [])) <= MAX_TRANSFORMATIONS,
              f"corpus transformations exceed the {MAX_TRANSFORMATIONS}-item limit")
        for t in d.get("transformations", []):
            t = _obj(t, "a transformation", ("name", "template", "copies", "when"), ("name", "template"))
            _need(isinstance(t["name"], str) and t["name"].strip() != "", "transformation names must not be empty")
            _need(t["name"] != "source", "transformation name `source` is reserved for canonical corpus views")
            _need(t["name"] not in seen, f"duplicate transformation name `{t['name']}`")
            seen.add(t["name"])
            _need(isinstance(t["template"], str) and "${text}" in t["template"], f"transformation `{t['name']}` template must contain `${{text}}`")
            copies = _uint(t.get("copies", 1), "transformation copies")
            _need(copies > 0, "every transformation must emit at least one copy")
            transforms.append(Transformation(t["name"], t["template"], copies, Predicate.decode(t.get("when"), "`when`", False)))
        rep = {"base_copies": 1, "max_copies_per_record": 1, "topic_copies": {}, "difficulty_copies": {}}
        rep.update(_obj(d.get("repetition", {}), "`repetition`", tuple(rep)))
        _need(_uint(rep["base_copies"], "base_copies") > 0, "base_copies must be positive")
        _need(rep["base_copies"] <= _uint(rep["max_copies_per_record"], "max_copies_per_record") <= MAX_COPIES_PER_RECORD,
              f"max_copies_per_record must cover base_copies and stay within {MAX_COPIES_PER_RECORD}")
        for table in ("topic_copies", "difficulty_copies"):
            _need(isinstance(rep[table], dict) and all(isinstance(k, str) and k.strip() and isinstance(c, int) and 0 < c <= rep["max_copies_per_record"]
                                                       for k, c in rep[table].items()),
                  "configured repetition copies must be positive, within max_copies_per_record, and keyed by non-empty labels")
        shard = _obj(d["sharding"], "`sharding`", ("max_tokens_per_shard",), ("max_tokens_per_shard",))
        _need(_uint(shard["max_tokens_per_shard"], "max_tokens_per_shard") > 0, "max_tokens_per_shard must be positive")
        return CorpusRecipe(build_id, queries, batch, norm, dedup, topic_rules, diff_rules, cls.get("default_topic"), cls.get("default_difficulty"),
                            transforms, rep, TokenTarget.decode(d["token_target"]), shard["max_tokens_per_shard"], raw=json.loads(json.dumps(d)))

    def sha256(self) -> str:
        return hashlib.sha256(json.dumps(self.raw, sort_keys=True, separators=(",", ":")).encode()).hexdigest()


# ------------------------------------------------------------------------------------------------ record steps
def normalize_text(text: str, cfg: Dict[str, Any]) -> Optional[str]:
    """None = rejected (a replacement character, or too short after normalisation)."""
    if cfg["reject_replacement_character"] and "�" in text:
        return None
    if cfg["normalize_newlines"]:
        text = text.replace("\r\n", "\n").replace("\r", "\n")
    if cfg["collapse_horizontal_whitespace"]:
        out, horizontal = [], False
        for ch in text:
            if ch != "\n" and ch.isspace():
                horizontal = True
            else:
                if horizontal and out and out[-1] not in (" ", "\n"):
                    out.append(" ")
                horizontal = False
                out.append(ch)
        text = "".join(out)
    keep, out, run = cfg["max_consecutive_blank_lines"] + 1, [], 0
    for ch in text:
        if ch == "\n":
            run += 1
            if run <= keep:
                out.append(ch)
        else:
            run = 0
            out.append(ch)
    text = "".join(out)
    if cfg["trim"]:
        text = text.strip()
    return text if len(text) >= cfg["minimum_characters"] else None


def classify(folded_text: str, metadata: Dict[str, Any], rules: Sequence[Rule], default: Optional[str]) -> Optional[str]:
    """The matching rule with the highest priority; ties by more metadata conditions, then more matched terms, then the
    lexicographically smaller label."""
    best = None
    for r in rules:
        any_t, all_t, none_t = r.folded()
        hit_any = sum(t in folded_text for t in any_t)
        hit_all = sum(t in folded_text for t in all_t)
        if not ((not any_t or hit_any > 0) and hit_all == len(all_t) and all(t not in folded_text for t in none_t)
                and all(metadata.get(k, _ABSENT) == v for k, v in r.metadata_equals.items())):
            continue
        key = (r.priority, len(r.metadata_equals), hit_any + hit_all + len(none_t), [-ord(c) for c in r.label])
        if best is None or key > best[0]:
            best = (key, r.label)
    return best[1] if best else default


def render_template(template: str, text: str, topic: Optional[str], difficulty: Optional[str], metadata: Dict[str, Any]) -> str:
    """Single pass over `${...}` placeholders: `text`, `topic`, `difficulty`, `metadata.<name>`; unknown placeholders
    stay as written, and substituted values are never re-scanned."""
    out, cursor = [], 0
    while True:
        start = template.find("${", cursor)
        if start < 0:
            out.append(template[cursor:])
            break
        out.append(template[cursor:start])
        close = template.find("}", start + 2)
        if close < 0:
            out.append(template[start:])
            break
        name = template[start + 2:close]
        if name == "text":
            value = text
        elif name == "topic":
            value = topic or ""
        elif name == "difficulty":
            value = difficulty or ""
        elif name.startswith("metadata.") and name[9:] in metadata:
            m = metadata[name[9:]]
            value = m if isinstance(m, str) else json.dumps(m, separators=(",", ":"))
        else:
            value = template[start:close + 1]
        out.append(value)
        cursor = close + 1
    rendered = "".join(out)
    _need(len(rendered.encode()) <= MAX_RENDERED_VIEW_TEXT_BYTES, f"rendered corpus view exceeds the {MAX_RENDERED_VIEW_TEXT_BYTES}-byte limit")
    return rendered


def render_views(recipe: CorpusRecipe, text: str, topic: Optional[str], difficulty: Optional[str], metadata: Dict[str, Any]):
    """([(view name, copy index, text index)], [distinct texts]); text 0 is the canonical one."""
    rep = recipe.repetition
    base = max(rep["base_copies"], rep["topic_copies"].get(topic, 0), rep["difficulty_copies"].get(difficulty, 0))
    views = [("source", c, 0) for c in range(base)]
    texts = [text]
    for t in recipe.transformations:
        room = max(rep["max_copies_per_record"] - len(views), 0)
        if room == 0:
            break
        if not t.when.matches(topic, difficulty, metadata):
            continue
        rendered = render_template(t.template, text, topic, difficulty, metadata)
        if rendered in texts:
            at = texts.index(rendered)
        else:
            texts.append(rendered)
            at = len(texts) - 1
        views += [(t.name, c, at) for c in range(min(t.copies, room))]
    return views, texts


# ------------------------------------------------------------------------------------------------ shards
class _ShardWriter:
    def __init__(self, directory: str, max_tokens: int, next_index: int):
        self.dir, self.max, self.index = directory, max_tokens, next_index
        self.rows: List[bytes] = []
        self.tokens = 0

    def push(self, row: Dict[str, Any]) -> Optional[Dict[str, Any]]:
        """Adds a row; returns the entry of a shard that had to be closed first (the row alone may exceed the size)."""
        n, closed = len(row["tokens"]), None
        if self.rows and self.tokens + n > self.max:
            closed = self.close()
        self.rows.append(json.dumps(row, sort_keys=True, separators=(",", ":"), ensure_ascii=False).encode() + b"\n")
        self.tokens += n
        return closed

    def close(self) -> Optional[Dict[str, Any]]:
        if not self.rows:
            return None
        name = f"shard-{self.index:06d}.jsonl"
        body = b"".join(self.rows)
        tmp = os.path.join(self.dir, name + ".partial")
        with open(tmp, "wb") as f:
            f.write(body)
            f.flush()
            os.fsync(f.fileno())
        os.replace(tmp, os.path.join(self.dir, name))
        entry = {"path": name, "sha256": hashlib.sha256(body).hexdigest(), "bytes": len(body), "records": len(self.rows), "tokens": self.tokens}
        self.index, self.rows, self.tokens = self.index + 1, [], 0
        return entry


def read_corpus_shard(path: str, expect_sha256: Optional[str] = None) -> Iterator[Dict[str, Any]]:
    with open(path, "rb") as f:
        body = f.read()
    if expect_sha256 is not None and hashlib.sha256(body).hexdigest() != expect_sha256:
        raise CorpusError(f"corpus shard {os.path.basename(path)} does not match its manifest hash")
    for line in body.splitlines():
        if line.strip():
            row = json.loads(line)
            _need(bool(row.get("record_key")) and bool(row.get("view")) and bool(row.get("tokens")), "corpus row lacks its key, view or tokens")
            yield row


def open_corpus_manifest(path: str) -> Tuple[Dict[str, Any], Callable[[], Iterator[Dict[str, Any]]]]:
    """Authenticates `<dir>/manifest.json` of a version-2 corpus (or curriculum stage); returns (manifest, row iterator)."""
    with open(path, "rb") as f:
        manifest = json.loads(f.read())
    build = manifest.get("build") or {}
    _need(build.get("version") == CORPUS_SCHEMA_VERSION, f"unsupported corpus manifest version {build.get('version')}")
    _need(manifest.get("manifest_sha256") == _canonical_sha256(build), "corpus manifest does not match its own hash")
    base = os.path.dirname(os.path.abspath(path))

    def rows():
        for sh in build["shards"]:
            _component(sh["path"], "shard path")
            yield from read_corpus_shard(os.path.join(base, sh["path"]), sh["sha256"])
    return manifest, rows


def _canonical_sha256(value: Any) -> str:
    return hashlib.sha256(json.dumps(value, sort_keys=True, separators=(",", ":"), ensure_ascii=False).encode()).hexdigest()


# ------------------------------------------------------------------------------------------------ build
def build_corpus(recipe: CorpusRecipe, search, materializer, tokenizer, output_root: str, vocabulary_size: Optional[int] = None,
                 max_batches: Optional[int] = None, work_directory: Optional[str] = None,
                 tokenizer_identity: Optional[str] = None) -> Optional[str]:
    """Builds (or resumes) `<output_root>/<build_id>/`. `search.discover_page(text, offset, limit, parameters)` returns a
    page of hits (`record_key`, `uris`, `metadata`, ...) with `total_hits`; `materializer.materialize(hits)` returns the
    records (`record_key`, `text`, `uris`, `metadata`) it could find; `tokenizer_identity` (the `sha256:<hex>` of the
    tokenizer file) is sealed into the manifest. Returns the published directory, or None when
    `max_batches` stopped the build early (call again to resume)."""
    final = os.path.join(output_root, recipe.build_id)
    if os.path.exists(os.path.join(final, "manifest.json")):
        return final
    stage = os.path.join(output_root, f".{recipe.build_id}.building")
    os.makedirs(stage, exist_ok=True)
    work = work_directory or stage                                      # restart state; never part of the published corpus
    os.makedirs(work, exist_ok=True)
    store = SqliteDeduplicator(os.path.join(work, "dedup.sqlite"))
    cur = store.load_cursor() or {"recipe_sha256": recipe.sha256(), "query": 0, "offset": 0, "taken": 0, "done": False, "shards": [],
                                  "topic_counts": {}, "difficulty_counts": {},
                                  "stats": {"discovered_hits": 0, "materialized_records": 0, "missing_records": 0, "normalization_rejections": 0,
                                            "duplicate_records": 0, "unique_records": 0, "unique_tokens": 0, "emitted_views": 0, "exposure_tokens": 0}}
    _need(cur["recipe_sha256"] == recipe.sha256(), "the staged corpus build belongs to another recipe")
    vocab = vocabulary_size if vocabulary_size is not None else (tokenizer.vocab_size() if hasattr(tokenizer, "vocab_size") else None)
    page = getattr(search, "page_size", lambda: recipe.materialization_batch_size)()
    batches = 0
    while not cur["done"] and cur["query"] < len(recipe.queries):
        if max_batches is not None and batches >= max_batches:
            return None
        q = recipe.queries[cur["query"]]
        want = min(recipe.materialization_batch_size, q["limit"] - cur["taken"])
        hits: Dict[str, Any] = {}
        offset, total = cur["offset"], None
        while len(hits) < want:
            got = search.discover_page(q["text"], offset, min(page, want - len(hits)), q["parameters"])
            total = got.total_hits
            if not got.hits:
                break
            for h in got.hits:
                if h.record_key in hits:                               # one hit per key inside a batch: metadata and uris merge
                    hits[h.record_key].metadata.update(h.metadata)
                    hits[h.record_key].uris = sorted(set(hits[h.record_key].uris) | set(h.uris))
                else:
                    hits[h.record_key] = h
            offset += len(got.hits)
            if total is not None and offset >= total:
                break
        st = cur["stats"]
        st["discovered_hits"] += offset - cur["offset"]
        writer = _ShardWriter(stage, recipe.max_tokens_per_shard, len(cur["shards"]))
        new_hashes: List[str] = []
        fresh = set()
        boundary = False
        if hits:
            records = materializer.materialize(list(hits.values()))
            st["materialized_records"] += len(records)
            st["missing_records"] += len(hits) - len(records)
            for rec in records:
                text = normalize_text(rec.text, recipe.normalization)
                if text is None:
                    st["normalization_rejections"] += 1
                    continue
                keys = ([f"k:{rec.record_key}"] if recipe.deduplication["by_record_key"] else []) + \
                       ([f"t:{hashlib.sha256(text.encode()).hexdigest()}"] if recipe.deduplication["by_normalized_text"] else [])
                if any(k in fresh or store.seen(k) for k in keys):
                    st["duplicate_records"] += 1
                    continue
                tokens = list(tokenizer.encode(text))
                _need(bool(tokens), f"tokenizer emitted no tokens for `{rec.record_key}`")
                _need(vocab is None or max(tokens) < vocab, f"tokenizer emitted a token outside vocabulary size {vocab} for `{rec.record_key}`")
                if st["unique_tokens"] + len(tokens) > recipe.token_target.maximum:
                    _need(st["unique_tokens"] >= recipe.token_target.minimum,
                          f"corpus has no legal canonical prefix: {st['unique_tokens']} unique tokens are below minimum {recipe.token_target.minimum}, "
                          f"but adding record `{rec.record_key}` ({len(tokens)} tokens) would exceed maximum {recipe.token_target.maximum}")
                    boundary = True
                    break
                new_hashes += keys
                fresh.update(keys)
                folded = text.lower()
                topic = classify(folded, rec.metadata, recipe.topic_rules, recipe.default_topic)
                difficulty = classify(folded, rec.metadata, recipe.difficulty_rules, recipe.default_difficulty)
                for table, label in (("topic_counts", topic), ("difficulty_counts", difficulty)):
                    if label is not None:
                        cur[table][label] = cur[table].get(label, 0) + 1
                st["unique_records"] += 1
                st["unique_tokens"] += len(tokens)
                views, texts = render_views(recipe, text, topic, difficulty, rec.metadata)
                encoded: List[Optional[List[int]]] = [tokens] + [None] * (len(texts) - 1)
                for name, copy, at in views:
                    if encoded[at] is None:
                        encoded[at] = list(tokenizer.encode(texts[at]))
                        _need(bool(encoded[at]), f"tokenizer emitted no tokens for view `{name}` of `{rec.record_key}`")
                    closed = writer.push({"record_key": rec.record_key, "uris": list(rec.uris), "topic": topic, "difficulty": difficulty,
                                          "view": name, "copy": copy, "metadata": rec.metadata, "tokens": encoded[at]})
                    if closed:
                        cur["shards"].append(closed)
                    st["emitted_views"] += 1
                    st["exposure_tokens"] += len(encoded[at])
                if st["unique_tokens"] >= recipe.token_target.desired:
                    boundary = True
                    break
        closed = writer.close()                                         # every commit names finished shards only
        if closed:
            cur["shards"].append(closed)
        cur["taken"] += offset - cur["offset"]
        cur["offset"] = offset
        exhausted = not hits or (total is not None and offset >= total) or cur["taken"] >= q["limit"]
        if boundary:
            cur["done"] = True
        elif exhausted:
            cur["query"], cur["offset"], cur["taken"] = cur["query"] + 1, 0, 0
        store.commit(new_hashes, cur)
        batches += 1
    st = cur["stats"]
    _need(recipe.token_target.accepts(st["unique_tokens"]),
          f"corpus holds {st['unique_tokens']} unique tokens, outside the target range {recipe.token_target.minimum}..={recipe.token_target.maximum}")
    _need(bool(cur["shards"]), "corpus build emitted no shards")
    build = {"version": CORPUS_SCHEMA_VERSION, "build_id": recipe.build_id, "config_sha256": recipe.sha256(), "config": recipe.raw,
             "discovery": _backend_entry(search), "materializer": _backend_entry(materializer),
             "deduplicator": {"type": "sqlite", **recipe.deduplication},
             "tokenizer": {"snapshot": tokenizer_identity or type(tokenizer).__name__, "vocabulary_size": vocab},
             "stats": st, "desired_token_target_reached": st["unique_tokens"] >= recipe.token_target.desired,
             "topic_counts": dict(sorted(cur["topic_counts"].items())), "difficulty_counts": dict(sorted(cur["difficulty_counts"].items())),
             "shards": cur["shards"]}
    _publish_manifest(stage, build)
    store.db.close()
    os.remove(os.path.join(work, "dedup.sqlite"))
    os.replace(stage, final)
    return final


def _backend_entry(backend) -> Dict[str, Any]:
    name = backend.name() if hasattr(backend, "name") else type(backend).__name__
    snap = backend.source_snapshot() if hasattr(backend, "source_snapshot") else None
    return {"backend": name, "snapshot": f"{snap.provider}@{snap.revision}" if snap is not None else None,
            "configuration": backend.configuration() if hasattr(backend, "configuration") else None}


def _publish_manifest(directory: str, build: Dict[str, Any]) -> Dict[str, Any]:
    manifest = {"manifest_sha256": _canonical_sha256(build), "build": build}
    path = os.path.join(directory, "manifest.json")
    with open(path, "wb") as f:
        f.write((json.dumps(manifest, indent=1, sort_keys=True, ensure_ascii=False) + "\n").encode())
        f.flush()
        os.fsync(f.fileno())
    return manifest


# ------------------------------------------------------------------------------------------------ composition
@dataclass
class StageConfig:
    name: str
    when: Predicate
    unmatched: str
    token_target: TokenTarget
    max_tokens_per_shard: int
    max_fraction_deviation: float
    strata: List[Tuple[str, int, Predicate]]


@dataclass
class CompositionConfig:
    build_id: str
    source_manifest: str
    source_manifest_sha256: Optional[str]
    seed: int
    stages: List[StageConfig]
    raw: Dict[str, Any] = field(default_factory=dict)

    @staticmethod
    def decode(v: Any, base: str = ".") -> "CompositionConfig":
        d = _obj(v, "the curriculum composition", ("version", "build_id", "source_manifest", "source_manifest_sha256", "seed", "stages"),
                 ("version", "build_id", "source_manifest", "seed", "stages"))
        _need(d["version"] == CORPUS_SCHEMA_VERSION, f"unsupported curriculum composition version {d['version']}")
        _need(isinstance(d["stages"], list) and d["stages"], "curriculum composition requires at least one stage")
        sha = d.get("source_manifest_sha256")
        _need(sha is None or (isinstance(sha, str) and len(sha) == 64 and all(c in "0123456789abcdef" for c in sha)),
              "source_manifest_sha256 must be 64 lower-case hex digits")
        stages, names = [], set()
        for s in d["stages"]:
            s = _obj(s, "a curriculum stage", ("name", "when", "unmatched", "token_target", "sharding", "max_fraction_deviation", "strata"),
                     ("name", "token_target", "sharding", "strata"))
            name = _component(s["name"], "curriculum stage name")
            _need(name not in names, f"curriculum composition repeats stage `{name}`")
            names.add(name)
            unmatched = s.get("unmatched", "error")
            _need(unmatched in ("error", "exclude"), f"stage `{name}` unmatched policy must be `error` or `exclude`")
            dev = s.get("max_fraction_deviation", 0.0)
            _need(isinstance(dev, (int, float)) and not isinstance(dev, bool) and math.isfinite(dev) and 0.0 <= dev <= 1.0,
                  f"stage `{name}` max_fraction_deviation must be finite and within [0, 1]")
            _need(isinstance(s["strata"], list) and 1 <= len(s["strata"]) <= MAX_STRATA_PER_STAGE, f"stage `{name}` requires 1..={MAX_STRATA_PER_STAGE} strata")
            strata, seen = [], set()
            for st in s["strata"]:
                st = _obj(st, "a curriculum stratum", ("name", "weight", "when"), ("name", "weight"))
                sname = _component(st["name"], "curriculum stratum name")
                _need(sname not in seen, f"stage `{name}` repeats stratum `{sname}`")
                seen.add(sname)
                _need(_uint(st["weight"], "stratum weight") > 0, f"stage `{name}` stratum `{sname}` weight must be positive")
                strata.append((sname, st["weight"], Predicate.decode(st.get("when"), "stratum predicate", True)))
            shard = _obj(s["sharding"], "`sharding`", ("max_tokens_per_shard",), ("max_tokens_per_shard",))
            _need(_uint(shard["max_tokens_per_shard"], "max_tokens_per_shard") > 0, "max_tokens_per_shard must be positive")
            stages.append(StageConfig(name, Predicate.decode(s.get("when"), "stage predicate", True), unmatched,
                                      TokenTarget.decode(s["token_target"], f"stage `{name}` token_target"), shard["max_tokens_per_shard"], float(dev), strata))
        src = d["source_manifest"]
        _need(isinstance(src, str) and src != "", "source_manifest must not be empty")
        return CompositionConfig(_component(d["build_id"], "curriculum build_id"), src if os.path.isabs(src) else os.path.normpath(os.path.join(base, src)),
                                 sha, _uint(d["seed"], "seed"), stages, raw=json.loads(json.dumps(d)))


def compose_curriculum(cfg: CompositionConfig, output_root: str, work_directory: Optional[str] = None) -> str:
    """Writes `<output_root>/<build_id>/<stage>/{shard-*.jsonl, manifest.json}` for every stage plus a root manifest."""
    source, rows = open_corpus_manifest(cfg.source_manifest)
    if cfg.source_manifest_sha256 is not None:
        _need(source["manifest_sha256"] == cfg.source_manifest_sha256, "the source corpus is not the pinned generation")
    final = os.path.join(output_root, cfg.build_id)
    _need(not os.path.exists(final), f"curriculum `{cfg.build_id}` is already published")
    staging = os.path.join(output_root, f".{cfg.build_id}.composing")
    if os.path.exists(staging):
        import shutil
        shutil.rmtree(staging)                                           # composition is cheap to redo from the sealed source
    os.makedirs(staging)
    composition_sha = _canonical_sha256(cfg.raw)
    # One pass over the sealed source spools every row into its (stage, stratum) file, so memory stays bounded by
    # one row whatever the corpus size; the spools are removed with the staging directory's work folder.
    work = work_directory or os.path.join(staging, ".spools")
    os.makedirs(work, exist_ok=True)
    spool_paths = [[os.path.join(work, f"{si:04d}-{qi:04d}.jsonl") for qi in range(len(st.strata))] for si, st in enumerate(cfg.stages)]
    spools = [[open(p, "wb") for p in row] for row in spool_paths]
    available = [[[0, 0] for _ in st.strata] for st in cfg.stages]      # [records, tokens]
    try:
        for row in rows():
            meta = row.get("metadata") or {}
            line = None
            for si, stage in enumerate(cfg.stages):
                if not stage.when.matches(row.get("topic"), row.get("difficulty"), meta, row.get("view")):
                    continue
                for qi, (_, _, pred) in enumerate(stage.strata):
                    if pred.matches(row.get("topic"), row.get("difficulty"), meta, row.get("view")):
                        line = line or json.dumps(row, sort_keys=True, separators=(",", ":"), ensure_ascii=False).encode() + b"\n"
                        spools[si][qi].write(line)
                        available[si][qi][0] += 1
                        available[si][qi][1] += len(row["tokens"])
                        break
                else:
                    _need(stage.unmatched == "exclude", f"stage `{stage.name}` matches record `{row['record_key']}` but no stratum does")
    finally:
        for row_files in spools:
            for f in row_files:
                f.close()
    summaries = []
    for index, stage in enumerate(cfg.stages):
        readers = [open(p, "rb") for p in spool_paths[index]]
        ties = [hashlib.sha256(f"{cfg.seed}\0{index}\0{stage.name}\0{name}".encode()).digest() for name, _, _ in stage.strata]
        emitted_tokens, emitted_records = [0] * len(stage.strata), [0] * len(stage.strata)
        total_tokens = total_records = 0
        topic_counts: Dict[str, int] = {}
        difficulty_counts: Dict[str, int] = {}
        root = os.path.join(staging, stage.name)
        os.makedirs(root)
        writer, shards = _ShardWriter(root, stage.max_tokens_per_shard, 0), []
        from functools import cmp_to_key

        def order(a: int, b: int) -> int:                               # emitted / weight, exactly (cross-multiplied), then the seeded tie-break
            left, right = emitted_tokens[a] * stage.strata[b][1], emitted_tokens[b] * stage.strata[a][1]
            return -1 if left < right else (1 if left > right else (-1 if ties[a] < ties[b] else 1))
        while total_tokens < stage.token_target.desired:
            pick = min(range(len(stage.strata)), key=cmp_to_key(order))
            name = stage.strata[pick][0]
            line = readers[pick].readline()
            _need(bool(line),
                  f"stage `{stage.name}` stratum `{name}` exhausted after {emitted_tokens[pick]} tokens; available={available[index][pick][1]} "
                  f"while stage target={stage.token_target.desired} (adjust weights, predicates, or target)")
            row = json.loads(line)
            n = len(row["tokens"])
            _need(total_tokens + n <= stage.token_target.maximum,
                  f"stage `{stage.name}` cannot reach desired target {stage.token_target.desired} without exceeding maximum "
                  f"{stage.token_target.maximum} (next record has {n} tokens)")
            closed = writer.push(row)
            if closed:
                shards.append(closed)
            emitted_tokens[pick] += n
            emitted_records[pick] += 1
            total_tokens += n
            total_records += 1
            for table, label in ((topic_counts, row.get("topic")), (difficulty_counts, row.get("difficulty"))):
                if label is not None:
                    table[label] = table.get(label, 0) + 1
        closed = writer.close()
        if closed:
            shards.append(closed)
        for f in readers:
            f.close()
        _need(total_tokens >= stage.token_target.minimum, f"stage `{stage.name}` emitted {total_tokens} tokens below minimum {stage.token_target.minimum}")
        weight_sum = sum(w for _, w, _ in stage.strata)
        for (name, w, _), got in zip(stage.strata, emitted_tokens):
            actual, expected = got / total_tokens, w / weight_sum
            _need(abs(actual - expected) <= stage.max_fraction_deviation,
                  f"stage `{stage.name}` stratum `{name}` token fraction {actual:.6f} differs from configured {expected:.6f} by more than "
                  f"{stage.max_fraction_deviation:.6f}")
        config = dict(source["build"]["config"], build_id=stage.name, token_target=stage.token_target.to_json(),
                      sharding={"max_tokens_per_shard": stage.max_tokens_per_shard})
        names = [n for n, _, _ in stage.strata]
        build = {"version": source["build"]["version"], "build_id": stage.name, "config_sha256": _canonical_sha256(config), "config": config,
                 "discovery": source["build"]["discovery"], "materializer": source["build"]["materializer"],
                 "deduplicator": {"type": "stratified_curriculum_composition", "composition_sha256": composition_sha,
                                  "source_manifest_sha256": source["manifest_sha256"], "seed": cfg.seed, "stage": stage.name,
                                  "stratum_records": dict(zip(names, emitted_records)), "stratum_tokens": dict(zip(names, emitted_tokens)),
                                  "available_stratum_records": dict(zip(names, (a[0] for a in available[index]))),
                                  "available_stratum_tokens": dict(zip(names, (a[1] for a in available[index])))},
                 "tokenizer": source["build"]["tokenizer"],
                 "stats": {"unique_records": total_records, "unique_tokens": total_tokens, "emitted_views": total_records, "exposure_tokens": total_tokens},
                 "desired_token_target_reached": True, "topic_counts": dict(sorted(topic_counts.items())),
                 "difficulty_counts": dict(sorted(difficulty_counts.items())), "shards": shards}
        manifest = _publish_manifest(root, build)
        summaries.append({"name": stage.name, "manifest_path": f"{stage.name}/manifest.json", "manifest_sha256": manifest["manifest_sha256"],
                          "records": total_records, "tokens": total_tokens, "stratum_records": dict(zip(names, emitted_records)),
                          "stratum_tokens": dict(zip(names, emitted_tokens))})
    body = {"version": CORPUS_SCHEMA_VERSION, "build_id": cfg.build_id, "composition_sha256": composition_sha,
            "source_manifest_sha256": source["manifest_sha256"], "seed": cfg.seed, "stages": summaries}
    for row_paths in spool_paths:
        for sp in row_paths:
            os.remove(sp)
    if work_directory is None:
        os.rmdir(work)
    with open(os.path.join(staging, "manifest.json"), "wb") as f:
        f.write((json.dumps({"manifest_sha256": _canonical_sha256(body), "build": body}, indent=1, sort_keys=True) + "\n").encode())
        f.flush()
        os.fsync(f.fileno())
    os.replace(staging, final)
    return final
