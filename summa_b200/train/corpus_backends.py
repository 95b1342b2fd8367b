"""Remote backends of the corpus pipeline behind narrow, fake-able interfaces.

`SearchApiClient` discovers record keys through a JSON search API whose request and response shapes are pure
configuration (JSON pointers), `PostgresRecordMaterializer` turns keys into authoritative text through a
statement executor. Both mirror the reference's contracts (`summa-train/src/corpus/search.rs:72-135,244-460,
603-845`, `corpus/materialize.rs:20-38,74-96,204-250,525-620`):

  * the request is the configured template with query / offset / limit / snapshot revision / named parameters
    written at their pointers, every configured reranker switch forced to `false`, the fusion marker and both
    vector fields rewritten, and both fusion clauses checked to be present AFTER all substitutions;
  * every response must prove the pinned source snapshot (provider and revision echoed at configured pointers)
    before any of its content is accepted; hits need a scalar, non-empty record key and a finite score;
  * the HTTP transport bounds the response body BEFORE parsing, retries with capped exponential back-off and
    resolves its secret from an environment variable at construction (the secret never enters a manifest);
  * the materializer rejects unrequested and duplicate rows and, by default, requires every requested record.

Both classes also satisfy the small interfaces `train/corpus.py::CorpusPipeline` consumes
(`snapshot()`, `discover(query, offset, limit) -> (keys, total)`; `fetch(keys) -> {key: text}`)."""
from __future__ import annotations

import copy
import json
import math
import os
import time
import urllib.error
import urllib.request
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

from .corpus import CorpusError

MAX_SEARCH_RESPONSE_BYTES = 256 * 1024 * 1024
MAX_SEARCH_RETRY_DELAY_MS = 300_000


# ---------------------------------------------------------------------------------------------- JSON pointers
def _tokens(pointer: str) -> List[str]:
    if pointer == "":
        return []
    if not pointer.startswith("/"):
        raise CorpusError(f"JSON pointer `{pointer}` must be empty or start with `/`")
    return [t.replace("~1", "/").replace("~0", "~") for t in pointer[1:].split("/")]


_MISSING = object()
_ABSENT = object()


def pointer_get(value: Any, pointer: str, default: Any = _MISSING) -> Any:
    cur = value
    for t in _tokens(pointer):
        if isinstance(cur, dict) and t in cur:
            cur = cur[t]
        elif isinstance(cur, list) and t.isdigit() and int(t) < len(cur):
            cur = cur[int(t)]
        else:
            if default is _MISSING:
                raise CorpusError(f"JSON pointer `{pointer}` does not exist")
            return default
    return cur


def pointer_set(root: Any, pointer: str, value: Any) -> None:
    toks = _tokens(pointer)
    if not toks:
        raise CorpusError("the empty JSON pointer cannot be written")
    parent = pointer_get(root, "/" + "/".join(t.replace("~", "~0").replace("/", "~1") for t in toks[:-1]) if len(toks) > 1 else "")
    last = toks[-1]
    if isinstance(parent, dict) and last in parent:
        parent[last] = value
    elif isinstance(parent, list) and last.isdigit() and int(last) < len(parent):
        parent[int(last)] = value
    else:
        raise CorpusError(f"JSON pointer `{pointer}` does not exist in the request")


def _scalar_string(v: Any) -> Optional[str]:
    if isinstance(v, bool) or v is None:
        return None
    if isinstance(v, str):
        return v
    if isinstance(v, (int, float)):
        return str(v)
    return None


# ---------------------------------------------------------------------------------------------- records
@dataclass
class SourceSnapshot:
    provider: str
    revision: str

    def validate(self) -> None:
        if not self.provider.strip() or not self.revision.strip():
            raise CorpusError("source snapshot provider and revision must not be empty")


@dataclass
class DiscoveryHit:
    record_key: str
    score: float = 0.0
    uris: List[str] = field(default_factory=list)
    metadata: Dict[str, Any] = field(default_factory=dict)
    inline_text: Optional[str] = None


@dataclass
class DiscoveryPage:
    hits: List[DiscoveryHit]
    total_hits: Optional[int]
    snapshot: SourceSnapshot


@dataclass
class MaterializedRecord:
    record_key: str
    text: str
    uris: List[str]
    metadata: Dict[str, Any]


# ---------------------------------------------------------------------------------------------- search API
_SEARCH_KEYS = {"endpoint", "request_template", "request_mapping", "response_mapping", "fusion", "snapshot", "page_size",
                "timeout_seconds", "max_retries", "retry_initial_ms", "retry_max_ms", "max_response_bytes", "auth"}
_REQ_KEYS = {"query_pointer", "offset_pointer", "limit_pointer", "parameter_pointers", "disabled_reranker_pointers",
             "return_documents_pointer"}
_RESP_KEYS = {"hits_pointer", "total_hits_pointer", "record_key_pointer", "score_pointer", "uris_pointer",
              "inline_text_pointer", "metadata_pointers"}
_SNAP_KEYS = {"provider", "revision", "request_revision_pointer", "response_provider_pointer", "response_revision_pointer"}
_FUSION_KEYS = {"marker_pointer", "marker_value", "sparse", "dense"}
_BRANCH_KEYS = {"clause_pointer", "vector_field_pointer", "vector_field"}
_AUTH_KEYS = {"header", "environment", "prefix"}


def _strict(d: Any, allowed: set, required: Sequence[str], what: str) -> Dict[str, Any]:
    if not isinstance(d, dict):
        raise CorpusError(f"{what} must be an object")
    unknown = set(d) - allowed
    if unknown:
        raise CorpusError(f"{what}: unknown field(s) {sorted(unknown)}")
    for k in required:
        if k not in d:
            raise CorpusError(f"{what}: missing field `{k}`")
    return d


def validate_search_api_config(cfg: Dict[str, Any]) -> Dict[str, Any]:
    """Checks a `search_api` configuration object the way the reference's typed decoder and `validate` do;
    returns it with the defaults filled in."""
    c = dict(_strict(cfg, _SEARCH_KEYS, ["endpoint", "request_template", "request_mapping", "response_mapping", "fusion",
                                         "snapshot", "page_size"], "search_api"))
    c.setdefault("timeout_seconds", 180)
    c.setdefault("max_retries", 3)
    c.setdefault("retry_initial_ms", 1000)
    c.setdefault("retry_max_ms", 30000)
    c.setdefault("max_response_bytes", 64 * 1024 * 1024)
    c.setdefault("auth", None)
    if not str(c["endpoint"]).startswith(("https://", "http://")):
        raise CorpusError("search_api endpoint must be an http(s) URL")
    if not isinstance(c["page_size"], int) or c["page_size"] <= 0:
        raise CorpusError("search_api page_size must be positive")
    if not (0 < c["max_response_bytes"] <= MAX_SEARCH_RESPONSE_BYTES):
        raise CorpusError("search_api max_response_bytes is out of range")
    if not (0 < c["retry_initial_ms"] <= c["retry_max_ms"] <= MAX_SEARCH_RETRY_DELAY_MS):
        raise CorpusError("search_api retry delays are out of range")
    tpl = c["request_template"]
    rm = _strict(c["request_mapping"], _REQ_KEYS, ["query_pointer", "offset_pointer", "limit_pointer",
                                                   "disabled_reranker_pointers"], "search_api request_mapping")
    for name in ("query_pointer", "offset_pointer", "limit_pointer"):
        pointer_get(tpl, rm[name])
    if not rm["disabled_reranker_pointers"]:
        raise CorpusError("search_api must configure at least one disabled reranker pointer")
    for p in rm["disabled_reranker_pointers"]:
        pointer_get(tpl, p)
    if rm.get("return_documents_pointer") is not None:
        pointer_get(tpl, rm["return_documents_pointer"])
    for name, p in (rm.get("parameter_pointers") or {}).items():
        if not name.strip():
            raise CorpusError("search_api parameter names must not be empty")
        pointer_get(tpl, p)
    resp = _strict(c["response_mapping"], _RESP_KEYS, ["hits_pointer", "record_key_pointer"], "search_api response_mapping")
    for k in ("hits_pointer", "total_hits_pointer", "record_key_pointer", "score_pointer", "uris_pointer", "inline_text_pointer"):
        if resp.get(k) is not None:
            _tokens(resp[k])
    snap = _strict(c["snapshot"], _SNAP_KEYS, list(_SNAP_KEYS), "search_api snapshot")
    SourceSnapshot(snap["provider"], snap["revision"]).validate()
    pointer_get(tpl, snap["request_revision_pointer"])
    if snap["response_provider_pointer"] == snap["response_revision_pointer"]:
        raise CorpusError("search_api snapshot provider and revision response pointers must be distinct")
    fus = _strict(c["fusion"], _FUSION_KEYS, list(_FUSION_KEYS), "search_api fusion")
    if pointer_get(tpl, fus["marker_pointer"]) != fus["marker_value"]:
        raise CorpusError("search_api fusion marker does not match request_template")
    for name in ("sparse", "dense"):
        br = _strict(fus[name], _BRANCH_KEYS, list(_BRANCH_KEYS), f"search_api fusion {name}")
        if pointer_get(tpl, br["clause_pointer"]) is None:
            raise CorpusError(f"search_api {name} fusion clause must not be null")
        pointer_get(tpl, br["vector_field_pointer"])
        if not br["vector_field_pointer"].startswith(br["clause_pointer"].rstrip("/") + "/"):
            raise CorpusError(f"search_api {name} vector-field pointer must be inside its fusion clause")
        if not str(br["vector_field"]).strip():
            raise CorpusError(f"search_api {name} vector field must not be empty")
    if fus["sparse"]["clause_pointer"] == fus["dense"]["clause_pointer"] or \
            fus["sparse"]["vector_field_pointer"] == fus["dense"]["vector_field_pointer"]:
        raise CorpusError("search_api sparse and dense fusion branches must be distinct")
    if c["auth"] is not None:
        _strict(c["auth"], _AUTH_KEYS, ["header", "environment"], "search_api auth")
    return c


class UrllibSearchApiTransport:
    """Blocking HTTP transport: POSTs JSON, bounds the response body before parsing, retries 5xx / transport errors
    with capped exponential back-off. The authentication secret is read from the configured environment variable
    here, once; it is never part of a configuration or a manifest."""

    def __init__(self, config: Dict[str, Any], opener: Optional[Callable] = None, sleep: Callable[[float], None] = time.sleep):
        self.timeout = config["timeout_seconds"]
        self.max_retries, self.delay0, self.delay_max = config["max_retries"], config["retry_initial_ms"], config["retry_max_ms"]
        self.max_bytes = config["max_response_bytes"]
        self.auth = None
        if config.get("auth"):
            secret = os.environ.get(config["auth"]["environment"])
            if secret is None:
                raise CorpusError(f"search_api authentication environment variable `{config['auth']['environment']}` is not set")
            self.auth = (config["auth"]["header"], config["auth"].get("prefix", "") + secret)
        self._open = opener or urllib.request.urlopen
        self._sleep = sleep

    def post_json(self, endpoint: str, body: Any) -> Any:
        data = json.dumps(body).encode()
        delay = self.delay0
        last = None
        for attempt in range(self.max_retries + 1):
            req = urllib.request.Request(endpoint, data=data, method="POST", headers={"content-type": "application/json"})
            if self.auth:
                req.add_header(*self.auth)
            try:
                with self._open(req, timeout=self.timeout) as resp:
                    raw = resp.read(self.max_bytes + 1)
                if len(raw) > self.max_bytes:
                    raise CorpusError(f"search_api response exceeds {self.max_bytes} bytes")
                return json.loads(raw)
            except urllib.error.HTTPError as e:
                if e.code < 500 and e.code != 429:
                    raise CorpusError(f"search_api request failed with HTTP {e.code}") from None
                last = e
            except (urllib.error.URLError, TimeoutError, ConnectionError) as e:
                last = e
            if attempt < self.max_retries:
                self._sleep(delay / 1000.0)
                delay = min(delay * 2, self.delay_max)
        raise CorpusError(f"search_api request failed after {self.max_retries + 1} attempts: {last}")


class SearchApiClient:
    def __init__(self, config: Dict[str, Any], transport=None):
        self.config = validate_search_api_config(config)
        self.transport = transport if transport is not None else UrllibSearchApiTransport(self.config)

    # ---- backend interface
    def name(self) -> str:
        return "search_api"

    def configuration(self) -> Dict[str, Any]:
        """Secret-free configuration for the build manifest (the auth block only names the environment variable)."""
        return copy.deepcopy(self.config)

    def source_snapshot(self) -> SourceSnapshot:
        s = self.config["snapshot"]
        return SourceSnapshot(s["provider"], s["revision"])

    def snapshot(self) -> str:
        s = self.source_snapshot()
        return f"{s.provider}@{s.revision}"

    def page_size(self) -> int:
        return self.config["page_size"]

    def request_for(self, query: str, offset: int, limit: int, parameters: Optional[Dict[str, Any]] = None,
                    query_name: str = "") -> Any:
        c = self.config
        if limit <= 0:
            raise CorpusError("search_api request limit must be positive")
        if limit > c["page_size"]:
            raise CorpusError(f"search_api request limit {limit} exceeds configured page_size {c['page_size']}")
        req = copy.deepcopy(c["request_template"])
        rm, fus = c["request_mapping"], c["fusion"]
        pointer_set(req, rm["query_pointer"], query)
        pointer_set(req, rm["offset_pointer"], int(offset))
        pointer_set(req, rm["limit_pointer"], int(limit))
        pointer_set(req, c["snapshot"]["request_revision_pointer"], c["snapshot"]["revision"])
        for name, value in (parameters or {}).items():
            ptr = (rm.get("parameter_pointers") or {}).get(name)
            if ptr is None:
                raise CorpusError(f"query `{query_name or query}` uses unmapped search_api parameter `{name}`")
            pointer_set(req, ptr, value)
        for ptr in rm["disabled_reranker_pointers"]:
            pointer_set(req, ptr, False)
        if rm.get("return_documents_pointer") is not None:
            pointer_set(req, rm["return_documents_pointer"], False)
        pointer_set(req, fus["marker_pointer"], fus["marker_value"])
        pointer_set(req, fus["sparse"]["vector_field_pointer"], fus["sparse"]["vector_field"])
        pointer_set(req, fus["dense"]["vector_field_pointer"], fus["dense"]["vector_field"])
        # after every substitution: a query parameter must not have replaced or removed either clause
        for name in ("sparse", "dense"):
            if pointer_get(req, fus[name]["clause_pointer"], None) is None:
                raise CorpusError(f"search_api {name} fusion clause `{fus[name]['clause_pointer']}` is absent from request")
        return req

    def parse_response(self, response: Any) -> DiscoveryPage:
        c, m = self.config, self.config["response_mapping"]
        prov = _scalar_string(pointer_get(response, c["snapshot"]["response_provider_pointer"], None))
        rev = _scalar_string(pointer_get(response, c["snapshot"]["response_revision_pointer"], None))
        if prov is None or rev is None:
            raise CorpusError("search_api response has no scalar snapshot proof")
        want = self.source_snapshot()
        if (prov, rev) != (want.provider, want.revision):
            raise CorpusError(f"search_api response snapshot mismatch: expected {want.provider}@{want.revision}, got {prov}@{rev}")
        raw_hits = pointer_get(response, m["hits_pointer"], None)
        if not isinstance(raw_hits, list):
            raise CorpusError(f"search_api response `{m['hits_pointer']}` is absent or not an array")
        hits = []
        for i, raw in enumerate(raw_hits):
            key = _scalar_string(pointer_get(raw, m["record_key_pointer"], None))
            if not key:
                raise CorpusError(f"search_api hit {i} has no scalar, non-empty record key")
            score = 0.0
            if m.get("score_pointer") is not None:
                sv = pointer_get(raw, m["score_pointer"], None)
                if isinstance(sv, bool) or not isinstance(sv, (int, float)) or not math.isfinite(float(sv)):
                    raise CorpusError(f"search_api hit {i} score `{m['score_pointer']}` must be a finite number")
                score = float(sv)
            uris: List[str] = []
            if m.get("uris_pointer") is not None:
                uv = pointer_get(raw, m["uris_pointer"], None)
                if isinstance(uv, str):
                    uris = [uv]
                elif isinstance(uv, list) and all(isinstance(u, str) for u in uv):
                    uris = list(uv)
                elif uv is not None:
                    raise CorpusError(f"search_api hit {i} uris must be a string or an array of strings")
            inline = None
            if m.get("inline_text_pointer") is not None:
                iv = pointer_get(raw, m["inline_text_pointer"], None)
                if iv is not None and not isinstance(iv, str):
                    raise CorpusError(f"search_api hit {i} inline text must be a string")
                inline = iv
            meta = {}
            for name, ptr in (m.get("metadata_pointers") or {}).items():
                mv = pointer_get(raw, ptr, _ABSENT)
                if mv is not _ABSENT:
                    meta[name] = mv
            hits.append(DiscoveryHit(key, score, uris, meta, inline))
        total = None
        if m.get("total_hits_pointer") is not None:
            total = pointer_get(response, m["total_hits_pointer"], None)
            if isinstance(total, bool) or not isinstance(total, int) or total < 0:
                raise CorpusError(f"search_api total_hits `{m['total_hits_pointer']}` must be a non-negative integer")
        return DiscoveryPage(hits, total, SourceSnapshot(prov, rev))

    def discover_page(self, query: str, offset: int, limit: int, parameters: Optional[Dict[str, Any]] = None) -> DiscoveryPage:
        return self.parse_response(self.transport.post_json(self.config["endpoint"], self.request_for(query, offset, limit, parameters)))

    def discover(self, query: str, offset: int, limit: int) -> Tuple[List[str], int]:
        page = self.discover_page(query, offset, limit)
        total = page.total_hits if page.total_hits is not None else offset + len(page.hits) + (1 if len(page.hits) == limit else 0)
        return [h.record_key for h in page.hits], total


# ---------------------------------------------------------------------------------------------- Postgres materializer
_PG_KEYS = {"connection_environment", "statement", "columns", "snapshot_statement", "transport_security", "require_every_record"}
_COL_KEYS = {"record_key", "text", "uris", "metadata"}


class PostgresRecordMaterializer:
    """Authoritative text by record key through a statement executor:
    `executor.snapshot_revision() -> str`, `executor.fetch(statement, columns, keys) -> rows` with rows as
    `{"record_key", "text", "uris": [...], "metadata": {...}}`. A live executor (a read-only repeatable-read
    transaction over a verified-TLS connection whose DSN comes from `connection_environment`) needs a database
    driver that this image does not ship; tests and offline builds pass their own executor."""

    def __init__(self, config: Dict[str, Any], executor):
        c = dict(_strict(config, _PG_KEYS, ["connection_environment", "statement", "columns", "snapshot_statement",
                                            "transport_security"], "postgres materializer"))
        cols = _strict(c["columns"], _COL_KEYS, ["record_key", "text"], "postgres columns")
        if not str(cols["record_key"]).strip() or not str(cols["text"]).strip():
            raise CorpusError("postgres record_key and text column mappings must not be empty")
        for k in ("uris", "metadata"):
            if cols.get(k) is not None and not str(cols[k]).strip():
                raise CorpusError("optional postgres column mappings must not be empty")
        if not str(c["statement"]).strip() or not str(c["snapshot_statement"]).strip():
            raise CorpusError("postgres statements must not be empty")
        c.setdefault("require_every_record", True)
        self.config, self.executor = c, executor

    def name(self) -> str:
        return "postgres"

    def configuration(self) -> Dict[str, Any]:
        return copy.deepcopy(self.config)          # names the environment variable, never its value

    def source_snapshot(self) -> SourceSnapshot:
        return SourceSnapshot("postgres", self.executor.snapshot_revision())

    def materialize(self, hits: Sequence[DiscoveryHit]) -> List[MaterializedRecord]:
        keys = [h.record_key for h in hits]
        by_key = {h.record_key: h for h in hits}
        rows = self.executor.fetch(self.config["statement"], self.config["columns"], keys)
        found, out = set(), []
        for row in rows:
            k = row["record_key"]
            if k not in by_key:
                raise CorpusError(f"postgres returned unrequested record key `{k}`")
            if k in found:
                raise CorpusError(f"postgres returned duplicate record key `{k}`")
            found.add(k)
            hit = by_key[k]
            meta = dict(hit.metadata)
            meta.update(row.get("metadata") or {})
            out.append(MaterializedRecord(k, row["text"], list(row.get("uris") or hit.uris), meta))
        if self.config["require_every_record"] and len(found) != len(by_key):
            raise CorpusError(f"postgres materialized {len(found)} of {len(by_key)} requested records")
        return out

    def fetch(self, keys: Sequence[str]) -> Dict[str, str]:
        return {r.record_key: r.text for r in self.materialize([DiscoveryHit(k) for k in keys])}


class InlineRecordMaterializer:
    """For discovery engines that are themselves the canonical text store: fails when a hit has no inline text."""

    def name(self) -> str:
        return "inline"

    def materialize(self, hits: Sequence[DiscoveryHit]) -> List[MaterializedRecord]:
        out = []
        for h in hits:
            if h.inline_text is None:
                raise CorpusError(f"discovery hit `{h.record_key}` has no inline text")
            out.append(MaterializedRecord(h.record_key, h.inline_text, list(h.uris), dict(h.metadata)))
        return out


# ---------------------------------------------------------------------------------------------- live Postgres executor
def postgres_connection_plan(config: Dict[str, Any], env: Optional[Dict[str, str]] = None) -> Dict[str, Any]:
    """Checks the `transport_security` block against the DSN in `connection_environment` and returns what a driver
    needs: `{dsn, sslmode, root_pem}`. Rules of `summa-train/src/corpus/materialize.rs:140-420`: `verified_tls` wants
    the DSN's hosts to equal `server_names` exactly (no Unix socket) and trusts either the system roots or exactly the
    PEM in `certificate_pem_environment`, whose bytes must hash to `certificate_sha256`; `plaintext_local_proxy`
    wants `acknowledge_plaintext: true` and numeric loopback hosts (or a Unix socket) only."""
    import hashlib
    import ipaddress
    import urllib.parse
    env = os.environ if env is None else env
    dsn = env.get(config["connection_environment"])
    if not dsn:
        raise CorpusError(f"postgres connection environment variable `{config['connection_environment']}` is not set")
    ts = config["transport_security"]
    if dsn.startswith(("postgres://", "postgresql://")):
        u = urllib.parse.urlsplit(dsn)
        netloc = u.netloc.rsplit("@", 1)[-1]
        hosts = [h.rsplit(":", 1)[0] if not h.startswith("[") else h[1:h.index("]")] for h in netloc.split(",") if h]
        hosts += urllib.parse.parse_qs(u.query).get("host", [])
    else:
        fields = dict(part.split("=", 1) for part in dsn.split() if "=" in part)
        hosts = [h for h in fields.get("host", "").split(",") if h]
    mode = ts.get("mode")
    if mode == "verified_tls":
        _strict(ts, {"mode", "server_names", "trust"}, ["server_names", "trust"], "postgres transport_security")
        names = ts["server_names"]
        if not isinstance(names, list) or not names or any((not isinstance(n, str)) or n != n.strip() or not n or
                                                           any(c in n for c in "*/\0") for n in names):
            raise CorpusError("postgres verified TLS server names must be exact DNS names or IP addresses")
        if any(h.startswith("/") for h in hosts):
            raise CorpusError("postgres verified TLS cannot use a Unix socket; select plaintext_local_proxy for a trusted local socket")
        if hosts != names:
            raise CorpusError("postgres DSN hosts must exactly match verified TLS server_names")
        trust, pem = ts["trust"], None
        if trust.get("source") == "pinned_pem":
            _strict(trust, {"source", "certificate_pem_environment", "certificate_sha256"},
                    ["certificate_pem_environment", "certificate_sha256"], "postgres TLS trust")
            pem = env.get(trust["certificate_pem_environment"])
            if pem is None:
                raise CorpusError(f"postgres TLS certificate environment variable `{trust['certificate_pem_environment']}` is not set")
            if "sha256:" + hashlib.sha256(pem.encode()).hexdigest() != trust["certificate_sha256"]:
                raise CorpusError("postgres TLS certificate digest does not match certificate_sha256")
            if "-----BEGIN CERTIFICATE-----" not in pem:
                raise CorpusError("postgres TLS certificate PEM must contain at least one certificate")
        elif trust.get("source") != "system":
            raise CorpusError("postgres TLS trust source must be `system` or `pinned_pem`")
        return {"dsn": dsn, "sslmode": "verify-full", "root_pem": pem}
    if mode == "plaintext_local_proxy":
        _strict(ts, {"mode", "acknowledge_plaintext"}, ["acknowledge_plaintext"], "postgres transport_security")
        if ts["acknowledge_plaintext"] is not True:
            raise CorpusError("postgres plaintext local-proxy mode requires acknowledge_plaintext=true")
        if not hosts:
            raise CorpusError("postgres plaintext local-proxy mode requires an explicit loopback IP or Unix socket host")
        for h in hosts:
            if h.startswith("/"):
                continue
            try:
                loop = ipaddress.ip_address(h).is_loopback
            except ValueError:
                raise CorpusError(f"postgres plaintext local-proxy host `{h}` must be a numeric loopback address")
            if not loop:
                raise CorpusError(f"postgres plaintext local-proxy host `{h}` is not loopback")
        return {"dsn": dsn, "sslmode": "disable", "root_pem": None}
    raise CorpusError("postgres transport_security mode must be `verified_tls` or `plaintext_local_proxy`")


class DbApiPostgresExecutor:
    """Statement executor over a DB-API connection (psycopg's `%s` parameter style): one read-only repeatable-read
    transaction for the whole build, so the snapshot revision and every fetched row belong to one database state."""

    def __init__(self, connection):
        self.connection = connection
        cur = connection.cursor()
        cur.execute("BEGIN TRANSACTION ISOLATION LEVEL REPEATABLE READ READ ONLY")
        self._revision: Optional[str] = None
        self._snapshot_statement: Optional[str] = None

    def bind(self, config: Dict[str, Any]) -> "DbApiPostgresExecutor":
        self._snapshot_statement = config["snapshot_statement"]
        return self

    def snapshot_revision(self) -> str:
        if self._revision is None:
            cur = self.connection.cursor()
            cur.execute(self._snapshot_statement)
            rows = cur.fetchall()
            if len(rows) != 1 or len(rows[0]) != 1 or rows[0][0] is None or not str(rows[0][0]).strip():
                raise CorpusError("postgres snapshot_statement must return exactly one non-empty value")
            self._revision = str(rows[0][0])
        return self._revision

    def fetch(self, statement: str, columns: Dict[str, Any], keys: Sequence[str]) -> List[Dict[str, Any]]:
        cur = self.connection.cursor()
        cur.execute(statement.replace("%", "%%").replace("$1", "%s"), (list(keys),))
        names = [d[0] for d in cur.description]
        for role in ("record_key", "text", "uris", "metadata"):
            if columns.get(role) is not None and columns[role] not in names:
                raise CorpusError(f"postgres statement returns no column `{columns[role]}`")
        at = {role: names.index(columns[role]) for role in ("record_key", "text", "uris", "metadata") if columns.get(role) is not None}
        out = []
        for row in cur.fetchall():
            key, text = row[at["record_key"]], row[at["text"]]
            if not isinstance(key, str) or not key or not isinstance(text, str):
                raise CorpusError("postgres rows need a non-empty string key and a string text")
            uris = row[at["uris"]] if "uris" in at else None
            meta = row[at["metadata"]] if "metadata" in at else None
            uris = json.loads(uris) if isinstance(uris, str) else uris
            meta = json.loads(meta) if isinstance(meta, str) else meta
            if uris is not None and not (isinstance(uris, list) and all(isinstance(u, str) for u in uris)):
                raise CorpusError(f"postgres uris of `{key}` must be an array of strings")
            if meta is not None and not isinstance(meta, dict):
                raise CorpusError(f"postgres metadata of `{key}` must be an object")
            out.append({"record_key": key, "text": text, "uris": uris or [], "metadata": meta or {}})
        return out


def connect_postgres(config: Dict[str, Any], env: Optional[Dict[str, str]] = None) -> DbApiPostgresExecutor:
    """Opens the database named by the configuration with whichever PostgreSQL driver is importable."""
    import tempfile
    plan = postgres_connection_plan(config, env)
    try:
        import psycopg as driver                                       # type: ignore
    except ImportError:
        try:
            import psycopg2 as driver                                  # type: ignore
        except ImportError:
            raise CorpusError("no PostgreSQL driver (psycopg or psycopg2) is importable; pass an executor of your own")
    extra = {"sslmode": plan["sslmode"]}
    if plan["root_pem"] is not None:
        f = tempfile.NamedTemporaryFile("w", suffix=".pem", delete=False)
        f.write(plan["root_pem"])
        f.close()
        extra["sslrootcert"] = f.name
    return DbApiPostgresExecutor(driver.connect(plan["dsn"], **extra)).bind(config)
