"""Corpus preparation: discovery -> materialisation -> normalisation -> dedup -> tokenisation ->
immutable token shards + manifest, resumable at every page, plus deterministic curriculum
composition (`summa-train/src/corpus/pipeline.rs:31-303,1358-1620`, `compose.rs:1-9`).

The pipeline is written against four small interfaces so that the search API and the database
of the reference deployment can be stubbed or replaced:

    SearchBackend       discover(query, offset, limit) -> (stable record keys, total hits);
                        snapshot() pins what was searched
    RecordMaterializer  fetch(keys) -> authoritative text by key
    Deduplicator        seen(content hash) / add(...) ; the SQLite one also stores the cursor
    tokenizer           anything with encode(text) -> ids

A build is identified by the hash of (config, source snapshot, tokenizer snapshot). It is
staged in `.<build_id>.building`, every page commits its dedup entries together with a
content-hashed cursor after the shard bytes are synced, and the directory is renamed into place
only when complete. `open_corpus` authenticates a published directory (manifest hash, shard
hashes) and yields documents for the trainer's packer.
"""
from __future__ import annotations

import hashlib
import json
import os
import sqlite3
import struct
import unicodedata
from dataclasses import asdict, dataclass, field
from typing import Callable, Dict, Iterable, Iterator, List, Optional, Sequence, Tuple

SHARD_MAGIC = b"HERTOK01"
MANIFEST_VERSION = 1


class CorpusError(RuntimeError):
    pass


def _sha(b: bytes) -> str:
    return hashlib.sha256(b).hexdigest()


def normalise_text(text: str) -> str:
    """NFC, unified newlines, control characters dropped, trailing whitespace trimmed per line."""
    text = unicodedata.normalize("NFC", text.replace("\r\n", "\n").replace("\r", "\n"))
    lines = ["".join(ch for ch in ln if ch == "\t" or unicodedata.category(ch)[0] != "C").rstrip()
             for ln in text.split("\n")]
    return "\n".join(lines).strip("\n")


# ---------------------------------------------------------------------------- interfaces
class ListSearchBackend:
    """In-memory stand-in for the search API: `queries[q]` is an ordered list of record keys."""

    def __init__(self, queries: Dict[str, List[str]]):
        self.queries = queries

    def snapshot(self) -> str:
        return _sha(json.dumps(self.queries, sort_keys=True).encode())

    def discover(self, query: str, offset: int, limit: int) -> Tuple[List[str], int]:
        keys = self.queries[query]
        return keys[offset:offset + limit], len(keys)


class DictMaterializer:
    def __init__(self, records: Dict[str, str]):
        self.records = records

    def fetch(self, keys: Sequence[str]) -> Dict[str, str]:
        return {k: self.records[k] for k in keys if k in self.records}


class InMemoryDeduplicator:
    def __init__(self):
        self.hashes = set()
        self.cursor: Optional[dict] = None

    def seen(self, h: str) -> bool:
        return h in self.hashes

    def commit(self, new_hashes: Sequence[str], cursor: dict) -> None:
        self.hashes.update(new_hashes)
        self.cursor = dict(cursor)

    def load_cursor(self) -> Optional[dict]:
        return self.cursor


class SqliteDeduplicator:
    """Content hashes and the resume cursor in one SQLite file: a page's hashes and its cursor
    commit in ONE transaction, so a crash can never record progress without its dedup state."""

    def __init__(self, path: str):
        self.db = sqlite3.connect(path)
        self.db.execute("CREATE TABLE IF NOT EXISTS seen (h TEXT PRIMARY KEY)")
        self.db.execute("CREATE TABLE IF NOT EXISTS cursor (id INTEGER PRIMARY KEY CHECK (id = 0), body TEXT)")
        self.db.commit()

    def seen(self, h: str) -> bool:
        return self.db.execute("SELECT 1 FROM seen WHERE h = ?", (h,)).fetchone() is not None

    def commit(self, new_hashes: Sequence[str], cursor: dict) -> None:
        with self.db:
            self.db.executemany("INSERT OR IGNORE INTO seen (h) VALUES (?)", [(h,) for h in new_hashes])
            self.db.execute("INSERT INTO cursor (id, body) VALUES (0, ?) ON CONFLICT(id) DO UPDATE SET body = excluded.body",
                            (json.dumps(cursor, sort_keys=True),))

    def load_cursor(self) -> Optional[dict]:
        row = self.db.execute("SELECT body FROM cursor WHERE id = 0").fetchone()
        return json.loads(row[0]) if row else None


# ---------------------------------------------------------------------------- shards
def write_shard(path: str, docs: Sequence[Sequence[int]]) -> dict:
    """`HERTOK01`, u64 doc count, then per doc u32 length + u32 little-endian ids. Returns its manifest entry."""
    body = bytearray(SHARD_MAGIC) + struct.pack("<Q", len(docs))
    tokens = 0
    for d in docs:
        body += struct.pack("<I", len(d)) + struct.pack(f"<{len(d)}I", *d)
        tokens += len(d)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(body)
        f.flush()
        os.fsync(f.fileno())
    os.replace(tmp, path)
    return {"file": os.path.basename(path), "sha256": _sha(bytes(body)), "documents": len(docs), "tokens": tokens}


def read_shard(path: str, expect_sha: Optional[str] = None) -> Iterator[List[int]]:
    with open(path, "rb") as f:
        body = f.read()
    if expect_sha is not None and _sha(body) != expect_sha:
        raise CorpusError(f"shard {os.path.basename(path)} does not match its manifest hash")
    if body[:8] != SHARD_MAGIC:
        raise CorpusError("not a token shard")
    (n,) = struct.unpack_from("<Q", body, 8)
    off = 16
    for _ in range(n):
        (ln,) = struct.unpack_from("<I", body, off)
        off += 4
        yield list(struct.unpack_from(f"<{ln}I", body, off))
        off += 4 * ln


# ---------------------------------------------------------------------------- pipeline
@dataclass
class CorpusConfig:
    name: str
    queries: List[str]
    page_size: int = 64
    docs_per_shard: int = 256
    min_chars: int = 1
    metadata: Dict[str, str] = field(default_factory=dict)


class CorpusPipeline:
    def __init__(self, cfg: CorpusConfig, search, materializer, tokenizer, dedup_factory: Callable[[str], object],
                 classify: Optional[Callable[[str, str], Dict[str, str]]] = None):
        if cfg.page_size <= 0 or cfg.docs_per_shard <= 0:
            raise CorpusError("page_size and docs_per_shard must be positive")
        self.cfg, self.search, self.mat, self.tok = cfg, search, materializer, tokenizer
        self.dedup_factory = dedup_factory
        self.classify = classify or (lambda key, text: {})

    def build_id(self) -> str:
        tok_snap = getattr(self.tok, "snapshot", lambda: type(self.tok).__name__)()
        return _sha(json.dumps({"config": asdict(self.cfg), "source": self.search.snapshot(), "tokenizer": tok_snap},
                               sort_keys=True).encode())[:24]

    def run(self, output_root: str, max_pages: Optional[int] = None) -> Optional[str]:
        """Builds (or resumes) the corpus. Returns the published directory, or None when
        `max_pages` stopped the build early (resume by calling again)."""
        bid = self.build_id()
        final = os.path.join(output_root, bid)
        if os.path.exists(os.path.join(final, "manifest.json")):
            return final
        stage = os.path.join(output_root, f".{bid}.building")
        os.makedirs(stage, exist_ok=True)
        dedup = self.dedup_factory(os.path.join(stage, "dedup.sqlite"))
        cur = dedup.load_cursor() or {"query_index": 0, "offset": 0, "shards": [], "pending": [], "stats": {
            "discovered": 0, "materialised": 0, "duplicates": 0, "too_short": 0, "kept": 0}}
        pages = 0
        while cur["query_index"] < len(self.cfg.queries):
            if max_pages is not None and pages >= max_pages:
                return None
            q = self.cfg.queries[cur["query_index"]]
            keys, total = self.search.discover(q, cur["offset"], self.cfg.page_size)
            if cur["offset"] + len(keys) > total or (not keys and cur["offset"] < total):
                raise CorpusError(f"search backend broke pagination for query `{q}` at offset {cur['offset']}")
            texts = self.mat.fetch(keys)
            st = cur["stats"]
            st["discovered"] += len(keys)
            new_hashes = []
            pending = [tuple(x) for x in cur["pending"]]
            for k in keys:
                if k not in texts:
                    continue
                st["materialised"] += 1
                text = normalise_text(texts[k])
                if len(text) < self.cfg.min_chars:
                    st["too_short"] += 1
                    continue
                h = _sha(text.encode())
                if dedup.seen(h) or h in new_hashes:
                    st["duplicates"] += 1
                    continue
                new_hashes.append(h)
                st["kept"] += 1
                pending.append((k, self.tok.encode(text), self.classify(k, text)))
            # full shards are written (and synced) BEFORE the cursor that mentions them commits
            while len(pending) >= self.cfg.docs_per_shard:
                chunk, pending = pending[:self.cfg.docs_per_shard], pending[self.cfg.docs_per_shard:]
                cur["shards"].append(self._write(stage, len(cur["shards"]), chunk))
            cur["pending"] = [list(x) for x in pending]
            cur["offset"] += len(keys)
            if cur["offset"] >= total:
                cur["query_index"] += 1
                cur["offset"] = 0
            dedup.commit(new_hashes, cur)
            pages += 1
        if cur["pending"]:
            cur["shards"].append(self._write(stage, len(cur["shards"]), [tuple(x) for x in cur["pending"]]))
            cur["pending"] = []
            dedup.commit([], cur)
        manifest = {"version": MANIFEST_VERSION, "name": self.cfg.name, "build_id": bid, "source_snapshot": self.search.snapshot(),
                    "stats": cur["stats"], "shards": cur["shards"], "metadata": self.cfg.metadata}
        body = json.dumps(manifest, sort_keys=True, indent=1).encode()
        with open(os.path.join(stage, "manifest.json"), "wb") as f:
            f.write(body)
            f.flush()
            os.fsync(f.fileno())
        os.replace(stage, final)
        return final

    @staticmethod
    def _write(stage: str, index: int, chunk) -> dict:
        entry = write_shard(os.path.join(stage, f"shard-{index:06d}.tok"), [ids for _, ids, _ in chunk])
        entry["records"] = [{"key": k, "tokens": len(ids), "labels": labels} for k, ids, labels in chunk]
        return entry


def open_corpus(path: str) -> Tuple[dict, Callable[[], Iterator[List[int]]]]:
    """Authenticates a published corpus directory; returns (manifest, document iterator factory)."""
    with open(os.path.join(path, "manifest.json"), "rb") as f:
        manifest = json.loads(f.read())
    if manifest.get("version") != MANIFEST_VERSION:
        raise CorpusError(f"unsupported corpus manifest version {manifest.get('version')}")

    def docs() -> Iterator[List[int]]:
        for sh in manifest["shards"]:
            yield from read_shard(os.path.join(path, sh["file"]), sh["sha256"])

    return manifest, docs


# ---------------------------------------------------------------------------- curriculum composition
@dataclass
class Stratum:
    name: str
    weight: float                                  # share of the stage's tokens
    predicate: Callable[[dict], bool]              # over a record's labels


def compose_stage(records: Iterable[Tuple[dict, List[int]]], strata: Sequence[Stratum], token_budget: int) -> List[Tuple[str, List[int]]]:
    """Deterministic interleave: every record goes to the first stratum whose predicate holds;
    strata are then drained in proportion to their token weights (largest deficit first, ties by
    declaration order) until the budget is met or the strata run dry."""
    if not strata or any(s.weight <= 0 for s in strata):
        raise CorpusError("strata need positive weights")
    queues: List[List[List[int]]] = [[] for _ in strata]
    for labels, ids in records:
        for qi, s in enumerate(strata):
            if s.predicate(labels):
                queues[qi].append(ids)
                break
    total_w = sum(s.weight for s in strata)
    taken = [0] * len(strata)
    heads = [0] * len(strata)
    out: List[Tuple[str, List[int]]] = []
    emitted = 0
    while emitted < token_budget:
        best, best_deficit = -1, None
        for qi, s in enumerate(strata):
            if heads[qi] >= len(queues[qi]):
                continue
            deficit = s.weight / total_w * (emitted + 1) - taken[qi]
            if best_deficit is None or deficit > best_deficit:
                best, best_deficit = qi, deficit
        if best < 0:
            break
        ids = queues[best][heads[best]]
        heads[best] += 1
        taken[best] += len(ids)
        emitted += len(ids)
        out.append((strata[best].name, ids))
    return out
