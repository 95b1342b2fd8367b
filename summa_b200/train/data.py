"""Training data: sources, EOS-joined packing, seeded reservoir shuffle, fixed-shape
batches, synthetic token streams.

Contracts kept from the reference (`summa-train/src/data.rs:1371-1448,1531-1575`,
`summa-train/src/data/batch.rs:124-181`):
  * causal JSONL rows are `{"text": ...}` (tokenised, EOS appended) or
    `{"tokens": [...]}` (validated < vocab, EOS appended); any other file is one text
    document; `.zst` files are decompressed when `zstandard` is importable;
  * packing concatenates `doc ⧺ EOS` and emits windows of `seq + 1` tokens with stride
    `seq` (inputs `[:seq]`, targets `[1:]`); a remainder shorter than `seq + 1` is dropped;
  * the shuffle buffer is a seeded reservoir (0 = source order), seed
    `seed + (phase << 32) + epoch`;
  * incomplete batches are dropped.
"""
from __future__ import annotations

import hashlib
import io
import json
import os
import random
import struct
from typing import Iterable, Iterator, List, Optional, Sequence

import torch

TOKEN_CACHE_MAGIC = b"HERTOK01"


class DataError(ValueError):
    pass


def file_sha256(path: str) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for chunk in iter(lambda: f.read(1 << 20), b""):
            h.update(chunk)
    return h.hexdigest()


def _open_text(path: str):
    if path.endswith(".zst"):
        try:
            import zstandard
        except ImportError as e:
            raise DataError(f"{path}: zstandard is not installed") from e
        return io.TextIOWrapper(zstandard.ZstdDecompressor().stream_reader(open(path, "rb")), encoding="utf-8")
    return open(path, "r", encoding="utf-8")


def iter_documents(path: str, tokenizer, vocab_size: int) -> Iterator[List[int]]:
    """Token lists of every document in a data file (without the trailing EOS). A corpus `manifest.json` (the file a
    corpus build or a curriculum stage publishes) stands for its authenticated shards, in manifest order."""
    base = path[:-4] if path.endswith(".zst") else path
    if os.path.basename(base) == "manifest.json":
        yield from _corpus_documents(path, vocab_size)
        return
    if base.endswith(".jsonl"):
        with _open_text(path) as f:
            for n, line in enumerate(f, 1):
                line = line.strip()
                if not line:
                    continue
                try:
                    row = json.loads(line)
                except json.JSONDecodeError as e:
                    raise DataError(f"{path}:{n}: invalid JSON: {e}")
                if "tokens" in row:
                    toks = row["tokens"]
                    if not isinstance(toks, list) or any((not isinstance(t, int)) or t < 0 or t >= vocab_size
                                                        for t in toks):
                        raise DataError(f"{path}:{n}: tokens must be integers in [0, {vocab_size})")
                    yield list(toks)
                elif "text" in row:
                    yield tokenizer.encode(row["text"], False)
                else:
                    raise DataError(f"{path}:{n}: row needs a 'text' or 'tokens' field")
    else:
        with _open_text(path) as f:
            yield tokenizer.encode(f.read(), False)


def _corpus_documents(path: str, vocab_size: int) -> Iterator[List[int]]:
    from . import corpus, corpus_recipe
    try:
        with open(path, "rb") as f:
            head = json.loads(f.read())
        if isinstance(head.get("build"), dict):                           # JSONL shards with one row per emitted view
            _, rows = corpus_recipe.open_corpus_manifest(path)
            docs = (row["tokens"] for row in rows())
        else:                                                             # binary token shards
            _, docs_fn = corpus.open_corpus(os.path.dirname(os.path.abspath(path)))
            docs = docs_fn()
        for n, toks in enumerate(docs):
            if any((not isinstance(t, int)) or t < 0 or t >= vocab_size for t in toks):
                raise DataError(f"{path}: document {n}: tokens must be integers in [0, {vocab_size})")
            yield list(toks)
    except corpus.CorpusError as e:
        raise DataError(f"{path}: {e}")


class SamplePacker:
    """Concatenates `doc ⧺ EOS` and yields `seq + 1`-token windows with stride `seq`."""

    def __init__(self, seq_len: int, eos_id: int):
        self.seq = seq_len
        self.eos = eos_id
        self.buf: List[int] = []

    def push(self, doc: Sequence[int]) -> Iterator[List[int]]:
        self.buf.extend(doc)
        self.buf.append(self.eos)
        need = self.seq + 1
        while len(self.buf) >= need:
            yield self.buf[:need]
            del self.buf[:self.seq]

    def remainder(self) -> int:
        return len(self.buf)


class ShuffleBuffer:
    """Seeded reservoir: holds `capacity` samples, emits a random one per arrival."""

    def __init__(self, capacity: int, seed: int):
        self.capacity = capacity
        self.rng = random.Random(seed)
        self.items: list = []

    def push(self, item):
        if self.capacity <= 0:
            return item
        if len(self.items) < self.capacity:
            self.items.append(item)
            return None
        j = self.rng.randrange(self.capacity)
        out, self.items[j] = self.items[j], item
        return out

    def drain(self) -> Iterator:
        self.rng.shuffle(self.items)
        while self.items:
            yield self.items.pop()


def shuffle_seed(seed: int, phase: int, epoch: int) -> int:
    return (seed + (phase << 32) + epoch) & 0xFFFFFFFFFFFFFFFF


def iter_samples(path: str, tokenizer, vocab_size: int, seq_len: int, eos_id: int, shuffle: int = 0,
                 seed: int = 0, skip: int = 0, token_cache: Optional[str] = None) -> Iterator[List[int]]:
    """Packed, shuffled `seq + 1` windows of a causal data file. `skip` replays the
    cursor of a resumed run by discarding that many samples. With `token_cache` the documents go through the
    derived cache of `train/token_cache.py` (tokenised once, replayed afterwards)."""
    packer = SamplePacker(seq_len, eos_id)
    buf = ShuffleBuffer(shuffle, seed)
    emitted = 0

    def out(sample):
        nonlocal emitted
        emitted += 1
        return emitted > skip

    if token_cache is not None:
        from .token_cache import cached_documents
        docs = cached_documents(lambda: iter_documents(path, tokenizer, vocab_size), token_cache, vocab_size)
    else:
        docs = iter_documents(path, tokenizer, vocab_size)
    for doc in docs:
        for window in packer.push(doc):
            got = buf.push(window)
            if got is not None and out(got):
                yield got
    for got in buf.drain():
        if out(got):
            yield got


def make_batch(samples: Sequence[Sequence[int]], device=None, pin: bool = False):
    """`[B, seq+1]` int64 → (inputs `[B, seq]`, targets `[B, seq]`)."""
    t = torch.tensor(samples, dtype=torch.int64)
    if pin and torch.cuda.is_available():
        t = t.pin_memory()
    if device is not None:
        t = t.to(device, non_blocking=True)
    return t[:, :-1], t[:, 1:]


def iter_batches(samples: Iterable[Sequence[int]], batch_size: int) -> Iterator[List[Sequence[int]]]:
    cur: List[Sequence[int]] = []
    for s in samples:
        cur.append(s)
        if len(cur) == batch_size:
            yield cur
            cur = []
    # an incomplete batch is dropped


# ------------------------------------------------------------------ token cache (derived)

def write_token_cache(path: str, docs: Iterable[Sequence[int]]) -> None:
    """`HERTOK01` + per document: u32 length, u32 tokens (little endian)."""
    with open(path, "wb") as f:
        f.write(TOKEN_CACHE_MAGIC)
        for d in docs:
            f.write(struct.pack("<I", len(d)))
            f.write(struct.pack(f"<{len(d)}I", *d))


def read_token_cache(path: str) -> Iterator[List[int]]:
    with open(path, "rb") as f:
        if f.read(8) != TOKEN_CACHE_MAGIC:
            raise DataError(f"{path}: not a token cache")
        while True:
            head = f.read(4)
            if not head:
                return
            (n,) = struct.unpack("<I", head)
            raw = f.read(4 * n)
            if len(raw) != 4 * n:
                raise DataError(f"{path}: truncated token cache")
            yield list(struct.unpack(f"<{n}I", raw))


# ------------------------------------------------------------------ synthetic streams

class SyntheticTokens:
    """Seeded uniform or Zipf(s) token batches (benchmark configs)."""

    def __init__(self, vocab_size: int, kind: str = "zipf", s: float = 1.1, seed: int = 0):
        self.vocab = vocab_size
        self.kind = kind
        self.gen = torch.Generator().manual_seed(seed)
        if kind == "zipf":
            ranks = torch.arange(1, vocab_size + 1, dtype=torch.float64)
            p = ranks.pow(-s)
            self.probs = p / p.sum()
        elif kind != "uniform":
            raise DataError(f"unknown synthetic kind {kind}")

    def batch(self, batch_size: int, seq_len: int) -> torch.Tensor:
        n = batch_size * (seq_len + 1)
        if self.kind == "zipf":
            t = torch.multinomial(self.probs, n, replacement=True, generator=self.gen)
        else:
            t = torch.randint(0, self.vocab, (n,), generator=self.gen)
        return t.view(batch_size, seq_len + 1).to(torch.int64)

    def write_jsonl(self, path: str, docs: int, doc_len: int) -> None:
        with open(path, "w") as f:
            for _ in range(docs):
                row = self.batch(1, doc_len - 1)[0].tolist()
                f.write(json.dumps({"tokens": row}) + "\n")
