"""Derived token cache of a causal data file: tokenise once, replay on every later epoch and resume.

Wire formats are the reference's (`summa-train/src/data.rs:44-50,502-548,590-742`):
  * cache `HERTOK01`, then per document a u32 length and that many u32 tokens, little endian;
  * sidecar `<cache>.index`, 144 bytes: `HERTIX01`, the indexed file's identity (length, device, inode, mtime s / ns,
    ctime s / ns, each 8 bytes LE), document count, stream length in tokens (each document counts its tokens plus
    one end-of-sequence token = cache bytes after the header / 4), the SHA-256 of the whole cache, and a SHA-256 of
    the preceding 112 bytes.
Behaviour follows `data.rs:1116-1330`: the cache is DERIVED data, so nothing about it is ever trusted over the
source and nothing wrong with it stops training. A torn final record is cut off and tokenisation resumes at the
first missing document; an unknown header, an out-of-vocabulary token, a cache that changed under a published
index, or a digest mismatch reset the cache; a torn or corrupt sidecar is dropped and rebuilt after a structural
scan; the sidecar is invalidated BEFORE the first append and republished (atomically) only after the cache is
synced; and a valid sidecar gives the packed-sample count of a finished cache without reading it. The cache and
its sidecar are opened relative to one directory descriptor without following symlinks."""
from __future__ import annotations

import hashlib
import os
import struct
from typing import Callable, Iterable, Iterator, List, Optional, Sequence, Tuple

from .data import DataError

CACHE_MAGIC = b"HERTOK01"
INDEX_MAGIC = b"HERTIX01"
INDEX_BYTES = 144
MAX_CACHED_DOCUMENT_TOKENS = 100_000_000
_IDENTITY = struct.Struct("<QQQqqqq")


def _identity(st: os.stat_result) -> Tuple[int, ...]:
    return (st.st_size, st.st_dev, st.st_ino, st.st_mtime_ns // 10**9, st.st_mtime_ns % 10**9, st.st_ctime_ns // 10**9, st.st_ctime_ns % 10**9)


def encode_index(identity: Sequence[int], documents: int, stream_tokens: int, cache_digest: bytes) -> bytes:
    body = INDEX_MAGIC + _IDENTITY.pack(*identity) + struct.pack("<QQ", documents, stream_tokens) + cache_digest
    out = body + hashlib.sha256(body).digest()
    assert len(out) == INDEX_BYTES
    return out


def decode_index(raw: bytes) -> Optional[Tuple[Tuple[int, ...], int, int, bytes]]:
    """(identity, documents, stream_tokens, cache digest), or None for anything that is not an intact index whose
    numbers agree with each other."""
    if len(raw) != INDEX_BYTES or raw[:8] != INDEX_MAGIC or hashlib.sha256(raw[:112]).digest() != raw[112:]:
        return None
    identity = _IDENTITY.unpack(raw[8:64])
    documents, stream_tokens = struct.unpack("<QQ", raw[64:80])
    size = identity[0]
    if size < 8 or (size - 8) % 4 or (size - 8) // 4 != stream_tokens or documents > stream_tokens:
        return None
    return identity, documents, stream_tokens, raw[80:112]


def token_cache_path(root: str, data_identity: str, source: str, tokenizer_identity: str, vocab_size: int, rank: int = 0, world: int = 1) -> str:
    """Cache file of one (data generation, source path, tokenizer) triple under `root`; another data file, another
    tokenizer or another vocabulary size names another file, so a finished cache is never replayed for inputs it
    was not derived from. Ranks of a multi-process run keep separate files."""
    key = hashlib.sha256("\0".join((data_identity, os.path.abspath(source), tokenizer_identity, str(vocab_size))).encode()).hexdigest()[:32]
    return os.path.join(root, key + (f".r{rank}of{world}" if world > 1 else "") + ".tok")


class TokenCache:
    """One cache file and its sidecar inside an opened directory."""

    def __init__(self, path: str, create_directory: bool = True):
        directory, self.name = os.path.split(os.path.abspath(path))
        self.index_name = self.name + ".index"
        self.path = path
        if create_directory:
            os.makedirs(directory, exist_ok=True)
        self.dir_fd = os.open(directory, os.O_RDONLY | os.O_DIRECTORY)

    def close(self) -> None:
        if self.dir_fd is not None:
            os.close(self.dir_fd)
            self.dir_fd = None

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    # ---- files, always relative to the opened directory and never through a symlink
    def _open(self, name: str, flags: int) -> Optional[int]:
        try:
            return os.open(name, flags | os.O_NOFOLLOW | os.O_CLOEXEC, 0o644, dir_fd=self.dir_fd)
        except FileNotFoundError:
            return None
        except OSError as e:
            raise DataError(f"{self.path}: token-cache entry `{name}` cannot be opened safely: {e}")

    def open_cache(self, create: bool) -> Optional[int]:
        return self._open(self.name, os.O_RDWR | (os.O_CREAT if create else 0))

    def read_index(self, cache_fd: int) -> Optional[Tuple[Tuple[int, ...], int, int, bytes]]:
        """The decoded sidecar if it is intact AND still describes the open cache file."""
        got = self._decode_index_file()
        if got in (None, "invalid"):
            return None
        return got if got[0] == _identity(os.fstat(cache_fd)) else None

    def _decode_index_file(self):
        fd = self._open(self.index_name, os.O_RDONLY)
        if fd is None:
            return None
        try:
            raw = os.read(fd, INDEX_BYTES + 1)
        finally:
            os.close(fd)
        return decode_index(raw) or "invalid"

    def invalidate_index(self) -> None:
        try:
            os.unlink(self.index_name, dir_fd=self.dir_fd)
        except FileNotFoundError:
            pass
        os.fsync(self.dir_fd)

    def write_index(self, raw: bytes) -> None:
        tmp = f".{self.index_name}.{os.getpid()}.tmp"
        fd = os.open(tmp, os.O_WRONLY | os.O_CREAT | os.O_EXCL | os.O_NOFOLLOW | os.O_CLOEXEC, 0o644, dir_fd=self.dir_fd)
        try:
            os.write(fd, raw)
            os.fsync(fd)
        finally:
            os.close(fd)
        os.rename(tmp, self.index_name, src_dir_fd=self.dir_fd, dst_dir_fd=self.dir_fd)
        os.fsync(self.dir_fd)

    def reset(self, cache_fd: int) -> None:
        """Back to an empty cache (header only), sidecar gone first."""
        self.invalidate_index()
        os.ftruncate(cache_fd, 0)
        os.pwrite(cache_fd, CACHE_MAGIC, 0)
        os.fsync(cache_fd)

    # ---- constant-time sample count of a finished cache
    def indexed_sample_count(self, seq_len: int) -> Optional[int]:
        if seq_len <= 0:
            raise DataError("sequence_length must be positive")
        fd = self.open_cache(False)
        if fd is None:
            return None
        try:
            idx = self.read_index(fd)
        finally:
            os.close(fd)
        if idx is None:
            return None
        return 0 if idx[2] == 0 else (idx[2] - 1) // seq_len


class _Writer:
    def __init__(self, cache: TokenCache, fd: int, digest, documents: int, stream_tokens: int):
        self.cache, self.fd, self.digest, self.documents, self.stream_tokens = cache, fd, digest, documents, stream_tokens
        self.index_invalidated = False
        self.buf = bytearray()

    def append(self, tokens: Sequence[int]) -> None:
        if not self.index_invalidated:                     # a published index must never describe a cache that grew
            self.cache.invalidate_index()
            self.index_invalidated = True
        if len(tokens) > MAX_CACHED_DOCUMENT_TOKENS:
            raise DataError("document is too large for the token cache")
        rec = struct.pack(f"<I{len(tokens)}I", len(tokens), *tokens)
        self.digest.update(rec)
        self.buf += rec
        self.documents += 1
        self.stream_tokens += len(tokens) + 1
        if len(self.buf) >= 1 << 20:
            self.flush()

    def flush(self) -> None:
        if self.buf:
            os.write(self.fd, self.buf)
            self.buf.clear()

    def publish_index(self) -> None:
        self.flush()
        os.fsync(self.fd)
        raw = encode_index(_identity(os.fstat(self.fd)), self.documents, self.stream_tokens, self.digest.copy().digest())
        if decode_index(raw) is None:
            raise DataError(f"{self.cache.path}: token cache and its counters disagree")
        fd = self.cache._open(self.cache.index_name, os.O_RDONLY)
        same = False
        if fd is not None:
            try:
                same = os.read(fd, INDEX_BYTES + 1) == raw
            finally:
                os.close(fd)
        if not same:
            self.cache.write_index(raw)
        self.index_invalidated = False

    def reset(self) -> None:
        self.buf.clear()
        self.cache.reset(self.fd)
        os.lseek(self.fd, 0, os.SEEK_END)
        self.digest = hashlib.sha256(CACHE_MAGIC)
        self.documents = self.stream_tokens = 0
        self.index_invalidated = True


def cached_documents(source: Callable[[], Iterable[List[int]]], cache_path: str, vocab_size: int,
                     stats: Optional[dict] = None) -> Iterator[List[int]]:
    """Documents of `source()` (token lists, no trailing EOS) through the cache at `cache_path`.

    Replays every complete cached document first, then tokenises the source from the first missing document on,
    appending as it goes, and publishes the index when the source ends. `stats` (if given) receives `replayed`,
    `tokenized`, `reset` (why the cache was discarded, or None), `torn_tail`, `completed_fast_path`.
    Stopping the iteration early leaves a valid, resumable cache (and checks a finished cache's identity)."""
    if vocab_size <= 0:
        raise DataError("tokenizer vocabulary must not be empty")
    stats = stats if stats is not None else {}
    stats.update(replayed=0, tokenized=0, reset=None, torn_tail=False, completed_fast_path=False)
    with TokenCache(cache_path) as cache:
        fd = cache.open_cache(True)
        try:
            state = cache._decode_index_file()
            expected = None
            if state == "invalid":
                cache.invalidate_index()               # derived metadata: drop it, keep the payload for a structural scan
            elif state is not None:
                if state[0] == _identity(os.fstat(fd)):
                    expected = state
                else:                                   # the cache changed under a published index: never re-bless it
                    cache.reset(fd)
                    stats["reset"] = "cache changed after its index was published"
            if os.fstat(fd).st_size < 8:
                os.ftruncate(fd, 0)
                os.pwrite(fd, CACHE_MAGIC, 0)
                os.fsync(fd)
            replay_identity = _identity(os.fstat(fd))
            f = os.fdopen(os.dup(fd), "rb", buffering=1 << 20)
            digest = hashlib.sha256(CACHE_MAGIC)
            documents = stream_tokens = 0
            valid_bytes = 8
            try:
                f.seek(0)
                if f.read(8) != CACHE_MAGIC:
                    cache.reset(fd)
                    stats["reset"] = "unrecognised header"
                    expected = None
                else:
                    while True:
                        head = f.read(4)
                        if not head:
                            break
                        if len(head) < 4:
                            stats["torn_tail"] = True
                            break
                        (n,) = struct.unpack("<I", head)
                        if n > MAX_CACHED_DOCUMENT_TOKENS:
                            raise DataError(f"{cache_path}: token cache contains an implausible {n}-token document")
                        raw = f.read(4 * n)
                        if len(raw) < 4 * n:
                            stats["torn_tail"] = True
                            break
                        doc = list(struct.unpack(f"<{n}I", raw))
                        if any(t >= vocab_size for t in doc):
                            cache.reset(fd)             # never emitted: the cache belongs to another vocabulary
                            stats["reset"] = "out-of-vocabulary token"
                            if stats["replayed"]:
                                raise DataError(f"{cache_path}: token cache held out-of-vocabulary tokens after {stats['replayed']} "
                                                f"documents were replayed; the derived cache was reset")
                            expected, documents, stream_tokens, valid_bytes = None, 0, 0, 8
                            digest = hashlib.sha256(CACHE_MAGIC)
                            break
                        digest.update(head + raw)
                        documents += 1
                        stream_tokens += n + 1
                        valid_bytes += 4 + 4 * n
                        stats["replayed"] += 1
                        try:
                            yield doc
                        except GeneratorExit:
                            if _identity(os.fstat(fd)) != replay_identity:
                                cache.reset(fd)
                            raise
                        if _identity(os.fstat(fd)) != replay_identity:
                            cache.reset(fd)
                            raise DataError(f"token cache {cache_path} changed while it was replayed; the derived cache was reset")
            finally:
                f.close()
            if stats["reset"] is None:
                if expected is not None:
                    # finished cache: every record was just re-hashed, so the digest decides
                    if (documents, stream_tokens, digest.digest()) == (expected[1], expected[2], expected[3]) and not stats["torn_tail"]:
                        stats["completed_fast_path"] = True
                        return
                    cache.reset(fd)
                    stats["reset"] = "cache digest differs from its index"
                    raise DataError(f"token cache {cache_path} does not match its index; the derived cache was reset")
                if stats["torn_tail"]:
                    os.ftruncate(fd, valid_bytes)       # derived data: the torn record is simply tokenised again
                    os.fsync(fd)
            os.lseek(fd, 0, os.SEEK_END)
            writer = _Writer(cache, fd, digest, documents, stream_tokens)
            skip = documents
            seen = 0
            try:
                for i, doc in enumerate(source()):
                    seen = i + 1
                    if i < skip:
                        continue
                    writer.append(doc)
                    stats["tokenized"] += 1
                    yield doc
                if seen < skip:
                    raise DataError(f"{cache_path}: the source has {seen} documents but its token cache replayed {skip}; "
                                    f"the derived cache was reset")
            except GeneratorExit:
                writer.flush()                          # stopped early: complete records stay, no index is published
                raise
            except BaseException:
                writer.reset()                          # a failing source must not leave a cache of unknown provenance
                raise
            writer.publish_index()
        finally:
            os.close(fd)
