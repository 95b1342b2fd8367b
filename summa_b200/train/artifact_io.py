"""Artifact reads and writes that cannot be redirected: no symlinks are followed, a file is
identified by (device, inode, size, mtime) from open to close, reads are bounded before they
allocate, new files are created exclusively and synced, and directories are pinned by a file
descriptor so that their members are opened relative to the directory object, not to a path
that could be swapped (`summa-train/src/artifact_io.rs:36-135,283-345,700-840`).
Content identities are `sha256:<64 lowercase hex>`.
"""
from __future__ import annotations

import hashlib
import json
import os
import stat
from dataclasses import dataclass
from typing import Any, List, Optional, Tuple

SHA256_PREFIX = "sha256:"
MAX_PINNED_DIRECTORY_ENTRIES = 4096
_CHUNK = 1 << 20


class ArtifactError(RuntimeError):
    pass


def sha256_hex(data: bytes) -> str:
    return hashlib.sha256(data).hexdigest()


def sha256_identity(data: bytes) -> str:
    return SHA256_PREFIX + sha256_hex(data)


def validate_sha256_hex(value: str, label: str) -> None:
    if len(value) != 64 or any(c not in "0123456789abcdef" for c in value):
        raise ArtifactError(f"{label} must use exactly 64 lowercase hexadecimal characters")


def validate_sha256_identity(value: str, label: str) -> None:
    if not isinstance(value, str) or not value.startswith(SHA256_PREFIX):
        raise ArtifactError(f"{label} must use the `sha256:<64 lowercase hex>` form")
    validate_sha256_hex(value[len(SHA256_PREFIX):], label)


def sha256_identity_from_hex(digest: str, label: str) -> str:
    validate_sha256_hex(digest, label)
    return SHA256_PREFIX + digest


def json_sha256_identity(value: Any) -> str:
    """Identity of the compact, key-sorted JSON bytes of a fixed-schema value."""
    return sha256_identity(json.dumps(value, sort_keys=True, separators=(",", ":")).encode())


@dataclass(frozen=True)
class StableIdentity:
    device: int
    inode: int
    size: int
    mtime_ns: int

    @staticmethod
    def of(st: os.stat_result) -> "StableIdentity":
        return StableIdentity(st.st_dev, st.st_ino, st.st_size, st.st_mtime_ns)

    def same_object(self, other: "StableIdentity") -> bool:
        return (self.device, self.inode) == (other.device, other.inode)


def ensure_real_directory(path: str, label: str) -> None:
    try:
        st = os.lstat(path)
    except OSError as e:
        raise ArtifactError(f"inspecting {label} {path}: {e}")
    if not stat.S_ISDIR(st.st_mode):
        raise ArtifactError(f"{label} {path} is not a real directory")


def ensure_directory(path: str, label: str) -> None:
    os.makedirs(path, exist_ok=True)
    ensure_real_directory(path, label)


def sync_directory(path: str) -> None:
    ensure_real_directory(path, "synced directory")
    fd = os.open(path, os.O_RDONLY | os.O_DIRECTORY)
    try:
        os.fsync(fd)
    finally:
        os.close(fd)


_OPEN_FLAGS = os.O_RDONLY | os.O_CLOEXEC | os.O_NOFOLLOW | os.O_NONBLOCK


def open_regular(path: str, label: str, dir_fd: Optional[int] = None) -> Tuple[int, StableIdentity]:
    """File descriptor of a regular, non-symlink file plus the identity it had when opened."""
    try:
        pst = os.stat(path, dir_fd=dir_fd, follow_symlinks=False)
    except OSError as e:
        raise ArtifactError(f"inspecting {label} {path}: {e}")
    if not stat.S_ISREG(pst.st_mode):
        raise ArtifactError(f"{label} {path} is not a regular file or is a symlink")
    try:
        fd = os.open(path, _OPEN_FLAGS, dir_fd=dir_fd)
    except OSError as e:
        raise ArtifactError(f"opening {label} {path}: {e}")
    ident = StableIdentity.of(os.fstat(fd))
    if ident != StableIdentity.of(pst):
        os.close(fd)
        raise ArtifactError(f"{label} {path} changed while it was opened")
    return fd, ident


def ensure_regular_file(path: str, label: str) -> None:
    fd, _ = open_regular(path, label)
    os.close(fd)


def hash_open_file(fd: int, ident: StableIdentity, label: str, capture_limit: Optional[int] = None):
    """(size, hex digest, bytes or None). The size is rejected against `capture_limit` before
    anything is read; a file that changes while it is read is refused."""
    if capture_limit is not None and ident.size > capture_limit:
        raise ArtifactError(f"{label} is {ident.size} bytes, limit {capture_limit}")
    h = hashlib.sha256()
    parts: Optional[List[bytes]] = [] if capture_limit is not None else None
    total = 0
    os.lseek(fd, 0, os.SEEK_SET)
    while True:
        chunk = os.read(fd, _CHUNK)
        if not chunk:
            break
        total += len(chunk)
        if total > ident.size:
            raise ArtifactError(f"{label} grew while it was read")
        h.update(chunk)
        if parts is not None:
            parts.append(chunk)
    if total != ident.size or StableIdentity.of(os.fstat(fd)) != ident:
        raise ArtifactError(f"{label} changed while it was read")
    return total, h.hexdigest(), (b"".join(parts) if parts is not None else None)


def read_regular_bounded(path: str, max_bytes: int, label: str) -> bytes:
    fd, ident = open_regular(path, label)
    try:
        return hash_open_file(fd, ident, label, max_bytes)[2]
    finally:
        os.close(fd)


def hash_regular_file_hex(path: str) -> Tuple[int, str]:
    fd, ident = open_regular(path, "hashed file")
    try:
        size, digest, _ = hash_open_file(fd, ident, f"hashed file {path}")
        return size, digest
    finally:
        os.close(fd)


def hash_regular_file(path: str) -> Tuple[int, str]:
    size, digest = hash_regular_file_hex(path)
    return size, SHA256_PREFIX + digest


def sync_regular_file(path: str, label: str) -> None:
    fd, _ = open_regular(path, label)
    try:
        os.fsync(fd)
    finally:
        os.close(fd)


def write_new_synced(path: str, data: bytes) -> None:
    """Creates `path` exclusively (an existing file or symlink is an error) and syncs it."""
    fd = os.open(path, os.O_WRONLY | os.O_CREAT | os.O_EXCL | os.O_CLOEXEC | os.O_NOFOLLOW, 0o644)
    try:
        view = memoryview(data)
        while view:
            n = os.write(fd, view[:_CHUNK])
            view = view[n:]
        os.fsync(fd)
    finally:
        os.close(fd)


def atomic_write_new(path: str, data: bytes) -> None:
    """Write-once publication of one file: staged beside the target, synced, hard-linked into
    place (a link fails if the name exists, so an existing artifact is never replaced)."""
    d = os.path.dirname(os.path.abspath(path))
    tmp = os.path.join(d, f".{os.path.basename(path)}.{os.getpid()}.{int.from_bytes(os.urandom(6), 'big')}.part")
    write_new_synced(tmp, data)
    try:
        os.link(tmp, path)
    except FileExistsError:
        raise ArtifactError(f"{path} already exists")
    finally:
        os.unlink(tmp)
    sync_directory(d)


class PinnedDirectory:
    """A directory held open by descriptor. Children are opened relative to it with no-follow
    semantics, so replacing the directory's path by another directory or a link after `open`
    cannot redirect later reads."""

    def __init__(self, fd: int, label: str):
        self.fd, self.label = fd, label

    @staticmethod
    def open(path: str, label: str) -> "PinnedDirectory":
        ensure_real_directory(path, label)
        try:
            fd = os.open(path, os.O_RDONLY | os.O_DIRECTORY | os.O_CLOEXEC | os.O_NOFOLLOW)
        except OSError as e:
            raise ArtifactError(f"opening {label} {path}: {e}")
        return PinnedDirectory(fd, label)

    def identity(self) -> StableIdentity:
        return StableIdentity.of(os.fstat(self.fd))

    def entries(self, maximum_entries: int = MAX_PINNED_DIRECTORY_ENTRIES) -> List[str]:
        names = sorted(os.listdir(self.fd))
        if len(names) > maximum_entries:
            raise ArtifactError(f"{self.label} holds more than {maximum_entries} entries")
        return names

    def _walk(self, relative: str) -> Tuple[int, str, List[int]]:
        parts = [p for p in relative.split("/")]
        if not parts or any(p in ("", ".", "..") for p in parts) or relative.startswith("/"):
            raise ArtifactError(f"{self.label}: `{relative}` is not a plain relative path")
        cur, opened = self.fd, []
        for p in parts[:-1]:
            try:
                nxt = os.open(p, os.O_RDONLY | os.O_DIRECTORY | os.O_CLOEXEC | os.O_NOFOLLOW, dir_fd=cur)
            except OSError as e:
                for f in opened:
                    os.close(f)
                raise ArtifactError(f"{self.label}: opening directory `{p}` of `{relative}`: {e}")
            opened.append(nxt)
            cur = nxt
        return cur, parts[-1], opened

    def read_bounded(self, relative: str, max_bytes: int) -> bytes:
        cur, leaf, opened = self._walk(relative)
        try:
            fd, ident = open_regular(leaf, f"{self.label} member {relative}", dir_fd=cur)
            try:
                return hash_open_file(fd, ident, f"{self.label} member {relative}", max_bytes)[2]
            finally:
                os.close(fd)
        finally:
            for f in opened:
                os.close(f)

    def hash_member(self, relative: str) -> Tuple[int, str]:
        cur, leaf, opened = self._walk(relative)
        try:
            fd, ident = open_regular(leaf, f"{self.label} member {relative}", dir_fd=cur)
            try:
                size, digest, _ = hash_open_file(fd, ident, f"{self.label} member {relative}")
                return size, SHA256_PREFIX + digest
            finally:
                os.close(fd)
        finally:
            for f in opened:
                os.close(f)

    def ensure_still_published(self, path: str) -> None:
        """The path must still name the directory object that was pinned."""
        try:
            st = os.lstat(path)
        except OSError as e:
            raise ArtifactError(f"{self.label} {path} disappeared: {e}")
        if not stat.S_ISDIR(st.st_mode) or not StableIdentity.of(st).same_object(self.identity()):
            raise ArtifactError(f"{self.label} {path} was replaced while it was read")

    def close(self) -> None:
        if self.fd >= 0:
            os.close(self.fd)
            self.fd = -1

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
