"""Derived token cache: replay, torn-tail repair, resets, the HERTIX01 sidecar and its constant-time sample count
(the cases of `summa-train/src/data.rs:2531-3060`, restated for this package)."""
import hashlib
import os
import struct

import pytest

from summa_b200.train import data as D
from summa_b200.train import token_cache as TC

DOCS = [[1, 2, 3], [4, 5], [], [6, 7, 8, 9], [10]]


def source_of(docs, calls=None, fail_at=None):
    def src():
        for i, d in enumerate(docs):
            if calls is not None:
                calls.append(i)
            if fail_at is not None and i == fail_at:
                raise ValueError("bad record")
            yield list(d)
    return src


def run(path, docs=DOCS, vocab=64, calls=None, **kw):
    stats = {}
    out = list(TC.cached_documents(source_of(docs, calls, **kw), path, vocab, stats))
    return out, stats


def test_first_pass_writes_cache_and_index_in_the_reference_wire_format(tmp_path):
    path = str(tmp_path / "cache" / "a.tok")
    out, st = run(path)
    assert out == DOCS and st["tokenized"] == 5 and st["replayed"] == 0
    raw = open(path, "rb").read()
    body = b"".join(struct.pack(f"<I{len(d)}I", len(d), *d) for d in DOCS)
    assert raw == b"HERTOK01" + body
    idx = open(path + ".index", "rb").read()
    assert len(idx) == 144 and idx[:8] == b"HERTIX01" and hashlib.sha256(idx[:112]).digest() == idx[112:]
    st_ = os.stat(path)
    assert struct.unpack("<QQQ", idx[8:32]) == (st_.st_size, st_.st_dev, st_.st_ino)
    documents, stream = struct.unpack("<QQ", idx[64:80])
    assert documents == 5 and stream == sum(len(d) + 1 for d in DOCS) == (len(raw) - 8) // 4
    assert idx[80:112] == hashlib.sha256(raw).digest()
    with TC.TokenCache(path) as c:
        assert c.indexed_sample_count(4) == (stream - 1) // 4 and c.indexed_sample_count(100) == 0
    # second pass: replay only, the source is never opened
    calls = []
    out, st = run(path, calls=calls)
    assert out == DOCS and st["completed_fast_path"] and st["replayed"] == 5 and calls == []


def test_torn_tail_is_cut_and_tokenisation_resumes_at_the_first_missing_document(tmp_path):
    path = str(tmp_path / "a.tok")
    gen = TC.cached_documents(source_of(DOCS), path, 64)
    assert [next(gen) for _ in range(3)] == DOCS[:3]
    gen.close()                                                   # stopped early: complete records stay, no index
    assert not os.path.exists(path + ".index")
    with open(path, "ab") as f:
        f.write(struct.pack("<I", 9) + b"\x01\x00")               # a torn final record
    with TC.TokenCache(path) as c:
        assert c.indexed_sample_count(2) is None
    calls = []
    out, st = run(path, calls=calls)
    assert out == DOCS and st["torn_tail"] and st["replayed"] == 3 and st["tokenized"] == 2 and calls == [0, 1, 2, 3, 4]
    assert os.path.exists(path + ".index") and run(path)[1]["completed_fast_path"]


def test_bad_headers_foreign_vocabularies_and_silent_edits_reset_the_cache(tmp_path):
    path = str(tmp_path / "a.tok")
    open(path, "wb").write(b"NOTACACHE" + b"\0" * 40)
    out, st = run(path)
    assert out == DOCS and st["reset"] == "unrecognised header" and run(path)[1]["completed_fast_path"]
    # a cache written for a larger vocabulary is never emitted
    with pytest.raises(D.DataError, match="out-of-vocabulary tokens after 3 documents"):      # found late: fail loudly, cache gone
        run(path, vocab=8)
    assert open(path, "rb").read() == b"HERTOK01"
    path2 = str(tmp_path / "b.tok")
    run(path2, docs=[[50, 60], [1]])
    with pytest.raises(D.DataError):
        list(TC.cached_documents(source_of([[1], [2]]), path2 + "x", 0))
    out, st = run(path2, docs=[[5, 6], [1]], vocab=10)
    assert out == [[5, 6], [1]] and st["reset"] == "out-of-vocabulary token" and st["tokenized"] == 2
    # an edit that keeps the index: the identity (length / mtime / ctime) no longer matches, the cache is rebuilt
    path3 = str(tmp_path / "c.tok")
    run(path3)
    with open(path3, "r+b") as f:
        f.seek(12)
        f.write(struct.pack("<I", 63))
    os.utime(path3, ns=(1, 1))
    out, st = run(path3)
    assert out == DOCS and st["reset"] == "cache changed after its index was published" and st["tokenized"] == 5
    # a corrupt sidecar alone does not cost the payload: structural scan, then a fresh index
    idx = bytearray(open(path3 + ".index", "rb").read())
    idx[70] ^= 1
    open(path3 + ".index", "wb").write(bytes(idx))
    with TC.TokenCache(path3) as c:
        assert c.indexed_sample_count(2) is None
    calls = []
    out, st = run(path3, calls=calls)
    assert out == DOCS and st["reset"] is None and st["replayed"] == 5 and st["tokenized"] == 0 and calls == [0, 1, 2, 3, 4]
    assert TC.decode_index(open(path3 + ".index", "rb").read()) is not None


def test_failing_source_resets_and_symlinks_are_refused(tmp_path):
    path = str(tmp_path / "a.tok")
    with pytest.raises(ValueError, match="bad record"):
        run(path, fail_at=3)
    assert open(path, "rb").read() == b"HERTOK01" and not os.path.exists(path + ".index")
    target = tmp_path / "precious.bin"
    target.write_bytes(b"do not touch")
    link = str(tmp_path / "link.tok")
    os.symlink(str(target), link)
    with pytest.raises(D.DataError, match="cannot be opened safely"):
        run(link)
    assert target.read_bytes() == b"do not touch"
    short = str(tmp_path / "s.tok")
    run(short)
    os.unlink(short + ".index")
    with pytest.raises(D.DataError, match="fewer|has 2 documents"):
        run(short, docs=DOCS[:2])


def test_iter_samples_and_cache_paths(tmp_path):
    class Tok:
        def encode(self, text, add_special_tokens=False):
            return [ord(c) % 50 for c in text]

    data = tmp_path / "d.jsonl"
    data.write_text("\n".join('{"text": "%s"}' % ("abcdefghij" * (i + 1)) for i in range(6)))
    plain = list(D.iter_samples(str(data), Tok(), 64, 8, 63, shuffle=4, seed=3))
    cache = TC.token_cache_path(str(tmp_path / ".token-cache"), "sha256:d", str(data), "sha256:t", 64)
    first = list(D.iter_samples(str(data), Tok(), 64, 8, 63, shuffle=4, seed=3, token_cache=cache))
    again = list(D.iter_samples(str(data), Tok(), 64, 8, 63, shuffle=4, seed=3, token_cache=cache))
    assert first == plain == again and len(plain) > 5
    with TC.TokenCache(cache) as c:
        assert c.indexed_sample_count(8) == len(plain)             # what the packer emits, without reading the cache
    assert cache != TC.token_cache_path(str(tmp_path / ".token-cache"), "sha256:e", str(data), "sha256:t", 64)
    assert cache != TC.token_cache_path(str(tmp_path / ".token-cache"), "sha256:d", str(data), "sha256:t", 65)
    assert TC.token_cache_path("r", "a", "b", "c", 1, rank=1, world=2).endswith(".r1of2.tok")
