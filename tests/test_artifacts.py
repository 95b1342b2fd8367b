"""No-follow artifact I/O and write-once QAT candidate publication (CPU)."""
import json
import os

import pytest
import torch


def test_artifact_io_refuses_links_growth_and_escapes(tmp_path):
    from summa_b200.train import artifact_io as A
    f = tmp_path / "a.bin"
    f.write_bytes(b"x" * 1000)
    link = tmp_path / "link.bin"
    os.symlink(f, link)
    assert A.read_regular_bounded(str(f), 1000, "file") == b"x" * 1000
    with pytest.raises(A.ArtifactError):
        A.read_regular_bounded(str(link), 1000, "file")                 # a symlink is never followed
    with pytest.raises(A.ArtifactError):
        A.read_regular_bounded(str(f), 999, "file")                     # size rejected before reading
    size, ident = A.hash_regular_file(str(f))
    assert size == 1000 and ident == A.sha256_identity(b"x" * 1000)
    A.validate_sha256_identity(ident, "id")
    for bad in ("sha256:ABC", ident.upper(), ident[7:], "md5:" + ident[7:]):
        with pytest.raises(A.ArtifactError):
            A.validate_sha256_identity(bad, "id")
    A.write_new_synced(str(tmp_path / "new.bin"), b"abc")
    with pytest.raises(FileExistsError):
        A.write_new_synced(str(tmp_path / "new.bin"), b"abc")
    A.atomic_write_new(str(tmp_path / "once.json"), b"{}")
    with pytest.raises(A.ArtifactError):
        A.atomic_write_new(str(tmp_path / "once.json"), b"{}")
    assert [n for n in os.listdir(tmp_path) if n.endswith(".part")] == []
    # a file that changes between open and read is refused
    fd, ident0 = A.open_regular(str(f), "file")
    with open(f, "ab") as g:
        g.write(b"y")
    with pytest.raises(A.ArtifactError):
        A.hash_open_file(fd, ident0, "file")
    os.close(fd)
    # pinned directory: relative, no-follow member access that survives a path swap
    d = tmp_path / "dir"
    (d / "sub").mkdir(parents=True)
    (d / "sub" / "m.txt").write_bytes(b"member")
    os.symlink(tmp_path / "a.bin", d / "evil")
    with A.PinnedDirectory.open(str(d), "dir") as pin:
        assert pin.read_bounded("sub/m.txt", 100) == b"member"
        for rel in ("../a.bin", "/etc/passwd", "sub/../sub/m.txt", "evil"):
            with pytest.raises(A.ArtifactError):
                pin.read_bounded(rel, 10000)
        os.rename(d, tmp_path / "moved")
        (tmp_path / "dir").mkdir()
        assert pin.read_bounded("sub/m.txt", 100) == b"member"        # still the pinned object
        with pytest.raises(A.ArtifactError):
            pin.ensure_still_published(str(d))
    with pytest.raises(A.ArtifactError):
        A.PinnedDirectory.open(str(tmp_path / "link.bin"), "dir")


def _model(seed=0):
    from summa_b200 import mal
    from summa_b200.models import Transformer
    cfg = mal.parse_mal("""attention a { num_heads: 2 } ffn f { hidden_dim: 128 }
      block b { attention: a ffn: f norm: rmsnorm { eps: 1e-5 } }
      model t { vocab_size: 200 max_seq_len: 32 hidden_size: 64 num_layers: 1 block: b }""")
    torch.manual_seed(seed)
    return Transformer(cfg, init_std=0.05)


def test_qat_candidate_is_write_once_and_authenticated(tmp_path):
    from summa_b200.train import qat_candidate as C
    root = str(tmp_path / "candidates")
    model = _model(0)
    recipe = C.Recipe("ternary_g128")
    factory = lambda: _model(99)
    pub = C.publish(model, root, "run-1.step-100", recipe, factory)
    assert not pub.reused and sorted(os.listdir(pub.candidate_root)) == ["candidate.json", "hquant", "weights.safetensors"]
    assert 2.0 < pub.metrics["average_bits_per_weight"] < 16 and pub.metrics["weighted_mean_squared_error"] > 0
    assert [n for n in os.listdir(root) if n.startswith(".")] == []          # no staging left behind
    # an identical retry adopts the published candidate; other bytes or another recipe are refused
    again = C.publish(model, root, "run-1.step-100", recipe, factory)
    assert again.reused and again.candidate_manifest_sha256 == pub.candidate_manifest_sha256
    again2 = C.publish(model, root, "run-1.step-100", recipe, factory, source_weights_sha256=pub.weights_sha256)
    assert again2.reused
    with pytest.raises(C.CandidateError, match="different model weights"):
        C.publish(_model(1), root, "run-1.step-100", recipe, factory)
    with pytest.raises(C.CandidateError, match="different quantization recipe"):
        C.publish(model, root, "run-1.step-100", C.Recipe("binary_g128"), factory)
    for bad in ("", "a/b", "..", "x" * 129, "sp ace", "é"):
        with pytest.raises(C.CandidateError):
            C.publish(model, root, bad, recipe, factory)
    # reopen: full reproduction, and the addressed fast path bound to the sealed receipt identity
    assert C.open_candidate(pub.candidate_root, factory).weights_sha256 == pub.weights_sha256
    assert C.open_addressed(pub.candidate_root, pub.candidate_manifest_sha256).metrics == pub.metrics
    with pytest.raises(C.CandidateError):
        C.open_addressed(pub.candidate_root, "sha256:" + "0" * 64)
    # a crash before the rename exposes nothing
    def crash(point, staging):
        if point == "manifest_synced":
            raise RuntimeError("power loss")
    with pytest.raises(RuntimeError):
        C.publish(model, root, "run-2", recipe, factory, hook=crash)
    assert not os.path.exists(os.path.join(root, "run-2"))
    assert [n for n in os.listdir(root) if n.startswith(".")] == []


def test_qat_candidate_detects_a_self_consistent_forgery(tmp_path):
    """An archive member replaced by other valid codes, with every hash in the manifests redone,
    passes the hash checks but is not the encoding of the stored weights."""
    import hashlib
    from summa_b200.train import artifact_io as A
    from summa_b200.train import qat_candidate as C
    from summa_b200.train import quantization as Q
    root = str(tmp_path / "c")
    factory = lambda: _model(99)
    pub = C.publish(_model(0), root, "k", C.Recipe("binary_g128"), factory)
    arch = pub.archive_path
    man = json.load(open(os.path.join(arch, "archive-manifest.json")))
    ent = next(e for e in man["files"] if e["path"].endswith(".hquant"))
    pt = Q.PackedTensor.from_bytes(open(os.path.join(arch, ent["path"]), "rb").read())
    forged = Q.quantize_tensor(-pt.decode(), "binary_g128").to_bytes()
    open(os.path.join(arch, ent["path"]), "wb").write(forged)
    # plain tampering is caught by the member hash
    with pytest.raises(C.CandidateError):
        C.open_addressed(pub.candidate_root, pub.candidate_manifest_sha256)
    # now make everything self-consistent again
    ent["bytes"], ent["sha256"] = len(forged), hashlib.sha256(forged).hexdigest()
    mbytes = json.dumps(man, indent=2, sort_keys=True).encode()
    open(os.path.join(arch, "archive-manifest.json"), "wb").write(mbytes)
    receipt = json.load(open(pub.candidate_manifest_path))
    receipt["archive_manifest_sha256"] = A.sha256_identity(mbytes)
    receipt["archive_content_sha256"] = C._archive_content_identity(arch, man)
    open(pub.candidate_manifest_path, "w").write(json.dumps(receipt, sort_keys=True, indent=2))
    with pytest.raises(C.CandidateError):                                  # the sealed receipt identity changed
        C.open_addressed(pub.candidate_root, pub.candidate_manifest_sha256)
    with pytest.raises(C.CandidateError, match="not the encoding"):        # and reproduction exposes the codes
        C.open_candidate(pub.candidate_root, factory)
