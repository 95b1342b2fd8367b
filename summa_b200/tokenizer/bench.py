"""Tokenizer throughput: `python -m summa_b200.tokenizer.bench [--tokenizer tokenizer.json] [--mib 16]`.

Encodes synthetic English-like text (or `--text FILE`) and prints one JSON line with MiB/s for the native core
(one thread and all threads), the pure-Python path, and HuggingFace `tokenizers` when it is importable. Without
`--tokenizer` a 2,000-entry byte-level BPE is trained on the spot (needs `tokenizers`). The reference's published
figure for the same kind of measurement is 22.71 MiB/s against 16.33 MiB/s for HuggingFace
(`docs/tokenizer-backends.md:39-40`)."""
from __future__ import annotations

import argparse
import json
import os
import random
import tempfile
import time


def _corpus(mib: float, seed: int = 0):
    rnd = random.Random(seed)
    words = ["the", "of", "and", "to", "in", "model", "training", "tokens", "attention", "state", "space", "gradient",
             "B200", "2026", "3.14", "don't", "it's", "über", "naïve", "data", "parallel", "kernel", "memory", "\n", ",", "."]
    docs, size = [], 0
    while size < mib * (1 << 20):
        d = " ".join(rnd.choice(words) for _ in range(rnd.randint(200, 1200)))
        docs.append(d)
        size += len(d.encode())
    return docs, size


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--tokenizer")
    ap.add_argument("--text")
    ap.add_argument("--mib", type=float, default=16.0)
    ap.add_argument("--python-mib", type=float, default=1.0, help="amount of text for the (slow) pure-Python path")
    a = ap.parse_args(argv)
    from . import Tokenizer
    if a.text:
        raw = open(a.text, encoding="utf-8", errors="replace").read()
        docs = [raw[i:i + 8192] for i in range(0, len(raw), 8192)]
        size = len(raw.encode())
    else:
        docs, size = _corpus(a.mib)
    hf = None
    path = a.tokenizer
    if path is None:
        from tokenizers import Tokenizer as HfTokenizer, decoders, models, pre_tokenizers, trainers
        hf = HfTokenizer(models.BPE())
        hf.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=True)
        hf.decoder = decoders.ByteLevel()
        hf.train_from_iterator(docs[:200], trainers.BpeTrainer(vocab_size=2000, show_progress=False,
                                                               initial_alphabet=pre_tokenizers.ByteLevel.alphabet()))
        path = os.path.join(tempfile.mkdtemp(), "tokenizer.json")
        hf.save(path)
    else:
        try:
            from tokenizers import Tokenizer as HfTokenizer
            hf = HfTokenizer.from_file(path)
        except Exception:
            hf = None
    tok = Tokenizer.from_file(path)
    out = {"bytes": size, "documents": len(docs), "native": tok.native, "cpus": os.cpu_count()}
    mib = size / (1 << 20)
    if tok.native:
        t0 = time.perf_counter()
        n1 = sum(len(x) for x in tok.encode_batch(docs, threads=1))
        out["native_1_thread_mib_s"] = round(mib / (time.perf_counter() - t0), 2)
        t0 = time.perf_counter()
        n2 = sum(len(x) for x in tok.encode_batch(docs))
        out["native_all_threads_mib_s"] = round(mib / (time.perf_counter() - t0), 2)
        assert n1 == n2
        out["tokens"] = n1
    py = Tokenizer.from_file(path)
    py._handle = None
    sub, sub_bytes = [], 0
    for d in docs:
        if sub_bytes >= a.python_mib * (1 << 20):
            break
        sub.append(d)
        sub_bytes += len(d.encode())
    t0 = time.perf_counter()
    for d in sub:
        py.encode(d)
    out["python_path_mib_s"] = round(sub_bytes / (1 << 20) / (time.perf_counter() - t0), 2)
    if hf is not None:
        t0 = time.perf_counter()
        hf.encode_batch(docs, add_special_tokens=False)
        out["huggingface_batch_mib_s"] = round(mib / (time.perf_counter() - t0), 2)
        t0 = time.perf_counter()
        for d in docs[:max(1, len(docs) // 8)]:
            hf.encode(d, add_special_tokens=False)
        out["huggingface_1_thread_mib_s"] = round(sum(len(d.encode()) for d in docs[:max(1, len(docs) // 8)]) / (1 << 20)
                                                  / (time.perf_counter() - t0), 2)
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
