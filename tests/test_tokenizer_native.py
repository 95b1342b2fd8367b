"""Native tokenizer core against its two oracles: the regex + Python merge loop of this package, and
HuggingFace `tokenizers` on a freshly trained byte-level BPE (the reference's differential-test method,
`summa-tokenizer/tests/parity.rs`)."""
import json
import os
import random

import pytest

from summa_b200 import tokenizer as T
from summa_b200.tokenizer import (CL100K_SPLIT, DEEPSEEK_V3_SPLITS, GPT2_SPLIT, O200K_SPLIT, QWEN2_SPLIT, QWEN35_SPLIT,
                                  Tokenizer, _native)

pytestmark = pytest.mark.skipif(_native() is None, reason="native tokenizer core not built")

PIECES = list("abcdefgXYZ 0123456789  \t\n\r'.,!?-_()é中文ßÑ١٢　 ") + [
    "'s", "'re", "'LL", "  ", "\r\n", "\n\n", " 12345", "don't", "Hello", " world", "über", "naïve", "日本語", "🙂", " the", "ing"]
# what separates the newer families: combining marks, title-case / modifier / other letters, letter-like numbers,
# Han non-letters, kana and the non-letters inside the kana block, control and format characters, `/` tails
HARD_PIECES = PIECES + ["\u0301", "\u0300\u0301", "\u01c5", "\u02b0", "\u00aa", "\u2180", "\u3007", "\u3005", "\u2e80", "カタカナ", "ひら",
                        "\u309b", "\u30a0", "\u30fb", "\u3040", "\x01", "\u200d", "\x7f", "McDonald", "HTTPServer", "iPhone", "A", "b",
                        "'S", "'T", "$", "+", "€", "//", "/\n", "한글", "İ", "\u0e31", "\u0e01", "½", "²", "\u9fa5", "\u9fa6"]


def _texts(n, seed, lo=1, hi=40):
    rnd = random.Random(seed)
    return ["".join(rnd.choice(PIECES) for _ in range(rnd.randint(lo, hi))) for _ in range(n)]


def _hard_texts(n, seed, lo=1, hi=24):
    rnd = random.Random(seed)
    return ["".join(rnd.choice(HARD_PIECES) for _ in range(rnd.randint(lo, hi))) for _ in range(n)]


def _train(tmp_path, split):
    tk = pytest.importorskip("tokenizers")
    from tokenizers import Regex, Tokenizer as HfTokenizer, decoders, models, pre_tokenizers, trainers
    hf = HfTokenizer(models.BPE())
    if split is None:
        hf.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=True)
    else:
        splits = [split] if isinstance(split, str) else list(split)
        hf.pre_tokenizer = pre_tokenizers.Sequence(
            [pre_tokenizers.Split(Regex(p), behavior="isolated", invert=False) for p in splits]
            + [pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False)])
    hf.decoder = decoders.ByteLevel()
    trainer = trainers.BpeTrainer(vocab_size=600, special_tokens=["<|endoftext|>"],
                                  initial_alphabet=pre_tokenizers.ByteLevel.alphabet(), show_progress=False)
    hf.train_from_iterator(_texts(3000, 1, 5, 80), trainer)
    path = str(tmp_path / "tokenizer.json")
    hf.save(path)
    return hf, path


@pytest.mark.parametrize("split", [None, CL100K_SPLIT, QWEN2_SPLIT, QWEN35_SPLIT, O200K_SPLIT, DEEPSEEK_V3_SPLITS],
                         ids=["gpt2", "cl100k", "qwen2", "qwen35", "o200k", "deepseek_v3"])
def test_native_matches_huggingface_and_python_paths(tmp_path, split, monkeypatch):
    hf, path = _train(tmp_path, split)
    ours = Tokenizer.from_file(path)
    assert ours.native and ours.vocab_size() == hf.get_vocab_size()
    texts = _texts(1500, 2) + _hard_texts(500, 5) + ["", " ", "\n", "a", "<|endoftext|>", "x<|endoftext|>y  z", "tab\tand  spaces   end "]
    oracle = Tokenizer.from_file(path)
    oracle._handle = None                                  # the regex + Python merge loop
    for t in texts:
        got = ours.encode(t)
        assert got == oracle.encode(t), repr(t)
        assert got == hf.encode(t, add_special_tokens=False).ids, repr(t)
        assert ours.decode(got) == t
    batch = ours.encode_batch(texts, threads=4)
    assert [list(b) for b in batch] == [ours.encode(t) for t in texts]      # input order, same ids


def test_split_offsets_cover_the_text_and_respect_families():
    base = Tokenizer.byte_level()
    for pat in (GPT2_SPLIT, CL100K_SPLIT, QWEN2_SPLIT):
        tk = Tokenizer(dict(base.vocab), [], {}, pat)
        import regex
        rx = regex.compile(pat)
        for s in _texts(3000, 3, 1, 24):
            data = s.encode()
            offs = tk.split_offsets(s)
            assert offs[0] == 0 and offs[-1] == len(data)
            assert [data[a:b].decode() for a, b in zip(offs, offs[1:])] == [m.group(0) for m in rx.finditer(s)], repr(s)
    digits = Tokenizer(dict(base.vocab), [], {}, QWEN2_SPLIT).split_offsets("12345")
    assert digits == [0, 1, 2, 3, 4, 5]
    assert Tokenizer(dict(base.vocab), [], {}, CL100K_SPLIT).split_offsets("12345") == [0, 3, 5]


@pytest.mark.parametrize("scheme", ["gpt2", "gpt4", "qwen2", "qwen35", "olmo3", "deepseek_v3", "o200k", "nemotron", "kimi"])
def test_every_named_scheme_splits_like_its_regexes(scheme):
    """The hand-written scanner of every family against the `regex` module running the family's own patterns
    (a sequence of isolated splits for DeepSeek), on text that mixes the code-point classes the families
    disagree on."""
    base = Tokenizer.byte_level()
    tk = Tokenizer.with_scheme(dict(base.vocab), [], {}, scheme)
    assert tk.native
    for s in _hard_texts(6000, 17):
        data = s.encode()
        offs = tk.split_offsets(s)
        assert offs[0] == 0 and offs[-1] == len(data)
        assert [data[a:b].decode() for a, b in zip(offs, offs[1:])] == T.split_isolated(tk.splits, s), repr(s)


def test_family_specific_cuts_and_round_trip():
    base = Tokenizer.byte_level()

    def cut(scheme, text):
        tk = Tokenizer.with_scheme(dict(base.vocab), [], {}, scheme)
        offs, data = tk.split_offsets(text), text.encode()
        return [data[a:b].decode() for a, b in zip(offs, offs[1:])]

    assert cut("o200k", "HTTPServer's McDonald") == ["HTTPServer's", " Mc", "Donald"]          # case structure + attached contraction
    assert cut("gpt4", "HTTPServer's McDonald") == ["HTTPServer", "'s", " McDonald"]
    assert cut("nemotron", "it's 123") == ["it", "'s", " ", "1", "2", "3"]
    assert cut("o200k", "a.\n/b") == ["a", ".\n/", "b"] and cut("kimi", "a.\n/b") == ["a", ".\n", "/b"]      # `/` in the tail or not
    assert cut("kimi", "汉字abc汉") == ["汉字", "abc", "汉"] and cut("o200k", "汉字abc汉") == ["汉字abc汉"]
    assert cut("deepseek_v3", "ab1234中文カナ x\x01\x01!") == ["ab", "123", "4", "中文カナ", " x", "\x01\x01", "!"]
    assert cut("qwen35", "e\u0301a..\u0301") == ["e\u0301a", "..", "\u0301"] and cut("qwen2", "e\u0301a..\u0301") == ["e", "\u0301a", "..\u0301"]
    with pytest.raises(T.TokenizerError, match="unknown pre-tokenizer scheme"):
        Tokenizer.with_scheme(dict(base.vocab), [], {}, "gpt5")
    for scheme in ("o200k", "deepseek_v3", "qwen35"):                                         # the patterns survive to_json
        tk = Tokenizer.with_scheme(dict(base.vocab), [], {}, scheme)
        again = Tokenizer.from_bytes(tk.to_json().encode())
        assert again.split_pattern == tk.split_pattern and again.native


def test_unknown_split_patterns_keep_the_regex_path():
    base = Tokenizer.byte_level()
    tk = Tokenizer(dict(base.vocab), [], {}, r"\w+|\W+")
    assert not tk.native and tk.encode("ab cd") == list(b"ab cd")


def test_piece_cache_is_not_shared_between_tables_that_reuse_an_address():
    """The per-thread piece cache belongs to one merge table: a table freed and another allocated at the same
    address must not see the first one's pieces."""
    base = Tokenizer.byte_level()
    a_id, b_id = base.vocab[base_token("a")], base.vocab[base_token("b")]
    for round_ in range(50):
        merged = dict(base.vocab)
        merged["ab"] = len(merged)
        with_merge = Tokenizer(merged, [("a", "b")], {}, GPT2_SPLIT)
        assert with_merge.native and with_merge.encode("ab") == [merged["ab"]]
        del with_merge                                     # sbt_free: the next table may land on the same address
        without = Tokenizer(dict(base.vocab), [], {}, GPT2_SPLIT)
        assert without.encode("ab") == [a_id, b_id], round_


def base_token(ch):
    return ch          # printable ASCII maps to itself in the byte-level alphabet
