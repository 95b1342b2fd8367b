"""Byte-level BPE tokenizer that loads HuggingFace `tokenizer.json` files.

API parity with the reference tokenizer (`summa-tokenizer/src/lib.rs:40-172`):
`from_file`, `from_bytes`, `encode`, `encode_batch`, `decode`, `id_to_token`,
`token_to_id`, `vocab_size`; plus the EOS-name resolution of the model-side wrapper
(`summa-llm/src/tokenizer.rs:7-36`).

Encoding runs on a native core (`csrc/fast_bpe.cpp`, built by `summa_b200.tokenizer.build`): per-family
pre-tokenizer scanners (r50k / GPT-2, cl100k / olmo3, qwen2, qwen3.5, o200k, nemotron, kimi, deepseek v3) instead of a regex engine, the merge loop over token
ids, and a multi-threaded `encode_batch`, the design of `summa-tokenizer/src/pretokenize/fast/*.rs` and
`summa-tokenizer/src/lib.rs:40-172`. Split patterns outside those families, or a missing library, take the
pure-Python path below, which is also the oracle the native core is tested against.

Accepted files (`summa-tokenizer/src/hf.rs:156-185,237-240,341-398`): `model.type`
= BPE with a ByteLevel pre-tokenizer (optionally behind a Sequence with a Split
regex) and a ByteLevel decoder. Rejected: dropout, unk tokens, byte_fallback,
`single_word` added tokens, sparse ids, non-NFC normalizers.
"""
from __future__ import annotations

import json
import re
import unicodedata
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

try:  # the `regex` module understands \p{L}; `re` is the fallback for simple patterns
    import regex as _re
except Exception:  # pragma: no cover
    _re = re

EOS_CANDIDATES = ["<eos>", "<|endoftext|>", "</s>", "<|end_of_text|>", "<|eot_id|>"]

GPT2_SPLIT = r"""'(?:[sdmt]|ll|ve|re)| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+"""
# the split patterns of the families the native scanners implement, as they appear in tokenizer.json files
# (`summa-tokenizer/src/pretokenize/options.rs:23-30,117-146`)
R50K_SPLITS = (GPT2_SPLIT, r"""'s|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+""")
_CONTRACTIONS = r"""(?i:'s|'t|'re|'ve|'m|'ll|'d)"""
_TAIL = r"""|\s*[\r\n]+|\s+(?!\S)|\s+"""
CL100K_SPLIT = _CONTRACTIONS + r"""|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n]*""" + _TAIL
CL100K_SPLITS = (CL100K_SPLIT,                                  # also the dolma2 / olmo3 pattern
                 _CONTRACTIONS + r"""|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]|\s+(?!\S)|\s+""",
                 r"""'(?i:[sdmt]|ll|ve|re)|[^\r\n\p{L}\p{N}]?+\p{L}++|\p{N}{1,3}+| ?[^\s\p{L}\p{N}]++[\r\n]*+|\s++$|\s*[\r\n]|\s+(?!\S)|\s+""")
QWEN2_SPLIT = _CONTRACTIONS + r"""|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n]*""" + _TAIL
QWEN35_SPLIT = _CONTRACTIONS + r"""|[^\r\n\p{L}\p{N}]?[\p{L}\p{M}]+|\p{N}| ?[^\s\p{L}\p{M}\p{N}]+[\r\n]*""" + _TAIL
_U, _W = r"""[\p{Lu}\p{Lt}\p{Lm}\p{Lo}\p{M}]""", r"""[\p{Ll}\p{Lm}\p{Lo}\p{M}]"""
O200K_SPLIT = (rf"""[^\r\n\p{{L}}\p{{N}}]?{_U}*{_W}+{_CONTRACTIONS}?|[^\r\n\p{{L}}\p{{N}}]?{_U}+{_W}*{_CONTRACTIONS}?"""
               r"""|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n/]*""" + _TAIL)
NEMOTRON_SPLIT = (rf"""[^\r\n\p{{L}}\p{{N}}]?{_U}*{_W}+|[^\r\n\p{{L}}\p{{N}}]?{_U}+{_W}*"""
                  r"""|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n/]*""" + _TAIL)
_UH, _WH = r"""[\p{Lu}\p{Lt}\p{Lm}\p{Lo}\p{M}&&[^\p{Han}]]""", r"""[\p{Ll}\p{Lm}\p{Lo}\p{M}&&[^\p{Han}]]"""
KIMI_SPLIT = (rf"""[\p{{Han}}]+|[^\r\n\p{{L}}\p{{N}}]?{_UH}*{_WH}+{_CONTRACTIONS}?|[^\r\n\p{{L}}\p{{N}}]?{_UH}+{_WH}*{_CONTRACTIONS}?"""
              r"""|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n]*""" + _TAIL)
DEEPSEEK_V3_SPLITS = (
    r"\p{N}{1,3}",
    "[一-龥぀-ゟ゠-ヿ]+",
    "[!\"#$%&'()*+,\\-./:;<=>?@\\[\\\\\\]^_`{|}~][A-Za-z]+|[^\r\n\\p{L}\\p{P}\\p{S}]?[\\p{L}\\p{M}]+| ?[\\p{P}\\p{S}]+[\r\n]*"
    "|\\s*[\r\n]+|\\s+(?!\\S)|\\s+",
)
(FAMILY_R50K, FAMILY_CL100K, FAMILY_QWEN2, FAMILY_WHOLE, FAMILY_QWEN35, FAMILY_O200K, FAMILY_NEMOTRON, FAMILY_KIMI,
 FAMILY_DEEPSEEK_V3) = range(9)

# scheme names for vocabularies whose source format carries no split regex (tiktoken rank files), with the
# common aliases (`options.rs:70-101`); each maps to (family, ordered split patterns of the regex path)
SCHEMES = {
    "gpt2": (FAMILY_R50K, (GPT2_SPLIT,)), "gpt4": (FAMILY_CL100K, (CL100K_SPLIT,)), "qwen2": (FAMILY_QWEN2, (QWEN2_SPLIT,)),
    "qwen35": (FAMILY_QWEN35, (QWEN35_SPLIT,)), "olmo3": (FAMILY_CL100K, (CL100K_SPLIT,)),
    "deepseek_v3": (FAMILY_DEEPSEEK_V3, DEEPSEEK_V3_SPLITS), "o200k": (FAMILY_O200K, (O200K_SPLIT,)),
    "nemotron": (FAMILY_NEMOTRON, (NEMOTRON_SPLIT,)), "kimi": (FAMILY_KIMI, (KIMI_SPLIT,)),
}
SCHEMES["r50k"], SCHEMES["cl100k"] = SCHEMES["gpt2"], SCHEMES["gpt4"]


def split_family(pattern) -> Optional[int]:
    """Native scanner family of a split pattern (a string, or the ordered patterns of a Sequence of Splits), or
    None when only the regex path implements it."""
    if pattern is None or pattern == ():
        return FAMILY_WHOLE
    if isinstance(pattern, (tuple, list)):
        if len(pattern) != 1:
            return FAMILY_DEEPSEEK_V3 if tuple(pattern) == DEEPSEEK_V3_SPLITS else None
        pattern = pattern[0]
    if pattern in R50K_SPLITS:
        return FAMILY_R50K
    if pattern in CL100K_SPLITS:
        return FAMILY_CL100K
    for pat, fam in ((QWEN2_SPLIT, FAMILY_QWEN2), (QWEN35_SPLIT, FAMILY_QWEN35), (O200K_SPLIT, FAMILY_O200K),
                     (NEMOTRON_SPLIT, FAMILY_NEMOTRON), (KIMI_SPLIT, FAMILY_KIMI)):
        if pattern == pat:
            return fam
    return None


def _compile_split(pattern: str):
    # set intersection (`&&`, the Kimi pattern) needs the `regex` module's version-1 syntax
    return _re.compile("(?V1)" + pattern if "&&" in pattern and _re is not re else pattern)


def split_isolated(patterns, text: str) -> List[str]:
    """Pieces of `text` under a sequence of `Split` pre-tokenizers with the `Isolated` behaviour: every stage
    re-splits every piece of the stage before, matches and the spans between them both stay pieces."""
    pieces = [text]
    for rx in patterns:
        nxt: List[str] = []
        for piece in pieces:
            pos = 0
            for m in rx.finditer(piece):
                if m.end() == m.start():
                    continue
                if m.start() > pos:
                    nxt.append(piece[pos:m.start()])
                nxt.append(m.group(0))
                pos = m.end()
            if pos < len(piece):
                nxt.append(piece[pos:])
        pieces = nxt
    return pieces


_native_lib = None


def _native():
    """ctypes handle of the native core, or None when it has not been built."""
    global _native_lib
    if _native_lib is None:
        import ctypes
        import os
        path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "libsumma_tokenizer.so")
        if os.environ.get("SUMMA_TOKENIZER_NATIVE", "1") != "1" or not os.path.exists(path):
            _native_lib = False
        else:
            lib = ctypes.CDLL(path)
            P, L, I = ctypes.c_void_p, ctypes.c_long, ctypes.c_int
            lib.sbt_new.restype, lib.sbt_new.argtypes = P, [P, P, L, I]
            lib.sbt_free.restype, lib.sbt_free.argtypes = None, [P]
            lib.sbt_split.restype, lib.sbt_split.argtypes = L, [P, ctypes.c_char_p, L, P, L]
            lib.sbt_encode.restype, lib.sbt_encode.argtypes = L, [P, ctypes.c_char_p, L, P, L]
            lib.sbt_encode_batch.restype, lib.sbt_encode_batch.argtypes = L, [P, P, P, L, P, L, P, I]
            _native_lib = lib
    return _native_lib or None


def _bytes_to_unicode() -> Dict[int, str]:
    """GPT-2's reversible byte → printable-codepoint alphabet."""
    bs = list(range(ord("!"), ord("~") + 1)) + list(range(0xA1, 0xAC + 1)) + list(range(0xAE, 0xFF + 1))
    cs = bs[:]
    n = 0
    for b in range(256):
        if b not in bs:
            bs.append(b)
            cs.append(256 + n)
            n += 1
    return {b: chr(c) for b, c in zip(bs, cs)}


_B2U = _bytes_to_unicode()
_U2B = {v: k for k, v in _B2U.items()}


class TokenizerError(ValueError):
    pass


class Tokenizer:
    def __init__(self, vocab: Dict[str, int], merges: List[Tuple[str, str]], added: Dict[str, int],
                 split_pattern, add_prefix_space: bool = False, nfc: bool = False):
        self.vocab = vocab
        self.added = added
        size = max(list(vocab.values()) + list(added.values())) + 1
        self.id_to_tok: List[Optional[str]] = [None] * size
        for t, i in vocab.items():
            self.id_to_tok[i] = t
        for t, i in added.items():
            self.id_to_tok[i] = t
        if any(t is None for t in self.id_to_tok):
            raise TokenizerError("sparse token ids are not supported")
        self.ranks = {pair: r for r, pair in enumerate(merges)}
        if isinstance(split_pattern, str):
            split_pattern = (split_pattern,)
        split_pattern = tuple(split_pattern) if split_pattern else None
        self.splits = [_compile_split(p) for p in split_pattern] if split_pattern else None
        self.add_prefix_space = add_prefix_space
        self.nfc = nfc
        self._added_re = None
        if added:
            alts = sorted(added, key=len, reverse=True)
            self._added_re = re.compile("|".join(re.escape(a) for a in alts))
        self._cache: Dict[str, List[int]] = {}
        self.split_pattern = split_pattern
        self._handle = None
        self._init_native()

    def _init_native(self) -> None:
        """Hands the vocabulary to the native core as id tables: byte -> id and (left, right, merged) per
        merge in rank order. Vocabularies the id form cannot express (a byte or a merge result missing from
        the vocabulary) keep the Python path, which reports such files at encode time."""
        lib, family = _native(), split_family(self.split_pattern)
        if lib is None or family is None:
            return
        import ctypes
        try:
            byte_ids = [self.vocab[_B2U[b]] for b in range(256)]
            rows = []
            for (a, b), _ in sorted(self.ranks.items(), key=lambda kv: kv[1]):
                rows.extend((self.vocab[a], self.vocab[b], self.vocab[a + b]))
        except KeyError:
            return
        self._byte_ids = (ctypes.c_int32 * 256)(*byte_ids)
        self._merge_rows = (ctypes.c_int32 * max(len(rows), 1))(*rows)
        self._lib = lib
        self._handle = lib.sbt_new(self._byte_ids, self._merge_rows, len(rows) // 3, family)

    def __del__(self):
        h, self._handle = getattr(self, "_handle", None), None
        if h:
            try:
                self._lib.sbt_free(h)
            except Exception:
                pass

    @property
    def native(self) -> bool:
        return self._handle is not None

    # ------------------------------------------------------------------ construction
    @staticmethod
    def from_file(path: str) -> "Tokenizer":
        with open(path, "rb") as f:
            return Tokenizer.from_bytes(f.read())

    @staticmethod
    def from_bytes(data: bytes) -> "Tokenizer":
        try:
            cfg = json.loads(data.decode("utf-8"))
        except Exception as e:
            raise TokenizerError(f"invalid tokenizer.json: {e}")
        model = cfg.get("model") or {}
        if model.get("type") != "BPE":
            raise TokenizerError("only model.type = BPE is supported")
        if model.get("dropout"):
            raise TokenizerError("BPE dropout is not supported")
        if model.get("unk_token"):
            raise TokenizerError("unk_token is not supported (byte-level BPE never needs one)")
        if model.get("byte_fallback"):
            raise TokenizerError("byte_fallback is not supported")
        norm = cfg.get("normalizer")
        nfc = False
        if norm is not None:
            if norm.get("type") == "NFC":
                nfc = True
            else:
                raise TokenizerError(f"normalizer {norm.get('type')} is not supported (only NFC)")
        pre = cfg.get("pre_tokenizer") or {}
        split_pattern, add_prefix_space, byte_level = [], False, False
        pres = pre.get("pretokenizers", [pre]) if pre.get("type") == "Sequence" else [pre]
        for p in pres:
            if p.get("type") == "ByteLevel":
                byte_level = True
                add_prefix_space = bool(p.get("add_prefix_space", False))
                if p.get("use_regex", True):
                    split_pattern.append(GPT2_SPLIT)
            elif p.get("type") == "Split":
                pat = p.get("pattern", {})
                if p.get("behavior", "Isolated") != "Isolated" or p.get("invert", False):
                    raise TokenizerError("only Split pre-tokenizers with the Isolated behaviour are supported")
                split_pattern.append(pat.get("Regex") or re.escape(pat.get("String", "")))
            elif p:
                raise TokenizerError(f"pre-tokenizer {p.get('type')} is not supported")
        if not byte_level:
            raise TokenizerError("a ByteLevel pre-tokenizer is required")
        dec = cfg.get("decoder") or {}
        if dec.get("type") != "ByteLevel":
            raise TokenizerError("a ByteLevel decoder is required")
        vocab = {str(k): int(v) for k, v in model.get("vocab", {}).items()}
        merges = []
        for m in model.get("merges", []):
            if isinstance(m, str):
                a, _, b = m.partition(" ")
            else:
                a, b = m
            merges.append((a, b))
        added = {}
        for t in cfg.get("added_tokens", []):
            if t.get("single_word"):
                raise TokenizerError("single_word added tokens are not supported")
            added[t["content"]] = int(t["id"])
        return Tokenizer(vocab, merges, added, tuple(split_pattern), add_prefix_space, nfc)

    @staticmethod
    def with_scheme(vocab: Dict[str, int], merges: List[Tuple[str, str]], added: Dict[str, int], scheme: str) -> "Tokenizer":
        """A tokenizer whose source format carries no split regex (tiktoken rank files): the pre-tokenizer is
        named, `gpt2 | gpt4 | qwen2 | qwen35 | olmo3 | deepseek_v3 | o200k | nemotron | kimi` (aliases `r50k`,
        `cl100k`), as in `summa-tokenizer/src/pretokenize/options.rs:70-101`."""
        if scheme not in SCHEMES:
            raise TokenizerError(f"unknown pre-tokenizer scheme `{scheme}`; accepted: {', '.join(sorted(SCHEMES))}")
        return Tokenizer(vocab, merges, added, SCHEMES[scheme][1])

    @staticmethod
    def byte_level(with_eos: bool = True) -> "Tokenizer":
        """The smallest real vocabulary: ids 0..255 = the byte alphabet, 256 = `<eos>`."""
        vocab = {_B2U[b]: b for b in range(256)}
        added = {"<eos>": 256} if with_eos else {}
        return Tokenizer(vocab, [], added, None)

    def to_json(self) -> str:
        """A `tokenizer.json` that `from_bytes` (and HuggingFace tokenizers) can load."""
        merges = [f"{a} {b}" for (a, b), _ in sorted(self.ranks.items(), key=lambda kv: kv[1])]
        return json.dumps({
            "version": "1.0", "truncation": None, "padding": None,
            "added_tokens": [{"id": i, "content": t, "single_word": False, "lstrip": False, "rstrip": False,
                              "normalized": False, "special": True} for t, i in self.added.items()],
            "normalizer": {"type": "NFC"} if self.nfc else None,
            "pre_tokenizer": self._pre_tokenizer_json(),
            "post_processor": None,
            "decoder": {"type": "ByteLevel", "add_prefix_space": True, "trim_offsets": True, "use_regex": True},
            "model": {"type": "BPE", "dropout": None, "unk_token": None, "continuing_subword_prefix": None,
                      "end_of_word_suffix": None, "fuse_unk": False, "byte_fallback": False,
                      "vocab": self.vocab, "merges": merges},
        })

    def _pre_tokenizer_json(self) -> dict:
        byte_level = {"type": "ByteLevel", "add_prefix_space": self.add_prefix_space, "trim_offsets": True,
                      "use_regex": self.split_pattern == (GPT2_SPLIT,)}
        if self.split_pattern is None or byte_level["use_regex"]:
            return byte_level
        splits = [{"type": "Split", "pattern": {"Regex": p}, "behavior": "Isolated", "invert": False} for p in self.split_pattern]
        return {"type": "Sequence", "pretokenizers": splits + [byte_level]}

    # ------------------------------------------------------------------ queries
    def vocab_size(self) -> int:
        return len(self.id_to_tok)

    def id_to_token(self, i: int) -> Optional[str]:
        return self.id_to_tok[i] if 0 <= i < len(self.id_to_tok) else None

    def token_to_id(self, t: str) -> Optional[int]:
        if t in self.added:
            return self.added[t]
        return self.vocab.get(t)

    def eos_id(self) -> Optional[int]:
        for name in EOS_CANDIDATES:
            i = self.token_to_id(name)
            if i is not None:
                return i
        return None

    # ------------------------------------------------------------------ encode / decode
    def _bpe(self, word: str) -> List[int]:
        hit = self._cache.get(word)
        if hit is not None:
            return hit
        parts = list(word)
        while len(parts) > 1:
            best, best_rank = None, None
            for i in range(len(parts) - 1):
                r = self.ranks.get((parts[i], parts[i + 1]))
                if r is not None and (best_rank is None or r < best_rank):
                    best, best_rank = i, r
            if best is None:
                break
            a, b = parts[best], parts[best + 1]
            merged, i = [], 0
            while i < len(parts):
                if i < len(parts) - 1 and parts[i] == a and parts[i + 1] == b:
                    merged.append(a + b)
                    i += 2
                else:
                    merged.append(parts[i])
                    i += 1
            parts = merged
        try:
            ids = [self.vocab[p] for p in parts]
        except KeyError as e:
            raise TokenizerError(f"token {e} missing from the vocabulary")
        if len(self._cache) < 200000:
            self._cache[word] = ids
        return ids

    def _encode_native(self, data: bytes) -> List[int]:
        import ctypes
        cap = len(data) + 8                                  # a piece never yields more ids than bytes
        buf = (ctypes.c_int32 * cap)()
        n = self._lib.sbt_encode(self._handle, data, len(data), buf, cap)
        if n < 0:
            raise TokenizerError("native encoder overflowed its output buffer")
        return buf[:n]

    def _encode_plain(self, text: str, out: List[int]) -> None:
        if not text:
            return
        if self.nfc:
            text = unicodedata.normalize("NFC", text)
        if self._handle is not None:
            out.extend(self._encode_native(text.encode("utf-8", errors="replace")))
            return
        pieces = split_isolated(self.splits, text) if self.splits is not None else [text]
        for piece in pieces:
            out.extend(self._bpe("".join(_B2U[b] for b in piece.encode("utf-8"))))

    def encode(self, text: str, add_special_tokens: bool = False) -> List[int]:
        if self.add_prefix_space and text and not text.startswith(" "):
            text = " " + text
        out: List[int] = []
        if self._added_re is None:
            self._encode_plain(text, out)
            return out
        pos = 0
        for m in self._added_re.finditer(text):
            self._encode_plain(text[pos:m.start()], out)
            out.append(self.added[m.group(0)])
            pos = m.end()
        self._encode_plain(text[pos:], out)
        return out

    def encode_batch(self, texts: Sequence[str], add_special_tokens: bool = False,
                     threads: Optional[int] = None) -> List[List[int]]:
        """Encodes many texts; with the native core (and no added tokens inside the texts) the batch is cut
        over worker threads, results stay in input order."""
        if self._handle is None or not texts:
            return [self.encode(t, add_special_tokens) for t in texts]
        import ctypes
        import os
        plain, slots = [], []
        out: List[Optional[List[int]]] = [None] * len(texts)
        for i, t in enumerate(texts):
            if (self._added_re is not None and self._added_re.search(t)) or not t:
                out[i] = self.encode(t, add_special_tokens)
                continue
            if self.add_prefix_space and not t.startswith(" "):
                t = " " + t
            if self.nfc:
                t = unicodedata.normalize("NFC", t)
            plain.append(t.encode("utf-8", errors="replace"))
            slots.append(i)
        if plain:
            n = len(plain)
            ptrs = (ctypes.c_char_p * n)(*plain)
            lens = (ctypes.c_long * n)(*[len(b) for b in plain])
            cap = sum(len(b) for b in plain) + 8
            buf = (ctypes.c_int32 * cap)()
            offs = (ctypes.c_long * (n + 1))()
            workers = threads if threads is not None else min(32, os.cpu_count() or 1)
            total = self._lib.sbt_encode_batch(self._handle, ptrs, lens, n, buf, cap, offs, workers)
            if total < 0:
                raise TokenizerError("native batch encoder overflowed its output buffer")
            for k, i in enumerate(slots):
                out[i] = buf[offs[k]:offs[k + 1]]
        return out      # type: ignore[return-value]

    def split_offsets(self, text: str) -> List[int]:
        """Byte offsets of the pre-tokenizer's pieces (native core only); used by the differential tests."""
        import ctypes
        data = text.encode("utf-8", errors="replace")
        cap = len(data) + 2
        buf = (ctypes.c_long * cap)()
        n = self._lib.sbt_split(self._handle, data, len(data), buf, cap)
        return list(buf[:n + 1])

    def decode(self, ids: Iterable[int], skip_special_tokens: bool = False) -> str:
        buf = bytearray()
        added_ids = set(self.added.values())
        for i in ids:
            tok = self.id_to_token(int(i))
            if tok is None:
                raise TokenizerError(f"token id {i} out of range")
            if int(i) in added_ids:
                if not skip_special_tokens:
                    buf.extend(tok.encode("utf-8"))
                continue
            for ch in tok:
                b = _U2B.get(ch)
                if b is None:
                    buf.extend(ch.encode("utf-8"))
                else:
                    buf.append(b)
        return buf.decode("utf-8", errors="replace")
