// Native core of the byte-level BPE tokenizer: hand-written pre-tokenizer scanners for the common split
// pattern families and the merge loop, with a multi-threaded batch entry point.
//
// The reference tokenizer gets its speed from per-family pre-tokenizers instead of a regex engine and from
// parallel batch encoding (`summa-tokenizer/src/pretokenize/fast/*.rs`, `summa-tokenizer/src/lib.rs:40-172`).
// This file restates that design in C++:
//   * a UTF-8 decoder plus a class mask per code point (letter, number, white space, mark, upper/title case,
//     lower case, modifier/other letter, punctuation-or-symbol, Han) from one generated range table
//     (`unicode_tables.h`, ASCII through a 128-entry table),
//   * one scanner per family that reproduces the leftmost-first / greedy-with-backtracking semantics of the
//     family's pattern without a regex engine (`summa-tokenizer/src/pretokenize/options.rs:8-21,117-146`):
//       0  r50k / GPT-2   's|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+
//       1  cl100k, olmo3  (?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,3}|
//                          ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+
//       2  qwen2          cl100k with single digits (\p{N} instead of \p{N}{1,3})
//       3  whole text     no split (ByteLevel with use_regex = false)
//       4  qwen3.5        qwen2 with [\p{L}\p{M}]+ letter runs and marks excluded from punctuation runs
//       5  o200k          [^\r\n\p{L}\p{N}]?U*W+C?|[^\r\n\p{L}\p{N}]?U+W*C?|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n/]*|
//                         \s*[\r\n]+|\s+(?!\S)|\s+   with U = [\p{Lu}\p{Lt}\p{Lm}\p{Lo}\p{M}],
//                         W = [\p{Ll}\p{Lm}\p{Lo}\p{M}], C = (?i:'s|'t|'re|'ve|'m|'ll|'d)
//       6  nemotron       o200k without C, single digits
//       7  kimi           [\p{Han}]+ first, Han removed from U and W, no `/` in the punctuation tail
//       8  deepseek v3    three isolated splits in sequence: \p{N}{1,3}; CJK ideograph / kana runs; then
//                         [ascii punct][A-Za-z]+|[^\r\n\p{L}\p{P}\p{S}]?[\p{L}\p{M}]+| ?[\p{P}\p{S}]+[\r\n]*|
//                         \s*[\r\n]+|\s+(?!\S)|\s+   inside each piece; unmatched spans stay pieces
//   * byte-level BPE over token ids: a piece starts as one id per byte; the adjacent pair with the lowest merge
//     rank (leftmost on ties) is merged until none is left; pieces are cached per thread.
// The C ABI takes and returns plain arrays so that the Python side needs only ctypes.
#include <stdint.h>
#include <string.h>

#include <algorithm>
#include <string>
#include <thread>
#include <atomic>
#include <unordered_map>
#include <vector>

#include "unicode_tables.h"

namespace {

enum : uint16_t {
  C_LETTER = 1, C_NUMBER = 2, C_SPACE = 4, C_MARK = 8, C_UPPER = 16, C_LOWER = 32, C_NEUTRAL = 64, C_PUNCT = 128, C_HAN = 256,
  C_U = C_UPPER | C_NEUTRAL | C_MARK,       // [\p{Lu}\p{Lt}\p{Lm}\p{Lo}\p{M}]
  C_W = C_LOWER | C_NEUTRAL | C_MARK,       // [\p{Ll}\p{Lm}\p{Lo}\p{M}]
};
enum { F_R50K = 0, F_CL100K = 1, F_QWEN2 = 2, F_WHOLE = 3, F_QWEN35 = 4, F_O200K = 5, F_NEMOTRON = 6, F_KIMI = 7, F_DEEPSEEK = 8 };

uint16_t g_ascii[128];
std::atomic<bool> g_ascii_ready{false};

uint16_t classify_slow(uint32_t cp) {
  int lo = 0, hi = SBT_RANGE_COUNT - 1;
  while (lo <= hi) {
    const int mid = (lo + hi) >> 1;
    if (cp < SBT_RANGES[mid].lo) hi = mid - 1;
    else if (cp > SBT_RANGES[mid].hi) lo = mid + 1;
    else return SBT_RANGES[mid].mask;
  }
  return 0;
}

void init_ascii() {
  if (g_ascii_ready.load(std::memory_order_acquire)) return;
  for (uint32_t c = 0; c < 128; ++c) g_ascii[c] = classify_slow(c);     // every writer stores the same values
  g_ascii_ready.store(true, std::memory_order_release);
}

inline uint16_t classify(uint32_t cp) { return cp < 128 ? g_ascii[cp] : classify_slow(cp); }

// Decodes one code point at s[i] (i < n); malformed bytes decode as themselves so that the scanners always
// advance and every input byte ends up in exactly one piece.
inline uint32_t decode(const uint8_t* s, long n, long i, int* len) {
  const uint8_t b = s[i];
  if (b < 0x80) { *len = 1; return b; }
  if ((b >> 5) == 6 && i + 1 < n && (s[i + 1] & 0xC0) == 0x80) { *len = 2; return ((b & 0x1F) << 6) | (s[i + 1] & 0x3F); }
  if ((b >> 4) == 14 && i + 2 < n && (s[i + 1] & 0xC0) == 0x80 && (s[i + 2] & 0xC0) == 0x80) {
    *len = 3;
    return ((b & 0x0F) << 12) | ((s[i + 1] & 0x3F) << 6) | (s[i + 2] & 0x3F);
  }
  if ((b >> 3) == 30 && i + 3 < n && (s[i + 1] & 0xC0) == 0x80 && (s[i + 2] & 0xC0) == 0x80 && (s[i + 3] & 0xC0) == 0x80) {
    *len = 4;
    return ((b & 0x07) << 18) | ((s[i + 1] & 0x3F) << 12) | ((s[i + 2] & 0x3F) << 6) | (s[i + 3] & 0x3F);
  }
  *len = 1;
  return 0xFFFD;
}

inline bool deepseek_cjk(uint32_t cp) { return (cp >= 0x4E00 && cp <= 0x9FA5) || (cp >= 0x3040 && cp <= 0x30FF); }

// One text (or, for the DeepSeek family, one region of it: `n` is then the region's end, which the patterns
// see as the end of input).
struct Scanner {
  const uint8_t* s;
  long n;
  int family;
  long region_hi = 0;                          // DeepSeek: end of the region that holds the current position

  // class mask of the code point at i as THIS family sees it (Kimi: a Han code point is in neither U nor W)
  inline uint16_t cls(long i, int* len) const {
    const uint32_t cp = decode(s, n, i, len);
    uint16_t c = classify(cp);
    if (family == F_KIMI && (c & C_HAN)) c &= ~(C_U | C_W);
    return c;
  }
  // end of the run of code points with (class & any) != 0, starting at i and ending before `end`
  inline long run_any(long i, uint16_t any, long end) const {
    while (i < end) {
      int len;
      if (!(cls(i, &len) & any)) break;
      i += len;
    }
    return i;
  }
  inline long run_none(long i, uint16_t none, long end) const {
    while (i < end) {
      int len;
      if (cls(i, &len) & none) break;
      i += len;
    }
    return i;
  }

  long contraction(long i, long end) const {
    if (i >= end || s[i] != '\'' || i + 1 >= end) return 0;
    const bool fold = family != F_R50K;
    auto lower = [&](uint8_t c) -> uint8_t { return (fold && c >= 'A' && c <= 'Z') ? c + 32 : c; };
    const uint8_t a = lower(s[i + 1]);
    if (a == 's' || a == 't' || a == 'm' || a == 'd') return 2;
    if (i + 2 < end) {
      const uint8_t b = lower(s[i + 2]);
      if ((a == 'r' && b == 'e') || (a == 'v' && b == 'e') || (a == 'l' && b == 'l')) return 3;
    }
    return 0;
  }

  // \s+(?!\S) then \s+ : a white-space run that is followed by a non-space gives up its last code point
  // (unless that would leave nothing, in which case \s+ takes the whole run)
  long spaces(long i, long end) const {
    long e = i, last = i;
    while (e < end) {
      int len;
      if (!(cls(e, &len) & C_SPACE)) break;
      last = e;
      e += len;
    }
    if (e == i) return 0;
    if (e == end) return e - i;                 // followed by nothing: the look-ahead holds
    if (last > i) return last - i;              // keep all but the last white-space code point
    return e - i;                               // single white-space code point before a non-space: \s+
  }

  // \s*[\r\n]+ : the longest prefix of the white-space run that ends in a line break
  long newline_run(long i, long end) const {
    long e = i, best = 0;
    while (e < end) {
      int l2;
      const uint32_t cp = decode(s, end, e, &l2);
      if (!(classify(cp) & C_SPACE)) break;
      e += l2;
      if (cp == '\r' || cp == '\n') best = e - i;
    }
    return best;
  }

  //  ?[^\s <excluded>]+ <tail>*   with tail = [\r\n] or [\r\n/]
  long punct_run(long i, long end, uint16_t excluded, bool slash_tail) const {
    long j = i;
    if (s[i] == ' ' && i + 1 < end) j = i + 1;
    int l2;
    if (j < end && !(cls(j, &l2) & excluded)) {
      long e = run_none(j, excluded, end);
      while (e < end && (s[e] == '\r' || s[e] == '\n' || (slash_tail && s[e] == '/'))) ++e;
      return e - i;
    }
    return 0;
  }

  long digits(long i, int first_len, int max_digits, long end) const {
    long j = i + first_len;
    for (int d = 1; d < max_digits && j < end; ++d) {
      int l2;
      if (!(cls(j, &l2) & C_NUMBER)) break;
      j += l2;
    }
    return j - i;
  }

  long next_gpt2(long i) const {
    long c = contraction(i, n);
    if (c) return c;
    int len;
    long j = i;
    if (s[i] == ' ' && i + 1 < n) j = i + 1;    // optional single space of ` ?X+`
    if (j < n) {
      const uint16_t k = cls(j, &len);
      if (k & C_LETTER) return run_any(j, C_LETTER, n) - i;
      if (k & C_NUMBER) return run_any(j, C_NUMBER, n) - i;
      if (!(k & (C_SPACE | C_LETTER | C_NUMBER))) return run_none(j, C_SPACE | C_LETTER | C_NUMBER, n) - i;
    }
    return spaces(i, n);
  }

  // cl100k / olmo3 / qwen2 / qwen3.5: `word` is the class of a letter run (\p{L} or [\p{L}\p{M}])
  long next_cl100k(long i) const {
    long c = contraction(i, n);
    if (c) return c;
    const uint16_t word = family == F_QWEN35 ? (C_LETTER | C_MARK) : C_LETTER;
    int len;
    const uint32_t cp0 = decode(s, n, i, &len);
    const uint16_t k0 = classify(cp0);
    // [^\r\n\p{L}\p{N}]?<word>+ : a mark that opens a run is the same span with or without the prefix
    if (k0 & word) return run_any(i, word, n) - i;
    if (cp0 != '\r' && cp0 != '\n' && !(k0 & (C_LETTER | C_NUMBER)) && i + len < n) {
      int l2;
      if (cls(i + len, &l2) & word) return run_any(i + len, word, n) - i;
    }
    if (k0 & C_NUMBER) return digits(i, len, (family == F_QWEN2 || family == F_QWEN35) ? 1 : 3, n);
    if (long p = punct_run(i, n, C_SPACE | word | C_LETTER | C_NUMBER, false)) return p;
    if (k0 & C_SPACE) {
      if (long b = newline_run(i, n)) return b;
    }
    return spaces(i, n);
  }

  // o200k body `U*W+` at q: greedy U*, then W+ where the regex engine first finds it while U* gives code
  // points back. Returns the end of the match or -1.
  long o200k_lower_body(long q) const {
    long u_end = q, last_shared_end = -1;
    while (u_end < n) {
      int l;
      const uint16_t c = cls(u_end, &l);
      if (!(c & C_U)) break;
      u_end += l;
      if (c & C_W) last_shared_end = u_end;      // in both classes: W+ can start here after U* backs off
    }
    if (u_end < n) {
      int l;
      if (cls(u_end, &l) & C_W) return run_any(u_end, C_W, n);
    }
    return last_shared_end;                       // W+ takes exactly that code point (the next one is not in W)
  }
  // o200k body `U+W*` at q
  long o200k_upper_body(long q) const {
    const long u_end = run_any(q, C_U, n);
    if (u_end == q) return -1;
    return run_any(u_end, C_W, n);
  }

  long next_o200k(long i) const {
    int len;
    const uint16_t k0 = cls(i, &len);
    if (family == F_KIMI && (classify(decode(s, n, i, &len)) & C_HAN)) return run_any_han(i) - i;
    const uint32_t cp0 = decode(s, n, i, &len);
    const bool prefix_ok = cp0 != '\r' && cp0 != '\n' && !(classify(cp0) & (C_LETTER | C_NUMBER)) && i + len < n;
    const bool with_contraction = family != F_NEMOTRON;
    for (int alt = 0; alt < 2; ++alt) {
      for (int pre = prefix_ok ? 1 : 0; pre >= 0; --pre) {
        const long q = pre ? i + len : i;
        const long e = alt == 0 ? o200k_lower_body(q) : o200k_upper_body(q);
        if (e > q) return e + (with_contraction ? contraction(e, n) : 0) - i;
      }
    }
    if (k0 & C_NUMBER) return digits(i, len, family == F_NEMOTRON ? 1 : 3, n);
    if (long p = punct_run(i, n, C_SPACE | C_LETTER | C_NUMBER, family != F_KIMI)) return p;
    if (k0 & C_SPACE) {
      if (long b = newline_run(i, n)) return b;
    }
    return spaces(i, n);
  }
  long run_any_han(long i) const {
    while (i < n) {
      int l;
      if (!(classify(decode(s, n, i, &l)) & C_HAN)) break;
      i += l;
    }
    return i;
  }

  // DeepSeek main pattern at i inside a region that ends at `end`; 0 when no alternative matches
  long deepseek_main(long i, long end) const {
    int len;
    const uint32_t cp0 = decode(s, end, i, &len);
    const uint16_t k0 = classify(cp0);
    auto ascii_alpha = [](uint8_t c) { return (c >= 'A' && c <= 'Z') || (c >= 'a' && c <= 'z'); };
    if (cp0 < 128 && (k0 & C_PUNCT) && i + 1 < end && ascii_alpha(s[i + 1])) {      // the ASCII \p{P}\p{S} set is exactly the listed one
      long e = i + 2;
      while (e < end && ascii_alpha(s[e])) ++e;
      return e - i;
    }
    if (k0 & (C_LETTER | C_MARK)) return run_any(i, C_LETTER | C_MARK, end) - i;
    if (cp0 != '\r' && cp0 != '\n' && !(k0 & (C_LETTER | C_PUNCT)) && i + len < end) {
      int l2;
      if (classify(decode(s, end, i + len, &l2)) & (C_LETTER | C_MARK)) return run_any(i + len, C_LETTER | C_MARK, end) - i;
    }
    {
      long j = i;
      if (s[i] == ' ' && i + 1 < end) j = i + 1;
      int l2;
      if (j < end && (classify(decode(s, end, j, &l2)) & C_PUNCT)) {
        long e = run_any(j, C_PUNCT, end);
        while (e < end && (s[e] == '\r' || s[e] == '\n')) ++e;
        return e - i;
      }
    }
    if (k0 & C_SPACE) {
      if (long b = newline_run(i, end)) return b;
    }
    return spaces(i, end);
  }

  long next_deepseek(long i) {
    int len;
    const uint32_t cp0 = decode(s, n, i, &len);
    if (classify(cp0) & C_NUMBER) return digits(i, len, 3, n);      // stage 1; called at piece starts only, so i opens a group
    if (i >= region_hi) {                                            // stages 1 + 2: the region ends at a digit or where CJK-ness flips
      const bool cjk = deepseek_cjk(cp0);
      long e = i + len;
      while (e < n) {
        int l;
        const uint32_t cp = decode(s, n, e, &l);
        if ((classify(cp) & C_NUMBER) || deepseek_cjk(cp) != cjk) break;
        e += l;
      }
      region_hi = e;
    }
    long m = deepseek_main(i, region_hi);
    if (m > 0) return m;
    long j = i + len;                                                // an unmatched span lasts until the next match starts
    while (j < region_hi && deepseek_main(j, region_hi) == 0) {
      int l;
      decode(s, region_hi, j, &l);
      j += l;
    }
    return j - i;
  }

  long next(long i) {
    long len;
    switch (family) {
      case F_WHOLE: return n - i;
      case F_R50K: len = next_gpt2(i); break;
      case F_O200K: case F_NEMOTRON: case F_KIMI: len = next_o200k(i); break;
      case F_DEEPSEEK: len = next_deepseek(i); break;
      default: len = next_cl100k(i); break;
    }
    if (len <= 0) {          // a code point no alternative accepts cannot exist, but never stall
      int l;
      decode(s, n, i, &l);
      len = l;
    }
    return len;
  }
};

struct PairHash {
  size_t operator()(uint64_t k) const {
    k ^= k >> 33; k *= 0xff51afd7ed558ccdULL; k ^= k >> 33;
    return (size_t)k;
  }
};

struct Bpe {
  int32_t byte_to_id[256];
  std::unordered_map<uint64_t, uint64_t, PairHash> merges;    // (a << 32 | b) -> (rank << 32 | merged id)
  int family;
  // Distinguishes this table from every other one ever built in the process: a per-thread piece cache is
  // keyed by it, not by the object's address, which the allocator hands out again after sbt_free.
  uint64_t serial;
};

typedef std::unordered_map<std::string, std::vector<int32_t>> PieceCache;

void bpe_piece(const Bpe& t, const uint8_t* p, long len, PieceCache& cache, std::vector<int32_t>& out) {
  if (len == 1) { out.push_back(t.byte_to_id[p[0]]); return; }
  std::string key(reinterpret_cast<const char*>(p), (size_t)len);
  auto hit = cache.find(key);
  if (hit != cache.end()) { out.insert(out.end(), hit->second.begin(), hit->second.end()); return; }
  std::vector<int32_t> ids((size_t)len);
  for (long i = 0; i < len; ++i) ids[(size_t)i] = t.byte_to_id[p[i]];
  while (ids.size() > 1) {
    uint64_t best = ~0ULL;
    size_t at = 0;
    for (size_t i = 0; i + 1 < ids.size(); ++i) {
      auto m = t.merges.find(((uint64_t)(uint32_t)ids[i] << 32) | (uint32_t)ids[i + 1]);
      if (m != t.merges.end() && m->second < best) { best = m->second; at = i; }     // rank in the high word
    }
    if (best == ~0ULL) break;
    ids[at] = (int32_t)(best & 0xFFFFFFFFu);
    ids.erase(ids.begin() + (long)at + 1);
  }
  if (cache.size() < 400000) cache.emplace(std::move(key), ids);
  out.insert(out.end(), ids.begin(), ids.end());
}

void encode_text(const Bpe& t, const uint8_t* s, long n, PieceCache& cache, std::vector<int32_t>& out) {
  Scanner sc{s, n, t.family};
  long i = 0;
  while (i < n) {
    const long len = sc.next(i);
    bpe_piece(t, s + i, len, cache, out);
    i += len;
  }
}

}  // namespace

extern "C" {

// merges: n rows of (left id, right id, merged id), in rank order.
void* sbt_new(const int32_t* byte_to_id, const int32_t* merges, long n_merges, int family) {
  init_ascii();
  static std::atomic<uint64_t> next_serial{1};
  Bpe* t = new Bpe();
  t->serial = next_serial.fetch_add(1);
  memcpy(t->byte_to_id, byte_to_id, sizeof(t->byte_to_id));
  t->family = family;
  t->merges.reserve((size_t)n_merges * 2);
  for (long r = 0; r < n_merges; ++r) {
    const uint64_t key = ((uint64_t)(uint32_t)merges[3 * r] << 32) | (uint32_t)merges[3 * r + 1];
    // the first occurrence of a pair defines its rank
    t->merges.emplace(key, ((uint64_t)r << 32) | (uint32_t)merges[3 * r + 2]);
  }
  return t;
}

void sbt_free(void* h) { delete static_cast<Bpe*>(h); }

// Byte offsets of the pieces the family's pre-tokenizer cuts `text` into: out[0..count] with out[0] = 0.
// Returns the piece count, or -(needed entries) when `cap` is too small.
long sbt_split(void* h, const char* text, long len, long* out, long cap) {
  const Bpe& t = *static_cast<Bpe*>(h);
  Scanner sc{reinterpret_cast<const uint8_t*>(text), len, t.family};
  long i = 0, k = 0;
  if (cap > 0) out[0] = 0;
  while (i < len) {
    i += sc.next(i);
    ++k;
    if (k < cap) out[k] = i;
  }
  return k + 1 <= cap ? k : -(k + 1);
}

// Encodes one UTF-8 text. Returns the id count, or -(needed) when `cap` is too small.
long sbt_encode(void* h, const char* text, long len, int32_t* out, long cap) {
  const Bpe& t = *static_cast<Bpe*>(h);
  thread_local PieceCache cache;
  thread_local uint64_t owner = 0;
  if (owner != t.serial) { cache.clear(); owner = t.serial; }
  std::vector<int32_t> ids;
  ids.reserve((size_t)len / 3 + 8);
  encode_text(t, reinterpret_cast<const uint8_t*>(text), len, cache, ids);
  if ((long)ids.size() > cap) return -(long)ids.size();
  memcpy(out, ids.data(), ids.size() * sizeof(int32_t));
  return (long)ids.size();
}

// Encodes `n` texts (texts[i], lens[i]) on `threads` worker threads. `out_offsets` has n + 1 entries; the ids of
// text i end up at out[out_offsets[i] .. out_offsets[i+1]). Returns the total id count, or -(needed) when `cap` is
// too small (nothing is written then).
long sbt_encode_batch(void* h, const char* const* texts, const long* lens, long n, int32_t* out, long cap,
                      long* out_offsets, int threads) {
  const Bpe& t = *static_cast<Bpe*>(h);
  std::vector<std::vector<int32_t>> results((size_t)n);
  if (threads < 1) threads = 1;
  if ((long)threads > n) threads = (int)std::max<long>(n, 1);
  auto work = [&](int w) {
    PieceCache cache;
    for (long i = w; i < n; i += threads) {
      results[(size_t)i].reserve((size_t)lens[i] / 3 + 8);
      encode_text(t, reinterpret_cast<const uint8_t*>(texts[i]), lens[i], cache, results[(size_t)i]);
    }
  };
  if (threads == 1) {
    work(0);
  } else {
    std::vector<std::thread> pool;
    for (int w = 0; w < threads; ++w) pool.emplace_back(work, w);
    for (auto& th : pool) th.join();
  }
  long total = 0;
  for (long i = 0; i < n; ++i) total += (long)results[(size_t)i].size();
  if (total > cap) return -total;
  long pos = 0;
  for (long i = 0; i < n; ++i) {
    out_offsets[i] = pos;
    memcpy(out + pos, results[(size_t)i].data(), results[(size_t)i].size() * sizeof(int32_t));
    pos += (long)results[(size_t)i].size();
  }
  out_offsets[n] = pos;
  return total;
}

}  // extern "C"
