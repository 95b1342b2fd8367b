// Native core of the byte-level BPE tokenizer: hand-written pre-tokenizer scanners for the common split
// pattern families and the merge loop, with a multi-threaded batch entry point.
//
// The reference tokenizer gets its speed from per-family pre-tokenizers instead of a regex engine and from
// parallel batch encoding (`summa-tokenizer/src/pretokenize/fast/*.rs`, `summa-tokenizer/src/lib.rs:40-172`).
// This file restates that design in C++:
//   * a UTF-8 decoder plus three code-point classes (letter, number, white space) from generated range
//     tables (`unicode_tables.h`, ASCII through a 128-entry table),
//   * one scanner per family that reproduces the leftmost-first / greedy-with-backtracking semantics of the
//     family's pattern without a regex engine:
//       0  r50k / GPT-2   's|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+
//       1  cl100k         (?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,3}|
//                          ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+
//       2  qwen2          cl100k with single digits (\p{N} instead of \p{N}{1,3})
//       3  whole text     no split (ByteLevel with use_regex = false)
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

enum : uint8_t { C_LETTER = 1, C_NUMBER = 2, C_SPACE = 4 };

uint8_t g_ascii[128];
bool g_ascii_ready = false;

bool in_ranges(const uint32_t (*r)[2], int n, uint32_t cp) {
  int lo = 0, hi = n - 1;
  while (lo <= hi) {
    const int mid = (lo + hi) >> 1;
    if (cp < r[mid][0]) hi = mid - 1;
    else if (cp > r[mid][1]) lo = mid + 1;
    else return true;
  }
  return false;
}

uint8_t classify_slow(uint32_t cp) {
  uint8_t c = 0;
  if (in_ranges(SBT_LETTER_RANGES, SBT_LETTER_COUNT, cp)) c |= C_LETTER;
  if (in_ranges(SBT_NUMBER_RANGES, SBT_NUMBER_COUNT, cp)) c |= C_NUMBER;
  if (in_ranges(SBT_SPACE_RANGES, SBT_SPACE_COUNT, cp)) c |= C_SPACE;
  return c;
}

void init_ascii() {
  if (g_ascii_ready) return;
  for (uint32_t c = 0; c < 128; ++c) g_ascii[c] = classify_slow(c);
  g_ascii_ready = true;
}

inline uint8_t classify(uint32_t cp) { return cp < 128 ? g_ascii[cp] : classify_slow(cp); }

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

struct Scanner {
  const uint8_t* s;
  long n;
  int family;

  inline uint8_t cls(long i, int* len) const {
    const uint32_t cp = decode(s, n, i, len);
    return classify(cp);
  }
  // end of the run of code points whose class satisfies `want` (mask any) starting at i
  template <class Pred>
  inline long run(long i, Pred pred) const {
    while (i < n) {
      int len;
      const uint32_t cp = decode(s, n, i, &len);
      if (!pred(cp, classify(cp))) break;
      i += len;
    }
    return i;
  }

  long contraction(long i) const {
    if (s[i] != '\'' || i + 1 >= n) return 0;
    const bool fold = family != 0;
    auto lower = [&](uint8_t c) -> uint8_t { return (fold && c >= 'A' && c <= 'Z') ? c + 32 : c; };
    const uint8_t a = lower(s[i + 1]);
    if (a == 's' || a == 't' || a == 'm' || a == 'd') return 2;
    if (i + 2 < n) {
      const uint8_t b = lower(s[i + 2]);
      if ((a == 'r' && b == 'e') || (a == 'v' && b == 'e') || (a == 'l' && b == 'l')) return 3;
    }
    return 0;
  }

  // \s+(?!\S) then \s+ : a white-space run that is followed by a non-space gives up its last code point
  // (unless that would leave nothing, in which case \s+ takes the whole run)
  long spaces(long i) const {
    long end = i, last = i;
    while (end < n) {
      int len;
      if (!(cls(end, &len) & C_SPACE)) break;
      last = end;
      end += len;
    }
    if (end == i) return 0;
    if (end == n) return end - i;               // followed by nothing: the look-ahead holds
    if (last > i) return last - i;              // keep all but the last white-space code point
    return end - i;                             // single white-space code point before a non-space: \s+
  }

  long next_gpt2(long i) const {
    long c = contraction(i);
    if (c) return c;
    int len;
    long j = i;
    if (s[i] == ' ' && i + 1 < n) j = i + 1;    // optional single space of ` ?X+`
    if (j < n) {
      const uint8_t k = cls(j, &len);
      if (k & C_LETTER) return run(j, [](uint32_t, uint8_t c) { return (c & C_LETTER) != 0; }) - i;
      if (k & C_NUMBER) return run(j, [](uint32_t, uint8_t c) { return (c & C_NUMBER) != 0; }) - i;
      if (!(k & (C_SPACE | C_LETTER | C_NUMBER)))
        return run(j, [](uint32_t, uint8_t c) { return (c & (C_SPACE | C_LETTER | C_NUMBER)) == 0; }) - i;
    }
    return spaces(i);
  }

  long next_cl100k(long i) const {
    long c = contraction(i);
    if (c) return c;
    int len;
    const uint32_t cp0 = decode(s, n, i, &len);
    const uint8_t k0 = classify(cp0);
    // [^\r\n\p{L}\p{N}]?\p{L}+
    if (k0 & C_LETTER) return run(i, [](uint32_t, uint8_t c) { return (c & C_LETTER) != 0; }) - i;
    if (cp0 != '\r' && cp0 != '\n' && !(k0 & C_NUMBER) && i + len < n) {
      int l2;
      if (cls(i + len, &l2) & C_LETTER) return run(i + len, [](uint32_t, uint8_t c) { return (c & C_LETTER) != 0; }) - i;
    }
    // \p{N}{1,3}  (qwen2: exactly one)
    if (k0 & C_NUMBER) {
      long j = i + len;
      const int max_digits = family == 2 ? 1 : 3;
      for (int d = 1; d < max_digits && j < n; ++d) {
        int l2;
        if (!(cls(j, &l2) & C_NUMBER)) break;
        j += l2;
      }
      return j - i;
    }
    //  ?[^\s\p{L}\p{N}]+[\r\n]*
    {
      long j = i;
      if (s[i] == ' ' && i + 1 < n) j = i + 1;
      int l2;
      if (j < n && !(cls(j, &l2) & (C_SPACE | C_LETTER | C_NUMBER))) {
        long e = run(j, [](uint32_t, uint8_t c) { return (c & (C_SPACE | C_LETTER | C_NUMBER)) == 0; });
        while (e < n && (s[e] == '\r' || s[e] == '\n')) ++e;
        return e - i;
      }
    }
    // \s*[\r\n]+ : the longest prefix of the white-space run that ends in a line break
    if (k0 & C_SPACE) {
      long end = i, best = 0;
      while (end < n) {
        int l2;
        const uint32_t cp = decode(s, n, end, &l2);
        if (!(classify(cp) & C_SPACE)) break;
        end += l2;
        if (cp == '\r' || cp == '\n') best = end - i;
      }
      if (best) return best;
    }
    return spaces(i);
  }

  long next(long i) const {
    if (family == 3) return n - i;
    long len = family == 0 ? next_gpt2(i) : next_cl100k(i);
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
