// Tokenizers for GGUF checkpoints: byte-level BPE (GPT-2 byte map + merge ranks) with the qwen2,
// llama-bpe / dbrx and case-aware (tekken, gpt-4o / o200k) pre-tokenizers, raw-UTF-8 BPE (Gemma) and
// classic SentencePiece score merging (tokenizer.ggml.model == "llama"), special-token splitting and
// UTF-8-safe decoding.
//
// Reference parity: src/tokenizer/tokenizer.cpp:58-726 (byte map, merge ranks, pre-tokenizers,
// ignore_merges, SPM, special tokens, decode with keep_special).  Own implementation: the
// pre-tokenizers are hand-written scanners over decoded code points with a compact Unicode class
// table instead of the reference's regex-shaped character tests.
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <limits>
#include <queue>
#include <string>
#include <string_view>
#include <unordered_map>
#include <unordered_set>
#include <vector>

namespace {

// ---- UTF-8 helpers -----------------------------------------------------------------------------
inline int utf8_len(unsigned char c) { return c < 0x80 ? 1 : (c >> 5) == 6 ? 2 : (c >> 4) == 14 ? 3 : (c >> 3) == 30 ? 4 : 1; }
inline uint32_t utf8_decode(const char* s, size_t n, int& len) {
  unsigned char c = (unsigned char)s[0];
  len = utf8_len(c);
  if ((size_t)len > n) { len = 1; return c; }
  if (len == 1) return c;
  uint32_t cp = c & (0xFF >> (len + 1));
  for (int i = 1; i < len; ++i) {
    if (((unsigned char)s[i] & 0xC0) != 0x80) { len = 1; return c; }
    cp = (cp << 6) | ((unsigned char)s[i] & 0x3F);
  }
  return cp;
}
inline void utf8_append(std::string& out, uint32_t cp) {
  if (cp < 0x80) out.push_back((char)cp);
  else if (cp < 0x800) { out.push_back((char)(0xC0 | (cp >> 6))); out.push_back((char)(0x80 | (cp & 0x3F))); }
  else if (cp < 0x10000) { out.push_back((char)(0xE0 | (cp >> 12))); out.push_back((char)(0x80 | ((cp >> 6) & 0x3F))); out.push_back((char)(0x80 | (cp & 0x3F))); }
  else { out.push_back((char)(0xF0 | (cp >> 18))); out.push_back((char)(0x80 | ((cp >> 12) & 0x3F))); out.push_back((char)(0x80 | ((cp >> 6) & 0x3F))); out.push_back((char)(0x80 | (cp & 0x3F))); }
}

// ---- coarse Unicode classes ----------------------------------------------------------------------
enum Cls : uint8_t { C_OTHER = 0, C_LOWER, C_UPPER, C_LETTER /* caseless letter / mark */, C_DIGIT, C_SPACE, C_NEWLINE };
inline Cls classify(uint32_t c) {
  if (c < 0x80) {
    if (c >= 'a' && c <= 'z') return C_LOWER;
    if (c >= 'A' && c <= 'Z') return C_UPPER;
    if (c >= '0' && c <= '9') return C_DIGIT;
    if (c == '\n' || c == '\r') return C_NEWLINE;
    if (c == ' ' || c == '\t' || c == '\v' || c == '\f') return C_SPACE;
    return C_OTHER;
  }
  if (c == 0x85 || c == 0x2028 || c == 0x2029) return C_SPACE;
  if (c == 0xA0 || c == 0x1680 || (c >= 0x2000 && c <= 0x200A) || c == 0x202F || c == 0x205F || c == 0x3000) return C_SPACE;
  // Latin-1 supplement / Latin extended, Greek, Cyrillic: cased letters (pairs mostly alternate upper/lower)
  if (c >= 0xC0 && c <= 0x24F) {
    if (c == 0xD7 || c == 0xF7) return C_OTHER;
    if (c <= 0xDE) return C_UPPER;
    if (c <= 0xFF) return C_LOWER;
    return (c & 1) ? C_LOWER : C_UPPER;
  }
  if (c >= 0x391 && c <= 0x3A9) return C_UPPER;
  if (c >= 0x3B1 && c <= 0x3C9) return C_LOWER;
  if (c >= 0x410 && c <= 0x42F) return C_UPPER;
  if (c >= 0x430 && c <= 0x44F) return C_LOWER;
  if (c >= 0x400 && c <= 0x40F) return C_UPPER;
  if (c >= 0x450 && c <= 0x45F) return C_LOWER;
  // digits of other scripts and number forms
  if ((c >= 0x660 && c <= 0x669) || (c >= 0x6F0 && c <= 0x6F9) || (c >= 0x966 && c <= 0x96F) || (c >= 0xFF10 && c <= 0xFF19) ||
      (c >= 0x2150 && c <= 0x218F) || (c >= 0x2460 && c <= 0x249B) || (c >= 0xB2 && c <= 0xB3) || c == 0xB9 || (c >= 0xBC && c <= 0xBE))
    return C_DIGIT;
  // punctuation / symbol blocks
  if ((c >= 0xA1 && c <= 0xBF) || (c >= 0x2010 && c <= 0x2BFF) || (c >= 0x3001 && c <= 0x303F) || (c >= 0xFE30 && c <= 0xFE6F) ||
      (c >= 0xFF01 && c <= 0xFF0F) || (c >= 0xFF1A && c <= 0xFF20) || (c >= 0xFF3B && c <= 0xFF40) || (c >= 0xFF5B && c <= 0xFF65) ||
      (c >= 0x1F000 && c <= 0x1FAFF) || (c >= 0xE000 && c <= 0xF8FF))
    return C_OTHER;
  return C_LETTER;
}
inline bool is_letter(Cls k) { return k == C_LOWER || k == C_UPPER || k == C_LETTER; }
inline bool is_space(Cls k) { return k == C_SPACE || k == C_NEWLINE; }

struct Cp { uint32_t c; Cls k; uint32_t off; };   // off = byte offset in the source chunk

enum PreType { PRE_QWEN2 = 0, PRE_LLAMA3 = 1, PRE_CASED = 2 /* tekken, gpt-4o */, PRE_GPT2 = 3 };

struct Tok {
  std::vector<std::string> vocab;
  std::unordered_map<std::string, int32_t> lookup;
  std::vector<int32_t> types;       // 1 normal, 2 unknown, 3 control, 4 user-defined, 5 unused, 6 byte
  std::vector<float> scores;
  std::unordered_map<std::string, int32_t> merge_rank;   // "a b" -> rank
  std::vector<std::pair<std::string, int32_t>> specials;  // sorted by length desc
  int model = 0;                     // 0 byte-level BPE, 1 SPM (scores), 2 raw-UTF-8 BPE (gemma)
  int pre = PRE_QWEN2;
  bool ignore_merges = false;
  bool add_space_prefix = true;
  std::string byte_to_uni[256];
  std::unordered_map<uint32_t, uint8_t> uni_to_byte;
  int32_t byte_tok[256];

  void build_byte_map() {
    // GPT-2: printable bytes map to themselves, the rest to U+0100.. in order
    std::vector<int> bs;
    for (int b = '!'; b <= '~'; ++b) bs.push_back(b);
    for (int b = 0xA1; b <= 0xAC; ++b) bs.push_back(b);
    for (int b = 0xAE; b <= 0xFF; ++b) bs.push_back(b);
    std::vector<bool> direct(256, false);
    for (int b : bs) direct[b] = true;
    int n = 0;
    for (int b = 0; b < 256; ++b) {
      uint32_t cp = direct[b] ? (uint32_t)b : (uint32_t)(256 + n++);
      std::string s; utf8_append(s, cp);
      byte_to_uni[b] = s;
      uni_to_byte[cp] = (uint8_t)b;
    }
  }
};

// ---- pre-tokenizers --------------------------------------------------------------------------------
// All follow the shape of the published GPT-family patterns:
//   contractions | [^\r\n L N]? L+ | N{1,k} | ' '? [^\s L N]+ [\r\n]* | \s*[\r\n]+ | \s+(?!\S) | \s+
// PRE_CASED splits letter runs at lower->upper boundaries (two alternatives of the o200k / tekken pattern)
// and lets the punctuation run absorb a trailing '/' as tekken does.
size_t match_contraction(const std::vector<Cp>& v, size_t i) {
  if (v[i].c != '\'' || i + 1 >= v.size()) return 0;
  auto lc = [&](size_t j) { uint32_t c = v[j].c; return (c >= 'A' && c <= 'Z') ? c + 32 : c; };
  uint32_t a = lc(i + 1);
  if (a == 's' || a == 't' || a == 'm' || a == 'd') return 2;
  if (i + 2 < v.size()) {
    uint32_t b = lc(i + 2);
    if ((a == 'r' && b == 'e') || (a == 'v' && b == 'e') || (a == 'l' && b == 'l')) return 3;
  }
  return 0;
}

void pretokenize(const Tok& t, std::string_view text, std::vector<std::string_view>& out) {
  std::vector<Cp> v;
  v.reserve(text.size());
  for (size_t i = 0; i < text.size();) {
    int len; uint32_t c = utf8_decode(text.data() + i, text.size() - i, len);
    v.push_back({c, classify(c), (uint32_t)i});
    i += len;
  }
  const size_t n = v.size();
  auto emit = [&](size_t a, size_t b) {
    size_t lo = v[a].off, hi = b < n ? v[b].off : text.size();
    out.push_back(text.substr(lo, hi - lo));
  };
  const int max_digits = (t.pre == PRE_QWEN2 || t.pre == PRE_GPT2) ? (t.pre == PRE_GPT2 ? 1 << 30 : 1) : 3;
  size_t i = 0;
  while (i < n) {
    // contractions (only directly after a letter run in the cased pattern; as a free alternative otherwise)
    if (t.pre != PRE_CASED) {
      size_t c = match_contraction(v, i);
      if (c) { emit(i, i + c); i += c; continue; }
    }
    // optional single non-letter/digit/newline prefix followed by letters
    {
      size_t j = i;
      if (!is_letter(v[j].k) && v[j].k != C_DIGIT && v[j].k != C_NEWLINE && j + 1 < n && is_letter(v[j + 1].k) && t.pre != PRE_GPT2) ++j;
      else if (t.pre == PRE_GPT2 && v[j].c == ' ' && j + 1 < n && is_letter(v[j + 1].k)) ++j;
      if (is_letter(v[j].k)) {
        size_t k = j;
        if (t.pre == PRE_CASED) {
          // [upper]* [lower]+   |   [upper]+ [lower]*
          size_t u = k;
          while (u < n && (v[u].k == C_UPPER || v[u].k == C_LETTER)) ++u;
          size_t l = u;
          while (l < n && (v[l].k == C_LOWER || v[l].k == C_LETTER)) ++l;
          if (l > u) {
            // upper run followed by lowers: if more than one upper precedes, the last upper starts the word ("HTMLParser" -> "HTML", "Parser")
            size_t ups = 0;
            for (size_t q = k; q < u; ++q) ups += v[q].k == C_UPPER;
            if (ups > 1 && v[u - 1].k == C_UPPER) { k = u - 1; }
            else k = l;
          } else k = u;
          if (k == j) k = j + 1;
          size_t c = k < n ? match_contraction(v, k) : 0;
          k += c;
        } else {
          while (k < n && is_letter(v[k].k)) ++k;
        }
        emit(i, k); i = k; continue;
      }
    }
    if (v[i].k == C_DIGIT) {
      size_t k = i; int cnt = 0;
      while (k < n && v[k].k == C_DIGIT && cnt < max_digits) { ++k; ++cnt; }
      emit(i, k); i = k; continue;
    }
    if (t.pre == PRE_GPT2 && v[i].c == ' ' && i + 1 < n && v[i + 1].k == C_DIGIT) {
      size_t k = i + 1;
      while (k < n && v[k].k == C_DIGIT) ++k;
      emit(i, k); i = k; continue;
    }
    // ' '? punctuation+ [\r\n]*
    {
      size_t j = i;
      if (v[j].c == ' ' && j + 1 < n && v[j + 1].k == C_OTHER) ++j;
      if (v[j].k == C_OTHER) {
        size_t k = j;
        while (k < n && v[k].k == C_OTHER) ++k;
        if (t.pre != PRE_GPT2) while (k < n && (v[k].k == C_NEWLINE || (t.pre == PRE_CASED && v[k].c == '/'))) ++k;
        emit(i, k); i = k; continue;
      }
    }
    // whitespace
    if (is_space(v[i].k)) {
      size_t k = i;
      while (k < n && is_space(v[k].k)) ++k;
      // \s*[\r\n]+ : cut after the last newline of the run
      size_t last_nl = n;
      for (size_t q = i; q < k; ++q) if (v[q].k == C_NEWLINE) last_nl = q;
      if (last_nl != n && t.pre != PRE_GPT2) { emit(i, last_nl + 1); i = last_nl + 1; continue; }
      // \s+(?!\S): leave the last space to prefix the next word, unless the run ends the text
      if (k < n && k - i > 1) { emit(i, k - 1); i = k - 1; continue; }
      emit(i, k); i = k; continue;
    }
    emit(i, i + 1); ++i;
  }
}

// ---- BPE over symbol strings -------------------------------------------------------------------------
void bpe_merge(const Tok& t, std::vector<std::string>& sym) {
  while (sym.size() > 1) {
    int best = std::numeric_limits<int>::max(); size_t bi = 0;
    std::string key;
    for (size_t i = 0; i + 1 < sym.size(); ++i) {
      key.assign(sym[i]); key.push_back(' '); key.append(sym[i + 1]);
      auto it = t.merge_rank.find(key);
      if (it != t.merge_rank.end() && it->second < best) { best = it->second; bi = i; }
    }
    if (best == std::numeric_limits<int>::max()) break;
    sym[bi] += sym[bi + 1];
    sym.erase(sym.begin() + bi + 1);
  }
}

void emit_symbols(const Tok& t, const std::vector<std::string>& sym, std::vector<int32_t>& out) {
  for (const auto& s : sym) {
    auto it = t.lookup.find(s);
    if (it != t.lookup.end()) { out.push_back(it->second); continue; }
    // unknown merged piece: fall back to its single characters, then bytes
    for (size_t i = 0; i < s.size();) {
      int len = utf8_len((unsigned char)s[i]);
      auto jt = t.lookup.find(s.substr(i, len));
      if (jt != t.lookup.end()) out.push_back(jt->second);
      else for (int b = 0; b < len && i + b < s.size(); ++b) { int32_t bt = t.byte_tok[(unsigned char)s[i + b]]; if (bt >= 0) out.push_back(bt); }
      i += len;
    }
  }
}

void encode_bytelevel_word(const Tok& t, std::string_view w, std::vector<int32_t>& out) {
  std::string enc;
  for (unsigned char c : w) enc += t.byte_to_uni[c];
  if (t.ignore_merges) { auto it = t.lookup.find(enc); if (it != t.lookup.end()) { out.push_back(it->second); return; } }
  std::vector<std::string> sym;
  for (size_t i = 0; i < enc.size();) { int len = utf8_len((unsigned char)enc[i]); sym.emplace_back(enc.substr(i, len)); i += len; }
  bpe_merge(t, sym);
  emit_symbols(t, sym, out);
}

void encode_rawbpe(const Tok& t, std::string_view seg, std::vector<int32_t>& out) {   // gemma: merges over raw UTF-8 symbols
  std::vector<std::string> sym;
  for (size_t i = 0; i < seg.size();) { int len = utf8_len((unsigned char)seg[i]); sym.emplace_back(seg.substr(i, len)); i += len; }
  bpe_merge(t, sym);
  emit_symbols(t, sym, out);
}

// SentencePiece: repeatedly merge the adjacent pair whose concatenation is a vocab piece with the highest score
void encode_spm(const Tok& t, std::string_view seg, std::vector<int32_t>& out) {
  struct Sym { std::string s; int prev, next; bool alive; };
  std::vector<Sym> sy;
  for (size_t i = 0; i < seg.size();) { int len = utf8_len((unsigned char)seg[i]); sy.push_back({std::string(seg.substr(i, len)), (int)sy.size() - 1, (int)sy.size() + 1, true}); i += len; }
  if (sy.empty()) return;
  sy.back().next = -1;
  struct Cand { float score; int left, right; size_t len; };
  auto cmp = [](const Cand& a, const Cand& b) { return a.score < b.score || (a.score == b.score && a.left > b.left); };
  std::priority_queue<Cand, std::vector<Cand>, decltype(cmp)> pq(cmp);
  auto try_add = [&](int l, int r) {
    if (l < 0 || r < 0) return;
    std::string m = sy[l].s + sy[r].s;
    auto it = t.lookup.find(m);
    if (it != t.lookup.end() && (size_t)it->second < t.scores.size()) pq.push({t.scores[it->second], l, r, m.size()});
  };
  for (int i = 0; i + 1 < (int)sy.size(); ++i) try_add(i, i + 1);
  while (!pq.empty()) {
    Cand c = pq.top(); pq.pop();
    if (!sy[c.left].alive || !sy[c.right].alive || sy[c.left].next != c.right || sy[c.left].s.size() + sy[c.right].s.size() != c.len) continue;
    sy[c.left].s += sy[c.right].s;
    sy[c.right].alive = false;
    sy[c.left].next = sy[c.right].next;
    if (sy[c.right].next >= 0) sy[sy[c.right].next].prev = c.left;
    try_add(sy[c.left].prev, c.left);
    try_add(c.left, sy[c.left].next);
  }
  for (int i = 0; i >= 0; i = sy[i].next) {
    auto it = t.lookup.find(sy[i].s);
    if (it != t.lookup.end()) out.push_back(it->second);
    else for (unsigned char b : sy[i].s) { int32_t bt = t.byte_tok[b]; if (bt >= 0) out.push_back(bt); }
  }
}

void encode_chunk(const Tok& t, std::string_view chunk, bool first_chunk, std::vector<int32_t>& out) {
  if (chunk.empty()) return;
  if (t.model == 0) {
    std::vector<std::string_view> words;
    pretokenize(t, chunk, words);
    for (auto w : words) encode_bytelevel_word(t, w, out);
  } else {
    std::string s;
    if (t.model == 1 && t.add_space_prefix && first_chunk) s = "\xE2\x96\x81";
    for (char c : chunk) { if (c == ' ') s += "\xE2\x96\x81"; else s.push_back(c); }
    if (t.model == 1) encode_spm(t, s, out); else encode_rawbpe(t, s, out);
  }
}

thread_local std::string g_out;

}  // namespace

extern "C" {

// model: 0 byte-level BPE ("gpt2"), 1 SentencePiece ("llama"), 2 raw-UTF-8 BPE (gemma).  pre: see PreType.
void* mx_tok_create(int model, int pre, int ignore_merges, int add_space_prefix, const char* tok_blob, const uint64_t* tok_lens, uint64_t n_tok,
                    const int32_t* types, const float* scores, const char* merge_blob, const uint64_t* merge_lens, uint64_t n_merges) {
  Tok* t = new Tok();
  t->model = model; t->pre = pre; t->ignore_merges = ignore_merges != 0; t->add_space_prefix = add_space_prefix != 0;
  t->build_byte_map();
  t->vocab.reserve(n_tok);
  const char* p = tok_blob;
  for (uint64_t i = 0; i < n_tok; ++i) { t->vocab.emplace_back(p, tok_lens[i]); p += tok_lens[i]; }
  t->lookup.reserve(n_tok * 2);
  for (uint64_t i = 0; i < n_tok; ++i) t->lookup.emplace(t->vocab[i], (int32_t)i);   // first id wins for duplicates
  if (types) t->types.assign(types, types + n_tok);
  if (scores) t->scores.assign(scores, scores + n_tok);
  p = merge_blob;
  t->merge_rank.reserve(n_merges * 2);
  for (uint64_t i = 0; i < n_merges; ++i) { t->merge_rank.emplace(std::string(p, merge_lens[i]), (int32_t)i); p += merge_lens[i]; }
  for (int b = 0; b < 256; ++b) {
    char name[8]; snprintf(name, sizeof name, "<0x%02X>", b);
    auto it = t->lookup.find(name);
    t->byte_tok[b] = it != t->lookup.end() ? it->second : -1;
    if (t->byte_tok[b] < 0 && model == 0) { auto jt = t->lookup.find(t->byte_to_uni[b]); if (jt != t->lookup.end()) t->byte_tok[b] = jt->second; }
  }
  for (uint64_t i = 0; i < n_tok; ++i) {
    int ty = t->types.empty() ? 1 : t->types[i];
    if ((ty == 3 || ty == 4) && !t->vocab[i].empty()) t->specials.emplace_back(t->vocab[i], (int32_t)i);
  }
  std::sort(t->specials.begin(), t->specials.end(), [](auto& a, auto& b) { return a.first.size() > b.first.size(); });
  return t;
}
void mx_tok_free(void* h) { delete (Tok*)h; }
int32_t mx_tok_find(void* h, const char* s, uint64_t n) { Tok* t = (Tok*)h; auto it = t->lookup.find(std::string(s, n)); return it == t->lookup.end() ? -1 : it->second; }
int mx_tok_is_special(void* h, int32_t id) { Tok* t = (Tok*)h; if (id < 0 || (size_t)id >= t->vocab.size() || t->types.empty()) return 0; return t->types[id] == 3 || t->types[id] == 4; }

// Returns the number of ids (which may exceed cap: call again with a larger buffer).
int64_t mx_tok_encode(void* h, const char* text, uint64_t len, int allow_special, int32_t* out, uint64_t cap) {
  Tok* t = (Tok*)h;
  std::vector<int32_t> ids;
  std::string_view s(text, len);
  size_t start = 0, i = 0;
  bool first = true;
  if (allow_special && !t->specials.empty()) {
    // index specials by first byte to keep the scan linear in practice
    std::vector<std::vector<int>> by_first(256);
    for (int k = 0; k < (int)t->specials.size(); ++k) by_first[(unsigned char)t->specials[k].first[0]].push_back(k);
    while (i < s.size()) {
      bool hit = false;
      for (int k : by_first[(unsigned char)s[i]]) {
        const std::string& sp = t->specials[k].first;
        if (s.compare(i, sp.size(), sp) == 0) {
          encode_chunk(*t, s.substr(start, i - start), first, ids);
          ids.push_back(t->specials[k].second);
          i += sp.size(); start = i; hit = true; first = false;
          break;
        }
      }
      if (!hit) ++i;
    }
  }
  encode_chunk(*t, s.substr(start), first, ids);
  for (size_t k = 0; k < ids.size() && k < cap; ++k) out[k] = ids[k];
  return (int64_t)ids.size();
}

// Returns the number of bytes (which may exceed cap).
int64_t mx_tok_decode(void* h, const int32_t* ids, uint64_t n, int skip_special, const int32_t* keep, uint64_t n_keep, char* out, uint64_t cap) {
  Tok* t = (Tok*)h;
  std::string& o = g_out;
  o.clear();
  std::unordered_set<int32_t> keepset(keep, keep + n_keep);
  for (uint64_t i = 0; i < n; ++i) {
    int32_t id = ids[i];
    if (id < 0 || (size_t)id >= t->vocab.size()) continue;
    int ty = t->types.empty() ? 1 : t->types[id];
    bool special = ty == 3 || ty == 4;
    if (special) { if (!skip_special || keepset.count(id)) o += t->vocab[id]; continue; }
    const std::string& s = t->vocab[id];
    if (ty == 6 && s.size() == 6 && s[0] == '<' && s[1] == '0' && s[2] == 'x') { o.push_back((char)strtol(s.c_str() + 3, nullptr, 16)); continue; }
    if (t->model == 0) {
      for (size_t k = 0; k < s.size();) {
        int len; uint32_t cp = utf8_decode(s.data() + k, s.size() - k, len);
        auto it = t->uni_to_byte.find(cp);
        if (it != t->uni_to_byte.end()) o.push_back((char)it->second); else o.append(s, k, len);
        k += len;
      }
    } else {
      for (size_t k = 0; k < s.size();) {
        if (s.compare(k, 3, "\xE2\x96\x81") == 0) { o.push_back(' '); k += 3; } else { o.push_back(s[k]); ++k; }
      }
    }
  }
  if (t->model == 1 && t->add_space_prefix && !o.empty() && o[0] == ' ') o.erase(0, 1);
  memcpy(out, o.data(), std::min<uint64_t>(cap, o.size()));
  return (int64_t)o.size();
}

}  // extern "C"
