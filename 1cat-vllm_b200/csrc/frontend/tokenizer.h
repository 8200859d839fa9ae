// Byte-level BPE tokenizer of the native front end. Reads a Hugging Face `tokenizer.json` (model type BPE with a ByteLevel
// pre-tokenizer: GPT-2, Llama-3, Qwen2/3 and relatives), a Mistral `tekken.json`, or the built-in byte vocabulary ("byte": ids
// 0..255 are raw bytes, 256 = BOS, 257 = EOS). The split pattern is not run through a regex engine: the known patterns are
// recognised by their text and executed by a hand-written scanner over Unicode classes (unicode_tables.h); a file with any
// other pattern is loaded for decoding only and text prompts are refused (token-id prompts still work).
// Merge order: `tokenizer.json` applies its `merges` list in order (pair ranks); `tekken.json` merges the adjacent pair whose
// concatenation has the lowest vocabulary rank (the tiktoken rule).
#pragma once
#include <fstream>
#include <sstream>
#include <unordered_map>

#include "unicode_tables.h"
#include "value.h"

namespace fe {

inline bool in_ranges(const uint32_t (*r)[2], int n, uint32_t cp) {
  int lo = 0, hi = n - 1;
  while (lo <= hi) {
    int mid = (lo + hi) >> 1;
    if (cp < r[mid][0]) hi = mid - 1;
    else if (cp > r[mid][1]) lo = mid + 1;
    else return true;
  }
  return false;
}
inline bool is_letter(uint32_t c) { return c < 128 ? ((c | 32) >= 'a' && (c | 32) <= 'z') : in_ranges(kLetter, kLetterCount, c); }
inline bool is_number(uint32_t c) { return c < 128 ? (c >= '0' && c <= '9') : in_ranges(kNumber, kNumberCount, c); }
inline bool is_space(uint32_t c) { return c < 128 ? (c == 0x20 || (c >= 9 && c <= 13)) : in_ranges(kSpace, kSpaceCount, c); }

inline std::string b64decode(const std::string& s) {
  static int8_t T[256];
  static bool init = false;
  if (!init) {
    memset(T, -1, sizeof T);
    const char* A = "ABCDEFGHIJKLMNOPQRSTUVWXYZabcdefghijklmnopqrstuvwxyz0123456789+/";
    for (int i = 0; i < 64; ++i) T[(unsigned char)A[i]] = (int8_t)i;
    init = true;
  }
  std::string o;
  uint32_t acc = 0;
  int bits = 0;
  for (unsigned char c : s) {
    if (T[c] < 0) continue;
    acc = (acc << 6) | (uint32_t)T[c];
    bits += 6;
    if (bits >= 8) { bits -= 8; o += (char)((acc >> bits) & 0xff); }
  }
  return o;
}

struct SplitOptions {
  bool contractions = false, ci = false;
  int letters = 0;        // 1: [^\r\n\p{L}\p{N}]?\p{L}+   2:  ?\p{L}+
  int digits = 0;         // 1: \p{N}   3: \p{N}{1,3}   -1:  ?\p{N}+
  int punct_tail = 0;     // 0: none   1: [\r\n]*   2: [\r\n/]*
  bool newline_alt = false;
  bool bracket_letters = false;  // letters written as [\p{L}]+
  std::string canonical() const {
    std::string p;
    if (contractions) p += ci ? "(?i:'s|'t|'re|'ve|'m|'ll|'d)|" : "'s|'t|'re|'ve|'m|'ll|'d|";
    p += letters == 1 ? (bracket_letters ? "[^\\r\\n\\p{L}\\p{N}]?[\\p{L}]+|" : "[^\\r\\n\\p{L}\\p{N}]?\\p{L}+|") : " ?\\p{L}+|";
    p += digits == 1 ? "\\p{N}|" : digits == 3 ? "\\p{N}{1,3}|" : " ?\\p{N}+|";
    p += " ?[^\\s\\p{L}\\p{N}]+";
    p += punct_tail == 1 ? "[\\r\\n]*|" : punct_tail == 2 ? "[\\r\\n/]*|" : "|";
    if (newline_alt) p += "\\s*[\\r\\n]+|";
    p += "\\s+(?!\\S)|\\s+";
    return p;
  }
  static bool recognise(const std::string& pat, SplitOptions& o) {
    auto has = [&](const char* s) { return pat.find(s) != std::string::npos; };
    o = SplitOptions();
    o.contractions = has("'s|'t|'re|'ve|'m|'ll|'d");
    o.ci = has("(?i:");
    o.bracket_letters = has("[\\p{L}]+");
    o.letters = has("[^\\r\\n\\p{L}\\p{N}]?") ? 1 : 2;
    o.digits = has("\\p{N}{1,3}") ? 3 : has(" ?\\p{N}+") ? -1 : 1;
    o.punct_tail = has("[\\r\\n/]*") ? 2 : has("]+[\\r\\n]*") ? 1 : 0;
    o.newline_alt = has("\\s*[\\r\\n]+");
    return o.canonical() == pat;
  }
};

class Tokenizer {
 public:
  int bos_id = -1, eos_id = -1;
  bool can_encode = false;
  std::string why_not;  // when !can_encode

  static uint32_t next_cp(const std::string& s, size_t& i) {
    unsigned char c = (unsigned char)s[i];
    if (c < 0x80) { ++i; return c; }
    int n = c >= 0xF0 ? 4 : c >= 0xE0 ? 3 : c >= 0xC0 ? 2 : 1;
    if (n == 1 || i + n > s.size()) { ++i; return 0xFFFD; }
    uint32_t cp = c & (0xFF >> (n + 1));
    for (int k = 1; k < n; ++k) cp = (cp << 6) | ((unsigned char)s[i + k] & 0x3F);
    i += n;
    return cp;
  }

  void load(const std::string& path) {
    if (path == "byte") {
      byte_mode_ = true;
      bos_id = 256;
      eos_id = 257;
      can_encode = true;
      vocab_size_ = 258;
      return;
    }
    std::string file = path;
    auto exists = [](const std::string& p) { std::ifstream f(p); return f.good(); };
    if (exists(path + "/tokenizer.json")) file = path + "/tokenizer.json";
    else if (exists(path + "/tekken.json")) file = path + "/tekken.json";
    std::ifstream f(file, std::ios::binary);
    if (!f) throw std::runtime_error("cannot open tokenizer file " + file);
    std::stringstream ss;
    ss << f.rdbuf();
    Val d = JsonParser(ss.str()).parse();
    if (d.get("config") && d.get("vocab") && d.get("vocab")->t == Val::ARR) load_tekken(d);
    else load_hf(d);
  }

  std::vector<int> encode(const std::string& text, bool add_bos) const {
    std::vector<int> out;
    if (add_bos && bos_id >= 0) out.push_back(bos_id);
    if (byte_mode_) {
      for (unsigned char c : text) out.push_back(c);
      return out;
    }
    if (!can_encode) throw std::runtime_error("this tokenizer cannot encode text here: " + why_not);
    size_t pos = 0;
    while (pos < text.size()) {  // added / special tokens are matched first, longest string wins
      size_t best_at = std::string::npos, best_len = 0;
      int best_id = -1;
      for (auto& kv : added_) {
        size_t at = text.find(kv.first, pos);
        if (at != std::string::npos && (at < best_at || (at == best_at && kv.first.size() > best_len))) {
          best_at = at; best_len = kv.first.size(); best_id = kv.second;
        }
      }
      size_t end = best_at == std::string::npos ? text.size() : best_at;
      if (end > pos) encode_plain(text.substr(pos, end - pos), out);
      if (best_at == std::string::npos) break;
      out.push_back(best_id);
      pos = best_at + best_len;
    }
    return out;
  }

  std::string decode(const std::vector<int>& ids, bool skip_special = true) const {
    std::string o;
    for (int id : ids) {
      if (byte_mode_) { if (id >= 0 && id < 256) o += (char)id; continue; }
      auto sp = special_by_id_.find(id);
      if (sp != special_by_id_.end()) { if (!skip_special) o += sp->second; continue; }
      if (id >= 0 && (size_t)id < bytes_.size()) o += bytes_[id];
    }
    return o;
  }
  int vocab_size() const { return vocab_size_; }

  // pieces of `text` as the split pattern cuts them (exposed for tests)
  std::vector<std::string> split(const std::string& text) const {
    std::vector<uint32_t> cps;
    std::vector<size_t> offs;
    for (size_t i = 0; i < text.size();) { offs.push_back(i); cps.push_back(next_cp(text, i)); }
    offs.push_back(text.size());
    std::vector<std::string> out;
    size_t p = 0;
    while (p < cps.size()) {
      size_t e = match(cps, p);
      if (e <= p) e = p + 1;
      out.push_back(text.substr(offs[p], offs[e] - offs[p]));
      p = e;
    }
    return out;
  }

 private:
  bool byte_mode_ = false, rank_merges_ = false;
  int vocab_size_ = 0;
  SplitOptions opt_;
  std::vector<std::string> bytes_;                         // id -> raw bytes
  std::unordered_map<std::string, int> id_of_;             // raw bytes -> id
  std::unordered_map<std::string, int> merge_rank_;        // HF: key(left, right) -> position in the merges list
  std::vector<std::pair<std::string, int>> added_;
  std::unordered_map<int, std::string> special_by_id_;

  static std::string pair_key(const std::string& l, const std::string& r) {
    std::string k;
    k += (char)(l.size() & 0xff);
    k += (char)((l.size() >> 8) & 0xff);
    k += l;
    k += r;
    return k;
  }
  int rank_of(const std::string& l, const std::string& r) const {
    if (rank_merges_) {
      auto it = id_of_.find(l + r);
      return it == id_of_.end() ? -1 : it->second;
    }
    auto it = merge_rank_.find(pair_key(l, r));
    return it == merge_rank_.end() ? -1 : it->second;
  }
  void bpe(const std::string& piece, std::vector<int>& out) const {
    auto whole = id_of_.find(piece);
    if (whole != id_of_.end()) { out.push_back(whole->second); return; }
    std::vector<std::string> parts;
    for (char c : piece) parts.emplace_back(1, c);
    while (parts.size() > 1) {
      int best = -1;
      size_t at = 0;
      for (size_t i = 0; i + 1 < parts.size(); ++i) {
        int r = rank_of(parts[i], parts[i + 1]);
        if (r >= 0 && (best < 0 || r < best)) { best = r; at = i; }
      }
      if (best < 0) break;
      parts[at] += parts[at + 1];
      parts.erase(parts.begin() + at + 1);
    }
    for (auto& p : parts) {
      auto it = id_of_.find(p);
      if (it != id_of_.end()) out.push_back(it->second);
      else for (char c : p) { auto b = id_of_.find(std::string(1, c)); if (b != id_of_.end()) out.push_back(b->second); }
    }
  }
  void encode_plain(const std::string& text, std::vector<int>& out) const {
    for (auto& piece : split(text)) bpe(piece, out);
  }

  // end (exclusive, in code points) of the piece that starts at p
  size_t match(const std::vector<uint32_t>& c, size_t p) const {
    const size_t n = c.size();
    auto L = [&](size_t i) { return i < n && is_letter(c[i]); };
    auto N = [&](size_t i) { return i < n && is_number(c[i]); };
    auto S = [&](size_t i) { return i < n && is_space(c[i]); };
    auto crlf = [&](size_t i) { return i < n && (c[i] == '\r' || c[i] == '\n'); };
    auto other = [&](size_t i) { return i < n && !is_space(c[i]) && !is_letter(c[i]) && !is_number(c[i]); };
    if (opt_.contractions && c[p] == '\'' && p + 1 < n) {
      auto lc = [&](size_t i) { uint32_t x = c[i]; return (opt_.ci && x >= 'A' && x <= 'Z') ? x + 32 : x; };
      uint32_t a = lc(p + 1), b = p + 2 < n ? lc(p + 2) : 0;
      if (a == 's' || a == 't') return p + 2;
      if ((a == 'r' && b == 'e') || (a == 'v' && b == 'e')) return p + 3;
      if (a == 'm') return p + 2;
      if (a == 'l' && b == 'l') return p + 3;
      if (a == 'd') return p + 2;
    }
    if (opt_.letters == 1) {
      if (!crlf(p) && !L(p) && !N(p) && L(p + 1)) { size_t e = p + 1; while (L(e)) ++e; return e; }
      if (L(p)) { size_t e = p; while (L(e)) ++e; return e; }
    } else {
      size_t s = (c[p] == ' ' && L(p + 1)) ? p + 1 : p;
      if (L(s)) { size_t e = s; while (L(e)) ++e; return e; }
    }
    if (opt_.digits == -1) {
      size_t s = (c[p] == ' ' && N(p + 1)) ? p + 1 : p;
      if (N(s)) { size_t e = s; while (N(e)) ++e; return e; }
    } else if (N(p)) {
      size_t e = p + 1;
      while (e < p + (size_t)opt_.digits && N(e)) ++e;
      return e;
    }
    {
      size_t s = (c[p] == ' ' && other(p + 1)) ? p + 1 : p;
      if (other(s)) {
        size_t e = s;
        while (other(e)) ++e;
        if (opt_.punct_tail >= 1) while (crlf(e) || (opt_.punct_tail == 2 && e < n && c[e] == '/')) ++e;
        return e;
      }
    }
    if (S(p)) {
      size_t e = p;
      while (S(e)) ++e;  // the whole whitespace run [p, e)
      if (opt_.newline_alt) {
        size_t last = n;
        for (size_t i = p; i < e; ++i) if (crlf(i)) last = i;
        if (last != n) return last + 1;   // \s*[\r\n]+ : up to and including the last line break of the run
      }
      if (e == n) return e;               // \s+(?!\S) at the end of the text
      if (e - p >= 2) return e - 1;       // \s+(?!\S): leave one space for the next piece
      return e;                           // \s+
    }
    return p + 1;
  }

  // GPT-2's byte <-> printable code point table, inverted: vocabulary strings back to raw bytes
  static std::unordered_map<uint32_t, unsigned char> byte_decoder() {
    std::unordered_map<uint32_t, unsigned char> m;
    int extra = 0;
    for (int b = 0; b < 256; ++b) {
      bool keep = (b >= 33 && b <= 126) || (b >= 161 && b <= 172) || (b >= 174 && b <= 255);
      m[keep ? (uint32_t)b : (uint32_t)(256 + extra++)] = (unsigned char)b;
    }
    return m;
  }
  static bool unmap(const std::unordered_map<uint32_t, unsigned char>& dec, const std::string& s, std::string& raw) {
    raw.clear();
    for (size_t i = 0; i < s.size();) {
      auto it = dec.find(next_cp(s, i));
      if (it == dec.end()) return false;
      raw += (char)it->second;
    }
    return true;
  }

  void add_special(const std::string& text, int id) {
    added_.emplace_back(text, id);
    special_by_id_[id] = text;
    if (text == "<s>" || text == "<|begin_of_text|>" || text == "<｜begin▁of▁sentence｜>") bos_id = id;
    if (text == "</s>" || text == "<|end_of_text|>" || text == "<|endoftext|>" || text == "<｜end▁of▁sentence｜>") eos_id = eos_id < 0 ? id : eos_id;
    if (id + 1 > vocab_size_) vocab_size_ = id + 1;
  }

  void load_hf(const Val& d) {
    const Val* model = d.get("model");
    if (!model || !model->get("vocab")) throw std::runtime_error("tokenizer.json has no BPE model");
    const Val* type = model->get("type");
    auto dec = byte_decoder();
    bool byte_level = true;
    const Val& vocab = *model->get("vocab");
    for (auto& kv : vocab.m) {
      int id = (int)kv.second.as_int();
      if ((size_t)id >= bytes_.size()) bytes_.resize(id + 1);
      std::string raw;
      if (!unmap(dec, kv.first, raw)) { byte_level = false; raw = kv.first; }
      bytes_[id] = raw;
      id_of_[raw] = id;
    }
    vocab_size_ = (int)bytes_.size();
    if (const Val* merges = model->get("merges")) {
      int rank = 0;
      for (auto& mg : merges->a) {
        std::string l, r;
        if (mg.t == Val::STR) {
          size_t sp = mg.s.find(' ');
          if (sp == std::string::npos) continue;
          l = mg.s.substr(0, sp);
          r = mg.s.substr(sp + 1);
        } else if (mg.t == Val::ARR && mg.a.size() == 2) {
          l = mg.a[0].s;
          r = mg.a[1].s;
        } else continue;
        std::string lr, rr;
        if (unmap(dec, l, lr) && unmap(dec, r, rr)) merge_rank_[pair_key(lr, rr)] = rank;
        ++rank;
      }
    }
    if (const Val* added = d.get("added_tokens"))
      for (auto& t : added->a) {
        const Val *c = t.get("content"), *id = t.get("id");
        if (c && id) add_special(c->s, (int)id->as_int());
      }
    // the split pattern: pre_tokenizer = ByteLevel{use_regex} | Sequence[Split{pattern.Regex}, ByteLevel]
    std::string pat;
    bool gpt2_default = false;
    std::vector<const Val*> pts;
    if (const Val* pt = d.get("pre_tokenizer")) {
      if (pt->get("pretokenizers")) for (auto& x : pt->get("pretokenizers")->a) pts.push_back(&x);
      else pts.push_back(pt);
    }
    for (const Val* pt : pts) {
      const Val* ty = pt->get("type");
      if (!ty) continue;
      if (ty->s == "Split" && pt->get("pattern") && pt->get("pattern")->get("Regex")) pat = pt->get("pattern")->get("Regex")->s;
      if (ty->s == "ByteLevel") { const Val* ur = pt->get("use_regex"); if (!ur || ur->b) gpt2_default = true; }
    }
    if (pat.empty() && gpt2_default) pat = "'s|'t|'re|'ve|'m|'ll|'d| ?\\p{L}+| ?\\p{N}+| ?[^\\s\\p{L}\\p{N}]+|\\s+(?!\\S)|\\s+";
    if (!type || type->s != "BPE" || !byte_level) why_not = "not a byte-level BPE model";
    else if (d.get("normalizer") && !d.get("normalizer")->is_nil()) why_not = "it has a normalizer";
    else if (!SplitOptions::recognise(pat, opt_)) why_not = "unknown split pattern";
    else can_encode = true;
  }

  void load_tekken(const Val& d) {
    const Val& cfg = *d.get("config");
    const Val* ns = cfg.get("default_num_special_tokens");
    int n_special = ns ? (int)ns->as_int() : (d.get("special_tokens") ? (int)d.get("special_tokens")->a.size() : 0);
    const Val* vs = cfg.get("default_vocab_size");
    int total = vs ? (int)vs->as_int() : (int)d.get("vocab")->a.size() + n_special;
    int n_regular = total - n_special;
    bytes_.assign(total, std::string());
    int k = 0;
    for (auto& t : d.get("vocab")->a) {
      if (k >= n_regular) break;
      std::string raw = b64decode(t.get("token_bytes")->s);
      bytes_[n_special + k] = raw;
      id_of_[raw] = n_special + k;   // ids grow with rank: comparing ids compares ranks
      ++k;
    }
    vocab_size_ = total;
    rank_merges_ = true;
    if (const Val* sp = d.get("special_tokens"))
      for (auto& t : sp->a) add_special(t.get("token_str")->s, (int)t.get("rank")->as_int());
    const Val* pat = cfg.get("pattern");
    if (!pat || !SplitOptions::recognise(pat->s, opt_)) why_not = "unknown split pattern";
    else can_encode = true;
  }
};

}  // namespace fe
