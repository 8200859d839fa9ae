// One value type for both codecs of the native front end: JSON (HTTP bodies) and msgpack (engine-core protocol).
#pragma once
#include <stdint.h>
#include <string.h>

#include <cmath>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace fe {

struct Val {
  enum T { NIL, BOOL, INT, DBL, STR, BIN, ARR, MAP } t = NIL;
  bool b = false;
  int64_t i = 0;
  double d = 0;
  std::string s;  // STR or BIN payload
  std::vector<Val> a;
  std::vector<std::pair<std::string, Val>> m;

  Val() {}
  static Val nil() { return Val(); }
  static Val boolean(bool v) { Val x; x.t = BOOL; x.b = v; return x; }
  static Val integer(int64_t v) { Val x; x.t = INT; x.i = v; return x; }
  static Val number(double v) { Val x; x.t = DBL; x.d = v; return x; }
  static Val str(std::string v) { Val x; x.t = STR; x.s = std::move(v); return x; }
  static Val bin(std::string v) { Val x; x.t = BIN; x.s = std::move(v); return x; }
  static Val array() { Val x; x.t = ARR; return x; }
  static Val map() { Val x; x.t = MAP; return x; }

  bool is_nil() const { return t == NIL; }
  bool is_num() const { return t == INT || t == DBL; }
  double as_double() const { return t == INT ? (double)i : d; }
  int64_t as_int() const { return t == INT ? i : (int64_t)d; }
  const Val* get(const std::string& k) const {
    if (t != MAP) return nullptr;
    for (auto& kv : m)
      if (kv.first == k) return &kv.second;
    return nullptr;
  }
  Val& set(const std::string& k, Val v) {
    for (auto& kv : m)
      if (kv.first == k) { kv.second = std::move(v); return kv.second; }
    m.emplace_back(k, std::move(v));
    return m.back().second;
  }
  Val& push(Val v) { a.push_back(std::move(v)); return a.back(); }
};

// ---------------------------------------------------------------------------------------------------------------------- JSON
class JsonParser {
 public:
  explicit JsonParser(const std::string& s) : p_(s.data()), e_(s.data() + s.size()) {}
  Val parse() {
    Val v = value();
    ws();
    if (p_ != e_) fail("trailing characters");
    return v;
  }

 private:
  const char *p_, *e_;
  int depth_ = 0;
  [[noreturn]] void fail(const char* what) { throw std::runtime_error(std::string("bad JSON: ") + what); }
  void ws() { while (p_ < e_ && (*p_ == ' ' || *p_ == '\t' || *p_ == '\n' || *p_ == '\r')) ++p_; }
  Val value() {
    ws();
    if (p_ >= e_) fail("unexpected end");
    if (++depth_ > 64) fail("nested too deeply");
    Val v;
    char c = *p_;
    if (c == '{') v = object();
    else if (c == '[') v = arr();
    else if (c == '"') v = Val::str(string());
    else if (c == 't') { lit("true"); v = Val::boolean(true); }
    else if (c == 'f') { lit("false"); v = Val::boolean(false); }
    else if (c == 'n') { lit("null"); }
    else v = num();
    --depth_;
    return v;
  }
  void lit(const char* w) {
    size_t n = strlen(w);
    if ((size_t)(e_ - p_) < n || memcmp(p_, w, n) != 0) fail("bad literal");
    p_ += n;
  }
  Val num() {
    const char* s = p_;
    bool isf = false;
    if (p_ < e_ && *p_ == '-') ++p_;
    while (p_ < e_ && ((*p_ >= '0' && *p_ <= '9') || *p_ == '.' || *p_ == 'e' || *p_ == 'E' || *p_ == '+' || *p_ == '-')) {
      if (*p_ == '.' || *p_ == 'e' || *p_ == 'E') isf = true;
      ++p_;
    }
    if (p_ == s) fail("bad number");
    std::string t(s, p_);
    try {
      if (!isf) return Val::integer(std::stoll(t));
      return Val::number(std::stod(t));
    } catch (...) {
      fail("bad number");
    }
  }
  static void utf8(std::string& o, uint32_t cp) {
    if (cp < 0x80) o += (char)cp;
    else if (cp < 0x800) { o += (char)(0xC0 | (cp >> 6)); o += (char)(0x80 | (cp & 63)); }
    else if (cp < 0x10000) { o += (char)(0xE0 | (cp >> 12)); o += (char)(0x80 | ((cp >> 6) & 63)); o += (char)(0x80 | (cp & 63)); }
    else { o += (char)(0xF0 | (cp >> 18)); o += (char)(0x80 | ((cp >> 12) & 63)); o += (char)(0x80 | ((cp >> 6) & 63)); o += (char)(0x80 | (cp & 63)); }
  }
  uint32_t hex4() {
    if (e_ - p_ < 4) fail("bad \\u escape");
    uint32_t v = 0;
    for (int k = 0; k < 4; ++k) {
      char c = *p_++;
      v <<= 4;
      if (c >= '0' && c <= '9') v |= c - '0';
      else if (c >= 'a' && c <= 'f') v |= c - 'a' + 10;
      else if (c >= 'A' && c <= 'F') v |= c - 'A' + 10;
      else fail("bad \\u escape");
    }
    return v;
  }
  std::string string() {
    ++p_;
    std::string o;
    while (true) {
      if (p_ >= e_) fail("unterminated string");
      char c = *p_++;
      if (c == '"') break;
      if (c != '\\') { o += c; continue; }
      if (p_ >= e_) fail("bad escape");
      char x = *p_++;
      switch (x) {
        case 'n': o += '\n'; break;
        case 't': o += '\t'; break;
        case 'r': o += '\r'; break;
        case 'b': o += '\b'; break;
        case 'f': o += '\f'; break;
        case '/': o += '/'; break;
        case '\\': o += '\\'; break;
        case '"': o += '"'; break;
        case 'u': {
          uint32_t cp = hex4();
          if (cp >= 0xD800 && cp < 0xDC00 && e_ - p_ >= 6 && p_[0] == '\\' && p_[1] == 'u') {
            p_ += 2;
            uint32_t lo = hex4();
            cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
          }
          utf8(o, cp);
          break;
        }
        default: fail("bad escape");
      }
    }
    return o;
  }
  Val arr() {
    ++p_;
    Val v = Val::array();
    ws();
    if (p_ < e_ && *p_ == ']') { ++p_; return v; }
    while (true) {
      v.a.push_back(value());
      ws();
      if (p_ >= e_) fail("unterminated array");
      if (*p_ == ',') { ++p_; continue; }
      if (*p_ == ']') { ++p_; break; }
      fail("expected , or ]");
    }
    return v;
  }
  Val object() {
    ++p_;
    Val v = Val::map();
    ws();
    if (p_ < e_ && *p_ == '}') { ++p_; return v; }
    while (true) {
      ws();
      if (p_ >= e_ || *p_ != '"') fail("expected a key");
      std::string k = string();
      ws();
      if (p_ >= e_ || *p_ != ':') fail("expected :");
      ++p_;
      v.m.emplace_back(std::move(k), value());
      ws();
      if (p_ >= e_) fail("unterminated object");
      if (*p_ == ',') { ++p_; continue; }
      if (*p_ == '}') { ++p_; break; }
      fail("expected , or }");
    }
    return v;
  }
};

inline void json_escape(std::string& o, const std::string& s) {
  o += '"';
  for (size_t k = 0; k < s.size(); ++k) {
    unsigned char c = (unsigned char)s[k];
    switch (c) {
      case '"': o += "\\\""; break;
      case '\\': o += "\\\\"; break;
      case '\n': o += "\\n"; break;
      case '\r': o += "\\r"; break;
      case '\t': o += "\\t"; break;
      default:
        if (c < 0x20) { char b[8]; snprintf(b, sizeof b, "\\u%04x", c); o += b; }
        else if (c < 0x80) o += (char)c;
        else {
          // bytes that are not well-formed UTF-8 (a model may emit any byte sequence) become U+FFFD: the document stays valid JSON
          int n = c >= 0xF0 ? 4 : c >= 0xE0 ? 3 : c >= 0xC2 ? 2 : 0;
          bool ok = n > 0 && k + n <= s.size() && c <= 0xF4;
          for (int q = 1; ok && q < n; ++q) ok = ((unsigned char)s[k + q] & 0xC0) == 0x80;
          if (ok && n == 3) { unsigned char d = (unsigned char)s[k + 1]; ok = !(c == 0xE0 && d < 0xA0) && !(c == 0xED && d >= 0xA0); }
          if (ok && n == 4) { unsigned char d = (unsigned char)s[k + 1]; ok = !(c == 0xF0 && d < 0x90) && !(c == 0xF4 && d >= 0x90); }
          if (ok) { o.append(s, k, n); k += n - 1; }
          else o += "\xEF\xBF\xBD";
        }
    }
  }
  o += '"';
}

inline void json_write(std::string& o, const Val& v) {
  switch (v.t) {
    case Val::NIL: o += "null"; break;
    case Val::BOOL: o += v.b ? "true" : "false"; break;
    case Val::INT: o += std::to_string(v.i); break;
    case Val::DBL: {
      if (!std::isfinite(v.d)) { o += "null"; break; }
      char b[40];
      snprintf(b, sizeof b, "%.17g", v.d);
      o += b;
      break;
    }
    case Val::STR: case Val::BIN: json_escape(o, v.s); break;
    case Val::ARR:
      o += '[';
      for (size_t k = 0; k < v.a.size(); ++k) { if (k) o += ','; json_write(o, v.a[k]); }
      o += ']';
      break;
    case Val::MAP:
      o += '{';
      for (size_t k = 0; k < v.m.size(); ++k) { if (k) o += ','; json_escape(o, v.m[k].first); o += ':'; json_write(o, v.m[k].second); }
      o += '}';
      break;
  }
}
inline std::string to_json(const Val& v) { std::string o; json_write(o, v); return o; }

// ------------------------------------------------------------------------------------------------------------------- msgpack
inline void mp_be(std::string& o, uint64_t v, int n) { for (int k = n - 1; k >= 0; --k) o += (char)((v >> (8 * k)) & 0xff); }
inline void mp_write(std::string& o, const Val& v) {
  switch (v.t) {
    case Val::NIL: o += (char)0xc0; break;
    case Val::BOOL: o += (char)(v.b ? 0xc3 : 0xc2); break;
    case Val::INT:
      if (v.i >= 0 && v.i < 128) o += (char)v.i;
      else if (v.i < 0 && v.i >= -32) o += (char)(0xe0 | (v.i + 32));
      else { o += (char)0xd3; mp_be(o, (uint64_t)v.i, 8); }
      break;
    case Val::DBL: { o += (char)0xcb; uint64_t u; memcpy(&u, &v.d, 8); mp_be(o, u, 8); break; }
    case Val::STR:
      if (v.s.size() < 32) o += (char)(0xa0 | v.s.size());
      else if (v.s.size() < 65536) { o += (char)0xda; mp_be(o, v.s.size(), 2); }
      else { o += (char)0xdb; mp_be(o, v.s.size(), 4); }
      o += v.s;
      break;
    case Val::BIN: o += (char)0xc6; mp_be(o, v.s.size(), 4); o += v.s; break;
    case Val::ARR:
      if (v.a.size() < 16) o += (char)(0x90 | v.a.size());
      else { o += (char)0xdd; mp_be(o, v.a.size(), 4); }
      for (auto& x : v.a) mp_write(o, x);
      break;
    case Val::MAP:
      if (v.m.size() < 16) o += (char)(0x80 | v.m.size());
      else { o += (char)0xdf; mp_be(o, v.m.size(), 4); }
      for (auto& kv : v.m) { mp_write(o, Val::str(kv.first)); mp_write(o, kv.second); }
      break;
  }
}
inline std::string to_msgpack(const Val& v) { std::string o; mp_write(o, v); return o; }

class MsgpackReader {
 public:
  MsgpackReader(const void* p, size_t n) : p_((const unsigned char*)p), e_((const unsigned char*)p + n) {}
  Val read() {
    if (++depth_ > 64) fail();
    Val v = read1();
    --depth_;
    return v;
  }

 private:
  const unsigned char *p_, *e_;
  int depth_ = 0;
  [[noreturn]] void fail() { throw std::runtime_error("bad msgpack"); }
  uint64_t be(int n) {
    if (e_ - p_ < n) fail();
    uint64_t v = 0;
    for (int k = 0; k < n; ++k) v = (v << 8) | *p_++;
    return v;
  }
  std::string bytes(size_t n) {
    if ((size_t)(e_ - p_) < n) fail();
    std::string s((const char*)p_, n);
    p_ += n;
    return s;
  }
  Val arr(size_t n) {
    Val v = Val::array();
    v.a.reserve(n < 4096 ? n : 4096);
    for (size_t k = 0; k < n; ++k) v.a.push_back(read());
    return v;
  }
  Val map(size_t n) {
    Val v = Val::map();
    for (size_t k = 0; k < n; ++k) {
      Val key = read();
      std::string ks = key.t == Val::STR || key.t == Val::BIN ? key.s : key.t == Val::INT ? std::to_string(key.i) : std::string("?");
      v.m.emplace_back(std::move(ks), read());
    }
    return v;
  }
  Val read1() {
    if (p_ >= e_) fail();
    unsigned char c = *p_++;
    if (c < 0x80) return Val::integer(c);
    if (c >= 0xe0) return Val::integer((int8_t)c);
    if (c >= 0xa0 && c < 0xc0) return Val::str(bytes(c & 31));
    if (c >= 0x90 && c < 0xa0) return arr(c & 15);
    if (c >= 0x80 && c < 0x90) return map(c & 15);
    switch (c) {
      case 0xc0: return Val::nil();
      case 0xc2: return Val::boolean(false);
      case 0xc3: return Val::boolean(true);
      case 0xc4: return Val::bin(bytes(be(1)));
      case 0xc5: return Val::bin(bytes(be(2)));
      case 0xc6: return Val::bin(bytes(be(4)));
      case 0xca: { uint32_t u = (uint32_t)be(4); float f; memcpy(&f, &u, 4); return Val::number(f); }
      case 0xcb: { uint64_t u = be(8); double d; memcpy(&d, &u, 8); return Val::number(d); }
      case 0xcc: return Val::integer((int64_t)be(1));
      case 0xcd: return Val::integer((int64_t)be(2));
      case 0xce: return Val::integer((int64_t)be(4));
      case 0xcf: return Val::integer((int64_t)be(8));
      case 0xd0: return Val::integer((int8_t)be(1));
      case 0xd1: return Val::integer((int16_t)be(2));
      case 0xd2: return Val::integer((int32_t)be(4));
      case 0xd3: return Val::integer((int64_t)be(8));
      case 0xd9: return Val::str(bytes(be(1)));
      case 0xda: return Val::str(bytes(be(2)));
      case 0xdb: return Val::str(bytes(be(4)));
      case 0xdc: return arr(be(2));
      case 0xdd: return arr(be(4));
      case 0xde: return map(be(2));
      case 0xdf: return map(be(4));
      default: fail();
    }
  }
};

}  // namespace fe
