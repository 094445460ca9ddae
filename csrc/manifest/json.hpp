// Minimal RFC 8259 JSON: ordered objects, exact 64-bit integers, duplicate keys rejected at parse
// (a manifest names everything once). Small on purpose: the manifest library depends on nothing else.
// (The reference's C++ consumer carries its own parser too: examples/cpp/json.hpp; duplicate-key
// rejection mirrors crates/kern-manifest/src/constants.rs:166-219.)
#pragma once
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace kern {

struct Json {
  enum Type { Null, Bool, Int, Float, Str, Arr, Obj };
  Type type = Null;
  bool b = false;
  bool neg = false;   // Int: sign
  uint64_t u = 0;     // Int: magnitude
  double d = 0;       // Float (also set for Int)
  std::string s;
  std::vector<Json> arr;
  std::vector<std::pair<std::string, Json>> obj;

  static Json null() { return Json(); }
  static Json boolean(bool v) { Json j; j.type = Bool; j.b = v; return j; }
  static Json uint(uint64_t v) { Json j; j.type = Int; j.u = v; j.d = (double)v; return j; }
  static Json sint(int64_t v) {
    Json j; j.type = Int; j.neg = v < 0;
    j.u = v < 0 ? (uint64_t)(-(v + 1)) + 1 : (uint64_t)v; j.d = (double)v; return j;
  }
  static Json number(double v) { Json j; j.type = Float; j.d = v; return j; }
  static Json str(std::string v) { Json j; j.type = Str; j.s = std::move(v); return j; }
  static Json array() { Json j; j.type = Arr; return j; }
  static Json object() { Json j; j.type = Obj; return j; }

  bool is_null() const { return type == Null; }
  bool is_bool() const { return type == Bool; }
  bool is_int() const { return type == Int; }
  bool is_uint() const { return type == Int && !neg; }
  bool is_number() const { return type == Int || type == Float; }
  bool is_str() const { return type == Str; }
  bool is_arr() const { return type == Arr; }
  bool is_obj() const { return type == Obj; }
  bool fits_i64() const {
    return type == Int && (neg ? u <= (uint64_t)INT64_MAX + 1 : u <= (uint64_t)INT64_MAX);
  }
  int64_t as_i64() const { return neg ? (int64_t)(0 - u) : (int64_t)u; }

  const Json* find(const std::string& k) const {
    for (auto& kv : obj) if (kv.first == k) return &kv.second;
    return nullptr;
  }
  Json* find(const std::string& k) {
    for (auto& kv : obj) if (kv.first == k) return &kv.second;
    return nullptr;
  }
  Json& set(const std::string& k, Json v) {
    if (Json* p = find(k)) { *p = std::move(v); return *p; }
    obj.emplace_back(k, std::move(v));
    return obj.back().second;
  }
  void push(Json v) { arr.push_back(std::move(v)); }

  // ---- serialisation ----
  static void escape(const std::string& s, std::string& out) {
    out.push_back('"');
    for (unsigned char c : s) {
      switch (c) {
        case '"': out += "\\\""; break;
        case '\\': out += "\\\\"; break;
        case '\n': out += "\\n"; break;
        case '\r': out += "\\r"; break;
        case '\t': out += "\\t"; break;
        default:
          if (c < 0x20) { char buf[8]; snprintf(buf, sizeof buf, "\\u%04x", c); out += buf; }
          else out.push_back((char)c);
      }
    }
    out.push_back('"');
  }
  void dump(std::string& out, int indent = -1, int depth = 0) const {
    auto nl = [&](int d) { if (indent >= 0) { out.push_back('\n'); out.append((size_t)(d * indent), ' '); } };
    switch (type) {
      case Null: out += "null"; break;
      case Bool: out += b ? "true" : "false"; break;
      case Int: if (neg) out.push_back('-'); out += std::to_string(u); break;
      case Float: {
        char buf[40];
        if (std::isfinite(d)) {
          snprintf(buf, sizeof buf, "%.17g", d);
          out += buf;
          if (!strpbrk(buf, ".eE")) out += ".0";
        } else out += "null";
        break;
      }
      case Str: escape(s, out); break;
      case Arr:
        out.push_back('[');
        for (size_t i = 0; i < arr.size(); ++i) {
          if (i) out.push_back(',');
          if (indent >= 0 && (arr[i].is_obj() || arr[i].is_arr())) nl(depth + 1);
          else if (i && indent >= 0) out.push_back(' ');
          arr[i].dump(out, indent, depth + 1);
        }
        out.push_back(']');
        break;
      case Obj:
        out.push_back('{');
        for (size_t i = 0; i < obj.size(); ++i) {
          if (i) out.push_back(',');
          nl(depth + 1);
          escape(obj[i].first, out);
          out += indent >= 0 ? ": " : ":";
          obj[i].second.dump(out, indent, depth + 1);
        }
        if (!obj.empty()) nl(depth);
        out.push_back('}');
        break;
    }
  }
  std::string dump(int indent = -1) const { std::string o; dump(o, indent, 0); return o; }
  static char* strpbrk(char* s, const char* set) { return ::strpbrk(s, set); }
};

class JsonParser {
 public:
  explicit JsonParser(const std::string& text) : p_(text.data()), end_(text.data() + text.size()), begin_(text.data()) {}
  Json parse() {
    Json v = value(0);
    ws();
    if (p_ != end_) fail("trailing characters after the document");
    return v;
  }

 private:
  const char* p_;
  const char* end_;
  const char* begin_;

  [[noreturn]] void fail(const std::string& msg) {
    size_t line = 1, col = 1;
    for (const char* q = begin_; q < p_; ++q) { if (*q == '\n') { ++line; col = 1; } else ++col; }
    throw std::runtime_error("JSON: " + msg + " at line " + std::to_string(line) + " column " + std::to_string(col));
  }
  void ws() { while (p_ < end_ && (*p_ == ' ' || *p_ == '\n' || *p_ == '\t' || *p_ == '\r')) ++p_; }
  bool lit(const char* w) {
    size_t n = strlen(w);
    if ((size_t)(end_ - p_) >= n && memcmp(p_, w, n) == 0) { p_ += n; return true; }
    return false;
  }
  Json value(int depth) {
    if (depth > 256) fail("nesting too deep");
    ws();
    if (p_ == end_) fail("unexpected end of input");
    switch (*p_) {
      case '{': return object(depth);
      case '[': return array(depth);
      case '"': return Json::str(string());
      case 't': if (lit("true")) return Json::boolean(true); break;
      case 'f': if (lit("false")) return Json::boolean(false); break;
      case 'n': if (lit("null")) return Json::null(); break;
      default: if (*p_ == '-' || (*p_ >= '0' && *p_ <= '9')) return number();
    }
    fail("unexpected character");
  }
  Json object(int depth) {
    Json j = Json::object();
    ++p_;
    ws();
    if (p_ < end_ && *p_ == '}') { ++p_; return j; }
    for (;;) {
      ws();
      if (p_ == end_ || *p_ != '"') fail("expected a string key");
      std::string k = string();
      if (j.find(k)) fail("duplicate key `" + k + "`");
      ws();
      if (p_ == end_ || *p_ != ':') fail("expected `:`");
      ++p_;
      j.obj.emplace_back(std::move(k), value(depth + 1));
      ws();
      if (p_ == end_) fail("unterminated object");
      if (*p_ == ',') { ++p_; continue; }
      if (*p_ == '}') { ++p_; return j; }
      fail("expected `,` or `}`");
    }
  }
  Json array(int depth) {
    Json j = Json::array();
    ++p_;
    ws();
    if (p_ < end_ && *p_ == ']') { ++p_; return j; }
    for (;;) {
      j.arr.push_back(value(depth + 1));
      ws();
      if (p_ == end_) fail("unterminated array");
      if (*p_ == ',') { ++p_; continue; }
      if (*p_ == ']') { ++p_; return j; }
      fail("expected `,` or `]`");
    }
  }
  static void utf8(uint32_t cp, std::string& out) {
    if (cp < 0x80) out.push_back((char)cp);
    else if (cp < 0x800) { out.push_back((char)(0xC0 | (cp >> 6))); out.push_back((char)(0x80 | (cp & 0x3F))); }
    else if (cp < 0x10000) {
      out.push_back((char)(0xE0 | (cp >> 12))); out.push_back((char)(0x80 | ((cp >> 6) & 0x3F)));
      out.push_back((char)(0x80 | (cp & 0x3F)));
    } else {
      out.push_back((char)(0xF0 | (cp >> 18))); out.push_back((char)(0x80 | ((cp >> 12) & 0x3F)));
      out.push_back((char)(0x80 | ((cp >> 6) & 0x3F))); out.push_back((char)(0x80 | (cp & 0x3F)));
    }
  }
  uint32_t hex4() {
    if (end_ - p_ < 4) fail("short \\u escape");
    uint32_t v = 0;
    for (int i = 0; i < 4; ++i) {
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
    std::string out;
    ++p_;
    for (;;) {
      if (p_ == end_) fail("unterminated string");
      unsigned char c = (unsigned char)*p_++;
      if (c == '"') return out;
      if (c < 0x20) fail("control character in string");
      if (c != '\\') { out.push_back((char)c); continue; }
      if (p_ == end_) fail("unterminated escape");
      char e = *p_++;
      switch (e) {
        case '"': out.push_back('"'); break;
        case '\\': out.push_back('\\'); break;
        case '/': out.push_back('/'); break;
        case 'b': out.push_back('\b'); break;
        case 'f': out.push_back('\f'); break;
        case 'n': out.push_back('\n'); break;
        case 'r': out.push_back('\r'); break;
        case 't': out.push_back('\t'); break;
        case 'u': {
          uint32_t cp = hex4();
          if (cp >= 0xD800 && cp < 0xDC00 && end_ - p_ >= 6 && p_[0] == '\\' && p_[1] == 'u') {
            p_ += 2;
            uint32_t lo = hex4();
            cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
          }
          utf8(cp, out);
          break;
        }
        default: fail("bad escape");
      }
    }
  }
  Json number() {
    const char* start = p_;
    bool neg = false, is_int = true;
    if (*p_ == '-') { neg = true; ++p_; }
    if (p_ == end_ || *p_ < '0' || *p_ > '9') fail("bad number");
    uint64_t mag = 0;
    bool overflow = false;
    while (p_ < end_ && *p_ >= '0' && *p_ <= '9') {
      uint64_t dgt = (uint64_t)(*p_ - '0');
      if (mag > (UINT64_MAX - dgt) / 10) overflow = true;
      mag = mag * 10 + dgt;
      ++p_;
    }
    if (p_ < end_ && *p_ == '.') { is_int = false; ++p_; while (p_ < end_ && *p_ >= '0' && *p_ <= '9') ++p_; }
    if (p_ < end_ && (*p_ == 'e' || *p_ == 'E')) {
      is_int = false; ++p_;
      if (p_ < end_ && (*p_ == '+' || *p_ == '-')) ++p_;
      while (p_ < end_ && *p_ >= '0' && *p_ <= '9') ++p_;
    }
    double d = strtod(std::string(start, p_).c_str(), nullptr);
    if (is_int && !overflow) {
      Json j; j.type = Json::Int; j.neg = neg && mag != 0; j.u = mag; j.d = d; return j;
    }
    return Json::number(d);
  }
};

inline Json parse_json(const std::string& text) { return JsonParser(text).parse(); }

}  // namespace kern
