// Minimal JSON value for the serving control plane: ordered objects (insertion order is part of the workflow
// semantics: nodes fire in document order), integers kept apart from floats (so "cfg": 1 stays 1 and 7.0 stays 7.0),
// strict UTF-8 pass-through, \uXXXX escapes decoded (surrogate pairs included).
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

namespace mdb {

class Json {
 public:
  enum Kind { Null, Bool, Int, Float, String, Array, Object };
  using Member = std::pair<std::string, Json>;

  Json() : kind_(Null) {}
  Json(std::nullptr_t) : kind_(Null) {}
  Json(bool b) : kind_(Bool), b_(b) {}
  Json(int v) : kind_(Int), i_(v) {}
  Json(int64_t v) : kind_(Int), i_(v) {}
  Json(long long v) : kind_(Int), i_(v) {}
  Json(size_t v) : kind_(Int), i_(static_cast<int64_t>(v)) {}
  Json(double v) : kind_(Float), d_(v) {}
  Json(const char* s) : kind_(String), s_(s) {}
  Json(std::string s) : kind_(String), s_(std::move(s)) {}
  static Json array() { Json j; j.kind_ = Array; return j; }
  static Json object() { Json j; j.kind_ = Object; return j; }

  Kind kind() const { return kind_; }
  bool is_null() const { return kind_ == Null; }
  bool is_bool() const { return kind_ == Bool; }
  bool is_int() const { return kind_ == Int; }
  bool is_number() const { return kind_ == Int || kind_ == Float; }
  bool is_string() const { return kind_ == String; }
  bool is_array() const { return kind_ == Array; }
  bool is_object() const { return kind_ == Object; }

  bool as_bool(bool d = false) const { return kind_ == Bool ? b_ : d; }
  int64_t as_int(int64_t d = 0) const { return kind_ == Int ? i_ : kind_ == Float ? static_cast<int64_t>(d_) : d; }
  double as_double(double d = 0) const { return kind_ == Float ? d_ : kind_ == Int ? static_cast<double>(i_) : d; }
  const std::string& as_string() const { static const std::string e; return kind_ == String ? s_ : e; }

  // ---- arrays
  std::vector<Json>& items() { return a_; }
  const std::vector<Json>& items() const { return a_; }
  void push(Json v) { if (kind_ != Array) { *this = array(); } a_.push_back(std::move(v)); }
  size_t size() const { return kind_ == Array ? a_.size() : kind_ == Object ? o_.size() : 0; }
  const Json& at(size_t i) const { static const Json n; return kind_ == Array && i < a_.size() ? a_[i] : n; }

  // ---- objects (ordered)
  std::vector<Member>& members() { return o_; }
  const std::vector<Member>& members() const { return o_; }
  const Json* find(const std::string& k) const {
    if (kind_ != Object) return nullptr;
    for (auto& m : o_) if (m.first == k) return &m.second;
    return nullptr;
  }
  Json* find(const std::string& k) { return const_cast<Json*>(static_cast<const Json*>(this)->find(k)); }
  bool has(const std::string& k) const { return find(k) != nullptr; }
  const Json& get(const std::string& k) const { static const Json n; auto* p = find(k); return p ? *p : n; }
  // present and not null
  bool present(const std::string& k) const { auto* p = find(k); return p && !p->is_null(); }
  void set(const std::string& k, Json v) {
    if (kind_ != Object) *this = object();
    if (auto* p = find(k)) { *p = std::move(v); return; }
    o_.emplace_back(k, std::move(v));
  }
  // the first writer of a key wins (an explicit null counts as absent)
  bool set_if_missing(const std::string& k, Json v) {
    if (present(k)) return false;
    set(k, std::move(v));
    return true;
  }
  bool erase(const std::string& k) {
    for (size_t i = 0; i < o_.size(); ++i) if (o_[i].first == k) { o_.erase(o_.begin() + i); return true; }
    return false;
  }
  std::string str(const std::string& k, const std::string& d = "") const {
    auto* p = find(k); return p && p->is_string() ? p->s_ : d;
  }

  // ---- serialisation
  std::string dump() const { std::string out; write(out); return out; }
  void write(std::string& out) const {
    switch (kind_) {
      case Null: out += "null"; break;
      case Bool: out += b_ ? "true" : "false"; break;
      case Int: out += std::to_string(i_); break;
      case Float: write_double(out, d_); break;
      case String: write_string(out, s_); break;
      case Array:
        out += '[';
        for (size_t i = 0; i < a_.size(); ++i) { if (i) out += ','; a_[i].write(out); }
        out += ']';
        break;
      case Object:
        out += '{';
        for (size_t i = 0; i < o_.size(); ++i) {
          if (i) out += ',';
          write_string(out, o_[i].first);
          out += ':';
          o_[i].second.write(out);
        }
        out += '}';
        break;
    }
  }
  static void write_string(std::string& out, const std::string& s) {
    out += '"';
    for (unsigned char c : s) {
      switch (c) {
        case '"': out += "\\\""; break;
        case '\\': out += "\\\\"; break;
        case '\n': out += "\\n"; break;
        case '\r': out += "\\r"; break;
        case '\t': out += "\\t"; break;
        case '\b': out += "\\b"; break;
        case '\f': out += "\\f"; break;
        default:
          if (c < 0x20) { char buf[8]; snprintf(buf, sizeof buf, "\\u%04x", c); out += buf; }
          else out += static_cast<char>(c);
      }
    }
    out += '"';
  }
  static void write_double(std::string& out, double d) {
    if (!std::isfinite(d)) { out += "null"; return; }
    char buf[40];
    for (int prec = 1; prec <= 17; ++prec) {           // shortest representation that round-trips
      snprintf(buf, sizeof buf, "%.*g", prec, d);
      if (strtod(buf, nullptr) == d) break;
    }
    out += buf;
    if (!strpbrk(buf, ".eEn")) out += ".0";             // keep it a float on the way back in
  }

  // ---- parsing
  static Json parse(const std::string& text) {
    Parser p{text.data(), text.data() + text.size()};
    p.ws();
    Json v = p.value(0);
    p.ws();
    if (p.cur != p.end) throw std::runtime_error("json: trailing characters");
    return v;
  }
  static bool try_parse(const std::string& text, Json* out, std::string* err = nullptr) {
    try { *out = parse(text); return true; }
    catch (const std::exception& e) { if (err) *err = e.what(); return false; }
  }

 private:
  struct Parser {
    const char* cur; const char* end;
    void ws() { while (cur < end && (*cur == ' ' || *cur == '\n' || *cur == '\r' || *cur == '\t')) ++cur; }
    [[noreturn]] void fail(const char* m) { throw std::runtime_error(std::string("json: ") + m); }
    Json value(int depth) {
      if (depth > 256) fail("nesting too deep");
      if (cur >= end) fail("unexpected end");
      switch (*cur) {
        case '{': return object(depth);
        case '[': return array(depth);
        case '"': return Json(string());
        case 't': lit("true"); return Json(true);
        case 'f': lit("false"); return Json(false);
        case 'n': lit("null"); return Json();
        default: return number();
      }
    }
    void lit(const char* w) {
      size_t n = strlen(w);
      if (static_cast<size_t>(end - cur) < n || memcmp(cur, w, n)) fail("bad literal");
      cur += n;
    }
    Json number() {
      const char* s = cur;
      if (cur < end && *cur == '-') ++cur;
      if (cur >= end || !(*cur >= '0' && *cur <= '9')) fail("bad number");
      while (cur < end && *cur >= '0' && *cur <= '9') ++cur;
      bool is_float = false;
      if (cur < end && *cur == '.') { is_float = true; ++cur; while (cur < end && *cur >= '0' && *cur <= '9') ++cur; }
      if (cur < end && (*cur == 'e' || *cur == 'E')) {
        is_float = true; ++cur;
        if (cur < end && (*cur == '+' || *cur == '-')) ++cur;
        while (cur < end && *cur >= '0' && *cur <= '9') ++cur;
      }
      std::string tok(s, cur);
      if (!is_float) {
        errno = 0;
        long long v = strtoll(tok.c_str(), nullptr, 10);
        if (errno == 0) return Json(static_cast<int64_t>(v));
      }
      return Json(strtod(tok.c_str(), nullptr));
    }
    static void utf8(std::string& out, uint32_t cp) {
      if (cp < 0x80) out += static_cast<char>(cp);
      else if (cp < 0x800) { out += static_cast<char>(0xC0 | (cp >> 6)); out += static_cast<char>(0x80 | (cp & 0x3F)); }
      else if (cp < 0x10000) {
        out += static_cast<char>(0xE0 | (cp >> 12)); out += static_cast<char>(0x80 | ((cp >> 6) & 0x3F));
        out += static_cast<char>(0x80 | (cp & 0x3F));
      } else {
        out += static_cast<char>(0xF0 | (cp >> 18)); out += static_cast<char>(0x80 | ((cp >> 12) & 0x3F));
        out += static_cast<char>(0x80 | ((cp >> 6) & 0x3F)); out += static_cast<char>(0x80 | (cp & 0x3F));
      }
    }
    uint32_t hex4() {
      if (end - cur < 4) fail("bad \\u escape");
      uint32_t v = 0;
      for (int i = 0; i < 4; ++i) {
        char c = *cur++;
        v <<= 4;
        if (c >= '0' && c <= '9') v |= c - '0';
        else if (c >= 'a' && c <= 'f') v |= c - 'a' + 10;
        else if (c >= 'A' && c <= 'F') v |= c - 'A' + 10;
        else fail("bad \\u escape");
      }
      return v;
    }
    std::string string() {
      ++cur;
      std::string out;
      while (true) {
        if (cur >= end) fail("unterminated string");
        char c = *cur++;
        if (c == '"') break;
        if (c != '\\') { out += c; continue; }
        if (cur >= end) fail("bad escape");
        char e = *cur++;
        switch (e) {
          case '"': out += '"'; break; case '\\': out += '\\'; break; case '/': out += '/'; break;
          case 'b': out += '\b'; break; case 'f': out += '\f'; break; case 'n': out += '\n'; break;
          case 'r': out += '\r'; break; case 't': out += '\t'; break;
          case 'u': {
            uint32_t cp = hex4();
            if (cp >= 0xD800 && cp <= 0xDBFF && end - cur >= 6 && cur[0] == '\\' && cur[1] == 'u') {
              cur += 2;
              uint32_t lo = hex4();
              if (lo >= 0xDC00 && lo <= 0xDFFF) cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
            }
            utf8(out, cp);
            break;
          }
          default: fail("bad escape");
        }
      }
      return out;
    }
    Json array(int depth) {
      ++cur;
      Json a = Json::array();
      ws();
      if (cur < end && *cur == ']') { ++cur; return a; }
      while (true) {
        ws();
        a.a_.push_back(value(depth + 1));
        ws();
        if (cur >= end) fail("unterminated array");
        if (*cur == ',') { ++cur; continue; }
        if (*cur == ']') { ++cur; return a; }
        fail("expected , or ]");
      }
    }
    Json object(int depth) {
      ++cur;
      Json o = Json::object();
      ws();
      if (cur < end && *cur == '}') { ++cur; return o; }
      while (true) {
        ws();
        if (cur >= end || *cur != '"') fail("expected key");
        std::string k = string();
        ws();
        if (cur >= end || *cur != ':') fail("expected :");
        ++cur;
        ws();
        Json v = value(depth + 1);
        o.set(k, std::move(v));                          // a repeated key keeps its first position, last value
        ws();
        if (cur >= end) fail("unterminated object");
        if (*cur == ',') { ++cur; continue; }
        if (*cur == '}') { ++cur; return o; }
        fail("expected , or }");
      }
    }
  };

  Kind kind_;
  bool b_ = false;
  int64_t i_ = 0;
  double d_ = 0;
  std::string s_;
  std::vector<Json> a_;
  std::vector<Member> o_;
};

}  // namespace mdb
