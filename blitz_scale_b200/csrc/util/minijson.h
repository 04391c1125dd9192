// Minimal JSON reader (RFC 8259 subset sufficient for tokenizer.json, safetensors headers and cluster
// configs): objects keep insertion order, numbers are doubles (integers exact up to 2^53), strings are
// UTF-8 with \uXXXX escapes (surrogate pairs included) decoded.  Errors throw std::runtime_error with the
// byte offset.  Plays the role of the reference's vendored minijson (src/model/safetensors.hh).
#pragma once
#include <cstdint>
#include <cstdlib>
#include <stdexcept>
#include <string>
#include <string_view>
#include <utility>
#include <vector>

namespace blitz::json {

struct Value {
  enum Type { Null, Bool, Number, String, Array, Object } type = Null;
  bool b = false;
  double num = 0.0;
  std::string str;
  std::vector<Value> arr;
  std::vector<std::pair<std::string, Value>> obj;

  const Value* find(std::string_view key) const {
    if (type != Object) return nullptr;
    for (const auto& kv : obj)
      if (kv.first == key) return &kv.second;
    return nullptr;
  }
  const Value& at(std::string_view key) const {
    const Value* v = find(key);
    if (!v) throw std::runtime_error("json: missing key '" + std::string(key) + "'");
    return *v;
  }
  bool is_null() const { return type == Null; }
  // saturating: a number outside the 64-bit range (or NaN) must not reach an undefined conversion
  int64_t as_int() const {
    if (!(num == num)) return 0;
    if (num >= 9.2e18) return INT64_MAX;
    if (num <= -9.2e18) return INT64_MIN;
    return static_cast<int64_t>(num);
  }
};

class Parser {
 public:
  explicit Parser(std::string_view s) : s_(s) {}
  Value parse() {
    Value v = value();
    ws();
    if (i_ != s_.size()) fail("trailing characters");
    return v;
  }

 private:
  std::string_view s_;
  size_t i_ = 0;
  int depth_ = 0;

  [[noreturn]] void fail(const char* what) const {
    throw std::runtime_error(std::string("json: ") + what + " at byte " + std::to_string(i_));
  }
  void ws() {
    while (i_ < s_.size() && (s_[i_] == ' ' || s_[i_] == '\n' || s_[i_] == '\t' || s_[i_] == '\r')) ++i_;
  }
  char peek() {
    if (i_ >= s_.size()) fail("unexpected end");
    return s_[i_];
  }
  void expect(char c) {
    if (peek() != c) fail("unexpected character");
    ++i_;
  }
  static void put_utf8(std::string& o, uint32_t cp) {
    if (cp < 0x80) o.push_back(static_cast<char>(cp));
    else if (cp < 0x800) { o.push_back(static_cast<char>(0xC0 | (cp >> 6))); o.push_back(static_cast<char>(0x80 | (cp & 0x3F))); }
    else if (cp < 0x10000) {
      o.push_back(static_cast<char>(0xE0 | (cp >> 12)));
      o.push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F)));
      o.push_back(static_cast<char>(0x80 | (cp & 0x3F)));
    } else {
      o.push_back(static_cast<char>(0xF0 | (cp >> 18)));
      o.push_back(static_cast<char>(0x80 | ((cp >> 12) & 0x3F)));
      o.push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F)));
      o.push_back(static_cast<char>(0x80 | (cp & 0x3F)));
    }
  }
  uint32_t hex4() {
    if (i_ + 4 > s_.size()) fail("short \\u escape");
    uint32_t v = 0;
    for (int k = 0; k < 4; ++k) {
      const char c = s_[i_++];
      v <<= 4;
      if (c >= '0' && c <= '9') v |= c - '0';
      else if (c >= 'a' && c <= 'f') v |= c - 'a' + 10;
      else if (c >= 'A' && c <= 'F') v |= c - 'A' + 10;
      else fail("bad \\u escape");
    }
    return v;
  }
  std::string string() {
    expect('"');
    std::string o;
    while (true) {
      if (i_ >= s_.size()) fail("unterminated string");
      const char c = s_[i_++];
      if (c == '"') break;
      if (c != '\\') { o.push_back(c); continue; }
      if (i_ >= s_.size()) fail("unterminated escape");
      const char e = s_[i_++];
      switch (e) {
        case '"': o.push_back('"'); break;
        case '\\': o.push_back('\\'); break;
        case '/': o.push_back('/'); break;
        case 'b': o.push_back('\b'); break;
        case 'f': o.push_back('\f'); break;
        case 'n': o.push_back('\n'); break;
        case 'r': o.push_back('\r'); break;
        case 't': o.push_back('\t'); break;
        case 'u': {
          uint32_t cp = hex4();
          if (cp >= 0xD800 && cp < 0xDC00 && i_ + 1 < s_.size() && s_[i_] == '\\' && s_[i_ + 1] == 'u') {
            i_ += 2;
            const uint32_t lo = hex4();
            if (lo >= 0xDC00 && lo < 0xE000) cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
          }
          put_utf8(o, cp);
          break;
        }
        default: fail("bad escape");
      }
    }
    return o;
  }
  Value value() {
    if (++depth_ > 256) fail("nesting too deep");
    ws();
    Value v;
    const char c = peek();
    if (c == '{') {
      ++i_;
      v.type = Value::Object;
      ws();
      if (peek() == '}') { ++i_; --depth_; return v; }
      while (true) {
        ws();
        std::string k = string();
        ws();
        expect(':');
        v.obj.emplace_back(std::move(k), value());
        ws();
        if (peek() == ',') { ++i_; continue; }
        expect('}');
        break;
      }
    } else if (c == '[') {
      ++i_;
      v.type = Value::Array;
      ws();
      if (peek() == ']') { ++i_; --depth_; return v; }
      while (true) {
        v.arr.push_back(value());
        ws();
        if (peek() == ',') { ++i_; continue; }
        expect(']');
        break;
      }
    } else if (c == '"') {
      v.type = Value::String;
      v.str = string();
    } else if (s_.compare(i_, 4, "true") == 0) { v.type = Value::Bool; v.b = true; i_ += 4; }
    else if (s_.compare(i_, 5, "false") == 0) { v.type = Value::Bool; v.b = false; i_ += 5; }
    else if (s_.compare(i_, 4, "null") == 0) { v.type = Value::Null; i_ += 4; }
    else {
      const size_t b = i_;
      while (i_ < s_.size() && (std::string_view("+-0123456789.eE").find(s_[i_]) != std::string_view::npos)) ++i_;
      if (b == i_) fail("unexpected character");
      v.type = Value::Number;
      v.num = std::strtod(std::string(s_.substr(b, i_ - b)).c_str(), nullptr);
    }
    --depth_;
    return v;
  }
};

inline Value parse(std::string_view s) { return Parser(s).parse(); }

}  // namespace blitz::json
