// A small JSON reader for safetensors headers and the quantization metadata blobs inside them: objects, arrays,
// strings (with escapes), numbers, true / false / null. Values keep insertion order; lookups are linear (headers
// have thousands of entries at most and are walked once).
#pragma once

#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace sfq::json {

struct Value {
  enum Kind { kNull, kBool, kNumber, kString, kArray, kObject } kind = kNull;
  bool boolean = false;
  double number = 0.0;
  std::string string;
  std::vector<Value> array;
  std::vector<std::pair<std::string, Value>> object;

  bool is_null() const { return kind == kNull; }
  bool is_object() const { return kind == kObject; }
  const Value* find(const std::string& key) const {
    if (kind != kObject) return nullptr;
    for (const auto& kv : object)
      if (kv.first == key) return &kv.second;
    return nullptr;
  }
  const std::string& as_string() const {
    if (kind != kString) throw std::runtime_error("json: not a string");
    return string;
  }
  bool as_bool() const {
    if (kind != kBool) throw std::runtime_error("json: not a boolean");
    return boolean;
  }
  double as_number() const {
    if (kind != kNumber) throw std::runtime_error("json: not a number");
    return number;
  }
  int64_t as_int() const {
    const double v = as_number();
    if (!std::isfinite(v) || std::floor(v) != v || std::fabs(v) > 9.0e15) throw std::runtime_error("json: not an integer");
    return int64_t(v);
  }
};

class Parser {
public:
  explicit Parser(const std::string& text) : s_(text) {}
  Value parse() {
    Value v = value();
    skip();
    if (i_ != s_.size()) fail("trailing characters");
    return v;
  }

private:
  const std::string& s_;
  size_t i_ = 0;
  int depth_ = 0;

  [[noreturn]] void fail(const char* what) const {
    throw std::runtime_error(std::string("json: ") + what + " at offset " + std::to_string(i_));
  }
  void skip() {
    while (i_ < s_.size() && (s_[i_] == ' ' || s_[i_] == '\n' || s_[i_] == '\t' || s_[i_] == '\r')) ++i_;
  }
  bool eat(char c) {
    skip();
    if (i_ < s_.size() && s_[i_] == c) {
      ++i_;
      return true;
    }
    return false;
  }
  void literal(const char* word) {
    for (const char* p = word; *p; ++p, ++i_)
      if (i_ >= s_.size() || s_[i_] != *p) fail("bad literal");
  }
  static void append_utf8(std::string& out, uint32_t cp) {
    if (cp < 0x80) {
      out += char(cp);
    } else if (cp < 0x800) {
      out += char(0xC0 | (cp >> 6));
      out += char(0x80 | (cp & 0x3F));
    } else if (cp < 0x10000) {
      out += char(0xE0 | (cp >> 12));
      out += char(0x80 | ((cp >> 6) & 0x3F));
      out += char(0x80 | (cp & 0x3F));
    } else {
      out += char(0xF0 | (cp >> 18));
      out += char(0x80 | ((cp >> 12) & 0x3F));
      out += char(0x80 | ((cp >> 6) & 0x3F));
      out += char(0x80 | (cp & 0x3F));
    }
  }
  uint32_t hex4() {
    if (i_ + 4 > s_.size()) fail("short \\u escape");
    uint32_t v = 0;
    for (int k = 0; k < 4; ++k, ++i_) {
      const char c = s_[i_];
      v <<= 4;
      if (c >= '0' && c <= '9') v |= uint32_t(c - '0');
      else if (c >= 'a' && c <= 'f') v |= uint32_t(c - 'a' + 10);
      else if (c >= 'A' && c <= 'F') v |= uint32_t(c - 'A' + 10);
      else fail("bad \\u escape");
    }
    return v;
  }
  std::string string() {
    if (!eat('"')) fail("expected a string");
    std::string out;
    for (;;) {
      if (i_ >= s_.size()) fail("unterminated string");
      const char c = s_[i_++];
      if (c == '"') return out;
      if (c != '\\') {
        out += c;
        continue;
      }
      if (i_ >= s_.size()) fail("unterminated escape");
      const char e = s_[i_++];
      switch (e) {
        case '"': out += '"'; break;
        case '\\': out += '\\'; break;
        case '/': out += '/'; break;
        case 'b': out += '\b'; break;
        case 'f': out += '\f'; break;
        case 'n': out += '\n'; break;
        case 'r': out += '\r'; break;
        case 't': out += '\t'; break;
        case 'u': {
          uint32_t cp = hex4();
          if (cp >= 0xD800 && cp < 0xDC00 && i_ + 1 < s_.size() && s_[i_] == '\\' && s_[i_ + 1] == 'u') {
            i_ += 2;
            const uint32_t lo = hex4();
            if (lo >= 0xDC00 && lo < 0xE000) cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
          }
          append_utf8(out, cp);
          break;
        }
        default: fail("unknown escape");
      }
    }
  }
  Value value() {
    if (++depth_ > 64) fail("nesting too deep");
    skip();
    if (i_ >= s_.size()) fail("unexpected end");
    Value v;
    const char c = s_[i_];
    if (c == '{') {
      ++i_;
      v.kind = Value::kObject;
      if (!eat('}')) {
        do {
          skip();
          std::string key = string();
          if (!eat(':')) fail("expected ':'");
          v.object.emplace_back(std::move(key), value());
        } while (eat(','));
        if (!eat('}')) fail("expected '}'");
      }
    } else if (c == '[') {
      ++i_;
      v.kind = Value::kArray;
      if (!eat(']')) {
        do v.array.push_back(value());
        while (eat(','));
        if (!eat(']')) fail("expected ']'");
      }
    } else if (c == '"') {
      v.kind = Value::kString;
      v.string = string();
    } else if (c == 't') {
      literal("true");
      v.kind = Value::kBool;
      v.boolean = true;
    } else if (c == 'f') {
      literal("false");
      v.kind = Value::kBool;
    } else if (c == 'n') {
      literal("null");
    } else {
      const char* begin = s_.c_str() + i_;
      char* end = nullptr;
      v.number = std::strtod(begin, &end);
      if (end == begin) fail("expected a value");
      v.kind = Value::kNumber;
      i_ += size_t(end - begin);
    }
    --depth_;
    return v;
  }
};

inline Value parse(const std::string& text) { return Parser(text).parse(); }

}  // namespace sfq::json
