// Minimal JSON reader for safetensors headers, the shard index and config.json (objects, arrays, strings with the
// usual escapes, numbers, true/false/null). Header-only; throws ijah::Error on malformed input.
#pragma once
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "common.hpp"

namespace ijah {

struct Json {
  enum Kind { Null, Bool, Num, Str, Arr, Obj } kind = Null;
  bool b = false;
  double num = 0;
  std::string str;
  std::vector<Json> arr;
  std::vector<std::pair<std::string, Json>> obj;  // insertion order kept

  const Json *get(const std::string &key) const {
    for (auto &kv : obj)
      if (kv.first == key) return &kv.second;
    return nullptr;
  }
  long long as_int() const { return (long long)num; }
};

class JsonParser {
 public:
  JsonParser(const char *s, size_t n) : p_(s), e_(s + n) {}
  Json parse() {
    Json j = value();
    ws();
    IJ_CHECK(p_ == e_, "json: trailing characters");
    return j;
  }

 private:
  const char *p_, *e_;
  void ws() {
    while (p_ < e_ && (*p_ == ' ' || *p_ == '\n' || *p_ == '\t' || *p_ == '\r')) p_++;
  }
  char peek() {
    ws();
    IJ_CHECK(p_ < e_, "json: unexpected end");
    return *p_;
  }
  void expect(char c) {
    IJ_CHECK(peek() == c, "json: expected '%c' got '%c'", c, *p_);
    p_++;
  }
  std::string string() {
    expect('"');
    std::string s;
    while (true) {
      IJ_CHECK(p_ < e_, "json: unterminated string");
      char c = *p_++;
      if (c == '"') break;
      if (c != '\\') { s.push_back(c); continue; }
      IJ_CHECK(p_ < e_, "json: bad escape");
      c = *p_++;
      switch (c) {
        case 'n': s.push_back('\n'); break;
        case 't': s.push_back('\t'); break;
        case 'r': s.push_back('\r'); break;
        case 'b': s.push_back('\b'); break;
        case 'f': s.push_back('\f'); break;
        case 'u': {
          IJ_CHECK(e_ - p_ >= 4, "json: bad \\u escape");
          unsigned cp = (unsigned)strtoul(std::string(p_, 4).c_str(), nullptr, 16);
          p_ += 4;
          if (cp < 0x80) s.push_back((char)cp);
          else if (cp < 0x800) { s.push_back((char)(0xC0 | (cp >> 6))); s.push_back((char)(0x80 | (cp & 0x3F))); }
          else { s.push_back((char)(0xE0 | (cp >> 12))); s.push_back((char)(0x80 | ((cp >> 6) & 0x3F))); s.push_back((char)(0x80 | (cp & 0x3F))); }
          break;
        }
        default: s.push_back(c);
      }
    }
    return s;
  }
  Json value() {
    Json j;
    const char c = peek();
    if (c == '{') {
      j.kind = Json::Obj;
      p_++;
      if (peek() == '}') { p_++; return j; }
      while (true) {
        std::string k = string();
        expect(':');
        j.obj.emplace_back(std::move(k), value());
        if (peek() == ',') { p_++; continue; }
        expect('}');
        break;
      }
    } else if (c == '[') {
      j.kind = Json::Arr;
      p_++;
      if (peek() == ']') { p_++; return j; }
      while (true) {
        j.arr.push_back(value());
        if (peek() == ',') { p_++; continue; }
        expect(']');
        break;
      }
    } else if (c == '"') {
      j.kind = Json::Str;
      j.str = string();
    } else if (c == 't' || c == 'f' || c == 'n') {
      const char *w = c == 't' ? "true" : c == 'f' ? "false" : "null";
      const size_t n = strlen(w);
      IJ_CHECK((size_t)(e_ - p_) >= n && std::string(p_, n) == w, "json: bad literal");
      p_ += n;
      j.kind = c == 'n' ? Json::Null : Json::Bool;
      j.b = c == 't';
    } else {
      char *end = nullptr;
      j.kind = Json::Num;
      j.num = strtod(p_, &end);
      IJ_CHECK(end != p_ && end <= e_, "json: bad number");
      p_ = end;
    }
    return j;
  }
};

}  // namespace ijah
