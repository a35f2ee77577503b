// Minimal JSON reader for the library's own calibration files (host only, no dependency).
// Objects, arrays, strings (with the common escapes), numbers, true / false / null.
#pragma once
#include <cstdlib>
#include <map>
#include <memory>
#include <string>
#include <utility>
#include <vector>

namespace ft {

struct Json {
  enum Kind { Null, Bool, Num, Str, Arr, Obj } kind = Null;
  bool b = false;
  double num = 0;
  std::string str;
  std::vector<Json> arr;
  std::map<std::string, Json> obj;

  const Json* get(const std::string& key) const {
    if (kind != Obj) return nullptr;
    auto it = obj.find(key);
    return it == obj.end() ? nullptr : &it->second;
  }
  double number_or(double dflt) const { return kind == Num ? num : dflt; }
};

class JsonParser {
 public:
  explicit JsonParser(std::string text) : s_(std::move(text)) {}   // owns its text: a temporary is a valid argument
  // false (and a reason in err()) on malformed input or trailing garbage
  bool parse(Json* out) {
    if (!value(out, 0)) return false;
    ws();
    if (i_ != s_.size()) return fail("trailing characters");
    return true;
  }
  const std::string& err() const { return err_; }

 private:
  const std::string s_;
  size_t i_ = 0;
  std::string err_;

  bool fail(const char* what) {
    if (err_.empty()) err_ = std::string(what) + " at offset " + std::to_string(i_);
    return false;
  }
  void ws() {
    while (i_ < s_.size() && (s_[i_] == ' ' || s_[i_] == '\n' || s_[i_] == '\t' || s_[i_] == '\r')) ++i_;
  }
  bool lit(const char* w) {
    size_t n = 0;
    while (w[n]) ++n;
    if (s_.compare(i_, n, w) != 0) return false;
    i_ += n;
    return true;
  }
  bool string(std::string* out) {
    if (i_ >= s_.size() || s_[i_] != '"') return fail("expected string");
    ++i_;
    out->clear();
    while (i_ < s_.size() && s_[i_] != '"') {
      char c = s_[i_++];
      if (c == '\\') {
        if (i_ >= s_.size()) return fail("dangling escape");
        char e = s_[i_++];
        switch (e) {
          case 'n': c = '\n'; break;
          case 't': c = '\t'; break;
          case 'r': c = '\r'; break;
          case 'b': c = '\b'; break;
          case 'f': c = '\f'; break;
          case 'u':   // the calibration files are ASCII; keep the escape readable instead of decoding it
            out->append("\\u");
            continue;
          default: c = e; break;   // \" \\ \/
        }
      }
      out->push_back(c);
    }
    if (i_ >= s_.size()) return fail("unterminated string");
    ++i_;
    return true;
  }
  bool value(Json* out, int depth) {
    if (depth > 64) return fail("nesting too deep");
    ws();
    if (i_ >= s_.size()) return fail("unexpected end");
    const char c = s_[i_];
    if (c == '{') {
      ++i_;
      out->kind = Json::Obj;
      ws();
      if (i_ < s_.size() && s_[i_] == '}') { ++i_; return true; }
      for (;;) {
        ws();
        std::string key;
        if (!string(&key)) return false;
        ws();
        if (i_ >= s_.size() || s_[i_] != ':') return fail("expected ':'");
        ++i_;
        if (!value(&out->obj[key], depth + 1)) return false;
        ws();
        if (i_ < s_.size() && s_[i_] == ',') { ++i_; continue; }
        if (i_ < s_.size() && s_[i_] == '}') { ++i_; return true; }
        return fail("expected ',' or '}'");
      }
    }
    if (c == '[') {
      ++i_;
      out->kind = Json::Arr;
      ws();
      if (i_ < s_.size() && s_[i_] == ']') { ++i_; return true; }
      for (;;) {
        out->arr.emplace_back();
        if (!value(&out->arr.back(), depth + 1)) return false;
        ws();
        if (i_ < s_.size() && s_[i_] == ',') { ++i_; continue; }
        if (i_ < s_.size() && s_[i_] == ']') { ++i_; return true; }
        return fail("expected ',' or ']'");
      }
    }
    if (c == '"') { out->kind = Json::Str; return string(&out->str); }
    if (lit("true")) { out->kind = Json::Bool; out->b = true; return true; }
    if (lit("false")) { out->kind = Json::Bool; out->b = false; return true; }
    if (lit("null")) { out->kind = Json::Null; return true; }
    if (lit("NaN")) { out->kind = Json::Num; out->num = 0; return true; }   // Python's json writes these for non-finite floats
    if (lit("Infinity")) { out->kind = Json::Num; out->num = 1e300; return true; }
    if (lit("-Infinity")) { out->kind = Json::Num; out->num = -1e300; return true; }
    char* end = nullptr;
    const double v = std::strtod(s_.c_str() + i_, &end);
    if (end == s_.c_str() + i_) return fail("unexpected character");
    i_ = (size_t)(end - s_.c_str());
    out->kind = Json::Num;
    out->num = v;
    return true;
  }
};

}  // namespace ft
