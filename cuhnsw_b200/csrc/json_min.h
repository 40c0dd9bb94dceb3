// Minimal reader for the flat JSON object the Python layer writes as its option
// file (cuhnsw/pyhnsw.py:36-39 dumps the option message; cpp/src/cuhnsw_base.cu:67-106
// reads it back).  Supports one object of string keys mapped to numbers, booleans,
// strings, null or arrays of numbers; anything else is a parse error.
#pragma once
#include <cctype>
#include <cstdlib>
#include <map>
#include <string>
#include <vector>

namespace hnsw {

struct JsonValue {
  enum Kind { kNull, kBool, kNumber, kString, kNumbers } kind = kNull;
  double num = 0.0;
  bool b = false;
  std::string str;
  std::vector<double> nums;
};

class FlatJson {
 public:
  bool parse(const std::string& text) {
    s_ = &text;
    i_ = 0;
    values_.clear();
    ws();
    if (!eat('{')) return false;
    ws();
    if (eat('}')) return tail();
    for (;;) {
      std::string key;
      ws();
      if (!str(&key)) return false;
      ws();
      if (!eat(':')) return false;
      ws();
      JsonValue v;
      if (!value(&v)) return false;
      values_[key] = v;
      ws();
      if (eat(',')) continue;
      if (eat('}')) return tail();
      return false;
    }
  }
  bool has(const std::string& k) const { return values_.count(k) != 0; }
  double number(const std::string& k, double dflt) const {
    auto it = values_.find(k);
    if (it == values_.end()) return dflt;
    if (it->second.kind == JsonValue::kNumber) return it->second.num;
    if (it->second.kind == JsonValue::kBool) return it->second.b ? 1.0 : 0.0;
    return dflt;
  }
  bool boolean(const std::string& k, bool dflt) const {
    auto it = values_.find(k);
    if (it == values_.end()) return dflt;
    if (it->second.kind == JsonValue::kBool) return it->second.b;
    if (it->second.kind == JsonValue::kNumber) return it->second.num != 0.0;
    return dflt;
  }
  // array of numbers; a single number reads as an array of one
  std::vector<double> numbers(const std::string& k) const {
    auto it = values_.find(k);
    if (it == values_.end()) return {};
    if (it->second.kind == JsonValue::kNumbers) return it->second.nums;
    if (it->second.kind == JsonValue::kNumber) return {it->second.num};
    return {};
  }
  std::string string(const std::string& k, const std::string& dflt) const {
    auto it = values_.find(k);
    if (it == values_.end() || it->second.kind != JsonValue::kString) return dflt;
    return it->second.str;
  }

 private:
  const std::string* s_ = nullptr;
  size_t i_ = 0;
  std::map<std::string, JsonValue> values_;

  bool end() const { return i_ >= s_->size(); }
  char cur() const { return (*s_)[i_]; }
  void ws() {
    while (!end() && std::isspace((unsigned char)cur())) ++i_;
  }
  bool eat(char c) {
    if (!end() && cur() == c) {
      ++i_;
      return true;
    }
    return false;
  }
  bool tail() {
    ws();
    return end();
  }
  bool str(std::string* out) {
    if (!eat('"')) return false;
    out->clear();
    while (!end()) {
      char c = cur();
      ++i_;
      if (c == '"') return true;
      if (c == '\\') {
        if (end()) return false;
        char e = cur();
        ++i_;
        switch (e) {
          case 'n': out->push_back('\n'); break;
          case 't': out->push_back('\t'); break;
          case 'r': out->push_back('\r'); break;
          case 'b': out->push_back('\b'); break;
          case 'f': out->push_back('\f'); break;
          case 'u': {
            if (i_ + 4 > s_->size()) return false;
            unsigned code = (unsigned)std::strtoul(s_->substr(i_, 4).c_str(), nullptr, 16);
            i_ += 4;
            out->push_back(code < 128 ? (char)code : '?');
            break;
          }
          default: out->push_back(e); break;
        }
      } else {
        out->push_back(c);
      }
    }
    return false;
  }
  bool literal(const char* w) {
    size_t n = std::char_traits<char>::length(w);
    if (s_->compare(i_, n, w) == 0) {
      i_ += n;
      return true;
    }
    return false;
  }
  bool value(JsonValue* v) {
    if (end()) return false;
    char c = cur();
    if (c == '"') {
      v->kind = JsonValue::kString;
      return str(&v->str);
    }
    if (c == '[') {
      ++i_;
      v->kind = JsonValue::kNumbers;
      ws();
      if (eat(']')) return true;
      for (;;) {
        ws();
        JsonValue item;
        if (end() || cur() == '[' || !value(&item) || item.kind != JsonValue::kNumber) return false;
        v->nums.push_back(item.num);
        ws();
        if (eat(',')) continue;
        return eat(']');
      }
    }
    if (literal("true")) {
      v->kind = JsonValue::kBool;
      v->b = true;
      return true;
    }
    if (literal("false")) {
      v->kind = JsonValue::kBool;
      v->b = false;
      return true;
    }
    if (literal("null")) {
      v->kind = JsonValue::kNull;
      return true;
    }
    const char* begin = s_->c_str() + i_;
    char* stop = nullptr;
    double x = std::strtod(begin, &stop);
    if (stop == begin) return false;
    i_ += (size_t)(stop - begin);
    v->kind = JsonValue::kNumber;
    v->num = x;
    return true;
  }
};

}  // namespace hnsw
