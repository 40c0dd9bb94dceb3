// Stand-in for the json11 header the reference includes (cpp/include/cuhnsw.hpp:29) but does
// not vendor (3rd/json11 is an empty submodule).  Written for this repository; implements only
// what cpp/src/cuhnsw_base.cu:67-128 calls: Json::parse(text, err), operator[](key),
// int_value(), bool_value(), number_value(), string_value() on one flat object.
// TEST INFRASTRUCTURE ONLY: used when compiling the reference's own sources into oracle/_ref/.
#pragma once
#include <cstdlib>
#include <map>
#include <memory>
#include <string>

namespace json11 {

class Json {
 public:
  Json() {}
  static Json parse(const std::string& in, std::string& err) {
    Json root;
    root.obj_ = std::make_shared<std::map<std::string, Json>>();
    size_t i = 0;
    auto ws = [&]() { while (i < in.size() && (in[i] == ' ' || in[i] == '\n' || in[i] == '\t' || in[i] == '\r')) ++i; };
    auto str = [&](std::string* out) {
      if (i >= in.size() || in[i] != '"') return false;
      ++i;
      out->clear();
      while (i < in.size() && in[i] != '"') {
        if (in[i] == '\\' && i + 1 < in.size()) ++i;
        out->push_back(in[i++]);
      }
      if (i >= in.size()) return false;
      ++i;
      return true;
    };
    ws();
    if (i >= in.size() || in[i] != '{') { err = "expected object"; return Json(); }
    ++i;
    ws();
    if (i < in.size() && in[i] == '}') return root;
    for (;;) {
      std::string key;
      ws();
      if (!str(&key)) { err = "expected key"; return Json(); }
      ws();
      if (i >= in.size() || in[i] != ':') { err = "expected ':'"; return Json(); }
      ++i;
      ws();
      Json v;
      if (i < in.size() && in[i] == '"') {
        if (!str(&v.str_)) { err = "bad string"; return Json(); }
        v.kind_ = 3;
      } else if (in.compare(i, 4, "true") == 0) { v.kind_ = 2; v.num_ = 1; i += 4; }
      else if (in.compare(i, 5, "false") == 0) { v.kind_ = 2; v.num_ = 0; i += 5; }
      else if (in.compare(i, 4, "null") == 0) { i += 4; }
      else {
        const char* b = in.c_str() + i;
        char* e = nullptr;
        v.num_ = std::strtod(b, &e);
        if (e == b) { err = "bad value"; return Json(); }
        v.kind_ = 1;
        i += (size_t)(e - b);
      }
      (*root.obj_)[key] = v;
      ws();
      if (i < in.size() && in[i] == ',') { ++i; continue; }
      if (i < in.size() && in[i] == '}') return root;
      err = "expected ',' or '}'";
      return Json();
    }
  }
  const Json& operator[](const std::string& key) const {
    static const Json none;
    if (!obj_) return none;
    auto it = obj_->find(key);
    return it == obj_->end() ? none : it->second;
  }
  int int_value() const { return kind_ == 1 ? (int)num_ : 0; }
  double number_value() const { return kind_ == 1 ? num_ : 0.0; }
  bool bool_value() const { return kind_ == 2 ? num_ != 0 : false; }
  const std::string& string_value() const { return str_; }

 private:
  int kind_ = 0;  // 0 null, 1 number, 2 bool, 3 string
  double num_ = 0.0;
  std::string str_;
  std::shared_ptr<std::map<std::string, Json>> obj_;
};

}  // namespace json11
