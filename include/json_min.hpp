// json_min.hpp -- a small JSON reader for model configurations and request lines (header only).
// Objects keep their keys in a map; numbers are doubles; no writer beyond what the callers print themselves.
#pragma once
#include <stdlib.h>

#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

class JsonValue {
 public:
  enum Kind { Null, Bool, Number, String, Array, Object };
  Kind kind = Null;
  bool b = false;
  double num = 0.0;
  std::string str;
  std::vector<JsonValue> arr;
  std::map<std::string, JsonValue> obj;

  bool is_null() const { return kind == Null; }
  bool has(const std::string& k) const { return kind == Object && obj.count(k) && !obj.at(k).is_null(); }
  const JsonValue& at(const std::string& k) const {
    if (kind != Object || !obj.count(k)) throw std::runtime_error("config: missing key '" + k + "'");
    return obj.at(k);
  }
  double number() const {
    if (kind != Number) throw std::runtime_error("config: a number was expected");
    return num;
  }
  int integer() const { return (int)number(); }
  const std::string& string() const {
    if (kind != String) throw std::runtime_error("config: a string was expected");
    return str;
  }
  double number_or(const std::string& k, double dflt) const { return has(k) ? at(k).number() : dflt; }

  static JsonValue parse(const std::string& text) {
    size_t i = 0;
    JsonValue v = value(text, i);
    skip(text, i);
    if (i != text.size()) throw std::runtime_error("json: trailing characters");
    return v;
  }

 private:
  static void skip(const std::string& s, size_t& i) {
    while (i < s.size() && (s[i] == ' ' || s[i] == '\n' || s[i] == '\t' || s[i] == '\r')) i++;
  }
  static JsonValue value(const std::string& s, size_t& i) {
    skip(s, i);
    if (i >= s.size()) throw std::runtime_error("json: unexpected end");
    JsonValue v;
    const char c = s[i];
    if (c == '{') {
      v.kind = Object;
      i++;
      skip(s, i);
      if (i < s.size() && s[i] == '}') { i++; return v; }
      while (true) {
        skip(s, i);
        JsonValue k = value(s, i);
        if (k.kind != String) throw std::runtime_error("json: a key must be a string");
        skip(s, i);
        if (i >= s.size() || s[i] != ':') throw std::runtime_error("json: ':' expected");
        i++;
        v.obj[k.str] = value(s, i);
        skip(s, i);
        if (i < s.size() && s[i] == ',') { i++; continue; }
        if (i < s.size() && s[i] == '}') { i++; return v; }
        throw std::runtime_error("json: ',' or '}' expected");
      }
    }
    if (c == '[') {
      v.kind = Array;
      i++;
      skip(s, i);
      if (i < s.size() && s[i] == ']') { i++; return v; }
      while (true) {
        v.arr.push_back(value(s, i));
        skip(s, i);
        if (i < s.size() && s[i] == ',') { i++; continue; }
        if (i < s.size() && s[i] == ']') { i++; return v; }
        throw std::runtime_error("json: ',' or ']' expected");
      }
    }
    if (c == '"') {
      v.kind = String;
      i++;
      while (i < s.size() && s[i] != '"') {
        if (s[i] == '\\' && i + 1 < s.size()) {
          const char e = s[i + 1];
          if (e == 'n') v.str += '\n';
          else if (e == 't') v.str += '\t';
          else if (e == 'r') v.str += '\r';
          else if (e == 'b') v.str += '\b';
          else if (e == 'f') v.str += '\f';
          else if (e == 'u' && i + 5 < s.size()) {   // code points above 127 are kept as '?': no caller needs them
            const long cp = strtol(s.substr(i + 2, 4).c_str(), nullptr, 16);
            v.str += cp < 128 ? (char)cp : '?';
            i += 4;
          } else v.str += e;
          i += 2;
        } else v.str += s[i++];
      }
      if (i >= s.size()) throw std::runtime_error("json: unterminated string");
      i++;
      return v;
    }
    if (s.compare(i, 4, "true") == 0) { v.kind = Bool; v.b = true; i += 4; return v; }
    if (s.compare(i, 5, "false") == 0) { v.kind = Bool; v.b = false; i += 5; return v; }
    if (s.compare(i, 4, "null") == 0) { i += 4; return v; }
    char* end = nullptr;
    v.num = strtod(s.c_str() + i, &end);
    if (end == s.c_str() + i) throw std::runtime_error("json: unexpected character");
    v.kind = Number;
    i = (size_t)(end - s.c_str());
    return v;
  }
};
