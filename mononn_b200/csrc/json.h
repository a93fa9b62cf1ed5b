// Minimal JSON value, parser and writer for tuning specs and backend_config strings.
// (The reference vendors nlohmann/json and converts protobuf <-> JSON with original field
// names, mononn_engine/helpers/protobuf.cc:32-88; only plain JSON is needed here.)
#pragma once
#include <cctype>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <map>
#include <memory>
#include <string>
#include <utility>
#include <vector>

namespace mononn {

class Json {
 public:
  enum Type { Null, Bool, Number, String, Array, Object };
  Type type = Null;
  bool b = false;
  double num = 0;
  std::string str;
  std::vector<Json> arr;
  std::vector<std::pair<std::string, Json>> obj;  // insertion order kept

  Json() = default;
  static Json number(double v) { Json j; j.type = Number; j.num = v; return j; }
  static Json string(const std::string& s) { Json j; j.type = String; j.str = s; return j; }
  static Json boolean(bool v) { Json j; j.type = Bool; j.b = v; return j; }
  static Json array() { Json j; j.type = Array; return j; }
  static Json object() { Json j; j.type = Object; return j; }

  bool is_object() const { return type == Object; }
  bool is_array() const { return type == Array; }
  const Json* find(const std::string& k) const {
    if (type != Object) return nullptr;
    for (const auto& kv : obj)
      if (kv.first == k) return &kv.second;
    return nullptr;
  }
  Json& set(const std::string& k, const Json& v) {
    for (auto& kv : obj)
      if (kv.first == k) { kv.second = v; return kv.second; }
    obj.emplace_back(k, v);
    return obj.back().second;
  }
  // Numbers may arrive as strings (XLA backend_config prints int64 as "123").
  double as_number(double dflt = 0) const {
    if (type == Number) return num;
    if (type == String) { char* e = nullptr; double v = std::strtod(str.c_str(), &e); return e != str.c_str() ? v : dflt; }
    if (type == Bool) return b ? 1 : 0;
    return dflt;
  }
  double get_number(const std::string& k, double dflt = 0) const {
    const Json* j = find(k);
    return j ? j->as_number(dflt) : dflt;
  }
  std::string get_string(const std::string& k, const std::string& dflt = "") const {
    const Json* j = find(k);
    return (j && j->type == String) ? j->str : dflt;
  }

  std::string dump(int indent = 0) const {
    std::string out;
    write(out, indent, 0);
    return out;
  }

  static bool parse(const std::string& text, Json* out, std::string* err) {
    size_t i = 0;
    if (!parse_value(text, i, out, err, 0)) return false;
    skip_ws(text, i);
    if (i != text.size()) {
      if (err) *err = "trailing characters at offset " + std::to_string(i);
      return false;
    }
    return true;
  }

 private:
  static void skip_ws(const std::string& s, size_t& i) {
    while (i < s.size() && std::isspace(static_cast<unsigned char>(s[i]))) ++i;
  }
  static bool fail(std::string* err, const std::string& m, size_t i) {
    if (err) *err = m + " at offset " + std::to_string(i);
    return false;
  }
  static bool parse_string(const std::string& s, size_t& i, std::string* out, std::string* err) {
    if (s[i] != '"') return fail(err, "expected string", i);
    ++i;
    out->clear();
    while (i < s.size() && s[i] != '"') {
      char c = s[i++];
      if (c == '\\') {
        if (i >= s.size()) return fail(err, "bad escape", i);
        char e = s[i++];
        switch (e) {
          case 'n': out->push_back('\n'); break;
          case 't': out->push_back('\t'); break;
          case 'r': out->push_back('\r'); break;
          case 'b': out->push_back('\b'); break;
          case 'f': out->push_back('\f'); break;
          case 'u': {
            if (i + 4 > s.size()) return fail(err, "bad \\u escape", i);
            unsigned v = static_cast<unsigned>(std::strtoul(s.substr(i, 4).c_str(), nullptr, 16));
            i += 4;
            if (v < 0x80) out->push_back(static_cast<char>(v));
            else if (v < 0x800) { out->push_back(static_cast<char>(0xC0 | (v >> 6))); out->push_back(static_cast<char>(0x80 | (v & 0x3F))); }
            else { out->push_back(static_cast<char>(0xE0 | (v >> 12))); out->push_back(static_cast<char>(0x80 | ((v >> 6) & 0x3F))); out->push_back(static_cast<char>(0x80 | (v & 0x3F))); }
            break;
          }
          default: out->push_back(e);
        }
      } else {
        out->push_back(c);
      }
    }
    if (i >= s.size()) return fail(err, "unterminated string", i);
    ++i;
    return true;
  }
  static bool parse_value(const std::string& s, size_t& i, Json* out, std::string* err, int depth) {
    if (depth > 64) return fail(err, "nesting too deep", i);
    skip_ws(s, i);
    if (i >= s.size()) return fail(err, "unexpected end", i);
    const char c = s[i];
    if (c == '{') {
      *out = object();
      ++i;
      skip_ws(s, i);
      if (i < s.size() && s[i] == '}') { ++i; return true; }
      for (;;) {
        skip_ws(s, i);
        std::string k;
        if (i >= s.size() || !parse_string(s, i, &k, err)) return fail(err, "expected key", i);
        skip_ws(s, i);
        if (i >= s.size() || s[i] != ':') return fail(err, "expected ':'", i);
        ++i;
        Json v;
        if (!parse_value(s, i, &v, err, depth + 1)) return false;
        out->obj.emplace_back(k, v);
        skip_ws(s, i);
        if (i < s.size() && s[i] == ',') { ++i; continue; }
        if (i < s.size() && s[i] == '}') { ++i; return true; }
        return fail(err, "expected ',' or '}'", i);
      }
    }
    if (c == '[') {
      *out = array();
      ++i;
      skip_ws(s, i);
      if (i < s.size() && s[i] == ']') { ++i; return true; }
      for (;;) {
        Json v;
        if (!parse_value(s, i, &v, err, depth + 1)) return false;
        out->arr.push_back(v);
        skip_ws(s, i);
        if (i < s.size() && s[i] == ',') { ++i; continue; }
        if (i < s.size() && s[i] == ']') { ++i; return true; }
        return fail(err, "expected ',' or ']'", i);
      }
    }
    if (c == '"') {
      out->type = String;
      return parse_string(s, i, &out->str, err);
    }
    if (s.compare(i, 4, "true") == 0) { *out = boolean(true); i += 4; return true; }
    if (s.compare(i, 5, "false") == 0) { *out = boolean(false); i += 5; return true; }
    if (s.compare(i, 4, "null") == 0) { *out = Json(); i += 4; return true; }
    char* e = nullptr;
    const double v = std::strtod(s.c_str() + i, &e);
    if (e == s.c_str() + i) return fail(err, "unexpected character", i);
    i = static_cast<size_t>(e - s.c_str());
    *out = number(v);
    return true;
  }
  static void escape(const std::string& s, std::string& out) {
    out.push_back('"');
    for (char c : s) {
      switch (c) {
        case '"': out += "\\\""; break;
        case '\\': out += "\\\\"; break;
        case '\n': out += "\\n"; break;
        case '\t': out += "\\t"; break;
        case '\r': out += "\\r"; break;
        default:
          if (static_cast<unsigned char>(c) < 0x20) { char b[8]; std::snprintf(b, sizeof(b), "\\u%04x", c); out += b; }
          else out.push_back(c);
      }
    }
    out.push_back('"');
  }
  void write(std::string& out, int indent, int level) const {
    auto nl = [&](int lv) {
      if (indent > 0) { out.push_back('\n'); out.append(static_cast<size_t>(indent * lv), ' '); }
    };
    switch (type) {
      case Null: out += "null"; break;
      case Bool: out += b ? "true" : "false"; break;
      case Number: {
        char buf[40];
        if (std::floor(num) == num && std::fabs(num) < 1e15) std::snprintf(buf, sizeof(buf), "%lld", static_cast<long long>(num));
        else std::snprintf(buf, sizeof(buf), "%.9g", num);
        out += buf;
        break;
      }
      case String: escape(str, out); break;
      case Array:
        out.push_back('[');
        for (size_t i = 0; i < arr.size(); ++i) {
          if (i) out.push_back(',');
          nl(level + 1);
          arr[i].write(out, indent, level + 1);
        }
        if (!arr.empty()) nl(level);
        out.push_back(']');
        break;
      case Object:
        out.push_back('{');
        for (size_t i = 0; i < obj.size(); ++i) {
          if (i) out.push_back(',');
          nl(level + 1);
          escape(obj[i].first, out);
          out += indent > 0 ? ": " : ":";
          obj[i].second.write(out, indent, level + 1);
        }
        if (!obj.empty()) nl(level);
        out.push_back('}');
        break;
    }
  }
};

}  // namespace mononn
