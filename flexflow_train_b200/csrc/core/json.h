// json.h -- a small self-contained JSON value, parser and writer.
//
// The compiler core uses it both as the on-disk format layer (the v1
// computation-graph / strategy files and the legacy substitution rule files)
// and as the attribute container of operators: an operator's attributes are a
// JSON object keyed by the field names of the corresponding reference struct
// (lib/op-attrs/include/op-attrs/ops/*_attrs.dtg.toml).
#pragma once
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <map>
#include <memory>
#include <sstream>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace ff {

class Json {
public:
  enum Kind { Null, Bool, Int, Float, String, Array, Object };
  using array_t = std::vector<Json>;
  using object_t = std::vector<std::pair<std::string, Json>>;  // insertion-ordered

  Json() : kind_(Null) {}
  Json(std::nullptr_t) : kind_(Null) {}
  Json(bool b) : kind_(Bool), b_(b) {}
  Json(int v) : kind_(Int), i_(v) {}
  Json(long v) : kind_(Int), i_(v) {}
  Json(long long v) : kind_(Int), i_(v) {}
  Json(unsigned v) : kind_(Int), i_(v) {}
  Json(unsigned long v) : kind_(Int), i_((long long)v) {}
  Json(unsigned long long v) : kind_(Int), i_((long long)v) {}
  Json(double v) : kind_(Float), d_(v) {}
  Json(float v) : kind_(Float), d_(v) {}
  Json(const char *s) : kind_(String), s_(s) {}
  Json(std::string s) : kind_(String), s_(std::move(s)) {}
  Json(array_t a) : kind_(Array), a_(std::move(a)) {}
  static Json array() { Json j; j.kind_ = Array; return j; }
  static Json object() { Json j; j.kind_ = Object; return j; }
  template <typename T>
  static Json from_ints(const std::vector<T> &v) {
    Json j = array();
    for (auto &x : v) j.a_.push_back(Json((long long)x));
    return j;
  }

  Kind kind() const { return kind_; }
  bool is_null() const { return kind_ == Null; }
  bool is_bool() const { return kind_ == Bool; }
  bool is_int() const { return kind_ == Int; }
  bool is_number() const { return kind_ == Int || kind_ == Float; }
  bool is_string() const { return kind_ == String; }
  bool is_array() const { return kind_ == Array; }
  bool is_object() const { return kind_ == Object; }

  bool as_bool() const { need(Bool); return b_; }
  long long as_int() const {
    if (kind_ == Float) return (long long)d_;
    need(Int);
    return i_;
  }
  double as_float() const {
    if (kind_ == Int) return (double)i_;
    need(Float);
    return d_;
  }
  const std::string &as_string() const { need(String); return s_; }
  const array_t &items() const { need(Array); return a_; }
  array_t &items() { need(Array); return a_; }
  const object_t &fields() const { need(Object); return o_; }
  std::vector<long long> as_ints() const {
    std::vector<long long> r;
    for (auto &x : items()) r.push_back(x.as_int());
    return r;
  }

  size_t size() const { return kind_ == Array ? a_.size() : kind_ == Object ? o_.size() : 0; }
  void push_back(Json v) { need(Array); a_.push_back(std::move(v)); }
  const Json &operator[](size_t i) const { need(Array); return a_.at(i); }

  bool contains(const std::string &k) const {
    if (kind_ != Object) return false;
    for (auto &kv : o_) if (kv.first == k) return true;
    return false;
  }
  const Json &at(const std::string &k) const {
    need(Object);
    for (auto &kv : o_) if (kv.first == k) return kv.second;
    throw std::runtime_error("json: missing key '" + k + "'");
  }
  // value of key k, or `dflt` when absent
  const Json &get(const std::string &k, const Json &dflt) const { return contains(k) ? at(k) : dflt; }
  long long get_int(const std::string &k, long long dflt) const { return contains(k) && !at(k).is_null() ? at(k).as_int() : dflt; }
  double get_float(const std::string &k, double dflt) const { return contains(k) && !at(k).is_null() ? at(k).as_float() : dflt; }
  bool get_bool(const std::string &k, bool dflt) const { return contains(k) && !at(k).is_null() ? at(k).as_bool() : dflt; }
  std::string get_string(const std::string &k, const std::string &dflt) const {
    return contains(k) && at(k).is_string() ? at(k).as_string() : dflt;
  }
  Json &operator[](const std::string &k) {
    if (kind_ == Null) kind_ = Object;
    need(Object);
    for (auto &kv : o_) if (kv.first == k) return kv.second;
    o_.emplace_back(k, Json());
    return o_.back().second;
  }
  void set(const std::string &k, Json v) { (*this)[k] = std::move(v); }

  bool operator==(const Json &o) const {
    if (is_number() && o.is_number()) {
      if (kind_ == Int && o.kind_ == Int) return i_ == o.i_;
      return as_float() == o.as_float();
    }
    if (kind_ != o.kind_) return false;
    switch (kind_) {
      case Null: return true;
      case Bool: return b_ == o.b_;
      case String: return s_ == o.s_;
      case Array: return a_ == o.a_;
      case Object: {
        if (o_.size() != o.o_.size()) return false;
        for (auto &kv : o_) {
          if (!o.contains(kv.first) || !(o.at(kv.first) == kv.second)) return false;
        }
        return true;
      }
      default: return false;
    }
  }
  bool operator!=(const Json &o) const { return !(*this == o); }

  // canonical text (object keys sorted) -- used for hashing / dedup keys
  std::string canonical() const {
    std::string out;
    write(out, -1, 0, true);
    return out;
  }
  std::string dump(int indent = -1) const {
    std::string out;
    write(out, indent, 0, false);
    return out;
  }
  static Json parse(const std::string &text) {
    size_t pos = 0;
    Json j = parse_value(text, pos);
    skip_ws(text, pos);
    if (pos != text.size()) throw std::runtime_error("json: trailing characters at " + std::to_string(pos));
    return j;
  }

private:
  Kind kind_;
  bool b_ = false;
  long long i_ = 0;
  double d_ = 0;
  std::string s_;
  array_t a_;
  object_t o_;

  void need(Kind k) const {
    if (kind_ != k) throw std::runtime_error(std::string("json: wrong kind, wanted ") + kind_name(k) + " got " + kind_name(kind_));
  }
  static const char *kind_name(Kind k) {
    static const char *n[] = {"null", "bool", "int", "float", "string", "array", "object"};
    return n[k];
  }
  static void write_string(std::string &out, const std::string &s) {
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
  void write(std::string &out, int indent, int depth, bool sorted) const {
    auto nl = [&](int d) {
      if (indent >= 0) { out.push_back('\n'); out.append((size_t)(indent * d), ' '); }
    };
    switch (kind_) {
      case Null: out += "null"; break;
      case Bool: out += b_ ? "true" : "false"; break;
      case Int: out += std::to_string(i_); break;
      case Float: {
        if (std::isfinite(d_)) {
          char buf[40];
          snprintf(buf, sizeof buf, "%.17g", d_);
          std::string t = buf;
          // shortest form that round-trips
          for (int prec = 1; prec < 17; ++prec) {
            char b2[40];
            snprintf(b2, sizeof b2, "%.*g", prec, d_);
            if (strtod(b2, nullptr) == d_) { t = b2; break; }
          }
          if (t.find_first_of(".eEn") == std::string::npos) t += ".0";
          out += t;
        } else out += "null";
        break;
      }
      case String: write_string(out, s_); break;
      case Array:
        out.push_back('[');
        for (size_t i = 0; i < a_.size(); ++i) {
          if (i) out.push_back(',');
          nl(depth + 1);
          a_[i].write(out, indent, depth + 1, sorted);
        }
        if (!a_.empty()) nl(depth);
        out.push_back(']');
        break;
      case Object: {
        out.push_back('{');
        std::vector<const std::pair<std::string, Json> *> order;
        for (auto &kv : o_) order.push_back(&kv);
        if (sorted) {
          std::sort(order.begin(), order.end(), [](auto *a, auto *b) { return a->first < b->first; });
        }
        for (size_t i = 0; i < order.size(); ++i) {
          if (i) out.push_back(',');
          nl(depth + 1);
          write_string(out, order[i]->first);
          out += indent >= 0 ? ": " : ":";
          order[i]->second.write(out, indent, depth + 1, sorted);
        }
        if (!order.empty()) nl(depth);
        out.push_back('}');
        break;
      }
    }
  }
  static void skip_ws(const std::string &t, size_t &p) {
    while (p < t.size() && (t[p] == ' ' || t[p] == '\n' || t[p] == '\t' || t[p] == '\r')) ++p;
  }
  static Json parse_value(const std::string &t, size_t &p) {
    skip_ws(t, p);
    if (p >= t.size()) throw std::runtime_error("json: unexpected end");
    char c = t[p];
    if (c == '{') {
      ++p;
      Json j = object();
      skip_ws(t, p);
      if (p < t.size() && t[p] == '}') { ++p; return j; }
      while (true) {
        skip_ws(t, p);
        std::string k = parse_string(t, p);
        skip_ws(t, p);
        if (p >= t.size() || t[p] != ':') throw std::runtime_error("json: expected ':' at " + std::to_string(p));
        ++p;
        j.o_.emplace_back(std::move(k), parse_value(t, p));
        skip_ws(t, p);
        if (p < t.size() && t[p] == ',') { ++p; continue; }
        if (p < t.size() && t[p] == '}') { ++p; break; }
        throw std::runtime_error("json: expected ',' or '}' at " + std::to_string(p));
      }
      return j;
    }
    if (c == '[') {
      ++p;
      Json j = array();
      skip_ws(t, p);
      if (p < t.size() && t[p] == ']') { ++p; return j; }
      while (true) {
        j.a_.push_back(parse_value(t, p));
        skip_ws(t, p);
        if (p < t.size() && t[p] == ',') { ++p; continue; }
        if (p < t.size() && t[p] == ']') { ++p; break; }
        throw std::runtime_error("json: expected ',' or ']' at " + std::to_string(p));
      }
      return j;
    }
    if (c == '"') return Json(parse_string(t, p));
    if (t.compare(p, 4, "true") == 0) { p += 4; return Json(true); }
    if (t.compare(p, 5, "false") == 0) { p += 5; return Json(false); }
    if (t.compare(p, 4, "null") == 0) { p += 4; return Json(); }
    // number
    size_t s = p;
    bool is_float = false;
    if (t[p] == '-' || t[p] == '+') ++p;
    while (p < t.size() && (isdigit((unsigned char)t[p]) || t[p] == '.' || t[p] == 'e' || t[p] == 'E' || t[p] == '-' || t[p] == '+')) {
      if (t[p] == '.' || t[p] == 'e' || t[p] == 'E') is_float = true;
      ++p;
    }
    if (s == p) throw std::runtime_error("json: unexpected character at " + std::to_string(p));
    std::string num = t.substr(s, p - s);
    if (is_float) return Json(strtod(num.c_str(), nullptr));
    return Json((long long)strtoll(num.c_str(), nullptr, 10));
  }
  static std::string parse_string(const std::string &t, size_t &p) {
    if (p >= t.size() || t[p] != '"') throw std::runtime_error("json: expected string at " + std::to_string(p));
    ++p;
    std::string out;
    while (p < t.size() && t[p] != '"') {
      if (t[p] == '\\') {
        ++p;
        if (p >= t.size()) break;
        switch (t[p]) {
          case 'n': out.push_back('\n'); break;
          case 't': out.push_back('\t'); break;
          case 'r': out.push_back('\r'); break;
          case 'b': out.push_back('\b'); break;
          case 'f': out.push_back('\f'); break;
          case 'u': {
            unsigned code = (unsigned)strtoul(t.substr(p + 1, 4).c_str(), nullptr, 16);
            p += 4;
            if (code < 0x80) out.push_back((char)code);
            else if (code < 0x800) { out.push_back((char)(0xC0 | (code >> 6))); out.push_back((char)(0x80 | (code & 0x3F))); }
            else { out.push_back((char)(0xE0 | (code >> 12))); out.push_back((char)(0x80 | ((code >> 6) & 0x3F))); out.push_back((char)(0x80 | (code & 0x3F))); }
            break;
          }
          default: out.push_back(t[p]);
        }
        ++p;
      } else out.push_back(t[p++]);
    }
    if (p >= t.size()) throw std::runtime_error("json: unterminated string");
    ++p;
    return out;
  }
};

}  // namespace ff
