// Minimal JSON document model, parser and serializer used by the serving runtime (configs,
// request/response bodies of the JSON FFI, metrics). Objects keep insertion order.
#pragma once
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <optional>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace mlcb {
namespace json {

class Value;
using Array = std::vector<Value>;
using Member = std::pair<std::string, Value>;

class Object {
 public:
  Value& operator[](const std::string& key);
  const Value* find(const std::string& key) const;
  Value* find(const std::string& key);
  bool contains(const std::string& key) const { return find(key) != nullptr; }
  size_t size() const { return members_.size(); }
  std::vector<Member>& members() { return members_; }
  const std::vector<Member>& members() const { return members_; }
  void erase(const std::string& key);

 private:
  std::vector<Member> members_;
};

enum class Type { Null, Bool, Int, Double, String, Array, Object };

class Value {
 public:
  Value() : type_(Type::Null) {}
  Value(std::nullptr_t) : type_(Type::Null) {}
  Value(bool b) : type_(Type::Bool), b_(b) {}
  Value(int v) : type_(Type::Int), i_(v) {}
  Value(int64_t v) : type_(Type::Int), i_(v) {}
  Value(uint64_t v) : type_(Type::Int), i_(static_cast<int64_t>(v)) {}
  Value(double v) : type_(Type::Double), d_(v) {}
  Value(const char* s) : type_(Type::String), s_(s) {}
  Value(std::string s) : type_(Type::String), s_(std::move(s)) {}
  Value(Array a) : type_(Type::Array), a_(std::make_shared<Array>(std::move(a))) {}
  Value(Object o) : type_(Type::Object), o_(std::make_shared<Object>(std::move(o))) {}

  Type type() const { return type_; }
  bool is_null() const { return type_ == Type::Null; }
  bool is_bool() const { return type_ == Type::Bool; }
  bool is_int() const { return type_ == Type::Int; }
  bool is_number() const { return type_ == Type::Int || type_ == Type::Double; }
  bool is_string() const { return type_ == Type::String; }
  bool is_array() const { return type_ == Type::Array; }
  bool is_object() const { return type_ == Type::Object; }

  bool as_bool() const { expect(Type::Bool); return b_; }
  int64_t as_int() const {
    if (type_ == Type::Double && d_ == std::floor(d_)) return static_cast<int64_t>(d_);
    expect(Type::Int);
    return i_;
  }
  double as_double() const {
    if (type_ == Type::Int) return static_cast<double>(i_);
    expect(Type::Double);
    return d_;
  }
  const std::string& as_string() const { expect(Type::String); return s_; }
  const Array& as_array() const { expect(Type::Array); return *a_; }
  Array& as_array() { expect(Type::Array); return *a_; }
  const Object& as_object() const { expect(Type::Object); return *o_; }
  Object& as_object() { expect(Type::Object); return *o_; }

  std::string dump() const {
    std::string out;
    write(out);
    return out;
  }
  void write(std::string& out) const;

 private:
  void expect(Type t) const {
    if (type_ != t) throw std::runtime_error("json: unexpected value type");
  }
  Type type_;
  bool b_ = false;
  int64_t i_ = 0;
  double d_ = 0;
  std::string s_;
  std::shared_ptr<Array> a_;
  std::shared_ptr<Object> o_;
};

inline Value& Object::operator[](const std::string& key) {
  for (auto& m : members_)
    if (m.first == key) return m.second;
  members_.emplace_back(key, Value());
  return members_.back().second;
}
inline const Value* Object::find(const std::string& key) const {
  for (auto& m : members_)
    if (m.first == key) return &m.second;
  return nullptr;
}
inline Value* Object::find(const std::string& key) {
  for (auto& m : members_)
    if (m.first == key) return &m.second;
  return nullptr;
}
inline void Object::erase(const std::string& key) {
  for (size_t i = 0; i < members_.size(); ++i)
    if (members_[i].first == key) {
      members_.erase(members_.begin() + i);
      return;
    }
}

inline void escape_to(const std::string& s, std::string& out) {
  out.push_back('"');
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
        if (c < 0x20) {
          char buf[8];
          snprintf(buf, sizeof(buf), "\\u%04x", c);
          out += buf;
        } else {
          out.push_back(static_cast<char>(c));
        }
    }
  }
  out.push_back('"');
}

inline void Value::write(std::string& out) const {
  switch (type_) {
    case Type::Null: out += "null"; break;
    case Type::Bool: out += b_ ? "true" : "false"; break;
    case Type::Int: out += std::to_string(i_); break;
    case Type::Double: {
      if (!std::isfinite(d_)) {
        out += "null";
      } else {
        char buf[40];
        snprintf(buf, sizeof(buf), "%.17g", d_);
        // prefer the shortest representation that round-trips
        for (int prec = 1; prec < 17; ++prec) {
          char b2[40];
          snprintf(b2, sizeof(b2), "%.*g", prec, d_);
          if (strtod(b2, nullptr) == d_) {
            memcpy(buf, b2, sizeof(b2));
            break;
          }
        }
        out += buf;
        if (!strpbrk(buf, ".eEn")) out += ".0";
      }
      break;
    }
    case Type::String: escape_to(s_, out); break;
    case Type::Array: {
      out.push_back('[');
      bool first = true;
      for (auto& v : *a_) {
        if (!first) out.push_back(',');
        first = false;
        v.write(out);
      }
      out.push_back(']');
      break;
    }
    case Type::Object: {
      out.push_back('{');
      bool first = true;
      for (auto& m : o_->members()) {
        if (!first) out.push_back(',');
        first = false;
        escape_to(m.first, out);
        out.push_back(':');
        m.second.write(out);
      }
      out.push_back('}');
      break;
    }
  }
}

class Parser {
 public:
  explicit Parser(const std::string& text) : s_(text) {}
  Value parse() {
    Value v = value();
    ws();
    if (p_ != s_.size()) fail("trailing characters");
    return v;
  }

 private:
  [[noreturn]] void fail(const char* msg) const {
    throw std::runtime_error(std::string("json parse error at ") + std::to_string(p_) + ": " + msg);
  }
  void ws() {
    while (p_ < s_.size() && (s_[p_] == ' ' || s_[p_] == '\n' || s_[p_] == '\t' || s_[p_] == '\r')) ++p_;
  }
  Value value() {
    ws();
    if (p_ >= s_.size()) fail("unexpected end");
    char c = s_[p_];
    if (c == '{') return object();
    if (c == '[') return array();
    if (c == '"') return Value(string());
    if (!s_.compare(p_, 4, "true")) { p_ += 4; return Value(true); }
    if (!s_.compare(p_, 5, "false")) { p_ += 5; return Value(false); }
    if (!s_.compare(p_, 4, "null")) { p_ += 4; return Value(); }
    return number();
  }
  Value number() {
    size_t start = p_;
    bool is_double = false;
    if (p_ < s_.size() && (s_[p_] == '-' || s_[p_] == '+')) ++p_;
    while (p_ < s_.size()) {
      char c = s_[p_];
      if (c >= '0' && c <= '9') { ++p_; }
      else if (c == '.' || c == 'e' || c == 'E' || c == '-' || c == '+') { is_double = true; ++p_; }
      else break;
    }
    if (start == p_) fail("invalid value");
    std::string tok = s_.substr(start, p_ - start);
    if (!is_double) {
      errno = 0;
      long long v = strtoll(tok.c_str(), nullptr, 10);
      if (errno == 0) return Value(static_cast<int64_t>(v));
    }
    return Value(strtod(tok.c_str(), nullptr));
  }
  static void append_utf8(std::string& out, uint32_t cp) {
    if (cp < 0x80) out.push_back(static_cast<char>(cp));
    else if (cp < 0x800) { out.push_back(0xC0 | (cp >> 6)); out.push_back(0x80 | (cp & 0x3F)); }
    else if (cp < 0x10000) {
      out.push_back(0xE0 | (cp >> 12)); out.push_back(0x80 | ((cp >> 6) & 0x3F)); out.push_back(0x80 | (cp & 0x3F));
    } else {
      out.push_back(0xF0 | (cp >> 18)); out.push_back(0x80 | ((cp >> 12) & 0x3F));
      out.push_back(0x80 | ((cp >> 6) & 0x3F)); out.push_back(0x80 | (cp & 0x3F));
    }
  }
  uint32_t hex4() {
    if (p_ + 4 > s_.size()) fail("bad \\u escape");
    uint32_t v = 0;
    for (int i = 0; i < 4; ++i) {
      char c = s_[p_++];
      v <<= 4;
      if (c >= '0' && c <= '9') v |= c - '0';
      else if (c >= 'a' && c <= 'f') v |= c - 'a' + 10;
      else if (c >= 'A' && c <= 'F') v |= c - 'A' + 10;
      else fail("bad hex digit");
    }
    return v;
  }
  std::string string() {
    ++p_;  // opening quote
    std::string out;
    while (true) {
      if (p_ >= s_.size()) fail("unterminated string");
      char c = s_[p_++];
      if (c == '"') break;
      if (c != '\\') { out.push_back(c); continue; }
      if (p_ >= s_.size()) fail("bad escape");
      char e = s_[p_++];
      switch (e) {
        case 'n': out.push_back('\n'); break;
        case 't': out.push_back('\t'); break;
        case 'r': out.push_back('\r'); break;
        case 'b': out.push_back('\b'); break;
        case 'f': out.push_back('\f'); break;
        case '/': out.push_back('/'); break;
        case '\\': out.push_back('\\'); break;
        case '"': out.push_back('"'); break;
        case 'u': {
          uint32_t cp = hex4();
          if (cp >= 0xD800 && cp < 0xDC00 && p_ + 1 < s_.size() && s_[p_] == '\\' && s_[p_ + 1] == 'u') {
            p_ += 2;
            uint32_t lo = hex4();
            cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
          }
          append_utf8(out, cp);
          break;
        }
        default: fail("unknown escape");
      }
    }
    return out;
  }
  Value array() {
    ++p_;
    Array a;
    ws();
    if (p_ < s_.size() && s_[p_] == ']') { ++p_; return Value(std::move(a)); }
    while (true) {
      a.push_back(value());
      ws();
      if (p_ >= s_.size()) fail("unterminated array");
      if (s_[p_] == ',') { ++p_; continue; }
      if (s_[p_] == ']') { ++p_; break; }
      fail("expected , or ]");
    }
    return Value(std::move(a));
  }
  Value object() {
    ++p_;
    Object o;
    ws();
    if (p_ < s_.size() && s_[p_] == '}') { ++p_; return Value(std::move(o)); }
    while (true) {
      ws();
      if (p_ >= s_.size() || s_[p_] != '"') fail("expected string key");
      std::string k = string();
      ws();
      if (p_ >= s_.size() || s_[p_] != ':') fail("expected :");
      ++p_;
      o[k] = value();
      ws();
      if (p_ >= s_.size()) fail("unterminated object");
      if (s_[p_] == ',') { ++p_; continue; }
      if (s_[p_] == '}') { ++p_; break; }
      fail("expected , or }");
    }
    return Value(std::move(o));
  }
  const std::string& s_;
  size_t p_ = 0;
};

inline Value parse(const std::string& text) { return Parser(text).parse(); }

// Typed lookups with defaults.
template <typename T>
inline T get_or(const Object& o, const std::string& key, T dflt);
template <>
inline int64_t get_or<int64_t>(const Object& o, const std::string& key, int64_t d) {
  auto* v = o.find(key);
  return (v && v->is_number()) ? v->as_int() : d;
}
template <>
inline int get_or<int>(const Object& o, const std::string& key, int d) {
  auto* v = o.find(key);
  return (v && v->is_number()) ? static_cast<int>(v->as_int()) : d;
}
template <>
inline double get_or<double>(const Object& o, const std::string& key, double d) {
  auto* v = o.find(key);
  return (v && v->is_number()) ? v->as_double() : d;
}
template <>
inline bool get_or<bool>(const Object& o, const std::string& key, bool d) {
  auto* v = o.find(key);
  return (v && v->is_bool()) ? v->as_bool() : d;
}
template <>
inline std::string get_or<std::string>(const Object& o, const std::string& key, std::string d) {
  auto* v = o.find(key);
  return (v && v->is_string()) ? v->as_string() : d;
}

}  // namespace json
}  // namespace mlcb
