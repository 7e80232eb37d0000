#include "json.hpp"

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>

namespace pk {

class JsonParser {
 public:
  JsonParser(const char* p, size_t n) : p_(p), end_(p + n) {}

  Json parse_document() {
    Json v = parse_value(0);
    skip_ws();
    if (p_ != end_) fail("trailing characters");
    return v;
  }

 private:
  const char* p_;
  const char* end_;

  [[noreturn]] void fail(const char* what) const { throw std::runtime_error(std::string("json: ") + what); }

  void skip_ws() {
    while (p_ < end_ && (*p_ == ' ' || *p_ == '\n' || *p_ == '\t' || *p_ == '\r')) ++p_;
  }

  Json parse_value(int depth) {
    if (depth > 256) fail("nesting too deep");
    skip_ws();
    if (p_ >= end_) fail("unexpected end");
    switch (*p_) {
      case '{': return parse_object(depth);
      case '[': return parse_array(depth);
      case '"': return Json(parse_string());
      case 't': literal("true"); return Json(true);
      case 'f': literal("false"); return Json(false);
      case 'n': literal("null"); return Json();
      default: return parse_number();
    }
  }

  void literal(const char* word) {
    const size_t n = strlen(word);
    if ((size_t)(end_ - p_) < n || memcmp(p_, word, n) != 0) fail("bad literal");
    p_ += n;
  }

  Json parse_number() {
    const char* s = p_;
    bool integral = true;
    if (p_ < end_ && (*p_ == '-' || *p_ == '+')) ++p_;
    while (p_ < end_ && ((*p_ >= '0' && *p_ <= '9') || *p_ == '.' || *p_ == 'e' || *p_ == 'E' || *p_ == '-' || *p_ == '+')) {
      if (*p_ == '.' || *p_ == 'e' || *p_ == 'E') integral = false;
      ++p_;
    }
    if (p_ == s) fail("bad number");
    std::string tok(s, p_ - s);
    if (integral && tok.size() < 19) return Json((int64_t)strtoll(tok.c_str(), nullptr, 10));
    return Json(strtod(tok.c_str(), nullptr));
  }

  static void append_utf8(std::string& out, uint32_t cp) {
    if (cp < 0x80) {
      out.push_back((char)cp);
    } else if (cp < 0x800) {
      out.push_back((char)(0xC0 | (cp >> 6)));
      out.push_back((char)(0x80 | (cp & 0x3F)));
    } else if (cp < 0x10000) {
      out.push_back((char)(0xE0 | (cp >> 12)));
      out.push_back((char)(0x80 | ((cp >> 6) & 0x3F)));
      out.push_back((char)(0x80 | (cp & 0x3F)));
    } else {
      out.push_back((char)(0xF0 | (cp >> 18)));
      out.push_back((char)(0x80 | ((cp >> 12) & 0x3F)));
      out.push_back((char)(0x80 | ((cp >> 6) & 0x3F)));
      out.push_back((char)(0x80 | (cp & 0x3F)));
    }
  }

  uint32_t hex4() {
    if (end_ - p_ < 4) fail("bad \\u escape");
    uint32_t v = 0;
    for (int i = 0; i < 4; ++i) {
      const char c = *p_++;
      v <<= 4;
      if (c >= '0' && c <= '9') v |= c - '0';
      else if (c >= 'a' && c <= 'f') v |= c - 'a' + 10;
      else if (c >= 'A' && c <= 'F') v |= c - 'A' + 10;
      else fail("bad \\u escape");
    }
    return v;
  }

  std::string parse_string() {
    ++p_;  // opening quote
    std::string out;
    while (true) {
      if (p_ >= end_) fail("unterminated string");
      const char c = *p_++;
      if (c == '"') break;
      if (c != '\\') {
        out.push_back(c);
        continue;
      }
      if (p_ >= end_) fail("bad escape");
      const char e = *p_++;
      switch (e) {
        case '"': out.push_back('"'); break;
        case '\\': out.push_back('\\'); break;
        case '/': out.push_back('/'); break;
        case 'b': out.push_back('\b'); break;
        case 'f': out.push_back('\f'); break;
        case 'n': out.push_back('\n'); break;
        case 'r': out.push_back('\r'); break;
        case 't': out.push_back('\t'); break;
        case 'u': {
          uint32_t cp = hex4();
          if (cp >= 0xD800 && cp <= 0xDBFF && end_ - p_ >= 6 && p_[0] == '\\' && p_[1] == 'u') {
            p_ += 2;
            const uint32_t lo = hex4();
            cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
          }
          append_utf8(out, cp);
          break;
        }
        default: fail("bad escape");
      }
    }
    return out;
  }

  Json parse_array(int depth) {
    ++p_;
    Json out = Json::array();
    skip_ws();
    if (p_ < end_ && *p_ == ']') { ++p_; return out; }
    while (true) {
      out.arr_.push_back(parse_value(depth + 1));
      skip_ws();
      if (p_ >= end_) fail("unterminated array");
      if (*p_ == ',') { ++p_; continue; }
      if (*p_ == ']') { ++p_; break; }
      fail("expected , or ]");
    }
    return out;
  }

  Json parse_object(int depth) {
    ++p_;
    Json out = Json::object();
    skip_ws();
    if (p_ < end_ && *p_ == '}') { ++p_; return out; }
    while (true) {
      skip_ws();
      if (p_ >= end_ || *p_ != '"') fail("expected key");
      std::string key = parse_string();
      skip_ws();
      if (p_ >= end_ || *p_ != ':') fail("expected :");
      ++p_;
      out.obj_.emplace_back(std::move(key), parse_value(depth + 1));
      skip_ws();
      if (p_ >= end_) fail("unterminated object");
      if (*p_ == ',') { ++p_; continue; }
      if (*p_ == '}') { ++p_; break; }
      fail("expected , or }");
    }
    return out;
  }
};

Json Json::parse(const std::string& text) { return JsonParser(text.data(), text.size()).parse_document(); }
Json Json::parse(const char* data, size_t len) { return JsonParser(data, len).parse_document(); }

const Json* Json::find(const std::string& key) const {
  if (type_ != Type::Object) return nullptr;
  for (const auto& kv : obj_)
    if (kv.first == key) return &kv.second;
  return nullptr;
}

const Json& Json::at(const std::string& key) const {
  const Json* v = find(key);
  if (!v) throw std::runtime_error("json: missing key " + key);
  return *v;
}

Json& Json::operator[](const std::string& key) {
  if (type_ == Type::Null) type_ = Type::Object;
  expect(Type::Object);
  for (auto& kv : obj_)
    if (kv.first == key) return kv.second;
  obj_.emplace_back(key, Json());
  return obj_.back().second;
}

int64_t Json::get_int(const std::string& key, int64_t dflt) const {
  const Json* v = find(key);
  return v && v->is_number() ? v->as_int() : dflt;
}
double Json::get_double(const std::string& key, double dflt) const {
  const Json* v = find(key);
  return v && v->is_number() ? v->as_double() : dflt;
}
bool Json::get_bool(const std::string& key, bool dflt) const {
  const Json* v = find(key);
  return v && v->is_bool() ? v->as_bool() : dflt;
}
std::string Json::get_string(const std::string& key, const std::string& dflt) const {
  const Json* v = find(key);
  return v && v->is_string() ? v->as_string() : dflt;
}

std::string json_escape(const std::string& s) {
  std::string out;
  out.reserve(s.size() + 2);
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
          snprintf(buf, sizeof buf, "\\u%04x", c);
          out += buf;
        } else {
          out.push_back((char)c);
        }
    }
  }
  return out;
}

void Json::dump_to(std::string& out) const {
  switch (type_) {
    case Type::Null: out += "null"; break;
    case Type::Bool: out += bool_ ? "true" : "false"; break;
    case Type::Number: {
      char buf[40];
      if (is_int_) snprintf(buf, sizeof buf, "%lld", (long long)int_);
      else if (std::isfinite(num_)) snprintf(buf, sizeof buf, "%.17g", num_);
      else snprintf(buf, sizeof buf, "null");
      out += buf;
      break;
    }
    case Type::String:
      out.push_back('"');
      out += json_escape(str_);
      out.push_back('"');
      break;
    case Type::Array: {
      out.push_back('[');
      bool first = true;
      for (const auto& v : arr_) {
        if (!first) out.push_back(',');
        first = false;
        v.dump_to(out);
      }
      out.push_back(']');
      break;
    }
    case Type::Object: {
      out.push_back('{');
      bool first = true;
      for (const auto& kv : obj_) {
        if (!first) out.push_back(',');
        first = false;
        out.push_back('"');
        out += json_escape(kv.first);
        out += "\":";
        kv.second.dump_to(out);
      }
      out.push_back('}');
      break;
    }
  }
}

std::string Json::dump() const {
  std::string out;
  dump_to(out);
  return out;
}

}  // namespace pk
