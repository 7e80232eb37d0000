// Small JSON document model and recursive-descent parser/serialiser for the engine's
// host side (model configs, Safetensors headers, tokenizer files, HTTP bodies, sidecar
// lines). Plays the role of the reference's cpp_engine/src/json_lite.cpp.
#pragma once

#include <cstdint>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace pk {

class Json {
 public:
  enum class Type { Null, Bool, Number, String, Array, Object };
  using Array = std::vector<Json>;
  // Insertion order matters for Safetensors headers and chat payloads.
  using Object = std::vector<std::pair<std::string, Json>>;

  Json() : type_(Type::Null) {}
  Json(bool b) : type_(Type::Bool), bool_(b) {}
  Json(double d) : type_(Type::Number), num_(d) {}
  Json(int64_t i) : type_(Type::Number), num_((double)i), int_(i), is_int_(true) {}
  Json(int i) : Json((int64_t)i) {}
  Json(const char* s) : type_(Type::String), str_(s) {}
  Json(std::string s) : type_(Type::String), str_(std::move(s)) {}
  static Json array() { Json j; j.type_ = Type::Array; return j; }
  static Json object() { Json j; j.type_ = Type::Object; return j; }

  static Json parse(const std::string& text);
  static Json parse(const char* data, size_t len);
  std::string dump() const;

  Type type() const { return type_; }
  bool is_null() const { return type_ == Type::Null; }
  bool is_object() const { return type_ == Type::Object; }
  bool is_array() const { return type_ == Type::Array; }
  bool is_string() const { return type_ == Type::String; }
  bool is_number() const { return type_ == Type::Number; }
  bool is_bool() const { return type_ == Type::Bool; }

  bool as_bool() const { expect(Type::Bool); return bool_; }
  double as_double() const { expect(Type::Number); return num_; }
  int64_t as_int() const { expect(Type::Number); return is_int_ ? int_ : (int64_t)num_; }
  const std::string& as_string() const { expect(Type::String); return str_; }
  const Array& items() const { expect(Type::Array); return arr_; }
  Array& items() { expect(Type::Array); return arr_; }
  const Object& members() const { expect(Type::Object); return obj_; }

  // Object access. find() returns nullptr when the key is absent.
  const Json* find(const std::string& key) const;
  const Json& at(const std::string& key) const;
  Json& operator[](const std::string& key);  // inserts null when absent
  bool contains(const std::string& key) const { return find(key) != nullptr; }
  void push_back(Json v) { expect(Type::Array); arr_.push_back(std::move(v)); }
  size_t size() const { return type_ == Type::Array ? arr_.size() : type_ == Type::Object ? obj_.size() : 0; }

  // Typed getters with defaults.
  int64_t get_int(const std::string& key, int64_t dflt) const;
  double get_double(const std::string& key, double dflt) const;
  bool get_bool(const std::string& key, bool dflt) const;
  std::string get_string(const std::string& key, const std::string& dflt) const;

 private:
  void expect(Type t) const {
    if (type_ != t) throw std::runtime_error("json: wrong value type");
  }
  void dump_to(std::string& out) const;

  Type type_;
  bool bool_ = false;
  double num_ = 0.0;
  int64_t int_ = 0;
  bool is_int_ = false;
  std::string str_;
  Array arr_;
  Object obj_;
  friend class JsonParser;
};

std::string json_escape(const std::string& s);

}  // namespace pk
