// A small JSON reader for model folders (config.json, the header of a safetensors file): objects, arrays, strings,
// numbers, true / false / null.  Header-only, no dependencies; values are immutable after parsing.
#ifndef KLLM_KUIPER_MODEL_JSON_H_
#define KLLM_KUIPER_MODEL_JSON_H_
#include <cmath>
#include <cstdlib>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace model {
namespace json {
class Value {
 public:
  enum class Kind { kNull, kBool, kNumber, kString, kArray, kObject };
  Kind kind = Kind::kNull;
  bool boolean = false;
  double number = 0;
  std::string string;
  std::vector<Value> array;
  std::vector<std::pair<std::string, Value>> object;  // in file order

  bool is_null() const { return kind == Kind::kNull; }
  bool is_object() const { return kind == Kind::kObject; }
  bool is_array() const { return kind == Kind::kArray; }
  // member of an object, or nullptr
  const Value* find(const std::string& key) const {
    if (kind != Kind::kObject) return nullptr;
    for (const auto& kv : object)
      if (kv.first == key) return &kv.second;
    return nullptr;
  }
  bool has(const std::string& key) const {
    const Value* v = find(key);
    return v != nullptr && !v->is_null();
  }
  const Value& at(const std::string& key) const {
    const Value* v = find(key);
    if (v == nullptr) throw std::runtime_error("json: missing key '" + key + "'");
    return *v;
  }
  double as_number() const {
    if (kind != Kind::kNumber) throw std::runtime_error("json: not a number");
    return number;
  }
  long long as_int() const {
    const double d = as_number();
    if (d != std::floor(d)) throw std::runtime_error("json: not an integer");
    return static_cast<long long>(d);
  }
  const std::string& as_string() const {
    if (kind != Kind::kString) throw std::runtime_error("json: not a string");
    return string;
  }
};

class Parser {
 public:
  explicit Parser(const std::string& text) : s_(text) {}
  Value parse() {
    Value v = value();
    ws();
    if (i_ != s_.size()) fail("trailing characters");
    return v;
  }

 private:
  const std::string& s_;
  size_t i_ = 0;
  [[noreturn]] void fail(const std::string& what) const {
    throw std::runtime_error("json: " + what + " at byte " + std::to_string(i_));
  }
  void ws() {
    while (i_ < s_.size() && (s_[i_] == ' ' || s_[i_] == '\n' || s_[i_] == '\t' || s_[i_] == '\r')) ++i_;
  }
  bool eat(char c) {
    ws();
    if (i_ < s_.size() && s_[i_] == c) {
      ++i_;
      return true;
    }
    return false;
  }
  void expect(char c) {
    if (!eat(c)) fail(std::string("expected '") + c + "'");
  }
  Value value() {
    ws();
    if (i_ >= s_.size()) fail("unexpected end");
    const char c = s_[i_];
    Value v;
    if (c == '{') {
      ++i_;
      v.kind = Value::Kind::kObject;
      if (eat('}')) return v;
      do {
        ws();
        std::string key = str();
        expect(':');
        v.object.emplace_back(std::move(key), value());
      } while (eat(','));
      expect('}');
    } else if (c == '[') {
      ++i_;
      v.kind = Value::Kind::kArray;
      if (eat(']')) return v;
      do v.array.push_back(value());
      while (eat(','));
      expect(']');
    } else if (c == '"') {
      v.kind = Value::Kind::kString;
      v.string = str();
    } else if (s_.compare(i_, 4, "true") == 0) {
      i_ += 4, v.kind = Value::Kind::kBool, v.boolean = true;
    } else if (s_.compare(i_, 5, "false") == 0) {
      i_ += 5, v.kind = Value::Kind::kBool;
    } else if (s_.compare(i_, 4, "null") == 0) {
      i_ += 4;
    } else {
      const char* b = s_.c_str() + i_;
      char* e = nullptr;
      v.number = std::strtod(b, &e);
      if (e == b) fail("unexpected character");
      i_ += static_cast<size_t>(e - b);
      v.kind = Value::Kind::kNumber;
    }
    return v;
  }
  std::string str() {
    if (i_ >= s_.size() || s_[i_] != '"') fail("expected a string");
    ++i_;
    std::string out;
    while (i_ < s_.size() && s_[i_] != '"') {
      char c = s_[i_++];
      if (c == '\\') {
        if (i_ >= s_.size()) fail("bad escape");
        const char e = s_[i_++];
        switch (e) {
          case 'n': c = '\n'; break;
          case 't': c = '\t'; break;
          case 'r': c = '\r'; break;
          case 'b': c = '\b'; break;
          case 'f': c = '\f'; break;
          case 'u': {  // keep the low byte of \uXXXX; names in model files are ASCII
            if (i_ + 4 > s_.size()) fail("bad \\u escape");
            c = static_cast<char>(std::strtol(s_.substr(i_, 4).c_str(), nullptr, 16) & 0xff);
            i_ += 4;
            break;
          }
          default: c = e;
        }
      }
      out.push_back(c);
    }
    if (i_ >= s_.size()) fail("unterminated string");
    ++i_;
    return out;
  }
};

inline Value parse(const std::string& text) { return Parser(text).parse(); }
}  // namespace json
}  // namespace model
#endif  // KLLM_KUIPER_MODEL_JSON_H_
