// Minimal JSON reader for <model>.json / <model>.profile.json (replaces the reference's
// src/reef/util/json.{h,cpp}; any conformant parser will do — this one is a recursive-descent
// reader into a small variant tree).
#pragma once
#include <cstdint>
#include <map>
#include <memory>
#include <string>
#include <vector>

namespace reef {
namespace util {

struct JsonValue {
    enum Kind { Null, Bool, Number, String, Array, Object } kind = Null;
    bool b = false;
    double num = 0;
    std::string str;
    std::vector<JsonValue> arr;
    std::vector<std::pair<std::string, JsonValue>> obj;   // keeps file order

    const JsonValue* find(const std::string& key) const;
    int64_t as_int() const { return (int64_t)num; }
    bool is(Kind k) const { return kind == k; }
};

// Returns false and fills *err on malformed input.
bool json_parse(const std::string& text, JsonValue* out, std::string* err);
bool json_parse_file(const std::string& path, JsonValue* out, std::string* err);

}  // namespace util
}  // namespace reef
