#include "json.h"

#include <cstdlib>
#include <fstream>
#include <sstream>

namespace reef {
namespace util {

const JsonValue* JsonValue::find(const std::string& key) const {
    if (kind != Object) return nullptr;
    for (auto& kv : obj)
        if (kv.first == key) return &kv.second;
    return nullptr;
}

namespace {
struct Reader {
    const std::string& s;
    size_t i = 0;
    std::string err;
    explicit Reader(const std::string& t) : s(t) {}

    void ws() {
        while (i < s.size() && (s[i] == ' ' || s[i] == '\n' || s[i] == '\t' || s[i] == '\r')) i++;
    }
    bool fail(const std::string& m) {
        if (err.empty()) err = m + " at offset " + std::to_string(i);
        return false;
    }
    bool value(JsonValue* v, int depth) {
        if (depth > 64) return fail("nesting too deep");
        ws();
        if (i >= s.size()) return fail("unexpected end");
        char c = s[i];
        if (c == '{') return object(v, depth);
        if (c == '[') return array(v, depth);
        if (c == '"') {
            v->kind = JsonValue::String;
            return string(&v->str);
        }
        if (s.compare(i, 4, "true") == 0) { v->kind = JsonValue::Bool; v->b = true; i += 4; return true; }
        if (s.compare(i, 5, "false") == 0) { v->kind = JsonValue::Bool; v->b = false; i += 5; return true; }
        if (s.compare(i, 4, "null") == 0) { v->kind = JsonValue::Null; i += 4; return true; }
        return number(v);
    }
    bool number(JsonValue* v) {
        const char* b = s.c_str() + i;
        char* e = nullptr;
        double d = strtod(b, &e);
        if (e == b) return fail("bad number");
        v->kind = JsonValue::Number;
        v->num = d;
        i += (size_t)(e - b);
        return true;
    }
    bool string(std::string* out) {
        i++;   // opening quote
        out->clear();
        while (i < s.size() && s[i] != '"') {
            char c = s[i++];
            if (c == '\\') {
                if (i >= s.size()) return fail("bad escape");
                char e = s[i++];
                switch (e) {
                    case 'n': out->push_back('\n'); break;
                    case 't': out->push_back('\t'); break;
                    case 'r': out->push_back('\r'); break;
                    case 'b': out->push_back('\b'); break;
                    case 'f': out->push_back('\f'); break;
                    case 'u': {
                        if (i + 4 > s.size()) return fail("bad \\u escape");
                        unsigned cp = (unsigned)strtoul(s.substr(i, 4).c_str(), nullptr, 16);
                        i += 4;
                        if (cp < 0x80) out->push_back((char)cp);
                        else if (cp < 0x800) { out->push_back((char)(0xC0 | (cp >> 6))); out->push_back((char)(0x80 | (cp & 0x3F))); }
                        else { out->push_back((char)(0xE0 | (cp >> 12))); out->push_back((char)(0x80 | ((cp >> 6) & 0x3F))); out->push_back((char)(0x80 | (cp & 0x3F))); }
                        break;
                    }
                    default: out->push_back(e);
                }
            } else {
                out->push_back(c);
            }
        }
        if (i >= s.size()) return fail("unterminated string");
        i++;
        return true;
    }
    bool array(JsonValue* v, int depth) {
        v->kind = JsonValue::Array;
        i++;
        ws();
        if (i < s.size() && s[i] == ']') { i++; return true; }
        for (;;) {
            v->arr.emplace_back();
            if (!value(&v->arr.back(), depth + 1)) return false;
            ws();
            if (i < s.size() && s[i] == ',') { i++; continue; }
            if (i < s.size() && s[i] == ']') { i++; return true; }
            return fail("expected , or ]");
        }
    }
    bool object(JsonValue* v, int depth) {
        v->kind = JsonValue::Object;
        i++;
        ws();
        if (i < s.size() && s[i] == '}') { i++; return true; }
        for (;;) {
            ws();
            if (i >= s.size() || s[i] != '"') return fail("expected key");
            std::string key;
            if (!string(&key)) return false;
            ws();
            if (i >= s.size() || s[i] != ':') return fail("expected :");
            i++;
            v->obj.emplace_back(key, JsonValue());
            if (!value(&v->obj.back().second, depth + 1)) return false;
            ws();
            if (i < s.size() && s[i] == ',') { i++; continue; }
            if (i < s.size() && s[i] == '}') { i++; return true; }
            return fail("expected , or }");
        }
    }
};
}  // namespace

bool json_parse(const std::string& text, JsonValue* out, std::string* err) {
    Reader r(text);
    if (!r.value(out, 0)) {
        if (err) *err = r.err;
        return false;
    }
    r.ws();
    if (r.i != text.size()) {
        if (err) *err = "trailing characters at offset " + std::to_string(r.i);
        return false;
    }
    return true;
}

bool json_parse_file(const std::string& path, JsonValue* out, std::string* err) {
    std::ifstream fs(path, std::ios::binary);
    if (!fs) {
        if (err) *err = "cannot open " + path;
        return false;
    }
    std::stringstream ss;
    ss << fs.rdbuf();
    return json_parse(ss.str(), out, err);
}

}  // namespace util
}  // namespace reef
