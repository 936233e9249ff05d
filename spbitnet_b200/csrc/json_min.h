// A small JSON reader for the host-side loaders (tokenizer.json, config.json, manifest.json): objects, arrays,
// strings with every escape (\uXXXX with surrogate pairs -> UTF-8), numbers, booleans, null.  Objects keep their
// members in file order (a tokenizer's vocabulary has over a hundred thousand).  The reference reads the same
// files with nlohmann/json (CMakeLists.txt:19-27); no third-party code is used here.
#pragma once

#include <cstdint>
#include <cstdlib>
#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace spb {
namespace json {

struct Value {
    enum Kind { Null, Bool, Number, String, Array, Object } kind = Null;
    bool b = false;
    double num = 0.0;
    std::string str;
    std::vector<Value> items;                              // Array
    std::vector<std::pair<std::string, Value>> members;    // Object, in file order

    const Value* find(const std::string& key) const {
        if (kind != Object) return nullptr;
        for (const auto& m : members)
            if (m.first == key) return &m.second;
        return nullptr;
    }
    bool is(Kind k) const { return kind == k; }
    long long as_int(long long fallback = 0) const { return kind == Number ? static_cast<long long>(num) : fallback; }
    double as_double(double fallback = 0.0) const { return kind == Number ? num : fallback; }
    bool as_bool(bool fallback = false) const { return kind == Bool ? b : fallback; }
};

class Parser {
public:
    explicit Parser(const std::string& text) : s_(text) {}

    Value parse() {
        Value v = value();
        skip_ws();
        if (p_ != s_.size()) fail("trailing characters");
        return v;
    }

private:
    const std::string& s_;
    size_t p_ = 0;

    [[noreturn]] void fail(const char* what) const {
        throw std::runtime_error(std::string("JSON: ") + what + " at byte " + std::to_string(p_));
    }
    void skip_ws() {
        while (p_ < s_.size() && (s_[p_] == ' ' || s_[p_] == '\n' || s_[p_] == '\t' || s_[p_] == '\r')) ++p_;
    }
    bool eat(char c) {
        skip_ws();
        if (p_ < s_.size() && s_[p_] == c) {
            ++p_;
            return true;
        }
        return false;
    }
    static void append_utf8(std::string& out, uint32_t cp) {
        if (cp < 0x80) {
            out += static_cast<char>(cp);
        } else if (cp < 0x800) {
            out += static_cast<char>(0xC0 | (cp >> 6));
            out += static_cast<char>(0x80 | (cp & 0x3F));
        } else if (cp < 0x10000) {
            out += static_cast<char>(0xE0 | (cp >> 12));
            out += static_cast<char>(0x80 | ((cp >> 6) & 0x3F));
            out += static_cast<char>(0x80 | (cp & 0x3F));
        } else {
            out += static_cast<char>(0xF0 | (cp >> 18));
            out += static_cast<char>(0x80 | ((cp >> 12) & 0x3F));
            out += static_cast<char>(0x80 | ((cp >> 6) & 0x3F));
            out += static_cast<char>(0x80 | (cp & 0x3F));
        }
    }
    uint32_t hex4() {
        if (p_ + 4 > s_.size()) fail("short \\u escape");
        uint32_t v = 0;
        for (int i = 0; i < 4; ++i) {
            const char c = s_[p_++];
            v <<= 4;
            if (c >= '0' && c <= '9') v |= static_cast<uint32_t>(c - '0');
            else if (c >= 'a' && c <= 'f') v |= static_cast<uint32_t>(c - 'a' + 10);
            else if (c >= 'A' && c <= 'F') v |= static_cast<uint32_t>(c - 'A' + 10);
            else fail("bad \\u escape");
        }
        return v;
    }
    std::string string_body() {  // after the opening quote
        std::string out;
        for (;;) {
            if (p_ >= s_.size()) fail("unterminated string");
            const char c = s_[p_++];
            if (c == '"') return out;
            if (c != '\\') {
                out += c;
                continue;
            }
            if (p_ >= s_.size()) fail("unterminated escape");
            const char e = s_[p_++];
            switch (e) {
                case '"': out += '"'; break;
                case '\\': out += '\\'; break;
                case '/': out += '/'; break;
                case 'b': out += '\b'; break;
                case 'f': out += '\f'; break;
                case 'n': out += '\n'; break;
                case 'r': out += '\r'; break;
                case 't': out += '\t'; break;
                case 'u': {
                    uint32_t cp = hex4();
                    if (cp >= 0xD800 && cp <= 0xDBFF && p_ + 1 < s_.size() && s_[p_] == '\\' && s_[p_ + 1] == 'u') {
                        p_ += 2;
                        const uint32_t lo = hex4();
                        if (lo >= 0xDC00 && lo <= 0xDFFF) cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
                        else fail("unpaired surrogate");
                    }
                    append_utf8(out, cp);
                    break;
                }
                default: fail("unknown escape");
            }
        }
    }
    Value value() {
        skip_ws();
        if (p_ >= s_.size()) fail("unexpected end");
        Value v;
        const char c = s_[p_];
        if (c == '{') {
            ++p_;
            v.kind = Value::Object;
            if (eat('}')) return v;
            do {
                skip_ws();
                if (p_ >= s_.size() || s_[p_] != '"') fail("expected a member name");
                ++p_;
                std::string key = string_body();
                if (!eat(':')) fail("expected ':'");
                v.members.emplace_back(std::move(key), value());
            } while (eat(','));
            if (!eat('}')) fail("expected '}'");
        } else if (c == '[') {
            ++p_;
            v.kind = Value::Array;
            if (eat(']')) return v;
            do {
                v.items.push_back(value());
            } while (eat(','));
            if (!eat(']')) fail("expected ']'");
        } else if (c == '"') {
            ++p_;
            v.kind = Value::String;
            v.str = string_body();
        } else if (s_.compare(p_, 4, "true") == 0) {
            p_ += 4;
            v.kind = Value::Bool;
            v.b = true;
        } else if (s_.compare(p_, 5, "false") == 0) {
            p_ += 5;
            v.kind = Value::Bool;
        } else if (s_.compare(p_, 4, "null") == 0) {
            p_ += 4;
        } else {
            char* end = nullptr;
            v.num = std::strtod(s_.c_str() + p_, &end);
            if (end == s_.c_str() + p_) fail("unexpected character");
            p_ = static_cast<size_t>(end - s_.c_str());
            v.kind = Value::Number;
        }
        return v;
    }
};

inline Value parse(const std::string& text) { return Parser(text).parse(); }

}  // namespace json
}  // namespace spb
