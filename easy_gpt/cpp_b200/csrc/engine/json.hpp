// A small JSON reader: enough for config.json, the header of a safetensors file and tokenizer.json.
// Values keep the order of an object's members; integers that fit 64 bits are kept exactly beside
// their double.  Errors carry the byte offset.  (The reference reads its files with a vendored
// nlohmann::json, include/third_party/json.hpp; this reader is written for this engine.)
#pragma once
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace easygpt::json {

struct ParseError : std::runtime_error {
    using std::runtime_error::runtime_error;
};

class Value {
public:
    enum Type { Null, Bool, Number, String, Array, Object };
    Type type = Null;
    bool boolean = false;
    double number = 0.0;
    int64_t integer = 0;
    bool is_integer = false;            // the number was written without fraction or exponent and fits int64
    std::string string;
    std::vector<Value> array;
    std::vector<std::pair<std::string, Value>> object;

    bool is_null() const { return type == Null; }
    bool is_object() const { return type == Object; }
    bool is_array() const { return type == Array; }
    bool is_string() const { return type == String; }
    bool is_number() const { return type == Number; }
    bool is_bool() const { return type == Bool; }

    const Value* find(const std::string& key) const {
        if (type != Object) return nullptr;
        for (auto& kv : object)
            if (kv.first == key) return &kv.second;
        return nullptr;
    }
    bool contains(const std::string& key) const { return find(key) != nullptr; }
};

class Parser {
public:
    explicit Parser(const char* data, size_t size) : p_(data), end_(data + size), begin_(data) {}

    Value parse() {
        Value v = value();
        space();
        if (p_ != end_) fail("text after the JSON value");
        return v;
    }

private:
    const char *p_, *end_, *begin_;

    [[noreturn]] void fail(const std::string& what) const {
        throw ParseError("JSON: " + what + " at byte " + std::to_string(p_ - begin_));
    }
    void space() {
        while (p_ != end_ && (*p_ == ' ' || *p_ == '\t' || *p_ == '\n' || *p_ == '\r')) ++p_;
    }
    bool literal(const char* word) {
        const char* q = p_;
        for (const char* w = word; *w; ++w, ++q)
            if (q == end_ || *q != *w) return false;
        p_ = q;
        return true;
    }
    static void append_utf8(std::string& out, uint32_t cp) {
        if (cp < 0x80) out += (char)cp;
        else if (cp < 0x800) { out += (char)(0xC0 | (cp >> 6)); out += (char)(0x80 | (cp & 0x3F)); }
        else if (cp < 0x10000) { out += (char)(0xE0 | (cp >> 12)); out += (char)(0x80 | ((cp >> 6) & 0x3F)); out += (char)(0x80 | (cp & 0x3F)); }
        else { out += (char)(0xF0 | (cp >> 18)); out += (char)(0x80 | ((cp >> 12) & 0x3F)); out += (char)(0x80 | ((cp >> 6) & 0x3F)); out += (char)(0x80 | (cp & 0x3F)); }
    }
    uint32_t hex4() {
        if (end_ - p_ < 4) fail("short \\u escape");
        uint32_t v = 0;
        for (int i = 0; i < 4; ++i, ++p_) {
            const char c = *p_;
            v <<= 4;
            if (c >= '0' && c <= '9') v |= c - '0';
            else if (c >= 'a' && c <= 'f') v |= c - 'a' + 10;
            else if (c >= 'A' && c <= 'F') v |= c - 'A' + 10;
            else fail("bad \\u escape");
        }
        return v;
    }
    std::string string_body() {
        std::string out;
        ++p_;                                            // the opening quote
        while (true) {
            if (p_ == end_) fail("unterminated string");
            const char c = *p_++;
            if (c == '"') return out;
            if (c != '\\') { out += c; continue; }
            if (p_ == end_) fail("unterminated escape");
            const char e = *p_++;
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
                    if (cp >= 0xD800 && cp <= 0xDBFF && end_ - p_ >= 6 && p_[0] == '\\' && p_[1] == 'u') {
                        p_ += 2;
                        const uint32_t low = hex4();
                        if (low >= 0xDC00 && low <= 0xDFFF) cp = 0x10000 + ((cp - 0xD800) << 10) + (low - 0xDC00);
                        else fail("bad surrogate pair");
                    }
                    append_utf8(out, cp);
                    break;
                }
                default: fail("unknown escape");
            }
        }
    }
    Value number() {
        const char* start = p_;
        bool integral = true;
        if (p_ != end_ && *p_ == '-') ++p_;
        while (p_ != end_ && ((*p_ >= '0' && *p_ <= '9') || *p_ == '.' || *p_ == 'e' || *p_ == 'E' || *p_ == '+' || *p_ == '-')) {
            if (*p_ == '.' || *p_ == 'e' || *p_ == 'E') integral = false;
            ++p_;
        }
        if (p_ == start) fail("a value was expected");
        const std::string text(start, p_);
        Value v;
        v.type = Value::Number;
        char* stop = nullptr;
        v.number = std::strtod(text.c_str(), &stop);
        if (stop == text.c_str() || *stop) fail("bad number '" + text + "'");
        if (integral && text.size() <= 19) {
            v.integer = std::strtoll(text.c_str(), nullptr, 10);
            v.is_integer = true;
        } else if (!integral && std::floor(v.number) == v.number && std::fabs(v.number) < 9e15) {
            v.integer = (int64_t)v.number;           // 1e6 and 4096.0 are whole numbers too, but not written as integers
        }
        return v;
    }
    Value value() {
        space();
        if (p_ == end_) fail("a value was expected");
        Value v;
        switch (*p_) {
            case '{': {
                v.type = Value::Object;
                ++p_;
                space();
                if (p_ != end_ && *p_ == '}') { ++p_; return v; }
                while (true) {
                    space();
                    if (p_ == end_ || *p_ != '"') fail("a member name was expected");
                    std::string key = string_body();
                    space();
                    if (p_ == end_ || *p_ != ':') fail("':' was expected");
                    ++p_;
                    v.object.emplace_back(std::move(key), value());
                    space();
                    if (p_ != end_ && *p_ == ',') { ++p_; continue; }
                    if (p_ != end_ && *p_ == '}') { ++p_; return v; }
                    fail("',' or '}' was expected");
                }
            }
            case '[': {
                v.type = Value::Array;
                ++p_;
                space();
                if (p_ != end_ && *p_ == ']') { ++p_; return v; }
                while (true) {
                    v.array.push_back(value());
                    space();
                    if (p_ != end_ && *p_ == ',') { ++p_; continue; }
                    if (p_ != end_ && *p_ == ']') { ++p_; return v; }
                    fail("',' or ']' was expected");
                }
            }
            case '"':
                v.type = Value::String;
                v.string = string_body();
                return v;
            case 't':
                if (!literal("true")) fail("a value was expected");
                v.type = Value::Bool;
                v.boolean = true;
                return v;
            case 'f':
                if (!literal("false")) fail("a value was expected");
                v.type = Value::Bool;
                return v;
            case 'n':
                if (!literal("null")) fail("a value was expected");
                return v;
            default:
                return number();
        }
    }
};

inline Value parse(const std::string& text) { return Parser(text.data(), text.size()).parse(); }
inline Value parse(const char* data, size_t size) { return Parser(data, size).parse(); }

}  // namespace easygpt::json
