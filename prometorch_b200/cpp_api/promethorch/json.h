// promethorch C++ API: a small JSON value with a parser and a writer.
//
// What the server, the Ollama manifest resolver and the tokenizer files need: objects keep their insertion order,
// numbers remember whether they were written as integers, strings are UTF-8 (\uXXXX escapes and surrogate pairs are
// decoded on input; output escapes only what JSON requires and replaces malformed UTF-8 by U+FFFD, so that every
// line the server streams is valid).  parse() throws std::runtime_error with the byte offset of the problem.
#pragma once
#include <cerrno>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace promethorch {
namespace json {

class Value {
 public:
    enum Kind { Null, Bool, Int, Float, String, Array, Object };
    Value() = default;
    Value(std::nullptr_t) {}
    Value(bool b) : kind_(Bool), b_(b) {}
    Value(int v) : kind_(Int), i_(v) {}
    Value(long v) : kind_(Int), i_(v) {}
    Value(long long v) : kind_(Int), i_(v) {}
    Value(unsigned long v) : kind_(Int), i_((long long)v) {}
    Value(double v) : kind_(Float), f_(v) {}
    Value(const char* s) : kind_(String), s_(s) {}
    Value(std::string s) : kind_(String), s_(std::move(s)) {}
    static Value array() { Value v; v.kind_ = Array; return v; }
    static Value object() { Value v; v.kind_ = Object; return v; }

    Kind kind() const { return kind_; }
    bool is_null() const { return kind_ == Null; }
    bool is_object() const { return kind_ == Object; }
    bool is_array() const { return kind_ == Array; }
    bool is_string() const { return kind_ == String; }
    bool is_number() const { return kind_ == Int || kind_ == Float; }
    bool is_bool() const { return kind_ == Bool; }

    bool as_bool(bool dflt = false) const { return kind_ == Bool ? b_ : (kind_ == Int ? i_ != 0 : dflt); }
    long long as_int(long long dflt = 0) const { return kind_ == Int ? i_ : (kind_ == Float ? (long long)f_ : dflt); }
    double as_double(double dflt = 0) const { return kind_ == Float ? f_ : (kind_ == Int ? (double)i_ : dflt); }
    const std::string& as_string() const { static const std::string empty; return kind_ == String ? s_ : empty; }

    // arrays
    size_t size() const { return kind_ == Array ? a_.size() : (kind_ == Object ? o_.size() : 0); }
    const Value& operator[](size_t i) const { return a_.at(i); }
    const Value& at(size_t i) const { return a_.at(i); }                       // for literal indices (0 is also a null pointer constant)
    void push_back(Value v) { if (kind_ != Array) { *this = array(); } a_.push_back(std::move(v)); }
    const std::vector<Value>& items() const { return a_; }
    // objects
    bool contains(const std::string& k) const { return find(k) != nullptr; }
    const Value* find(const std::string& k) const {
        if (kind_ != Object) return nullptr;
        for (const auto& kv : o_)
            if (kv.first == k) return &kv.second;
        return nullptr;
    }
    // Missing keys read as null.
    const Value& operator[](const std::string& k) const { static const Value none; const Value* v = find(k); return v ? *v : none; }
    const Value& operator[](const char* k) const { return (*this)[std::string(k)]; }
    Value& set(const std::string& k, Value v) {
        if (kind_ != Object) *this = object();
        for (auto& kv : o_)
            if (kv.first == k) { kv.second = std::move(v); return kv.second; }
        o_.emplace_back(k, std::move(v));
        return o_.back().second;
    }
    const std::vector<std::pair<std::string, Value>>& members() const { return o_; }

    std::string dump() const { std::string out; write(out); return out; }

 private:
    static void write_string(const std::string& s, std::string& out) {
        out.push_back('"');
        const size_t n = s.size();
        for (size_t i = 0; i < n;) {
            const unsigned char c = (unsigned char)s[i];
            if (c == '"') { out += "\\\""; ++i; }
            else if (c == '\\') { out += "\\\\"; ++i; }
            else if (c == '\n') { out += "\\n"; ++i; }
            else if (c == '\r') { out += "\\r"; ++i; }
            else if (c == '\t') { out += "\\t"; ++i; }
            else if (c < 0x20) { char b[8]; std::snprintf(b, sizeof b, "\\u%04x", c); out += b; ++i; }
            else if (c < 0x80) { out.push_back((char)c); ++i; }
            else {
                int len = c >= 0xF0 && c <= 0xF4 ? 4 : (c >= 0xE0 ? 3 : (c >= 0xC2 && c < 0xE0 ? 2 : 0));
                bool ok = len != 0 && i + (size_t)len <= n;
                for (int k = 1; ok && k < len; ++k) ok = ((unsigned char)s[i + (size_t)k] & 0xC0) == 0x80;
                if (ok) { out.append(s, i, (size_t)len); i += (size_t)len; }
                else { out += "\xEF\xBF\xBD"; ++i; }
            }
        }
        out.push_back('"');
    }
    void write(std::string& out) const {
        switch (kind_) {
            case Null: out += "null"; break;
            case Bool: out += b_ ? "true" : "false"; break;
            case Int: out += std::to_string(i_); break;
            case Float: {
                if (!std::isfinite(f_)) { out += "null"; break; }
                char b[32];
                std::snprintf(b, sizeof b, "%.17g", f_);
                std::string t(b);
                if (t.find_first_of(".eE") == std::string::npos) t += ".0";
                out += t;
                break;
            }
            case String: write_string(s_, out); break;
            case Array:
                out.push_back('[');
                for (size_t i = 0; i < a_.size(); ++i) { if (i) out += ", "; a_[i].write(out); }
                out.push_back(']');
                break;
            case Object:
                out.push_back('{');
                for (size_t i = 0; i < o_.size(); ++i) {
                    if (i) out += ", ";
                    write_string(o_[i].first, out);
                    out += ": ";
                    o_[i].second.write(out);
                }
                out.push_back('}');
                break;
        }
    }
    Kind kind_ = Null;
    bool b_ = false;
    long long i_ = 0;
    double f_ = 0;
    std::string s_;
    std::vector<Value> a_;
    std::vector<std::pair<std::string, Value>> o_;
};

namespace detail {
class Parser {
 public:
    explicit Parser(const std::string& s) : s_(s) {}
    Value run() {
        Value v = value(0);
        ws();
        if (p_ != s_.size()) fail("trailing characters");
        return v;
    }

 private:
    [[noreturn]] void fail(const char* what) const { throw std::runtime_error(std::string("JSON: ") + what + " at byte " + std::to_string(p_)); }
    void ws() { while (p_ < s_.size() && (s_[p_] == ' ' || s_[p_] == '\t' || s_[p_] == '\n' || s_[p_] == '\r')) ++p_; }
    bool lit(const char* w) {
        size_t n = 0;
        while (w[n]) ++n;
        if (s_.compare(p_, n, w) == 0) { p_ += n; return true; }
        return false;
    }
    static void utf8(uint32_t c, std::string& out) {
        if (c < 0x80) out.push_back((char)c);
        else if (c < 0x800) { out.push_back((char)(0xC0 | (c >> 6))); out.push_back((char)(0x80 | (c & 0x3F))); }
        else if (c < 0x10000) { out.push_back((char)(0xE0 | (c >> 12))); out.push_back((char)(0x80 | ((c >> 6) & 0x3F))); out.push_back((char)(0x80 | (c & 0x3F))); }
        else { out.push_back((char)(0xF0 | (c >> 18))); out.push_back((char)(0x80 | ((c >> 12) & 0x3F))); out.push_back((char)(0x80 | ((c >> 6) & 0x3F))); out.push_back((char)(0x80 | (c & 0x3F))); }
    }
    uint32_t hex4() {
        if (p_ + 4 > s_.size()) fail("truncated \\u escape");
        uint32_t v = 0;
        for (int k = 0; k < 4; ++k) {
            const char c = s_[p_++];
            v <<= 4;
            if (c >= '0' && c <= '9') v |= (uint32_t)(c - '0');
            else if (c >= 'a' && c <= 'f') v |= (uint32_t)(c - 'a' + 10);
            else if (c >= 'A' && c <= 'F') v |= (uint32_t)(c - 'A' + 10);
            else fail("bad \\u escape");
        }
        return v;
    }
    std::string string() {
        std::string out;
        ++p_;                                   // the opening quote
        for (;;) {
            if (p_ >= s_.size()) fail("unterminated string");
            const char c = s_[p_++];
            if (c == '"') return out;
            if (c != '\\') { out.push_back(c); continue; }
            if (p_ >= s_.size()) fail("unterminated escape");
            const char e = s_[p_++];
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
                    uint32_t c1 = hex4();
                    if (c1 >= 0xD800 && c1 < 0xDC00 && p_ + 1 < s_.size() && s_[p_] == '\\' && s_[p_ + 1] == 'u') {
                        p_ += 2;
                        const uint32_t c2 = hex4();
                        if (c2 >= 0xDC00 && c2 < 0xE000) c1 = 0x10000 + ((c1 - 0xD800) << 10) + (c2 - 0xDC00);
                        else { utf8(0xFFFD, out); c1 = c2; }
                    }
                    if (c1 >= 0xD800 && c1 < 0xE000) c1 = 0xFFFD;
                    utf8(c1, out);
                    break;
                }
                default: fail("unknown escape");
            }
        }
    }
    Value number() {
        const size_t start = p_;
        bool is_float = false;
        if (p_ < s_.size() && s_[p_] == '-') ++p_;
        while (p_ < s_.size() && ((s_[p_] >= '0' && s_[p_] <= '9') || s_[p_] == '.' || s_[p_] == 'e' || s_[p_] == 'E' || s_[p_] == '+' || s_[p_] == '-')) {
            is_float |= s_[p_] == '.' || s_[p_] == 'e' || s_[p_] == 'E';
            ++p_;
        }
        const std::string t = s_.substr(start, p_ - start);
        if (t.empty() || t == "-") fail("bad number");
        char* end = nullptr;
        if (!is_float) {
            errno = 0;
            const long long v = std::strtoll(t.c_str(), &end, 10);
            if (*end == 0 && errno == 0) return Value(v);
        }
        const double d = std::strtod(t.c_str(), &end);
        if (*end != 0) fail("bad number");
        return Value(d);
    }
    Value value(int depth) {
        if (depth > 256) fail("nesting too deep");
        ws();
        if (p_ >= s_.size()) fail("unexpected end");
        const char c = s_[p_];
        if (c == '{') {
            Value o = Value::object();
            ++p_;
            ws();
            if (p_ < s_.size() && s_[p_] == '}') { ++p_; return o; }
            for (;;) {
                ws();
                if (p_ >= s_.size() || s_[p_] != '"') fail("expected a key");
                std::string k = string();
                ws();
                if (p_ >= s_.size() || s_[p_] != ':') fail("expected ':'");
                ++p_;
                o.set(k, value(depth + 1));
                ws();
                if (p_ < s_.size() && s_[p_] == ',') { ++p_; continue; }
                if (p_ < s_.size() && s_[p_] == '}') { ++p_; return o; }
                fail("expected ',' or '}'");
            }
        }
        if (c == '[') {
            Value a = Value::array();
            ++p_;
            ws();
            if (p_ < s_.size() && s_[p_] == ']') { ++p_; return a; }
            for (;;) {
                a.push_back(value(depth + 1));
                ws();
                if (p_ < s_.size() && s_[p_] == ',') { ++p_; continue; }
                if (p_ < s_.size() && s_[p_] == ']') { ++p_; return a; }
                fail("expected ',' or ']'");
            }
        }
        if (c == '"') return Value(string());
        if (lit("true")) return Value(true);
        if (lit("false")) return Value(false);
        if (lit("null")) return Value();
        return number();
    }
    const std::string& s_;
    size_t p_ = 0;
};
}  // namespace detail

inline Value parse(const std::string& text) { return detail::Parser(text).run(); }

}  // namespace json
}  // namespace promethorch
