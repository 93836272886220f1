// A small JSON value with a strict reader and a writer.
//
// config.json, the safetensors header, the shard index and a part's parameters are all held as Json values.
// Objects keep the order of their keys (a safetensors header is written back in the order it was made).
// The reader accepts exactly RFC 8259 plus the bare tokens NaN / Infinity / -Infinity that Python's json
// module writes; every error names the byte offset.  The reference scans config files for a key by substring
// (src/safetensors_mmap.cpp:334-346), which cannot see into nested objects such as rope_parameters.
#pragma once

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace qe {

struct JsonError : std::runtime_error {
    using std::runtime_error::runtime_error;
};

class Json {
public:
    enum Kind { Null, Bool, Int, Real, String, Array, Object };
    using Member = std::pair<std::string, Json>;

    Json() = default;
    Json(std::nullptr_t) {}
    Json(bool b) : kind_(Bool), b_(b) {}
    Json(int v) : kind_(Int), i_(v) {}
    Json(long v) : kind_(Int), i_(v) {}
    Json(long long v) : kind_(Int), i_(v) {}
    Json(unsigned long v) : kind_(Int), i_((long long)v) {}
    Json(double v) : kind_(Real), d_(v) {}
    Json(const char* s) : kind_(String), s_(s) {}
    Json(std::string s) : kind_(String), s_(std::move(s)) {}

    static Json array() { Json j; j.kind_ = Array; return j; }
    static Json object() { Json j; j.kind_ = Object; return j; }

    Kind kind() const { return kind_; }
    bool is_null() const { return kind_ == Null; }
    bool is_bool() const { return kind_ == Bool; }
    bool is_int() const { return kind_ == Int; }
    bool is_number() const { return kind_ == Int || kind_ == Real; }
    bool is_string() const { return kind_ == String; }
    bool is_array() const { return kind_ == Array; }
    bool is_object() const { return kind_ == Object; }

    bool as_bool() const { need(Bool, "a boolean"); return b_; }
    long long as_int() const {
        if (kind_ == Real && d_ == std::floor(d_) && std::fabs(d_) < 9e15) return (long long)d_;
        need(Int, "an integer");
        return i_;
    }
    double as_double() const {
        if (kind_ == Int) return (double)i_;
        need(Real, "a number");
        return d_;
    }
    const std::string& as_string() const { need(String, "a string"); return s_; }

    // arrays
    const std::vector<Json>& items() const { need(Array, "an array"); return a_; }
    std::vector<Json>& items() { need(Array, "an array"); return a_; }
    void push(Json v) { need(Array, "an array"); a_.push_back(std::move(v)); }
    size_t size() const { return kind_ == Array ? a_.size() : kind_ == Object ? o_.size() : 0; }
    const Json& operator[](size_t i) const { need(Array, "an array"); return a_.at(i); }

    // objects
    const std::vector<Member>& members() const { need(Object, "an object"); return o_; }
    const Json* find(const std::string& key) const {
        if (kind_ != Object) return nullptr;
        for (const auto& m : o_) if (m.first == key) return &m.second;
        return nullptr;
    }
    bool has(const std::string& key) const { return find(key) != nullptr; }
    const Json& at(const std::string& key) const {
        const Json* j = find(key);
        if (!j) throw JsonError("missing key '" + key + "'");
        return *j;
    }
    Json& set(const std::string& key, Json v) {
        need(Object, "an object");
        for (auto& m : o_) if (m.first == key) { m.second = std::move(v); return m.second; }
        o_.emplace_back(key, std::move(v));
        return o_.back().second;
    }
    // typed reads with defaults, for a part's parameters
    long long get_int(const std::string& key, long long dflt) const {
        const Json* j = find(key);
        return (j && !j->is_null()) ? j->as_int() : dflt;
    }
    double get_double(const std::string& key, double dflt) const {
        const Json* j = find(key);
        return (j && !j->is_null()) ? j->as_double() : dflt;
    }
    bool get_bool(const std::string& key, bool dflt) const {
        const Json* j = find(key);
        return (j && !j->is_null()) ? j->as_bool() : dflt;
    }
    std::string get_string(const std::string& key, const std::string& dflt) const {
        const Json* j = find(key);
        return (j && !j->is_null()) ? j->as_string() : dflt;
    }

    bool operator==(const Json& o) const {
        if (kind_ != o.kind_) {
            if (is_number() && o.is_number()) return as_double() == o.as_double();
            return false;
        }
        switch (kind_) {
            case Null: return true;
            case Bool: return b_ == o.b_;
            case Int: return i_ == o.i_;
            case Real: return d_ == o.d_;
            case String: return s_ == o.s_;
            case Array: return a_ == o.a_;
            case Object: return o_ == o.o_;
        }
        return false;
    }
    bool operator!=(const Json& o) const { return !(*this == o); }

    // ---- reading ------------------------------------------------------------------------------------------
    static Json parse(const char* text, size_t len) {
        Reader r{text, len, 0};
        r.skip();
        Json v = r.value(0);
        r.skip();
        if (r.pos != r.len) r.fail("text after the value");
        return v;
    }
    static Json parse(const std::string& text) { return parse(text.data(), text.size()); }

    // ---- writing ------------------------------------------------------------------------------------------
    std::string dump(int indent = -1) const {
        std::string out;
        write(out, indent, 0);
        return out;
    }

private:
    Kind kind_ = Null;
    bool b_ = false;
    long long i_ = 0;
    double d_ = 0.0;
    std::string s_;
    std::vector<Json> a_;
    std::vector<Member> o_;

    void need(Kind k, const char* what) const {
        if (kind_ != k) throw JsonError(std::string("value is not ") + what);
    }

    struct Reader {
        const char* s;
        size_t len, pos;
        [[noreturn]] void fail(const std::string& what) const {
            throw JsonError(what + " at byte " + std::to_string(pos));
        }
        void skip() {
            while (pos < len && (s[pos] == ' ' || s[pos] == '\t' || s[pos] == '\n' || s[pos] == '\r')) pos++;
        }
        bool take(const char* word) {
            size_t n = strlen(word);
            if (len - pos >= n && memcmp(s + pos, word, n) == 0) { pos += n; return true; }
            return false;
        }
        Json value(int depth) {
            if (depth > 200) fail("nesting too deep");
            if (pos >= len) fail("unexpected end");
            char c = s[pos];
            if (c == '{') return object(depth);
            if (c == '[') return array(depth);
            if (c == '"') return Json(string());
            if (take("true")) return Json(true);
            if (take("false")) return Json(false);
            if (take("null")) return Json();
            if (take("NaN")) return Json(std::nan(""));
            if (take("Infinity")) return Json(HUGE_VAL);
            if (take("-Infinity")) return Json(-HUGE_VAL);
            if (c == '-' || (c >= '0' && c <= '9')) return number();
            fail("unexpected character");
        }
        Json number() {
            size_t start = pos;
            bool real = false;
            if (s[pos] == '-') pos++;
            if (pos >= len || s[pos] < '0' || s[pos] > '9') fail("malformed number");
            while (pos < len && s[pos] >= '0' && s[pos] <= '9') pos++;
            if (pos < len && s[pos] == '.') {
                real = true; pos++;
                if (pos >= len || s[pos] < '0' || s[pos] > '9') fail("malformed number");
                while (pos < len && s[pos] >= '0' && s[pos] <= '9') pos++;
            }
            if (pos < len && (s[pos] == 'e' || s[pos] == 'E')) {
                real = true; pos++;
                if (pos < len && (s[pos] == '+' || s[pos] == '-')) pos++;
                if (pos >= len || s[pos] < '0' || s[pos] > '9') fail("malformed number");
                while (pos < len && s[pos] >= '0' && s[pos] <= '9') pos++;
            }
            std::string t(s + start, pos - start);
            if (!real && t.size() < 19) return Json((long long)strtoll(t.c_str(), nullptr, 10));
            return Json(strtod(t.c_str(), nullptr));
        }
        static void utf8(std::string& out, unsigned cp) {
            if (cp < 0x80) out += (char)cp;
            else if (cp < 0x800) { out += (char)(0xC0 | (cp >> 6)); out += (char)(0x80 | (cp & 0x3F)); }
            else if (cp < 0x10000) {
                out += (char)(0xE0 | (cp >> 12)); out += (char)(0x80 | ((cp >> 6) & 0x3F)); out += (char)(0x80 | (cp & 0x3F));
            } else {
                out += (char)(0xF0 | (cp >> 18)); out += (char)(0x80 | ((cp >> 12) & 0x3F));
                out += (char)(0x80 | ((cp >> 6) & 0x3F)); out += (char)(0x80 | (cp & 0x3F));
            }
        }
        unsigned hex4() {
            if (len - pos < 4) fail("short \\u escape");
            unsigned v = 0;
            for (int i = 0; i < 4; i++) {
                char c = s[pos++];
                v <<= 4;
                if (c >= '0' && c <= '9') v |= c - '0';
                else if (c >= 'a' && c <= 'f') v |= c - 'a' + 10;
                else if (c >= 'A' && c <= 'F') v |= c - 'A' + 10;
                else fail("bad \\u escape");
            }
            return v;
        }
        std::string string() {
            pos++;  // opening quote
            std::string out;
            while (true) {
                if (pos >= len) fail("unterminated string");
                unsigned char c = (unsigned char)s[pos++];
                if (c == '"') return out;
                if (c < 0x20) fail("control character in a string");
                if (c != '\\') { out += (char)c; continue; }
                if (pos >= len) fail("unterminated escape");
                char e = s[pos++];
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
                        unsigned cp = hex4();
                        if (cp >= 0xD800 && cp < 0xDC00 && len - pos >= 6 && s[pos] == '\\' && s[pos + 1] == 'u') {
                            pos += 2;
                            unsigned lo = hex4();
                            if (lo >= 0xDC00 && lo < 0xE000) cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
                            else fail("bad surrogate pair");
                        }
                        utf8(out, cp);
                        break;
                    }
                    default: fail("unknown escape");
                }
            }
        }
        Json array(int depth) {
            pos++;
            Json j = Json::array();
            skip();
            if (pos < len && s[pos] == ']') { pos++; return j; }
            while (true) {
                skip();
                j.a_.push_back(value(depth + 1));
                skip();
                if (pos >= len) fail("unterminated array");
                if (s[pos] == ',') { pos++; continue; }
                if (s[pos] == ']') { pos++; return j; }
                fail("expected ',' or ']'");
            }
        }
        Json object(int depth) {
            pos++;
            Json j = Json::object();
            skip();
            if (pos < len && s[pos] == '}') { pos++; return j; }
            while (true) {
                skip();
                if (pos >= len || s[pos] != '"') fail("expected a key");
                std::string key = string();
                skip();
                if (pos >= len || s[pos] != ':') fail("expected ':'");
                pos++;
                skip();
                Json v = value(depth + 1);
                j.set(key, std::move(v));     // a repeated key keeps its last value, as Python's reader does
                skip();
                if (pos >= len) fail("unterminated object");
                if (s[pos] == ',') { pos++; continue; }
                if (s[pos] == '}') { pos++; return j; }
                fail("expected ',' or '}'");
            }
        }
    };

    static void write_string(std::string& out, const std::string& s) {
        out += '"';
        for (unsigned char c : s) {
            switch (c) {
                case '"': out += "\\\""; break;
                case '\\': out += "\\\\"; break;
                case '\n': out += "\\n"; break;
                case '\r': out += "\\r"; break;
                case '\t': out += "\\t"; break;
                default:
                    if (c < 0x20) { char b[8]; snprintf(b, sizeof b, "\\u%04x", c); out += b; }
                    else out += (char)c;
            }
        }
        out += '"';
    }
    void write(std::string& out, int indent, int level) const {
        auto nl = [&](int lv) {
            if (indent < 0) return;
            out += '\n';
            out.append((size_t)(indent * lv), ' ');
        };
        switch (kind_) {
            case Null: out += "null"; break;
            case Bool: out += b_ ? "true" : "false"; break;
            case Int: out += std::to_string(i_); break;
            case Real: {
                if (std::isnan(d_)) { out += "NaN"; break; }
                if (std::isinf(d_)) { out += d_ > 0 ? "Infinity" : "-Infinity"; break; }
                char b[40];
                snprintf(b, sizeof b, "%.17g", d_);
                out += b;
                if (!strpbrk(b, ".eE")) out += ".0";
                break;
            }
            case String: write_string(out, s_); break;
            case Array:
                out += '[';
                for (size_t i = 0; i < a_.size(); i++) {
                    if (i) out += indent < 0 ? ", " : ",";
                    nl(level + 1);
                    a_[i].write(out, indent, level + 1);
                }
                if (!a_.empty()) nl(level);
                out += ']';
                break;
            case Object:
                out += '{';
                for (size_t i = 0; i < o_.size(); i++) {
                    if (i) out += indent < 0 ? ", " : ",";
                    nl(level + 1);
                    write_string(out, o_[i].first);
                    out += ": ";
                    o_[i].second.write(out, indent, level + 1);
                }
                if (!o_.empty()) nl(level);
                out += '}';
                break;
        }
    }
};

}  // namespace qe
