// Small JSON reader for the three documents the weight store parses: config.json, the weight index and
// safetensors headers. Integers that fit in 64 bits are kept exactly (tensor offsets exceed 2^53 in no real
// file, but nothing here depends on that). Objects keep document order; on duplicate keys the last one wins,
// which is what a map-building reader does.
#pragma once
#include <stdint.h>

#include <cstdlib>
#include <cstring>
#include <string>
#include <utility>
#include <vector>

namespace q4json {

struct Value {
    enum Type { Null, Bool, Number, String, Array, Object } type = Null;
    bool boolean = false;
    bool is_u64 = false;  // a non-negative integer literal without fraction or exponent that fits in 64 bits
    uint64_t u64 = 0;
    double number = 0;
    std::string string;
    std::vector<Value> array;
    std::vector<std::pair<std::string, Value>> object;

    const Value *find(const char *key) const {
        if (type != Object) return nullptr;
        for (size_t i = object.size(); i-- > 0;)
            if (object[i].first == key) return &object[i].second;
        return nullptr;
    }
};

class Parser {
public:
    Parser(const char *data, size_t len) : p_(data), end_(data + len), begin_(data) {}

    bool parse(Value *out, std::string *error) {
        if (!value(out, 0)) {
            *error = error_ + " at byte " + std::to_string((size_t)(p_ - begin_));
            return false;
        }
        skip_ws();
        if (p_ != end_) {
            *error = "trailing characters at byte " + std::to_string((size_t)(p_ - begin_));
            return false;
        }
        return true;
    }

private:
    const char *p_, *end_, *begin_;
    std::string error_;
    static constexpr int kMaxDepth = 64;

    bool fail(const char *what) {
        error_ = what;
        return false;
    }
    void skip_ws() {
        while (p_ < end_ && (*p_ == ' ' || *p_ == '\t' || *p_ == '\n' || *p_ == '\r')) ++p_;
    }
    bool literal(const char *word) {
        const size_t n = strlen(word);
        if ((size_t)(end_ - p_) < n || memcmp(p_, word, n) != 0) return fail("unknown literal");
        p_ += n;
        return true;
    }
    static void append_utf8(std::string *s, uint32_t cp) {
        if (cp < 0x80) {
            s->push_back((char)cp);
        } else if (cp < 0x800) {
            s->push_back((char)(0xC0 | (cp >> 6)));
            s->push_back((char)(0x80 | (cp & 0x3F)));
        } else if (cp < 0x10000) {
            s->push_back((char)(0xE0 | (cp >> 12)));
            s->push_back((char)(0x80 | ((cp >> 6) & 0x3F)));
            s->push_back((char)(0x80 | (cp & 0x3F)));
        } else {
            s->push_back((char)(0xF0 | (cp >> 18)));
            s->push_back((char)(0x80 | ((cp >> 12) & 0x3F)));
            s->push_back((char)(0x80 | ((cp >> 6) & 0x3F)));
            s->push_back((char)(0x80 | (cp & 0x3F)));
        }
    }
    bool hex4(uint32_t *out) {
        if (end_ - p_ < 4) return fail("truncated \\u escape");
        uint32_t v = 0;
        for (int i = 0; i < 4; ++i) {
            const char c = *p_++;
            v <<= 4;
            if (c >= '0' && c <= '9') v |= (uint32_t)(c - '0');
            else if (c >= 'a' && c <= 'f') v |= (uint32_t)(c - 'a' + 10);
            else if (c >= 'A' && c <= 'F') v |= (uint32_t)(c - 'A' + 10);
            else return fail("bad \\u escape");
        }
        *out = v;
        return true;
    }
    bool string(std::string *out) {
        if (p_ >= end_ || *p_ != '"') return fail("expected a string");
        ++p_;
        out->clear();
        while (true) {
            if (p_ >= end_) return fail("unterminated string");
            const unsigned char c = (unsigned char)*p_++;
            if (c == '"') return true;
            if (c < 0x20) return fail("control character in string");
            if (c != '\\') {
                out->push_back((char)c);
                continue;
            }
            if (p_ >= end_) return fail("unterminated escape");
            const char e = *p_++;
            switch (e) {
                case '"': out->push_back('"'); break;
                case '\\': out->push_back('\\'); break;
                case '/': out->push_back('/'); break;
                case 'b': out->push_back('\b'); break;
                case 'f': out->push_back('\f'); break;
                case 'n': out->push_back('\n'); break;
                case 'r': out->push_back('\r'); break;
                case 't': out->push_back('\t'); break;
                case 'u': {
                    uint32_t cp;
                    if (!hex4(&cp)) return false;
                    if (cp >= 0xD800 && cp < 0xDC00) {
                        if (end_ - p_ < 2 || p_[0] != '\\' || p_[1] != 'u') return fail("lone surrogate");
                        p_ += 2;
                        uint32_t lo;
                        if (!hex4(&lo)) return false;
                        if (lo < 0xDC00 || lo > 0xDFFF) return fail("bad surrogate pair");
                        cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
                    } else if (cp >= 0xDC00 && cp <= 0xDFFF) {
                        return fail("lone surrogate");
                    }
                    append_utf8(out, cp);
                    break;
                }
                default: return fail("unknown escape");
            }
        }
    }
    bool number(Value *out) {
        const char *start = p_;
        bool integral = true, negative = false;
        if (p_ < end_ && *p_ == '-') {
            negative = true;
            ++p_;
        }
        if (p_ >= end_ || *p_ < '0' || *p_ > '9') return fail("expected a digit");
        if (*p_ == '0') {
            ++p_;
        } else {
            while (p_ < end_ && *p_ >= '0' && *p_ <= '9') ++p_;
        }
        if (p_ < end_ && *p_ == '.') {
            integral = false;
            ++p_;
            if (p_ >= end_ || *p_ < '0' || *p_ > '9') return fail("expected a fraction digit");
            while (p_ < end_ && *p_ >= '0' && *p_ <= '9') ++p_;
        }
        if (p_ < end_ && (*p_ == 'e' || *p_ == 'E')) {
            integral = false;
            ++p_;
            if (p_ < end_ && (*p_ == '+' || *p_ == '-')) ++p_;
            if (p_ >= end_ || *p_ < '0' || *p_ > '9') return fail("expected an exponent digit");
            while (p_ < end_ && *p_ >= '0' && *p_ <= '9') ++p_;
        }
        const std::string text(start, p_);
        out->type = Value::Number;
        out->number = strtod(text.c_str(), nullptr);
        if (integral && !negative) {
            uint64_t v = 0;
            bool fits = true;
            for (char c : text) {
                const uint64_t d = (uint64_t)(c - '0');
                if (v > (UINT64_MAX - d) / 10) {
                    fits = false;
                    break;
                }
                v = v * 10 + d;
            }
            out->is_u64 = fits;
            out->u64 = fits ? v : 0;
        }
        return true;
    }
    bool value(Value *out, int depth) {
        if (depth > kMaxDepth) return fail("nesting too deep");
        skip_ws();
        if (p_ >= end_) return fail("unexpected end of document");
        const char c = *p_;
        if (c == '{') {
            ++p_;
            out->type = Value::Object;
            skip_ws();
            if (p_ < end_ && *p_ == '}') {
                ++p_;
                return true;
            }
            while (true) {
                skip_ws();
                std::string key;
                if (!string(&key)) return false;
                skip_ws();
                if (p_ >= end_ || *p_ != ':') return fail("expected ':'");
                ++p_;
                out->object.emplace_back(std::move(key), Value());
                if (!value(&out->object.back().second, depth + 1)) return false;
                skip_ws();
                if (p_ < end_ && *p_ == ',') {
                    ++p_;
                    continue;
                }
                if (p_ < end_ && *p_ == '}') {
                    ++p_;
                    return true;
                }
                return fail("expected ',' or '}'");
            }
        }
        if (c == '[') {
            ++p_;
            out->type = Value::Array;
            skip_ws();
            if (p_ < end_ && *p_ == ']') {
                ++p_;
                return true;
            }
            while (true) {
                out->array.emplace_back();
                if (!value(&out->array.back(), depth + 1)) return false;
                skip_ws();
                if (p_ < end_ && *p_ == ',') {
                    ++p_;
                    continue;
                }
                if (p_ < end_ && *p_ == ']') {
                    ++p_;
                    return true;
                }
                return fail("expected ',' or ']'");
            }
        }
        if (c == '"') {
            out->type = Value::String;
            return string(&out->string);
        }
        if (c == 't') {
            out->type = Value::Bool;
            out->boolean = true;
            return literal("true");
        }
        if (c == 'f') {
            out->type = Value::Bool;
            out->boolean = false;
            return literal("false");
        }
        if (c == 'n') {
            out->type = Value::Null;
            return literal("null");
        }
        return number(out);
    }
};

inline bool parse(const char *data, size_t len, Value *out, std::string *error) {
    Parser parser(data, len);
    return parser.parse(out, error);
}

}  // namespace q4json
