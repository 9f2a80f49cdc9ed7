// prima.cpp_b200/csrc/json.h — a small JSON reader for model configuration files and safetensors headers (host only).
// Values are kept as a tree; numbers as double (integers up to 2^53 survive, which covers byte offsets of any file that fits a GPU).
#pragma once
#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <utility>
#include <vector>

namespace pb {

struct Json {
    enum Kind { NUL, BOOL, NUM, STR, ARR, OBJ } kind = NUL;
    bool b = false;
    double num = 0;
    std::string str;
    std::vector<Json> arr;
    std::vector<std::pair<std::string, Json>> obj;   // file order kept (tensor tables are walked in order)

    const Json * get(const char * key) const {
        if (kind != OBJ) return nullptr;
        for (const auto & kv : obj)
            if (kv.first == key) return &kv.second;
        return nullptr;
    }
    bool is_null() const { return kind == NUL; }
    bool has(const char * key) const { const Json * j = get(key); return j && !j->is_null(); }
    double number(const char * key, double dflt) const {
        const Json * j = get(key);
        return (j && j->kind == NUM) ? j->num : dflt;
    }
    long long integer(const char * key, long long dflt) const {
        const Json * j = get(key);
        return (j && j->kind == NUM) ? (long long) llround(j->num) : dflt;
    }
    std::string string(const char * key, const char * dflt = "") const {
        const Json * j = get(key);
        return (j && j->kind == STR) ? j->str : std::string(dflt);
    }
};

class JsonParser {
   public:
    JsonParser(const char * s, size_t n) : p_(s), e_(s + n) {}
    bool parse(Json & out) {
        if (!value(out, 0)) return false;
        ws();
        return p_ == e_;
    }

   private:
    const char *p_, *e_;
    void ws() {
        while (p_ < e_ && (*p_ == ' ' || *p_ == '\n' || *p_ == '\t' || *p_ == '\r')) p_++;
    }
    bool lit(const char * w) {
        const size_t n = strlen(w);
        if ((size_t) (e_ - p_) < n || memcmp(p_, w, n) != 0) return false;
        p_ += n;
        return true;
    }
    static void utf8(std::string & s, unsigned cp) {
        if (cp < 0x80) s += (char) cp;
        else if (cp < 0x800) { s += (char) (0xC0 | (cp >> 6)); s += (char) (0x80 | (cp & 0x3F)); }
        else if (cp < 0x10000) { s += (char) (0xE0 | (cp >> 12)); s += (char) (0x80 | ((cp >> 6) & 0x3F)); s += (char) (0x80 | (cp & 0x3F)); }
        else { s += (char) (0xF0 | (cp >> 18)); s += (char) (0x80 | ((cp >> 12) & 0x3F)); s += (char) (0x80 | ((cp >> 6) & 0x3F)); s += (char) (0x80 | (cp & 0x3F)); }
    }
    bool hex4(unsigned & v) {
        if (e_ - p_ < 4) return false;
        v = 0;
        for (int i = 0; i < 4; i++) {
            const char c = *p_++;
            v <<= 4;
            if (c >= '0' && c <= '9') v |= (unsigned) (c - '0');
            else if (c >= 'a' && c <= 'f') v |= (unsigned) (c - 'a' + 10);
            else if (c >= 'A' && c <= 'F') v |= (unsigned) (c - 'A' + 10);
            else return false;
        }
        return true;
    }
    bool string(std::string & s) {
        if (p_ >= e_ || *p_ != '"') return false;
        p_++;
        while (p_ < e_ && *p_ != '"') {
            if (*p_ == '\\') {
                if (++p_ >= e_) return false;
                const char c = *p_++;
                switch (c) {
                    case 'n': s += '\n'; break;
                    case 't': s += '\t'; break;
                    case 'r': s += '\r'; break;
                    case 'b': s += '\b'; break;
                    case 'f': s += '\f'; break;
                    case 'u': {
                        unsigned cp = 0;
                        if (!hex4(cp)) return false;
                        if (cp >= 0xD800 && cp < 0xDC00 && e_ - p_ >= 6 && p_[0] == '\\' && p_[1] == 'u') {
                            p_ += 2;
                            unsigned lo = 0;
                            if (!hex4(lo)) return false;
                            cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
                        }
                        utf8(s, cp);
                        break;
                    }
                    default: s += c;   // \" \\ \/
                }
            } else {
                s += *p_++;
            }
        }
        if (p_ >= e_) return false;
        p_++;
        return true;
    }
    bool value(Json & out, int depth) {
        if (depth > 64) return false;
        ws();
        if (p_ >= e_) return false;
        const char c = *p_;
        if (c == '{') {
            p_++;
            out.kind = Json::OBJ;
            ws();
            if (p_ < e_ && *p_ == '}') { p_++; return true; }
            for (;;) {
                ws();
                std::string k;
                if (!string(k)) return false;
                ws();
                if (p_ >= e_ || *p_++ != ':') return false;
                Json v;
                if (!value(v, depth + 1)) return false;
                out.obj.emplace_back(std::move(k), std::move(v));
                ws();
                if (p_ >= e_) return false;
                if (*p_ == ',') { p_++; continue; }
                if (*p_ == '}') { p_++; return true; }
                return false;
            }
        }
        if (c == '[') {
            p_++;
            out.kind = Json::ARR;
            ws();
            if (p_ < e_ && *p_ == ']') { p_++; return true; }
            for (;;) {
                Json v;
                if (!value(v, depth + 1)) return false;
                out.arr.push_back(std::move(v));
                ws();
                if (p_ >= e_) return false;
                if (*p_ == ',') { p_++; continue; }
                if (*p_ == ']') { p_++; return true; }
                return false;
            }
        }
        if (c == '"') { out.kind = Json::STR; return string(out.str); }
        if (lit("true")) { out.kind = Json::BOOL; out.b = true; return true; }
        if (lit("false")) { out.kind = Json::BOOL; out.b = false; return true; }
        if (lit("null")) { out.kind = Json::NUL; return true; }
        if (lit("Infinity")) { out.kind = Json::NUM; out.num = INFINITY; return true; }
        char * end = nullptr;
        std::string tmp(p_, (size_t) std::min<ptrdiff_t>(e_ - p_, 64));
        const double v = strtod(tmp.c_str(), &end);
        if (end == tmp.c_str()) return false;
        p_ += end - tmp.c_str();
        out.kind = Json::NUM;
        out.num = v;
        return true;
    }
};

inline bool json_parse(const std::string & text, Json & out) { return JsonParser(text.data(), text.size()).parse(out); }

}  // namespace pb
