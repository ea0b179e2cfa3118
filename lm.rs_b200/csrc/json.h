// json.h -- a small JSON reader for model folders (config.json, the header of a safetensors file).
// Values are parsed into a tree; numbers are kept as double, object keys keep their order of appearance.
#pragma once
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <memory>
#include <string>
#include <utility>
#include <vector>

namespace lmrs {

struct Json {
    enum Kind { NUL, BOOL, NUM, STR, ARR, OBJ } kind = NUL;
    bool b = false;
    double num = 0.0;
    std::string str;
    std::vector<Json> arr;
    std::vector<std::pair<std::string, Json>> obj;

    bool is_null() const { return kind == NUL; }
    bool is_obj() const { return kind == OBJ; }
    const Json* find(const char* key) const {
        if (kind != OBJ) return nullptr;
        for (const auto& kv : obj)
            if (kv.first == key) return &kv.second;
        return nullptr;
    }
    // present and not null
    bool has(const char* key) const { const Json* j = find(key); return j && !j->is_null(); }
    const Json& at(const char* key) const {
        static const Json null_value;
        const Json* j = find(key);
        return j ? *j : null_value;
    }
    double number(double dflt) const { return kind == NUM ? num : (kind == BOOL ? (b ? 1.0 : 0.0) : dflt); }
    bool truth() const { return kind == BOOL ? b : (kind == NUM ? num != 0.0 : false); }
};

class JsonParser {
  public:
    JsonParser(const char* p, size_t n) : p_(p), e_(p + n) {}
    bool parse(Json& out, std::string& err) {
        if (!value(out, 0)) { err = err_.empty() ? "malformed JSON" : err_; return false; }
        ws();
        if (p_ != e_) { err = "trailing characters after the JSON value"; return false; }
        return true;
    }

  private:
    const char *p_, *e_;
    std::string err_;
    void ws() { while (p_ < e_ && (*p_ == ' ' || *p_ == '\t' || *p_ == '\n' || *p_ == '\r')) p_++; }
    bool lit(const char* s) {
        size_t n = strlen(s);
        if ((size_t)(e_ - p_) < n || memcmp(p_, s, n) != 0) return false;
        p_ += n;
        return true;
    }
    bool string(std::string& s) {
        if (p_ >= e_ || *p_ != '"') return false;
        p_++;
        while (p_ < e_ && *p_ != '"') {
            if (*p_ == '\\') {
                if (++p_ >= e_) return false;
                switch (*p_) {
                    case 'n': s += '\n'; break;
                    case 't': s += '\t'; break;
                    case 'r': s += '\r'; break;
                    case 'b': s += '\b'; break;
                    case 'f': s += '\f'; break;
                    case 'u': {   // code points above 0x7f are kept as UTF-8 of the BMP value; surrogate pairs are not joined
                        if (e_ - p_ < 5) return false;
                        unsigned cp = (unsigned)strtoul(std::string(p_ + 1, 4).c_str(), nullptr, 16);
                        p_ += 4;
                        if (cp < 0x80) s += (char)cp;
                        else if (cp < 0x800) { s += (char)(0xC0 | (cp >> 6)); s += (char)(0x80 | (cp & 0x3F)); }
                        else { s += (char)(0xE0 | (cp >> 12)); s += (char)(0x80 | ((cp >> 6) & 0x3F)); s += (char)(0x80 | (cp & 0x3F)); }
                        break;
                    }
                    default: s += *p_;
                }
                p_++;
            } else {
                s += *p_++;
            }
        }
        if (p_ >= e_) return false;
        p_++;
        return true;
    }
    bool value(Json& v, int depth) {
        if (depth > 64) { err_ = "JSON nested too deeply"; return false; }
        ws();
        if (p_ >= e_) return false;
        const char c = *p_;
        if (c == '{') {
            p_++;
            v.kind = Json::OBJ;
            ws();
            if (p_ < e_ && *p_ == '}') { p_++; return true; }
            for (;;) {
                ws();
                std::string k;
                if (!string(k)) return false;
                ws();
                if (p_ >= e_ || *p_++ != ':') return false;
                v.obj.emplace_back(std::move(k), Json());
                if (!value(v.obj.back().second, depth + 1)) return false;
                ws();
                if (p_ < e_ && *p_ == ',') { p_++; continue; }
                if (p_ < e_ && *p_ == '}') { p_++; return true; }
                return false;
            }
        }
        if (c == '[') {
            p_++;
            v.kind = Json::ARR;
            ws();
            if (p_ < e_ && *p_ == ']') { p_++; return true; }
            for (;;) {
                v.arr.emplace_back();
                if (!value(v.arr.back(), depth + 1)) return false;
                ws();
                if (p_ < e_ && *p_ == ',') { p_++; continue; }
                if (p_ < e_ && *p_ == ']') { p_++; return true; }
                return false;
            }
        }
        if (c == '"') { v.kind = Json::STR; return string(v.str); }
        if (lit("true")) { v.kind = Json::BOOL; v.b = true; return true; }
        if (lit("false")) { v.kind = Json::BOOL; v.b = false; return true; }
        if (lit("null")) { v.kind = Json::NUL; return true; }
        if (lit("NaN")) { v.kind = Json::NUM; v.num = strtod("nan", nullptr); return true; }
        if (lit("Infinity")) { v.kind = Json::NUM; v.num = strtod("inf", nullptr); return true; }
        if (lit("-Infinity")) { v.kind = Json::NUM; v.num = -strtod("inf", nullptr); return true; }
        const std::string num(p_, (size_t)std::min<ptrdiff_t>(e_ - p_, 63));
        char* end = nullptr;
        const double d = strtod(num.c_str(), &end);
        if (end == num.c_str()) return false;
        p_ += end - num.c_str();
        v.kind = Json::NUM;
        v.num = d;
        return true;
    }
};

}  // namespace lmrs
