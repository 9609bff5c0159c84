// A small JSON reader over one document held in memory: enough for a SafeTensors header and for the checkpoint meta.
// Strings are unescaped (\uXXXX to UTF-8, surrogate pairs included); numbers are handed out as text, as u64 or as f64;
// any value can be skipped. `ok` turns false at the first thing that is not JSON and stays false.
#pragma once

#include <cerrno>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <string>

namespace oxz {

struct JsonReader {
    const char* p;
    const char* e;
    bool ok = true;
    void ws() { while (p < e && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) p++; }
    bool eat(char c) { ws(); if (p < e && *p == c) { p++; return true; } return false; }
    bool peek(char c) { ws(); return p < e && *p == c; }
    bool word(const char* w) {
        ws();
        const size_t n = strlen(w);
        if ((size_t)(e - p) >= n && memcmp(p, w, n) == 0) { p += n; return true; }
        return false;
    }
    static void utf8(std::string& out, uint32_t cp) {
        if (cp < 0x80) out += (char)cp;
        else if (cp < 0x800) { out += (char)(0xC0 | (cp >> 6)); out += (char)(0x80 | (cp & 0x3F)); }
        else if (cp < 0x10000) { out += (char)(0xE0 | (cp >> 12)); out += (char)(0x80 | ((cp >> 6) & 0x3F)); out += (char)(0x80 | (cp & 0x3F)); }
        else { out += (char)(0xF0 | (cp >> 18)); out += (char)(0x80 | ((cp >> 12) & 0x3F)); out += (char)(0x80 | ((cp >> 6) & 0x3F)); out += (char)(0x80 | (cp & 0x3F)); }
    }
    bool hex4(uint32_t* v) {
        if (e - p < 4) return false;
        uint32_t x = 0;
        for (int i = 0; i < 4; i++) {
            const char c = p[i];
            x <<= 4;
            if (c >= '0' && c <= '9') x |= (uint32_t)(c - '0');
            else if (c >= 'a' && c <= 'f') x |= (uint32_t)(c - 'a' + 10);
            else if (c >= 'A' && c <= 'F') x |= (uint32_t)(c - 'A' + 10);
            else return false;
        }
        p += 4;
        *v = x;
        return true;
    }
    std::string str() {
        std::string out;
        ws();
        if (p >= e || *p != '"') { ok = false; return out; }
        p++;
        while (p < e && *p != '"') {
            if (*p != '\\') { out += *p++; continue; }
            if (++p >= e) break;
            const char c = *p++;
            switch (c) {
                case 'n': out += '\n'; break;
                case 't': out += '\t'; break;
                case 'r': out += '\r'; break;
                case 'b': out += '\b'; break;
                case 'f': out += '\f'; break;
                case 'u': {
                    uint32_t cp = 0, lo = 0;
                    if (!hex4(&cp)) { ok = false; return out; }
                    if (cp >= 0xD800 && cp < 0xDC00 && e - p >= 6 && p[0] == '\\' && p[1] == 'u') {
                        p += 2;
                        if (!hex4(&lo)) { ok = false; return out; }
                        cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
                    }
                    utf8(out, cp);
                    break;
                }
                default: out += c;  // \" \\ \/
            }
        }
        if (p >= e) { ok = false; return out; }
        p++;
        return out;
    }
    // a JSON number as text; serde_json prints f64 so that it reads back to the same bits
    std::string number() {
        ws();
        const char* s = p;
        while (p < e && (strchr("+-.eE", *p) || (*p >= '0' && *p <= '9'))) p++;
        if (p == s) ok = false;
        return std::string(s, p);
    }
    bool u64(uint64_t* v) {
        const std::string t = number();
        if (!ok || t.empty() || t.find_first_not_of("0123456789") != std::string::npos || t.size() > 20) { ok = false; return false; }
        errno = 0;
        *v = strtoull(t.c_str(), nullptr, 10);
        if (errno) ok = false;
        return ok;
    }
    bool f64(double* v) {
        const std::string t = number();
        if (!ok) return false;
        char* end = nullptr;
        *v = strtod(t.c_str(), &end);
        if (!end || *end) ok = false;
        return ok;
    }
    void skip() {
        ws();
        if (p >= e) { ok = false; return; }
        if (*p == '"') { str(); return; }
        if (*p == '{' || *p == '[') {
            const char open = *p, close = open == '{' ? '}' : ']';
            p++;
            if (eat(close)) return;
            do {
                if (open == '{') { str(); if (!ok || !eat(':')) { ok = false; return; } }
                skip();
                if (!ok) return;
            } while (eat(','));
            if (!eat(close)) ok = false;
            return;
        }
        if (word("null") || word("true") || word("false")) return;
        number();
    }
    // calls fn(key) for every member of the object at the cursor; fn must consume the value
    template <class F>
    bool object(F fn) {
        if (!eat('{')) { ok = false; return false; }
        if (eat('}')) return true;
        do {
            const std::string key = str();
            if (!ok || !eat(':')) { ok = false; return false; }
            fn(key);
            if (!ok) return false;
        } while (eat(','));
        if (!eat('}')) ok = false;
        return ok;
    }
};

}  // namespace oxz
