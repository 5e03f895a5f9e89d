// Minimal JSON reader for encoding configurations: one flat object whose values are strings,
// numbers, booleans or null.  Nested containers are rejected; unknown keys are kept (the
// reference only warns about them, include/encodings/encoding_factory.h:150-158).
#pragma once
#include <cctype>
#include <cstdlib>
#include <cstring>
#include <map>
#include <stdexcept>
#include <string>

namespace tnn {

struct JsonValue {
    bool is_string = false;
    bool is_bool = false;
    std::string str;
    double num = 0.0;
    bool truthy() const { return is_string ? !str.empty() : num != 0.0; }
};

struct JsonObject {
    std::map<std::string, JsonValue> items;
    bool has(const std::string &k) const { return items.count(k) != 0; }
    const JsonValue &at(const std::string &k) const {
        auto it = items.find(k);
        if (it == items.end()) throw std::invalid_argument("Config misses " + k);
        return it->second;
    }
    double number(const std::string &k, double dflt) const {
        auto it = items.find(k);
        if (it == items.end()) return dflt;
        if (it->second.is_string) throw std::invalid_argument("Config key " + k + " must be a number");
        return it->second.num;
    }
};

namespace json_detail {
inline void skip_ws(const char *&p) {
    for (;;) {
        while (*p && std::isspace((unsigned char)*p)) ++p;
        if (p[0] == '/' && p[1] == '/') { // comments are tolerated like the reference's loader (io.h:50)
            while (*p && *p != '\n') ++p;
            continue;
        }
        return;
    }
}
inline std::string parse_string(const char *&p) {
    if (*p != '"') throw std::invalid_argument("JSON: expected string");
    ++p;
    std::string s;
    while (*p && *p != '"') {
        if (*p == '\\') {
            ++p;
            switch (*p) {
            case 'n': s += '\n'; break;
            case 't': s += '\t'; break;
            case '"': s += '"'; break;
            case '\\': s += '\\'; break;
            case '/': s += '/'; break;
            default: throw std::invalid_argument("JSON: unsupported escape");
            }
            ++p;
        } else {
            s += *p++;
        }
    }
    if (*p != '"') throw std::invalid_argument("JSON: unterminated string");
    ++p;
    return s;
}
} // namespace json_detail

inline JsonObject parse_json_object(const char *text) {
    using namespace json_detail;
    JsonObject obj;
    const char *p = text;
    skip_ws(p);
    if (*p != '{') throw std::invalid_argument("JSON: expected '{'");
    ++p;
    skip_ws(p);
    if (*p == '}') return obj;
    for (;;) {
        skip_ws(p);
        const std::string key = parse_string(p);
        skip_ws(p);
        if (*p != ':') throw std::invalid_argument("JSON: expected ':' after key " + key);
        ++p;
        skip_ws(p);
        JsonValue v;
        if (*p == '"') {
            v.is_string = true;
            v.str = parse_string(p);
        } else if (!std::strncmp(p, "true", 4)) {
            v.is_bool = true, v.num = 1.0, p += 4;
        } else if (!std::strncmp(p, "false", 5)) {
            v.is_bool = true, v.num = 0.0, p += 5;
        } else if (!std::strncmp(p, "null", 4)) {
            p += 4;
        } else if (*p == '{' || *p == '[') {
            throw std::invalid_argument("JSON: nested values are not supported for key " + key);
        } else {
            char *end = nullptr;
            v.num = std::strtod(p, &end);
            if (end == p) throw std::invalid_argument("JSON: bad value for key " + key);
            p = end;
        }
        obj.items[key] = v;
        skip_ws(p);
        if (*p == ',') {
            ++p;
            continue;
        }
        if (*p == '}') break;
        throw std::invalid_argument("JSON: expected ',' or '}'");
    }
    return obj;
}

} // namespace tnn
