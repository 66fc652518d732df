// gm_host_json.cpp -- the optimizer part of a checkpoint as JSON text.
//
// checkpoints/checkpoint.go:74-86 gives the payload its field names ("type",
// "parameters", "state_data"; per tensor "name", "shape", "data", "state_type")
// and Go's encoding/json decides what comes back: every number inside
// "parameters" decodes into interface{} as float64, whatever it was when it was
// saved, while "data" decodes into []float32.  Encode writes what GetState
// produced; Decode returns what a Go reader would hand to LoadState -- Float64
// parameters and float32 tensors with exactly the saved bits (nine significant
// digits round-trip every binary32 value).  NaN and infinities are refused, as
// json.Marshal refuses them.
#include <errno.h>
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "gm_host.hpp"

namespace gometal {
namespace checkpoints {

namespace {

void put_string(std::string* out, const std::string& s) {
    out->push_back('"');
    for (unsigned char c : s) {
        switch (c) {
            case '"': *out += "\\\""; break;
            case '\\': *out += "\\\\"; break;
            case '\n': *out += "\\n"; break;
            case '\r': *out += "\\r"; break;
            case '\t': *out += "\\t"; break;
            default:
                if (c < 0x20) { char b[8]; snprintf(b, sizeof b, "\\u%04x", c); *out += b; }
                else out->push_back((char)c);
        }
    }
    out->push_back('"');
}

bool put_number(std::string* out, double v, int digits) {
    if (!isfinite(v)) return false;
    char b[40];
    snprintf(b, sizeof b, "%.*g", digits, v);
    *out += b;
    return true;
}

struct Parser {
    const char* p;
    const char* end;
    std::string err;

    void ws() { while (p < end && (*p == ' ' || *p == '\n' || *p == '\r' || *p == '\t')) ++p; }
    bool fail(const char* what) { if (err.empty()) err = std::string("invalid checkpoint JSON: ") + what; return false; }
    bool eat(char c) { ws(); if (p < end && *p == c) { ++p; return true; } return false; }
    bool expect(char c) { if (eat(c)) return true; char m[32]; snprintf(m, sizeof m, "expected '%c'", c); return fail(m); }

    bool string(std::string* out) {
        ws();
        if (p >= end || *p != '"') return fail("expected a string");
        ++p;
        out->clear();
        while (p < end && *p != '"') {
            if (*p == '\\') {
                if (++p >= end) return fail("unterminated escape");
                switch (*p) {
                    case 'n': out->push_back('\n'); break;
                    case 'r': out->push_back('\r'); break;
                    case 't': out->push_back('\t'); break;
                    case 'b': out->push_back('\b'); break;
                    case 'f': out->push_back('\f'); break;
                    case 'u': {
                        if (end - p < 5) return fail("short \\u escape");
                        char hex[5] = {p[1], p[2], p[3], p[4], 0};
                        unsigned cp = (unsigned)strtoul(hex, nullptr, 16);
                        if (cp < 0x80) out->push_back((char)cp);
                        else if (cp < 0x800) { out->push_back((char)(0xc0 | (cp >> 6))); out->push_back((char)(0x80 | (cp & 0x3f))); }
                        else { out->push_back((char)(0xe0 | (cp >> 12))); out->push_back((char)(0x80 | ((cp >> 6) & 0x3f))); out->push_back((char)(0x80 | (cp & 0x3f))); }
                        p += 4;
                        break;
                    }
                    default: out->push_back(*p);          // \" \\ \/
                }
                ++p;
            } else {
                out->push_back(*p++);
            }
        }
        if (p >= end) return fail("unterminated string");
        ++p;
        return true;
    }

    // The text of one number; the caller converts it at the precision it needs.
    bool number_text(std::string* out) {
        ws();
        const char* s = p;
        if (p < end && (*p == '-' || *p == '+')) ++p;
        while (p < end && ((*p >= '0' && *p <= '9') || *p == '.' || *p == 'e' || *p == 'E' || *p == '-' || *p == '+')) ++p;
        if (p == s) return fail("expected a number");
        out->assign(s, p);
        return true;
    }

    bool skip_value() {
        ws();
        if (p >= end) return fail("unexpected end");
        if (*p == '"') { std::string s; return string(&s); }
        if (*p == '{') {
            ++p;
            if (eat('}')) return true;
            do { std::string k; if (!string(&k) || !expect(':') || !skip_value()) return false; } while (eat(','));
            return expect('}');
        }
        if (*p == '[') {
            ++p;
            if (eat(']')) return true;
            do { if (!skip_value()) return false; } while (eat(','));
            return expect(']');
        }
        if (!strncmp(p, "true", 4)) { p += 4; return true; }
        if (!strncmp(p, "false", 5)) { p += 5; return true; }
        if (!strncmp(p, "null", 4)) { p += 4; return true; }
        std::string n;
        return number_text(&n);
    }

    bool parameters(std::map<std::string, Param>* out) {
        if (!expect('{')) return false;
        if (eat('}')) return true;
        do {
            std::string key;
            if (!string(&key) || !expect(':')) return false;
            ws();
            Param v;
            if (p < end && !strncmp(p, "true", 4)) { p += 4; v.kind = Param::Bool; v.b = true; }
            else if (p < end && !strncmp(p, "false", 5)) { p += 5; v.kind = Param::Bool; v.b = false; }
            else if (p < end && (*p == '-' || (*p >= '0' && *p <= '9'))) {
                std::string n;
                if (!number_text(&n)) return false;
                v.kind = Param::Float64;                      // interface{} receives float64 for every JSON number
                v.f = strtod(n.c_str(), nullptr);
            } else {
                if (!skip_value()) return false;              // strings, null, nested values: not optimizer parameters
                continue;
            }
            (*out)[key] = v;
        } while (eat(','));
        return expect('}');
    }

    bool tensor(OptimizerTensor* t) {
        if (!expect('{')) return false;
        if (eat('}')) return true;
        do {
            std::string key;
            if (!string(&key) || !expect(':')) return false;
            if (key == "name") { if (!string(&t->Name)) return false; }
            else if (key == "state_type") { if (!string(&t->StateType)) return false; }
            else if (key == "shape" || key == "data") {
                if (eat('n')) { if (strncmp(p, "ull", 3)) return fail("expected null"); p += 3; continue; }   // a nil slice encodes as null
                if (!expect('[')) return false;
                if (!eat(']')) {
                    do {
                        std::string n;
                        if (!number_text(&n)) return false;
                        if (key == "shape") t->Shape.push_back((int)strtol(n.c_str(), nullptr, 10));
                        else t->Data.push_back(strtof(n.c_str(), nullptr));        // []float32: parsed at binary32 precision
                    } while (eat(','));
                    if (!expect(']')) return false;
                }
            } else if (!skip_value()) return false;
        } while (eat(','));
        return expect('}');
    }
};

}  // namespace

std::string EncodeOptimizerState(const OptimizerState& st, std::string* out) {
    out->clear();
    *out += "{\"type\":";
    put_string(out, st.Type);
    *out += ",\"parameters\":{";
    bool first = true;
    for (const auto& kv : st.Parameters) {                    // std::map iterates in key order, like Go's encoder
        if (!first) out->push_back(',');
        first = false;
        put_string(out, kv.first);
        out->push_back(':');
        const Param& v = kv.second;
        bool ok = true;
        switch (v.kind) {
            case Param::Bool: *out += v.b ? "true" : "false"; break;
            case Param::Uint64: { char b[32]; snprintf(b, sizeof b, "%llu", (unsigned long long)v.u); *out += b; break; }
            case Param::Float32: ok = put_number(out, (double)(float)v.f, 9); break;
            default: ok = put_number(out, v.f, 17); break;
        }
        if (!ok) return "json: unsupported value: parameter " + kv.first + " is not finite";
    }
    *out += "},\"state_data\":[";
    for (size_t i = 0; i < st.StateData.size(); ++i) {
        const OptimizerTensor& t = st.StateData[i];
        if (i) out->push_back(',');
        *out += "{\"name\":";
        put_string(out, t.Name);
        *out += ",\"shape\":[";
        for (size_t k = 0; k < t.Shape.size(); ++k) { if (k) out->push_back(','); *out += std::to_string(t.Shape[k]); }
        *out += "],\"data\":[";
        for (size_t k = 0; k < t.Data.size(); ++k) {
            if (k) out->push_back(',');
            if (!put_number(out, (double)t.Data[k], 9))
                return "json: unsupported value: " + t.Name + " holds a value that is not finite";
        }
        *out += "],\"state_type\":";
        put_string(out, t.StateType);
        out->push_back('}');
    }
    *out += "]}";
    return "";
}

std::string DecodeOptimizerState(const std::string& text, OptimizerState* out) {
    *out = OptimizerState();
    Parser ps{text.data(), text.data() + text.size(), ""};
    if (!ps.expect('{')) return ps.err;
    if (!ps.eat('}')) {
        do {
            std::string key;
            if (!ps.string(&key) || !ps.expect(':')) return ps.err;
            if (key == "type") { if (!ps.string(&out->Type)) return ps.err; }
            else if (key == "parameters") { if (!ps.parameters(&out->Parameters)) return ps.err; }
            else if (key == "state_data") {
                if (ps.eat('n')) { if (strncmp(ps.p, "ull", 3)) return "invalid checkpoint JSON: expected null"; ps.p += 3; continue; }
                if (!ps.expect('[')) return ps.err;
                if (!ps.eat(']')) {
                    do {
                        OptimizerTensor t;
                        if (!ps.tensor(&t)) return ps.err;
                        out->StateData.push_back(std::move(t));
                    } while (ps.eat(','));
                    if (!ps.expect(']')) return ps.err;
                }
            } else if (!ps.skip_value()) return ps.err;
        } while (ps.eat(','));
        if (!ps.expect('}')) return ps.err;
    }
    ps.ws();
    if (ps.p != ps.end) return "invalid checkpoint JSON: trailing characters";
    return "";
}

}  // namespace checkpoints
}  // namespace gometal
