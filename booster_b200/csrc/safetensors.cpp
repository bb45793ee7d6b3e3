// safetensors.cpp — JSON parser + safetensors container reader (see safetensors.hpp)
#include "safetensors.hpp"

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fcntl.h>
#include <stdexcept>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

namespace b200 {

// ---- JSON ---------------------------------------------------------------------------------------------------
namespace {
struct Parser {
    const char * s; size_t n, i = 0;
    [[noreturn]] void fail(const char * what) const { throw std::runtime_error(std::string("JSON: ") + what + " at byte " + std::to_string(i)); }
    void ws() { while (i < n && (s[i] == ' ' || s[i] == '\n' || s[i] == '\t' || s[i] == '\r')) i++; }
    bool lit(const char * w) { const size_t l = std::strlen(w); if (i + l <= n && std::memcmp(s + i, w, l) == 0) { i += l; return true; } return false; }
    static void utf8(std::string & o, uint32_t cp) {
        if (cp < 0x80) o += (char) cp;
        else if (cp < 0x800) { o += (char) (0xC0 | (cp >> 6)); o += (char) (0x80 | (cp & 0x3F)); }
        else if (cp < 0x10000) { o += (char) (0xE0 | (cp >> 12)); o += (char) (0x80 | ((cp >> 6) & 0x3F)); o += (char) (0x80 | (cp & 0x3F)); }
        else { o += (char) (0xF0 | (cp >> 18)); o += (char) (0x80 | ((cp >> 12) & 0x3F)); o += (char) (0x80 | ((cp >> 6) & 0x3F)); o += (char) (0x80 | (cp & 0x3F)); }
    }
    uint32_t hex4() {
        if (i + 4 > n) fail("short \\u escape");
        uint32_t v = 0;
        for (int k = 0; k < 4; k++) {
            const char c = s[i++];
            v = v * 16 + (uint32_t) (c >= '0' && c <= '9' ? c - '0' : c >= 'a' && c <= 'f' ? c - 'a' + 10 : c >= 'A' && c <= 'F' ? c - 'A' + 10 : (fail("bad hex digit"), 0));
        }
        return v;
    }
    std::string str() {
        if (s[i] != '"') fail("expected a string");
        i++;
        std::string o;
        while (i < n && s[i] != '"') {
            if (s[i] != '\\') { o += s[i++]; continue; }
            if (++i >= n) fail("short escape");
            const char c = s[i++];
            switch (c) {
                case 'n': o += '\n'; break; case 't': o += '\t'; break; case 'r': o += '\r'; break;
                case 'b': o += '\b'; break; case 'f': o += '\f'; break;
                case 'u': {
                    uint32_t cp = hex4();
                    if (cp >= 0xD800 && cp < 0xDC00 && i + 1 < n && s[i] == '\\' && s[i + 1] == 'u') { i += 2; cp = 0x10000 + ((cp - 0xD800) << 10) + (hex4() - 0xDC00); }
                    utf8(o, cp);
                    break;
                }
                default: o += c;
            }
        }
        if (i >= n) fail("unterminated string");
        i++;
        return o;
    }
    Json value(int depth) {
        if (depth > 64) fail("nesting too deep");
        ws();
        if (i >= n) fail("unexpected end");
        Json v;
        const char c = s[i];
        if (c == '{') {
            v.kind = Json::Obj; i++; ws();
            if (i < n && s[i] == '}') { i++; return v; }
            for (;;) {
                ws();
                std::string k = str();
                ws();
                if (i >= n || s[i] != ':') fail("expected ':'");
                i++;
                v.obj[k] = value(depth + 1);
                ws();
                if (i < n && s[i] == ',') { i++; continue; }
                if (i < n && s[i] == '}') { i++; return v; }
                fail("expected ',' or '}'");
            }
        }
        if (c == '[') {
            v.kind = Json::Arr; i++; ws();
            if (i < n && s[i] == ']') { i++; return v; }
            for (;;) {
                v.arr.push_back(value(depth + 1));
                ws();
                if (i < n && s[i] == ',') { i++; continue; }
                if (i < n && s[i] == ']') { i++; return v; }
                fail("expected ',' or ']'");
            }
        }
        if (c == '"') { v.kind = Json::Str; v.str = str(); return v; }
        if (lit("true")) { v.kind = Json::Bool; v.b = true; return v; }
        if (lit("false")) { v.kind = Json::Bool; return v; }
        if (lit("null")) return v;
        if (lit("NaN")) { v.kind = Json::Num; v.num = NAN; return v; }
        if (lit("Infinity")) { v.kind = Json::Num; v.num = INFINITY; return v; }
        if (lit("-Infinity")) { v.kind = Json::Num; v.num = -INFINITY; return v; }
        // number
        const size_t b = i;
        while (i < n && (std::strchr("+-0123456789.eE", s[i]) != nullptr)) i++;
        if (b == i) fail("unexpected character");
        const std::string t(s + b, i - b);
        char * end = nullptr;
        v.kind = Json::Num;
        v.num = std::strtod(t.c_str(), &end);
        if (!end || *end) fail("bad number");
        return v;
    }
};
}  // namespace

Json json_parse(const char * text, size_t n) {
    Parser p{text, n};
    Json v = p.value(0);
    p.ws();
    if (p.i != n) p.fail("trailing characters");
    return v;
}

Json json_parse_file(const std::string & path) {
    FILE * f = std::fopen(path.c_str(), "rb");
    if (!f) throw std::runtime_error("cannot open " + path);
    std::string s;
    char buf[1 << 14];
    size_t r;
    while ((r = std::fread(buf, 1, sizeof buf, f)) > 0) s.append(buf, r);
    std::fclose(f);
    return json_parse(s.data(), s.size());
}

const Json & Json::at(const std::string & k) const {
    if (kind != Obj) throw std::runtime_error("config: '" + k + "' looked up in something that is not an object");
    auto it = obj.find(k);
    if (it == obj.end()) throw std::runtime_error("config: missing key '" + k + "'");
    return it->second;
}
double Json::number(const std::string & k) const {
    const Json & v = at(k);
    if (v.kind != Num) throw std::runtime_error("config: '" + k + "' must be a number");
    return v.num;
}
int64_t Json::integer(const std::string & k) const {
    const double d = number(k);
    if (d != std::floor(d) || std::fabs(d) > 9e15) throw std::runtime_error("config: '" + k + "' must be an integer");
    return (int64_t) d;
}
std::string Json::string(const std::string & k, const std::string & def) const {
    if (!has(k)) return def;
    const Json & v = at(k);
    if (v.kind != Str) throw std::runtime_error("config: '" + k + "' must be a string");
    return v.str;
}

// ---- safetensors ----------------------------------------------------------------------------------------------
safetensors_file::~safetensors_file() {
    if (base) munmap((void *) base, size);
    if (fd >= 0) close(fd);
}

void safetensors_file::open(const std::string & path) {
    fd = ::open(path.c_str(), O_RDONLY);
    if (fd < 0) throw std::runtime_error("cannot open " + path);
    struct stat sb;
    if (fstat(fd, &sb) != 0 || sb.st_size < 8) throw std::runtime_error(path + ": too short for a safetensors file");
    size = (uint64_t) sb.st_size;
    void * p = mmap(nullptr, size, PROT_READ, MAP_PRIVATE, fd, 0);
    if (p == MAP_FAILED) { base = nullptr; throw std::runtime_error("mmap failed for " + path); }
    base = (const uint8_t *) p;
    uint64_t hn = 0;
    for (int k = 7; k >= 0; k--) hn = (hn << 8) | base[k];
    if (hn > size - 8) throw std::runtime_error(path + ": header length exceeds the file");
    const Json head = json_parse((const char *) base + 8, hn);
    if (head.kind != Json::Obj) throw std::runtime_error(path + ": header is not a JSON object");
    const uint64_t data0 = 8 + hn, avail = size - data0;
    for (const auto & kv : head.obj) {
        if (kv.first == "__metadata__") continue;
        st_tensor t;
        t.name = kv.first;
        const std::string dt = kv.second.string("dtype", "");
        t.dtype = dt == "BF16" ? ST_BF16 : dt == "F32" ? ST_F32 : dt == "F16" ? ST_F16 : dt == "I32" ? ST_I32 : ST_OTHER;
        for (const Json & d : kv.second.at("shape").arr) {
            if (d.kind != Json::Num || d.num < 0 || d.num != std::floor(d.num)) throw std::runtime_error(path + ": bad shape of " + t.name);
            t.shape.push_back((int64_t) d.num);
        }
        const Json & off = kv.second.at("data_offsets");
        if (off.kind != Json::Arr || off.arr.size() != 2) throw std::runtime_error(path + ": bad data_offsets of " + t.name);
        const double a = off.arr[0].num, b = off.arr[1].num;
        if (!(a >= 0 && b >= a && b <= (double) avail)) throw std::runtime_error(path + ": tensor " + t.name + " lies outside the file");
        t.data = base + data0 + (uint64_t) a;
        t.nbytes = (uint64_t) b - (uint64_t) a;
        const uint64_t esz = t.dtype == ST_F32 || t.dtype == ST_I32 ? 4 : t.dtype == ST_OTHER ? 0 : 2;
        if (esz && (uint64_t) t.numel() * esz != t.nbytes) throw std::runtime_error(path + ": tensor " + t.name + " has a size that does not fit its shape");
        tensors[t.name] = std::move(t);
    }
}

const st_tensor * safetensors_file::find(const std::string & name) const {
    auto it = tensors.find(name);
    return it == tensors.end() ? nullptr : &it->second;
}

static float half_to_float(uint16_t h) {
    const uint32_t s = (uint32_t) (h & 0x8000) << 16, e = (h >> 10) & 0x1F, m = h & 0x3FF;
    uint32_t u;
    if (e == 0) {
        if (m == 0) u = s;
        else { int sh = 0; uint32_t mm = m; while (!(mm & 0x400)) { mm <<= 1; sh++; } u = s | ((uint32_t) (113 - sh) << 23) | ((mm & 0x3FF) << 13); }
    } else if (e == 31) u = s | 0x7F800000u | (m << 13);
    else u = s | ((e + 112) << 23) | (m << 13);
    float f; std::memcpy(&f, &u, 4); return f;
}

std::vector<float> safetensors_file::read_f32(const std::string & name, const std::vector<int64_t> & shape) const {
    const st_tensor * t = find(name);
    if (!t) throw std::runtime_error("missing tensor " + name);
    if (t->shape != shape) {
        std::string have, want;
        for (int64_t d : t->shape) have += std::to_string(d) + " ";
        for (int64_t d : shape) want += std::to_string(d) + " ";
        throw std::runtime_error("tensor " + name + " has shape [ " + have + "], expected [ " + want + "]");
    }
    const int64_t n = t->numel();
    std::vector<float> out((size_t) n);
    if (t->dtype == ST_F32) std::memcpy(out.data(), t->data, (size_t) n * 4);
    else if (t->dtype == ST_BF16) {
        for (int64_t i = 0; i < n; i++) { uint16_t h; std::memcpy(&h, t->data + 2 * i, 2); const uint32_t u = (uint32_t) h << 16; std::memcpy(&out[(size_t) i], &u, 4); }
    } else if (t->dtype == ST_F16) {
        for (int64_t i = 0; i < n; i++) { uint16_t h; std::memcpy(&h, t->data + 2 * i, 2); out[(size_t) i] = half_to_float(h); }
    } else throw std::runtime_error("tensor " + name + " is not a floating-point tensor");
    return out;
}

bool is_model_dir(const std::string & path, std::string * dir_out) {
    struct stat sb;
    if (stat(path.c_str(), &sb) != 0) return false;
    std::string dir = path;
    if (!S_ISDIR(sb.st_mode)) {
        const size_t sl = path.find_last_of('/');
        const std::string file = sl == std::string::npos ? path : path.substr(sl + 1);
        if (file != "config.json") return false;
        dir = sl == std::string::npos ? "." : path.substr(0, sl);
    }
    if (stat((dir + "/config.json").c_str(), &sb) != 0) return false;
    if (dir_out) *dir_out = dir;
    return true;
}

}  // namespace b200
