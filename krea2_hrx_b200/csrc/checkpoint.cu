// Reading a ComfyUI int8 ConvRot checkpoint into the resident weights block:
//   krea2_checkpoint_*            (src/checkpoint/file.rs: Checkpoint::{open, has, get, names, block_count})
//   krea2_checkpoint_plan/_span.. (src/checkpoint/plan.rs: Plan::for_checkpoint, operand, vector)
//   krea2_weights_load_checkpoint (src/session/weights.rs: Weights::{plan, load, upload})
// Host code only.  The safetensors container itself is read by a dependency of the reference
// that is not part of its tree (hrx-rs 0.12.0, `hrx::artifacts::safetensors`); the format is
// public: an 8-byte little-endian header length, a JSON object mapping tensor names to
// {dtype, shape, data_offsets} (plus an optional "__metadata__" object of strings), then the
// tensor bytes, offsets relative to the end of the header.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cerrno>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "common.cuh"

using namespace krea2;

namespace {

struct Entry {
    std::string dtype;
    std::vector<size_t> shape;
    size_t begin = 0, end = 0;  // within the data section
};

// Rows to copy from one checkpoint tensor, in order (plan.rs:14-21).
struct Segment {
    std::string tensor;
    size_t row_begin = 0, row_end = 0;
};

// One destination on the device (plan.rs:23-43).
struct PlanSpan {
    size_t device_offset = 0, device_bytes = 0, rows = 0, row_bytes = 0, device_row_bytes = 0;
    std::vector<Segment> segments;
    std::vector<uint8_t> host;  // bytes assembled on the host instead: the gathered f32 scale vectors
    size_t file_bytes() const { return host.empty() ? rows * row_bytes : host.size(); }
};

struct Plan {
    std::map<std::string, PlanSpan> spans;  // byte-wise name order, as the reference's BTreeMap
    std::vector<const std::string *> order;
    size_t total_bytes = 0, layers = 0;
    bool built = false;
};

}  // namespace

struct krea2_checkpoint {
    std::string path;
    const uint8_t *map = nullptr;
    size_t file_bytes = 0, data_start = 0;
    std::map<std::string, Entry> entries;  // under unwrapped names
    std::vector<const std::string *> names;
    Plan plan;
    ~krea2_checkpoint() {
        if (map) munmap(const_cast<uint8_t *>(map), file_bytes);
    }
    const uint8_t *bytes(const Entry &e) const { return map + data_start + e.begin; }
};

namespace {

// ---------------------------------------------------------------- a small JSON reader
struct Json {
    enum Kind { Null, Bool, Number, String, Array, Object } kind = Null;
    double number = 0;
    bool integral = false;
    uint64_t integer = 0;
    std::string text;
    std::vector<Json> items;
    std::vector<std::pair<std::string, Json>> members;
};

struct Parser {
    const char *p, *end;
    std::string error;
    bool fail_at(const char *what) {
        if (error.empty()) error = what;
        return false;
    }
    void space() {
        while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) p++;
    }
    // Four hex digits after the 'u' that p points at; leaves p on the last digit.
    bool hex4(unsigned &code) {
        if (end - p < 5) return fail_at("short \\u escape in the header");
        code = 0;
        for (int i = 1; i <= 4; i++) {
            const char c = p[i];
            code = code * 16 + (c >= '0' && c <= '9' ? c - '0' : c >= 'a' && c <= 'f' ? c - 'a' + 10
                                : c >= 'A' && c <= 'F' ? c - 'A' + 10 : 0x10000);
        }
        if (code > 0xffff) return fail_at("bad \\u escape in the header");
        p += 4;
        return true;
    }
    bool string(std::string &out) {
        if (p >= end || *p != '"') return fail_at("a string was expected in the header");
        p++;
        while (p < end && *p != '"') {
            if (*p == '\\') {
                if (++p >= end) return fail_at("unterminated escape in the header");
                switch (*p) {
                    case '"': out += '"'; break;
                    case '\\': out += '\\'; break;
                    case '/': out += '/'; break;
                    case 'b': out += '\b'; break;
                    case 'f': out += '\f'; break;
                    case 'n': out += '\n'; break;
                    case 'r': out += '\r'; break;
                    case 't': out += '\t'; break;
                    case 'u': {
                        unsigned code = 0;
                        if (!hex4(code)) return false;
                        if (code >= 0xdc00 && code <= 0xdfff) return fail_at("lone surrogate in the header");
                        if (code >= 0xd800 && code <= 0xdbff) {  // a pair encodes one character above U+FFFF
                            unsigned low = 0;
                            if (end - p < 3 || p[1] != '\\' || p[2] != 'u') return fail_at("lone surrogate in the header");
                            p += 2;
                            if (!hex4(low)) return false;
                            if (low < 0xdc00 || low > 0xdfff) return fail_at("lone surrogate in the header");
                            code = 0x10000 + ((code - 0xd800) << 10) + (low - 0xdc00);
                        }
                        if (code < 0x80) out += static_cast<char>(code);
                        else if (code < 0x800) {
                            out += static_cast<char>(0xc0 | (code >> 6));
                            out += static_cast<char>(0x80 | (code & 0x3f));
                        } else if (code < 0x10000) {
                            out += static_cast<char>(0xe0 | (code >> 12));
                            out += static_cast<char>(0x80 | ((code >> 6) & 0x3f));
                            out += static_cast<char>(0x80 | (code & 0x3f));
                        } else {
                            out += static_cast<char>(0xf0 | (code >> 18));
                            out += static_cast<char>(0x80 | ((code >> 12) & 0x3f));
                            out += static_cast<char>(0x80 | ((code >> 6) & 0x3f));
                            out += static_cast<char>(0x80 | (code & 0x3f));
                        }
                        break;
                    }
                    default: return fail_at("unknown escape in the header");
                }
                p++;
            } else {
                if (static_cast<unsigned char>(*p) < 0x20) return fail_at("control character in a header string");
                out += *p++;
            }
        }
        if (p >= end) return fail_at("unterminated string in the header");
        p++;
        return true;
    }
    bool value(Json &out, int depth) {
        if (depth > 16) return fail_at("the header nests too deeply");
        space();
        if (p >= end) return fail_at("the header ends early");
        if (*p == '{') {
            out.kind = Json::Object;
            p++;
            space();
            if (p < end && *p == '}') return p++, true;
            for (;;) {
                space();
                std::string key;
                if (!string(key)) return false;
                space();
                if (p >= end || *p != ':') return fail_at("':' was expected in the header");
                p++;
                Json member;
                if (!value(member, depth + 1)) return false;
                out.members.emplace_back(std::move(key), std::move(member));
                space();
                if (p < end && *p == ',') { p++; continue; }
                if (p < end && *p == '}') return p++, true;
                return fail_at("',' or '}' was expected in the header");
            }
        }
        if (*p == '[') {
            out.kind = Json::Array;
            p++;
            space();
            if (p < end && *p == ']') return p++, true;
            for (;;) {
                Json item;
                if (!value(item, depth + 1)) return false;
                out.items.push_back(std::move(item));
                space();
                if (p < end && *p == ',') { p++; continue; }
                if (p < end && *p == ']') return p++, true;
                return fail_at("',' or ']' was expected in the header");
            }
        }
        if (*p == '"') {
            out.kind = Json::String;
            return string(out.text);
        }
        if (end - p >= 4 && std::strncmp(p, "true", 4) == 0) return out.kind = Json::Bool, out.integer = 1, p += 4, true;
        if (end - p >= 5 && std::strncmp(p, "false", 5) == 0) return out.kind = Json::Bool, p += 5, true;
        if (end - p >= 4 && std::strncmp(p, "null", 4) == 0) return p += 4, true;
        const char *start = p;
        bool digits_only = true;
        uint64_t integer = 0;
        bool overflow = false;
        while (p < end && (std::strchr("+-.eE", *p) || (*p >= '0' && *p <= '9'))) {
            if (*p >= '0' && *p <= '9') {
                const uint64_t next = integer * 10 + static_cast<uint64_t>(*p - '0');
                if (next / 10 != integer) overflow = true;
                integer = next;
            } else {
                digits_only = false;
            }
            p++;
        }
        if (p == start) return fail_at("unexpected character in the header");
        out.kind = Json::Number;
        out.integral = digits_only && !overflow;
        out.integer = integer;
        out.number = std::strtod(std::string(start, p).c_str(), nullptr);
        return true;
    }
};

// Whether the bytes are well-formed UTF-8 (no overlong forms, no surrogates, nothing above U+10FFFF):
// JSON text is UTF-8, and tensor names leave this library as C strings.
bool valid_utf8(const uint8_t *p, const uint8_t *end) {
    while (p < end) {
        const uint8_t lead = *p++;
        if (lead < 0x80) continue;
        int tail;
        uint32_t code, least;
        if ((lead & 0xe0) == 0xc0) tail = 1, code = lead & 0x1f, least = 0x80;
        else if ((lead & 0xf0) == 0xe0) tail = 2, code = lead & 0x0f, least = 0x800;
        else if ((lead & 0xf8) == 0xf0) tail = 3, code = lead & 0x07, least = 0x10000;
        else return false;
        if (end - p < tail) return false;
        for (int i = 0; i < tail; i++) {
            if ((*p & 0xc0) != 0x80) return false;
            code = (code << 6) | (*p++ & 0x3f);
        }
        if (code < least || code > 0x10ffff || (code >= 0xd800 && code <= 0xdfff)) return false;
    }
    return true;
}

size_t dtype_bytes(const std::string &dtype) {
    static const std::pair<const char *, size_t> kTable[] = {
        {"BOOL", 1}, {"U8", 1}, {"I8", 1}, {"F8_E5M2", 1}, {"F8_E4M3", 1}, {"I16", 2}, {"U16", 2}, {"F16", 2},
        {"BF16", 2}, {"I32", 4}, {"U32", 4}, {"F32", 4}, {"F64", 8}, {"I64", 8}, {"U64", 8}};
    for (const auto &row : kTable)
        if (dtype == row.first) return row.second;
    return 0;
}

int unreadable(const std::string &path, const std::string &why) {
    return fail(KREA2_INVALID_ARGUMENT, "cannot read %s: %s", path.c_str(), why.c_str());
}

// A tensor every transformer checkpoint carries, whatever wraps its names (file.rs:39-57): the
// prefix before it is removed when every tensor shares it.
constexpr const char *kAnchor = "blocks.0.attn.wq.weight";

void unwrap_model(std::map<std::string, Entry> &entries) {
    const size_t anchor = std::strlen(kAnchor);
    std::string prefix;
    for (const auto &e : entries) {
        const std::string &name = e.first;
        if (name.size() >= anchor && name.compare(name.size() - anchor, anchor, kAnchor) == 0) {
            prefix = name.substr(0, name.size() - anchor);
            break;
        }
    }
    if (prefix.empty() || prefix.back() != '.') return;
    for (const auto &e : entries)
        if (e.first.compare(0, prefix.size(), prefix) != 0) return;
    std::map<std::string, Entry> renamed;
    for (auto &e : entries) renamed.emplace(e.first.substr(prefix.size()), std::move(e.second));
    entries.swap(renamed);
}

int read_header(krea2_checkpoint &c) {
    if (c.file_bytes < 8) return unreadable(c.path, "the file is shorter than a header length");
    uint64_t header_bytes = 0;
    for (int i = 7; i >= 0; i--) header_bytes = (header_bytes << 8) | c.map[i];
    if (header_bytes > c.file_bytes - 8) return unreadable(c.path, "the header is longer than the file");
    c.data_start = 8 + static_cast<size_t>(header_bytes);
    const size_t data_bytes = c.file_bytes - c.data_start;
    if (!valid_utf8(c.map + 8, c.map + c.data_start)) return unreadable(c.path, "the header is not UTF-8");
    Parser parser{reinterpret_cast<const char *>(c.map + 8), reinterpret_cast<const char *>(c.map + c.data_start), {}};
    Json root;
    if (!parser.value(root, 0)) return unreadable(c.path, parser.error);
    parser.space();
    if (parser.p != parser.end) return unreadable(c.path, "text follows the header object");
    if (root.kind != Json::Object) return unreadable(c.path, "the header is not an object");
    for (auto &member : root.members) {
        if (member.first == "__metadata__") continue;  // not a tensor
        const Json &t = member.second;
        if (t.kind != Json::Object) return unreadable(c.path, "tensor " + member.first + " is not an object");
        Entry entry;
        bool have_dtype = false, have_shape = false, have_offsets = false;
        for (const auto &field : t.members) {
            const Json &v = field.second;
            if (field.first == "dtype" && v.kind == Json::String) {
                entry.dtype = v.text;
                have_dtype = true;
            } else if (field.first == "shape" && v.kind == Json::Array) {
                for (const Json &d : v.items) {
                    if (d.kind != Json::Number || !d.integral) return unreadable(c.path, "bad shape of " + member.first);
                    entry.shape.push_back(static_cast<size_t>(d.integer));
                }
                have_shape = true;
            } else if (field.first == "data_offsets" && v.kind == Json::Array && v.items.size() == 2 &&
                       v.items[0].integral && v.items[1].integral) {
                entry.begin = static_cast<size_t>(v.items[0].integer);
                entry.end = static_cast<size_t>(v.items[1].integer);
                have_offsets = true;
            }
        }
        if (!have_dtype || !have_shape || !have_offsets)
            return unreadable(c.path, "tensor " + member.first + " lacks dtype, shape or data_offsets");
        const size_t element = dtype_bytes(entry.dtype);
        if (element == 0) return unreadable(c.path, "tensor " + member.first + " has unknown dtype " + entry.dtype);
        if (entry.begin > entry.end || entry.end > data_bytes)
            return unreadable(c.path, "tensor " + member.first + " reaches past the data");
        size_t count = 1;
        for (size_t d : entry.shape) {
            if (d != 0 && count > SIZE_MAX / d) return unreadable(c.path, "shape of " + member.first + " overflows");
            count *= d;
        }
        if (count > SIZE_MAX / element || count * element != entry.end - entry.begin)
            return unreadable(c.path, "tensor " + member.first + " does not fill its data span");
        if (!c.entries.emplace(member.first, std::move(entry)).second)
            return unreadable(c.path, "tensor " + member.first + " appears twice");
    }
    unwrap_model(c.entries);
    for (const auto &e : c.entries) c.names.push_back(&e.first);
    return KREA2_OK;
}

const Entry *find(const krea2_checkpoint &c, const std::string &name) {
    auto it = c.entries.find(name);
    return it == c.entries.end() ? nullptr : &it->second;
}

int get(const krea2_checkpoint &c, const std::string &name, const Entry **out) {
    *out = find(c, name);
    if (!*out) return fail(KREA2_INVALID_ARGUMENT, "missing tensor %s in %s", name.c_str(), c.path.c_str());
    return KREA2_OK;
}

size_t block_count(const krea2_checkpoint &c) {
    size_t n = 0;
    while (n < c.entries.size() && find(c, "blocks." + std::to_string(n) + ".attn.wq.weight")) n++;
    return n;
}

// ---------------------------------------------------------------- the plan (plan.rs)
int row_bytes_of(const Entry &t, size_t *out) {  // file.rs:30-37
    KREA2_REQUIRE(!t.shape.empty(), "a tensor with no shape");
    const size_t rows = t.shape[0], bytes = t.end - t.begin;
    KREA2_REQUIRE(rows != 0 && bytes % rows == 0, "tensor size is not a whole number of rows");
    *out = bytes / rows;
    return KREA2_OK;
}

int int8_rows(const krea2_checkpoint &c, const std::string &name, const Entry **out) {  // plan.rs:59-72
    if (int s = get(c, name + ".weight", out)) return s;
    const Entry &t = **out;
    if (t.dtype != "I8" || t.shape.size() != 2)
        return fail(KREA2_INVALID_ARGUMENT, "%s.weight is %s, not int8 ConvRot rows (%s)", name.c_str(), t.dtype.c_str(),
                    c.path.c_str());
    size_t row = 0;
    if (t.shape[0] == 0 || t.shape[1] == 0 || row_bytes_of(t, &row) != KREA2_OK || row != t.shape[1])
        return fail(KREA2_INVALID_ARGUMENT, "invalid weight shape or size in %s", name.c_str());
    return KREA2_OK;
}

int scales_of(const krea2_checkpoint &c, const std::string &name, size_t rows, const Entry **out) {  // plan.rs:74-83
    if (int s = get(c, name + ".weight_scale", out)) return s;
    KREA2_REQUIRE((*out)->dtype == "F32", "%s.weight_scale is not float32", name.c_str());
    KREA2_REQUIRE((*out)->end - (*out)->begin == rows * 4, "scale count in %s", name.c_str());
    return KREA2_OK;
}

// One GEMM operand and its scale vector (plan.rs:150-232): `group` 0 concatenates the parts' rows,
// `group` n interleaves them n rows at a time.
int operand(const krea2_checkpoint &c, const std::string &out, const std::vector<std::string> &parts, size_t group,
            PlanSpan *weights, PlanSpan *scales) {
    std::vector<const Entry *> tensors(parts.size());
    for (size_t i = 0; i < parts.size(); i++)
        if (int s = int8_rows(c, parts[i], &tensors[i])) return s;
    size_t row_bytes = 0;
    if (int s = row_bytes_of(*tensors[0], &row_bytes)) return s;
    size_t rows = 0;
    for (const Entry *t : tensors) {
        KREA2_REQUIRE(t->shape[1] == tensors[0]->shape[1], "mismatched K in %s", out.c_str());
        rows += t->shape[0];
    }
    const size_t pitch = krea2_shape_gemm_pitch(row_bytes);
    KREA2_REQUIRE(pitch != 0 && rows <= SIZE_MAX / pitch, "%s spans more than the address space", out.c_str());
    weights->device_bytes = rows * pitch;
    weights->rows = rows, weights->row_bytes = row_bytes, weights->device_row_bytes = pitch;
    scales->host.assign(rows * 4, 0);
    size_t written = 0;
    if (group == 0) {
        for (size_t i = 0; i < parts.size(); i++) {
            const size_t count = tensors[i]->shape[0];
            weights->segments.push_back({parts[i] + ".weight", 0, count});
            const Entry *source = nullptr;
            if (int s = scales_of(c, parts[i], count, &source)) return s;
            std::memcpy(scales->host.data() + written * 4, c.bytes(*source), count * 4);
            written += count;
        }
    } else {
        KREA2_REQUIRE(tensors.size() == 2 && tensors[0]->shape[0] == tensors[1]->shape[0] && tensors[0]->shape[0] % group == 0,
                      "interleave shape in %s", out.c_str());
        const Entry *sources[2] = {nullptr, nullptr};
        for (size_t i = 0; i < 2; i++)
            if (int s = scales_of(c, parts[i], tensors[0]->shape[0], &sources[i])) return s;
        for (size_t start = 0; start < tensors[0]->shape[0]; start += group)
            for (size_t i = 0; i < 2; i++) {
                weights->segments.push_back({parts[i] + ".weight", start, start + group});
                std::memcpy(scales->host.data() + written * 4, c.bytes(*sources[i]) + start * 4, group * 4);
                written += group;
            }
    }
    scales->device_bytes = scales->host.size();
    return KREA2_OK;
}

// An f32 vector: copied as it is, or upcast exactly from bf16 (plan.rs:234-268).
int vector_span(const krea2_checkpoint &c, const std::string &name, PlanSpan *span) {
    const Entry *t = nullptr;
    if (int s = get(c, name, &t)) return s;
    const size_t bytes = t->end - t->begin;
    if (t->dtype == "BF16") {
        span->host.resize(bytes * 2);
        const uint8_t *src = c.bytes(*t);
        for (size_t i = 0; i < bytes / 2; i++) {
            span->host[4 * i] = 0, span->host[4 * i + 1] = 0;
            span->host[4 * i + 2] = src[2 * i], span->host[4 * i + 3] = src[2 * i + 1];
        }
        span->device_bytes = span->host.size();
        return KREA2_OK;
    }
    KREA2_REQUIRE(t->dtype == "F32", "%s is %s, not float32", name.c_str(), t->dtype.c_str());
    span->device_bytes = bytes;
    span->rows = 1, span->row_bytes = bytes, span->device_row_bytes = bytes;
    span->segments.push_back({name, 0, 1});
    return KREA2_OK;
}

int build_plan(krea2_checkpoint &c) {  // plan.rs:85-144
    if (c.plan.built) return KREA2_OK;
    Plan plan;
    plan.layers = block_count(c);
    KREA2_REQUIRE(plan.layers != 0, "no transformer blocks in %s", c.path.c_str());
    for (size_t block = 0; block < plan.layers; block++) {
        const std::string p = "blocks." + std::to_string(block);
        PlanSpan q, s;
        if (int st = operand(c, p + ".qkvg", {p + ".attn.wq", p + ".attn.wk", p + ".attn.wv", p + ".attn.gate"}, 0, &q, &s))
            return st;
        plan.spans[p + ".qkvg.q"] = std::move(q);
        plan.spans[p + ".qkvg.s"] = std::move(s);
        const std::pair<const char *, std::string> single[2] = {{"wo", p + ".attn.wo"}, {"down", p + ".mlp.down"}};
        for (const auto &item : single) {
            PlanSpan wq, ws;
            if (int st = operand(c, p + "." + item.first, {item.second}, 0, &wq, &ws)) return st;
            plan.spans[p + "." + item.first + ".q"] = std::move(wq);
            plan.spans[p + "." + item.first + ".s"] = std::move(ws);
        }
        PlanSpan gq, gs;
        if (int st = operand(c, p + ".gu", {p + ".mlp.gate", p + ".mlp.up"}, 16, &gq, &gs)) return st;
        plan.spans[p + ".gu.q"] = std::move(gq);
        plan.spans[p + ".gu.s"] = std::move(gs);
        const std::pair<const char *, std::string> vectors[4] = {{"prenorm", p + ".prenorm.scale"},
                                                                 {"postnorm", p + ".postnorm.scale"},
                                                                 {"qnorm", p + ".attn.qknorm.qnorm.scale"},
                                                                 {"knorm", p + ".attn.qknorm.knorm.scale"}};
        for (const auto &item : vectors) {
            PlanSpan v;
            if (int st = vector_span(c, item.second, &v)) return st;
            plan.spans[p + "." + item.first] = std::move(v);
        }
    }
    // Tensors start at 256-byte boundaries in name order; sessions use these offsets.
    size_t total = 0;
    for (auto &entry : plan.spans) {
        entry.second.device_offset = total;
        total += (entry.second.device_bytes + 255) / 256 * 256;
        plan.order.push_back(&entry.first);
    }
    plan.total_bytes = total;
    plan.built = true;
    c.plan = std::move(plan);
    c.plan.order.clear();
    for (auto &entry : c.plan.spans) c.plan.order.push_back(&entry.first);
    return KREA2_OK;
}

int find_span(const krea2_checkpoint &c, const char *name, const PlanSpan **out) {
    auto it = c.plan.spans.find(name);
    if (it == c.plan.spans.end()) return fail(KREA2_INVALID_ARGUMENT, "no span named %s", name);
    *out = &it->second;
    return KREA2_OK;
}

// The device image of a span: rows at the device pitch with zero padding, or the host-assembled
// bytes (src/session/weights.rs:47-98 without the bounded staging).
int assemble(const krea2_checkpoint &c, const PlanSpan &span, uint8_t *out) {
    if (!span.host.empty()) {
        std::memcpy(out, span.host.data(), span.host.size());
        return KREA2_OK;
    }
    const size_t pitch = span.rows > 0 ? span.device_row_bytes : span.row_bytes, width = span.row_bytes;
    std::memset(out, 0, span.device_bytes);
    size_t row_out = 0;
    for (const Segment &segment : span.segments) {
        const Entry *t = nullptr;
        if (int s = get(c, segment.tensor, &t)) return s;
        const uint8_t *src = c.bytes(*t);
        KREA2_REQUIRE(segment.row_end * width <= t->end - t->begin, "segment of %s reaches past its tensor",
                      segment.tensor.c_str());
        for (size_t row = segment.row_begin; row < segment.row_end; row++, row_out++)
            std::memcpy(out + row_out * pitch, src + row * width, width);
    }
    return KREA2_OK;
}

}  // namespace

// ---------------------------------------------------------------- C entry points
extern "C" int krea2_checkpoint_open(const char *path, krea2_checkpoint **out) {
    clear_error();
    KREA2_REQUIRE(path && out, "checkpoint_open: null argument");
    const std::string name(path);
    const size_t dot = name.rfind('.'), slash = name.rfind('/');
    const bool has_extension = dot != std::string::npos && (slash == std::string::npos || dot > slash + 1);
    if (!has_extension || name.substr(dot + 1) != "safetensors")
        return fail(KREA2_INVALID_ARGUMENT, "%s is not a ComfyUI checkpoint (.safetensors)", path);
    std::unique_ptr<krea2_checkpoint> c(new krea2_checkpoint);
    c->path = name;
    const int fd = open(path, O_RDONLY);
    if (fd < 0) return unreadable(name, std::strerror(errno));
    struct stat info {};
    if (fstat(fd, &info) != 0 || info.st_size < 0) {
        const std::string why = std::strerror(errno);
        close(fd);
        return unreadable(name, why);
    }
    c->file_bytes = static_cast<size_t>(info.st_size);
    if (c->file_bytes == 0) {
        close(fd);
        return unreadable(name, "the file is empty");
    }
    void *map = mmap(nullptr, c->file_bytes, PROT_READ, MAP_PRIVATE, fd, 0);
    const std::string why = std::strerror(errno);
    close(fd);
    if (map == MAP_FAILED) return unreadable(name, why);
    c->map = static_cast<const uint8_t *>(map);
    if (int s = read_header(*c)) return s;
    *out = c.release();
    return KREA2_OK;
}

extern "C" void krea2_checkpoint_close(krea2_checkpoint *checkpoint) { delete checkpoint; }

extern "C" int krea2_checkpoint_has(const krea2_checkpoint *c, const char *name) {
    return c && name && find(*c, name) ? 1 : 0;
}

extern "C" size_t krea2_checkpoint_block_count(const krea2_checkpoint *c) { return c ? block_count(*c) : 0; }

extern "C" size_t krea2_checkpoint_names(const krea2_checkpoint *c, const char **names, size_t capacity) {
    if (!c) return 0;
    for (size_t i = 0; names && i < c->names.size() && i < capacity; i++) names[i] = c->names[i]->c_str();
    return c->names.size();
}

extern "C" int krea2_checkpoint_tensor(const krea2_checkpoint *c, const char *name, const char **dtype,
                                       const size_t **shape, size_t *rank, const void **bytes, size_t *byte_count) {
    clear_error();
    KREA2_REQUIRE(c && name, "checkpoint_tensor: null argument");
    const Entry *entry = nullptr;
    if (int s = get(*c, name, &entry)) return s;
    if (dtype) *dtype = entry->dtype.c_str();
    if (shape) *shape = entry->shape.data();
    if (rank) *rank = entry->shape.size();
    if (bytes) *bytes = c->bytes(*entry);
    if (byte_count) *byte_count = entry->end - entry->begin;
    return KREA2_OK;
}

extern "C" int krea2_checkpoint_plan(krea2_checkpoint *c, size_t *total_bytes, size_t *layers, size_t *span_count) {
    clear_error();
    KREA2_REQUIRE(c, "checkpoint_plan: null checkpoint");
    if (int s = build_plan(*c)) return s;
    if (total_bytes) *total_bytes = c->plan.total_bytes;
    if (layers) *layers = c->plan.layers;
    if (span_count) *span_count = c->plan.spans.size();
    return KREA2_OK;
}

extern "C" int krea2_checkpoint_span_name(krea2_checkpoint *c, size_t index, const char **name) {
    clear_error();
    KREA2_REQUIRE(c && name, "checkpoint_span_name: null argument");
    if (int s = build_plan(*c)) return s;
    KREA2_REQUIRE(index < c->plan.order.size(), "span index %zu of %zu", index, c->plan.order.size());
    *name = c->plan.order[index]->c_str();
    return KREA2_OK;
}

extern "C" int krea2_checkpoint_span(krea2_checkpoint *c, const char *name, krea2_span_info *info) {
    clear_error();
    KREA2_REQUIRE(c && name && info, "checkpoint_span: null argument");
    if (int s = build_plan(*c)) return s;
    const PlanSpan *span = nullptr;
    if (int s = find_span(*c, name, &span)) return s;
    info->device_offset = span->device_offset, info->device_bytes = span->device_bytes;
    info->rows = span->rows, info->row_bytes = span->row_bytes, info->device_row_bytes = span->device_row_bytes;
    info->segments = span->segments.size(), info->file_bytes = span->file_bytes();
    return KREA2_OK;
}

extern "C" int krea2_checkpoint_segment(krea2_checkpoint *c, const char *span_name, size_t index, const char **tensor,
                                        size_t *row_begin, size_t *row_end) {
    clear_error();
    KREA2_REQUIRE(c && span_name && tensor && row_begin && row_end, "checkpoint_segment: null argument");
    if (int s = build_plan(*c)) return s;
    const PlanSpan *span = nullptr;
    if (int s = find_span(*c, span_name, &span)) return s;
    KREA2_REQUIRE(index < span->segments.size(), "segment index %zu of %zu", index, span->segments.size());
    *tensor = span->segments[index].tensor.c_str();
    *row_begin = span->segments[index].row_begin, *row_end = span->segments[index].row_end;
    return KREA2_OK;
}

extern "C" int krea2_checkpoint_assemble(krea2_checkpoint *c, const char *span_name, void *host_bytes, size_t bytes) {
    clear_error();
    KREA2_REQUIRE(c && span_name && host_bytes, "checkpoint_assemble: null argument");
    if (int s = build_plan(*c)) return s;
    const PlanSpan *span = nullptr;
    if (int s = find_span(*c, span_name, &span)) return s;
    KREA2_REQUIRE(bytes == span->device_bytes, "%s spans %zu bytes on the device, got %zu", span_name, span->device_bytes,
                  bytes);
    return assemble(*c, *span, static_cast<uint8_t *>(host_bytes));
}

extern "C" int krea2_checkpoint_dims(krea2_checkpoint *c, krea2_dims *dims, size_t *layers) {
    clear_error();
    KREA2_REQUIRE(c && dims, "checkpoint_dims: null argument");
    if (int s = build_plan(*c)) return s;
    const Entry *wq = nullptr, *wk = nullptr, *gate = nullptr;
    if (int s = get(*c, "blocks.0.attn.wq.weight", &wq)) return s;
    if (int s = get(*c, "blocks.0.attn.wk.weight", &wk)) return s;
    if (int s = get(*c, "blocks.0.mlp.gate.weight", &gate)) return s;
    const PlanSpan *qnorm = nullptr;
    if (int s = find_span(*c, "blocks.0.qnorm", &qnorm)) return s;
    dims->hidden = wq->shape[1];
    dims->head_dim = qnorm->device_bytes / 4;
    KREA2_REQUIRE(dims->head_dim != 0 && wk->shape[0] % dims->head_dim == 0, "key rows are not whole heads in %s",
                  c->path.c_str());
    dims->kv_heads = wk->shape[0] / dims->head_dim;
    dims->inter = gate->shape[0];
    if (layers) *layers = c->plan.layers;
    return KREA2_OK;
}

// Session::validate (src/session/mod.rs:249-261): the session dimensions, then the checkpoint's header
// and layout.  Host work only: a refusal costs nothing and leaves the driver library unloaded.
extern "C" int krea2_session_validate(const char *checkpoint_path, size_t tokens, size_t layers) {
    clear_error();
    if (int s = krea2_session_validate_dimensions(tokens, layers)) return s;
    krea2_checkpoint *c = nullptr;
    if (int s = krea2_checkpoint_open(checkpoint_path, &c)) return s;
    const int status = build_plan(*c);
    delete c;
    return status;
}

// Weights::load (src/session/weights.rs:40-98): the plan of the file must be the plan the
// kernels' block shape implies (same names, offsets and extents); then every span is assembled at
// its device pitch and uploaded.
extern "C" int krea2_weights_load_checkpoint(krea2_checkpoint *c, krea2_stream stream, krea2_weights **out) {
    clear_error();
    KREA2_REQUIRE(c && out, "weights_load_checkpoint: null argument");
    krea2_dims dims{};
    size_t layers = 0;
    if (int s = krea2_checkpoint_dims(c, &dims, &layers)) return s;
    size_t planned = 0;
    if (int s = krea2_weights_plan_bytes(&dims, layers, &planned)) return s;
    KREA2_REQUIRE(planned == c->plan.total_bytes,
                  "%s lays out %zu bytes, the block shape it declares (hidden %zu, %zu kv heads of %zu, inter %zu) %zu",
                  c->path.c_str(), c->plan.total_bytes, dims.hidden, dims.kv_heads, dims.head_dim, dims.inter, planned);
    krea2_weights *weights = nullptr;
    if (int s = krea2_weights_create(&dims, layers, &weights)) return s;
    void *base = nullptr;
    size_t first_bytes = 0;
    int status = krea2_weights_locate(weights, c->plan.order.front()->c_str(), &base, &first_bytes);
    std::vector<uint8_t> staging;
    for (const auto &entry : c->plan.spans) {
        if (status) break;
        const PlanSpan &span = entry.second;
        void *ptr = nullptr;
        size_t bytes = 0;
        if ((status = krea2_weights_locate(weights, entry.first.c_str(), &ptr, &bytes))) break;
        if (bytes != span.device_bytes ||
            static_cast<size_t>(static_cast<uint8_t *>(ptr) - static_cast<uint8_t *>(base)) != span.device_offset) {
            status = fail(KREA2_INVALID_ARGUMENT, "%s: span %s does not have the extent the kernels expect", c->path.c_str(),
                          entry.first.c_str());
            break;
        }
        staging.resize(span.device_bytes);
        if ((status = assemble(*c, span, staging.data()))) break;
        if ((status = krea2_weights_upload(weights, entry.first.c_str(), staging.data(), staging.size(), stream))) break;
        // The staging vector is reused: the copy must have left it before the next span is assembled.
        cudaError_t sync = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
        if (sync != cudaSuccess) status = fail(KREA2_RUNTIME, "upload of %s failed: %s", entry.first.c_str(), cudaGetErrorString(sync));
    }
    if (status) {
        const std::string message = krea2_last_error();
        krea2_weights_release(weights);
        return fail(static_cast<krea2_status>(status), "%s", message.c_str());
    }
    *out = weights;
    return KREA2_OK;
}
