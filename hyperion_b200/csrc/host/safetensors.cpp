#include "safetensors.hpp"

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <utility>

#include "cache_index.hpp"  // Failure

namespace hb {
namespace {

constexpr int64_t MAX_HEADER_BYTES = 64ll << 20;
constexpr int MAX_DEPTH = 32;

[[noreturn]] void fail(const std::string& text) { throw Failure{BAD_FILE, text}; }

// ------------------------------------------------------------------ a small JSON reader
// Enough for a header: objects keep their members in order (so that a name that comes twice is seen), integers are
// kept exact, everything else a header may legally carry (metadata strings, reals, literals) is parsed and skipped.
struct Json {
    enum Kind { Null, Bool, Int, Real, String, Array, Object } kind = Null;
    bool boolean = false;
    long long integer = 0;
    std::string text;
    std::vector<Json> items;
    std::vector<std::pair<std::string, Json>> members;

    const Json* find(const char* key) const {
        for (const auto& member : members)
            if (member.first == key) return &member.second;
        return nullptr;
    }
};

class JsonReader {
  public:
    JsonReader(const char* data, size_t size) : p_(data), end_(data + size) {}

    Json document() {
        Json value = this->value(0);
        skip_space();
        if (p_ != end_) bad("text after the document");
        return value;
    }

  private:
    const char* p_;
    const char* end_;

    [[noreturn]] void bad(const char* what) const { fail(std::string("header is not JSON (") + what + ")"); }

    void skip_space() {
        while (p_ != end_ && (*p_ == ' ' || *p_ == '\t' || *p_ == '\n' || *p_ == '\r')) ++p_;
    }

    bool take(char c) {
        skip_space();
        if (p_ != end_ && *p_ == c) { ++p_; return true; }
        return false;
    }

    void literal(const char* word) {
        const size_t n = std::strlen(word);
        if ((size_t)(end_ - p_) < n || std::memcmp(p_, word, n) != 0) bad("unknown literal");
        p_ += n;
    }

    static void append_utf8(std::string& out, unsigned code) {
        if (code < 0x80) out += (char)code;
        else if (code < 0x800) { out += (char)(0xC0 | (code >> 6)); out += (char)(0x80 | (code & 0x3F)); }
        else if (code < 0x10000) { out += (char)(0xE0 | (code >> 12)); out += (char)(0x80 | ((code >> 6) & 0x3F)); out += (char)(0x80 | (code & 0x3F)); }
        else { out += (char)(0xF0 | (code >> 18)); out += (char)(0x80 | ((code >> 12) & 0x3F)); out += (char)(0x80 | ((code >> 6) & 0x3F)); out += (char)(0x80 | (code & 0x3F)); }
    }

    unsigned hex4() {
        if (end_ - p_ < 4) bad("short \\u escape");
        unsigned code = 0;
        for (int i = 0; i < 4; ++i) {
            const char c = *p_++;
            code <<= 4;
            if (c >= '0' && c <= '9') code |= (unsigned)(c - '0');
            else if (c >= 'a' && c <= 'f') code |= (unsigned)(c - 'a' + 10);
            else if (c >= 'A' && c <= 'F') code |= (unsigned)(c - 'A' + 10);
            else bad("bad \\u escape");
        }
        return code;
    }

    std::string string() {
        // the opening quote has been taken
        std::string out;
        while (true) {
            if (p_ == end_) bad("unterminated string");
            const unsigned char c = (unsigned char)*p_++;
            if (c == '"') return out;
            if (c < 0x20) bad("control character in a string");
            if (c != '\\') { out += (char)c; continue; }
            if (p_ == end_) bad("unterminated escape");
            const char e = *p_++;
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
                    unsigned code = hex4();
                    if (code >= 0xD800 && code < 0xDC00 && end_ - p_ >= 6 && p_[0] == '\\' && p_[1] == 'u') {
                        p_ += 2;
                        const unsigned low = hex4();
                        if (low >= 0xDC00 && low < 0xE000) code = 0x10000 + ((code - 0xD800) << 10) + (low - 0xDC00);
                        else bad("bad surrogate pair");
                    }
                    append_utf8(out, code);
                    break;
                }
                default: bad("unknown escape");
            }
        }
    }

    Json number() {
        const char* start = p_;
        if (p_ != end_ && *p_ == '-') ++p_;
        if (p_ == end_ || *p_ < '0' || *p_ > '9') bad("bad number");
        while (p_ != end_ && *p_ >= '0' && *p_ <= '9') ++p_;
        bool real = false;
        if (p_ != end_ && *p_ == '.') {
            real = true;
            ++p_;
            if (p_ == end_ || *p_ < '0' || *p_ > '9') bad("bad number");
            while (p_ != end_ && *p_ >= '0' && *p_ <= '9') ++p_;
        }
        if (p_ != end_ && (*p_ == 'e' || *p_ == 'E')) {
            real = true;
            ++p_;
            if (p_ != end_ && (*p_ == '+' || *p_ == '-')) ++p_;
            if (p_ == end_ || *p_ < '0' || *p_ > '9') bad("bad number");
            while (p_ != end_ && *p_ >= '0' && *p_ <= '9') ++p_;
        }
        Json value;
        if (real) { value.kind = Json::Real; return value; }
        // an integer: exact while it fits 63 bits, else kept as a real (no offset or extent is that large)
        const bool negative = *start == '-';
        unsigned long long magnitude = 0;
        for (const char* q = start + (negative ? 1 : 0); q != p_; ++q) {
            const unsigned digit = (unsigned)(*q - '0');
            if (magnitude > (0x7fffffffffffffffull - digit) / 10ull) { value.kind = Json::Real; return value; }
            magnitude = magnitude * 10ull + digit;
        }
        value.kind = Json::Int;
        value.integer = negative ? -(long long)magnitude : (long long)magnitude;
        return value;
    }

    Json value(int depth) {
        if (depth > MAX_DEPTH) bad("nested too deeply");
        skip_space();
        if (p_ == end_) bad("unexpected end");
        Json out;
        const char c = *p_;
        if (c == '{') {
            ++p_;
            out.kind = Json::Object;
            if (take('}')) return out;
            while (true) {
                if (!take('"')) bad("a member name was expected");
                std::string key = string();
                if (!take(':')) bad("':' was expected");
                out.members.emplace_back(std::move(key), value(depth + 1));
                if (take(',')) continue;
                if (take('}')) return out;
                bad("',' or '}' was expected");
            }
        }
        if (c == '[') {
            ++p_;
            out.kind = Json::Array;
            if (take(']')) return out;
            while (true) {
                out.items.push_back(value(depth + 1));
                if (take(',')) continue;
                if (take(']')) return out;
                bad("',' or ']' was expected");
            }
        }
        if (c == '"') { ++p_; out.kind = Json::String; out.text = string(); return out; }
        if (c == 't') { literal("true"); out.kind = Json::Bool; out.boolean = true; return out; }
        if (c == 'f') { literal("false"); out.kind = Json::Bool; return out; }
        if (c == 'n') { literal("null"); return out; }
        return number();
    }
};

std::string quoted(const std::string& name) { return "'" + name + "'"; }

std::string shape_text(const std::vector<int64_t>& shape) {
    std::string out = "[";
    for (size_t i = 0; i < shape.size(); ++i) out += (i ? ", " : "") + std::to_string(shape[i]);
    return out + "]";
}

struct FileCloser {
    std::FILE* file;
    ~FileCloser() { if (file) std::fclose(file); }
};

}  // namespace

int safetensors_element_size(const std::string& dtype) {
    static const std::pair<const char*, int> sizes[] = {{"BF16", 2}, {"F16", 2}, {"F32", 4}, {"F64", 8}, {"I8", 1},
                                                        {"U8", 1},   {"I16", 2}, {"I32", 4}, {"I64", 8}, {"BOOL", 1}};
    for (const auto& entry : sizes)
        if (dtype == entry.first) return entry.second;
    return 0;
}

TensorTable read_safetensors_header(const std::string& path) {
    FileCloser closer{std::fopen(path.c_str(), "rb")};
    if (!closer.file) fail("cannot be opened");
    if (std::fseek(closer.file, 0, SEEK_END) != 0) fail("cannot be read");
    const long long size = std::ftell(closer.file);
    if (size < 0 || std::fseek(closer.file, 0, SEEK_SET) != 0) fail("cannot be read");
    unsigned char prefix[8];
    if (std::fread(prefix, 1, 8, closer.file) != 8) fail("shorter than its 8-byte header length");
    unsigned long long header_len = 0;
    for (int i = 7; i >= 0; --i) header_len = (header_len << 8) | prefix[i];
    if (header_len > (unsigned long long)MAX_HEADER_BYTES || 8ull + header_len > (unsigned long long)size)
        fail("header length " + std::to_string(header_len) + " does not fit the file (" + std::to_string(size) + " bytes)");
    std::string text((size_t)header_len, '\0');
    if (header_len && std::fread(&text[0], 1, (size_t)header_len, closer.file) != (size_t)header_len) fail("cannot be read");

    const Json document = JsonReader(text.data(), text.size()).document();
    if (document.kind != Json::Object) fail("header must be a JSON object");

    TensorTable table;
    table.payload_start = 8 + (int64_t)header_len;
    table.payload_bytes = (int64_t)size - table.payload_start;
    std::vector<std::string> names;
    for (const auto& member : document.members) names.push_back(member.first);
    std::sort(names.begin(), names.end());
    for (size_t i = 1; i < names.size(); ++i)
        if (names[i] == names[i - 1]) fail("the header names " + quoted(names[i]) + " twice");

    for (const auto& member : document.members) {
        const std::string& name = member.first;
        if (name == "__metadata__") continue;
        const Json& meta = member.second;
        const Json* dtype = meta.kind == Json::Object ? meta.find("dtype") : nullptr;
        const Json* shape = meta.kind == Json::Object ? meta.find("shape") : nullptr;
        const Json* offsets = meta.kind == Json::Object ? meta.find("data_offsets") : nullptr;
        if (!dtype || !shape || !offsets || dtype->kind != Json::String || shape->kind != Json::Array || offsets->kind != Json::Array ||
            offsets->items.size() != 2 || offsets->items[0].kind != Json::Int || offsets->items[1].kind != Json::Int)
            fail("tensor " + quoted(name) + " lacks dtype, shape or data_offsets");
        TensorRecord record;
        record.name = name;
        record.dtype = dtype->text;
        const int element = safetensors_element_size(record.dtype);
        if (!element) fail("tensor " + quoted(name) + " has unsupported dtype " + quoted(record.dtype));
        bool shape_ok = true;
        for (const Json& extent : shape->items) {
            if (extent.kind != Json::Int || extent.integer < 0) { shape_ok = false; break; }
            record.shape.push_back(extent.integer);
        }
        if (!shape_ok) fail("tensor " + quoted(name) + " has a bad shape");
        record.begin = offsets->items[0].integer;
        record.end = offsets->items[1].integer;
        if (!(0 <= record.begin && record.begin <= record.end && record.end <= table.payload_bytes))
            fail("tensor " + quoted(name) + " range [" + std::to_string(record.begin) + ", " + std::to_string(record.end) +
                 ") lies outside the payload (" + std::to_string(table.payload_bytes) + " bytes)");
        // shape x element size, without overflow: more than the payload can hold is enough to know
        unsigned __int128 needed = (unsigned __int128)element;
        const bool empty = std::find(record.shape.begin(), record.shape.end(), (int64_t)0) != record.shape.end();
        for (int64_t extent : record.shape) {
            if (needed > ((unsigned __int128)1 << 64)) break;  // extents are below 2^63: the product stays inside 128 bits
            needed *= (unsigned __int128)extent;
        }
        if (empty) needed = 0;
        if (needed != (unsigned __int128)(record.end - record.begin)) {
            const std::string wanted = needed > ((unsigned __int128)1 << 62) ? std::string("more than 2^62") : std::to_string((unsigned long long)needed);
            fail("tensor " + quoted(name) + " holds " + std::to_string(record.end - record.begin) + " bytes but shape " + shape_text(record.shape) +
                 " of " + record.dtype + " needs " + wanted);
        }
        table.tensors.push_back(std::move(record));
    }
    std::vector<const TensorRecord*> ordered;
    for (const TensorRecord& record : table.tensors) ordered.push_back(&record);
    std::sort(ordered.begin(), ordered.end(), [](const TensorRecord* a, const TensorRecord* b) {
        return a->begin != b->begin ? a->begin < b->begin : a->end < b->end;
    });
    for (size_t i = 1; i < ordered.size(); ++i)
        if (ordered[i]->begin < ordered[i - 1]->end)
            fail("tensors " + quoted(ordered[i - 1]->name) + " and " + quoted(ordered[i]->name) + " overlap");
    return table;
}

}  // namespace hb
