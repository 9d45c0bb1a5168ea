// Weights in, images out: safetensors reader / writer, OpenEXR and PNG writers, the tone-mapping curve.
// Host code behind the C ABI of include/rfk_io.h; stands where the reference has src/io/safetensors.cpp and
// src/io/image_writer.cpp (BANANASJIM/renderformer-cuda). Written against the formats' specifications:
//   safetensors: u64 little-endian header length, JSON header, data section;
//   OpenEXR 2 single-part scan-line file, no compression, FLOAT channels;
//   PNG: signature, IHDR, one IDAT holding a zlib stream of filter-0 rows, IEND.
#include "rfk_io.h"

#include <cuda_runtime.h>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>
#include <zlib.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <vector>

namespace {

// ---------------------------------------------------------------- dtype table
struct DtypeName { const char* name; int code; int bytes; };
constexpr DtypeName kDtypes[] = {
    {"F32", RFK_DTYPE_F32, 4}, {"F16", RFK_DTYPE_F16, 2}, {"BF16", RFK_DTYPE_BF16, 2}, {"F64", RFK_DTYPE_F64, 8},
    {"I64", RFK_DTYPE_I64, 8}, {"I32", RFK_DTYPE_I32, 4}, {"I16", RFK_DTYPE_I16, 2}, {"I8", RFK_DTYPE_I8, 1},
    {"U8", RFK_DTYPE_U8, 1}, {"BOOL", RFK_DTYPE_BOOL, 1}, {"U16", RFK_DTYPE_U16, 2}, {"U32", RFK_DTYPE_U32, 4},
    {"U64", RFK_DTYPE_U64, 8}, {"F8_E4M3", RFK_DTYPE_F8_E4M3, 1}, {"F8_E5M2", RFK_DTYPE_F8_E5M2, 1},
};
const DtypeName* dtype_by_name(const std::string& s) {
    for (const auto& d : kDtypes) if (s == d.name) return &d;
    return nullptr;
}
const DtypeName* dtype_by_code(int c) {
    for (const auto& d : kDtypes) if (c == d.code) return &d;
    return nullptr;
}

// ---------------------------------------------------------------- a JSON reader for the header
// Enough JSON for any conforming header: objects, arrays, strings with escapes, non-negative integers, and a
// generic skip for values the format does not define. Every step checks the end of the buffer; a malformed header
// makes `ok` false and parsing stops.
struct Json {
    const char* p; const char* end; bool ok = true;
    void ws() { while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p; }
    bool peek(char c) { ws(); return p < end && *p == c; }
    bool take(char c) { ws(); if (p < end && *p == c) { ++p; return true; } return false; }
    void need(char c) { if (!take(c)) ok = false; }
    std::string string() {
        std::string s;
        ws();
        if (p >= end || *p != '"') { ok = false; return s; }
        ++p;
        while (p < end && *p != '"') {
            if (*p == '\\') {
                if (++p >= end) break;
                switch (*p) {
                    case 'n': s += '\n'; break; case 't': s += '\t'; break; case 'r': s += '\r'; break;
                    case 'b': s += '\b'; break; case 'f': s += '\f'; break;
                    case 'u': {  // \uXXXX -> UTF-8 (surrogate pairs are passed through as two 3-byte sequences)
                        if (end - p < 5) { ok = false; return s; }
                        unsigned v = 0;
                        for (int i = 1; i <= 4; ++i) {
                            const char h = p[i];
                            v = v * 16 + (h >= '0' && h <= '9' ? h - '0' : h >= 'a' && h <= 'f' ? h - 'a' + 10 : h >= 'A' && h <= 'F' ? h - 'A' + 10 : (ok = false, 0));
                        }
                        p += 4;
                        if (v < 0x80) s += (char)v;
                        else if (v < 0x800) { s += (char)(0xC0 | (v >> 6)); s += (char)(0x80 | (v & 0x3F)); }
                        else { s += (char)(0xE0 | (v >> 12)); s += (char)(0x80 | ((v >> 6) & 0x3F)); s += (char)(0x80 | (v & 0x3F)); }
                        break;
                    }
                    default: s += *p;  // \" \\ \/
                }
                ++p;
            } else {
                s += *p++;
            }
        }
        if (p >= end) { ok = false; return s; }
        ++p;  // closing quote
        return s;
    }
    uint64_t uint() {
        ws();
        if (p >= end || *p < '0' || *p > '9') { ok = false; return 0; }
        uint64_t v = 0;
        while (p < end && *p >= '0' && *p <= '9') {
            if (v > (UINT64_MAX - 9) / 10) { ok = false; return 0; }
            v = v * 10 + (uint64_t)(*p++ - '0');
        }
        return v;
    }
    void skip_value(int depth = 0) {  // any JSON value
        ws();
        if (p >= end || depth > 64) { ok = false; return; }
        if (*p == '"') { string(); return; }
        if (*p == '{' || *p == '[') {
            const char close = *p == '{' ? '}' : ']';
            const bool object = *p == '{';
            ++p;
            if (take(close)) return;
            do {
                if (object) { string(); need(':'); }
                skip_value(depth + 1);
            } while (ok && take(','));
            need(close);
            return;
        }
        while (p < end && *p != ',' && *p != '}' && *p != ']' && *p != ' ' && *p != '\n' && *p != '\t' && *p != '\r') ++p;  // number / literal
    }
};

struct Entry {
    std::string name;
    int dtype = 0;
    std::vector<int64_t> shape;
    size_t offset = 0, bytes = 0;
};

}  // namespace

struct rfk_safetensors {
    int fd = -1;
    const unsigned char* map = nullptr;  // whole file
    size_t file_bytes = 0, data_offset = 0, data_bytes = 0;
    std::vector<Entry> entries;                       // by offset
    std::map<std::string, int> by_name;
    std::map<std::string, std::string> metadata;
};

namespace {

void fill(const rfk_safetensors* f, const Entry& e, rfk_tensor_info* info) {
    info->name = e.name.c_str();
    info->dtype = e.dtype;
    info->ndim = (int)e.shape.size();
    info->shape = e.shape.data();
    info->offset = e.offset;
    info->bytes = e.bytes;
    info->host = f->map + f->data_offset + e.offset;
}

int parse_header(rfk_safetensors* f) {
    if (f->file_bytes < 8) return RFK_EFORMAT;
    uint64_t hlen = 0;
    for (int i = 7; i >= 0; --i) hlen = (hlen << 8) | f->map[i];  // little-endian, whatever the host
    if (hlen < 2 || hlen > f->file_bytes - 8) return RFK_EFORMAT;
    f->data_offset = 8 + (size_t)hlen;
    f->data_bytes = f->file_bytes - f->data_offset;
    Json j{reinterpret_cast<const char*>(f->map) + 8, reinterpret_cast<const char*>(f->map) + 8 + hlen};
    j.need('{');
    if (!j.peek('}')) {
        do {
            const std::string key = j.string();
            j.need(':');
            if (!j.ok) return RFK_EFORMAT;
            if (key == "__metadata__") {  // string -> string
                j.need('{');
                if (!j.peek('}')) {
                    do {
                        const std::string k = j.string();
                        j.need(':');
                        if (j.peek('"')) f->metadata[k] = j.string();
                        else j.skip_value();
                    } while (j.ok && j.take(','));
                }
                j.need('}');
                continue;
            }
            Entry e;
            e.name = key;
            bool have_dtype = false, have_shape = false, have_offsets = false;
            uint64_t begin = 0, end = 0;
            j.need('{');
            do {
                const std::string field = j.string();
                j.need(':');
                if (field == "dtype") {
                    const DtypeName* d = dtype_by_name(j.string());
                    if (!d) return RFK_EFORMAT;
                    e.dtype = d->code;
                    have_dtype = true;
                } else if (field == "shape") {
                    j.need('[');
                    if (!j.peek(']')) {
                        do {
                            const uint64_t v = j.uint();
                            if (v > (uint64_t)INT64_MAX) return RFK_EFORMAT;
                            e.shape.push_back((int64_t)v);
                        } while (j.ok && j.take(','));
                    }
                    j.need(']');
                    have_shape = true;
                } else if (field == "data_offsets") {
                    j.need('[');
                    begin = j.uint();
                    j.need(',');
                    end = j.uint();
                    j.need(']');
                    have_offsets = true;
                } else {
                    j.skip_value();
                }
            } while (j.ok && j.take(','));
            j.need('}');
            if (!j.ok || !have_dtype || !have_shape || !have_offsets) return RFK_EFORMAT;
            if (end < begin || end > f->data_bytes) return RFK_EFORMAT;
            // byte size must be what dtype and shape say (with overflow checked)
            uint64_t n = (uint64_t)dtype_by_code(e.dtype)->bytes;
            for (int64_t d : e.shape) {
                if (d != 0 && n > UINT64_MAX / (uint64_t)d) return RFK_EFORMAT;
                n *= (uint64_t)d;
            }
            if (n != end - begin) return RFK_EFORMAT;
            e.offset = (size_t)begin;
            e.bytes = (size_t)(end - begin);
            if (f->by_name.count(e.name)) return RFK_EFORMAT;
            f->by_name[e.name] = 0;
            f->entries.push_back(std::move(e));
        } while (j.ok && j.take(','));
    }
    j.need('}');
    if (!j.ok) return RFK_EFORMAT;
    std::stable_sort(f->entries.begin(), f->entries.end(), [](const Entry& a, const Entry& b) { return a.offset < b.offset; });
    for (size_t i = 0; i < f->entries.size(); ++i) f->by_name[f->entries[i].name] = (int)i;
    return RFK_OK;
}

}  // namespace

extern "C" int rfk_safetensors_open(const char* path, rfk_safetensors** out) {
    if (!path || !out) return RFK_EINVAL;
    *out = nullptr;
    std::unique_ptr<rfk_safetensors> f(new (std::nothrow) rfk_safetensors());
    if (!f) return RFK_EIO;
    f->fd = ::open(path, O_RDONLY | O_CLOEXEC);
    if (f->fd < 0) return RFK_EIO;
    struct stat st;
    if (fstat(f->fd, &st) != 0 || st.st_size < 0) { ::close(f->fd); return RFK_EIO; }
    f->file_bytes = (size_t)st.st_size;
    if (f->file_bytes == 0) { ::close(f->fd); return RFK_EFORMAT; }
    void* m = mmap(nullptr, f->file_bytes, PROT_READ, MAP_PRIVATE, f->fd, 0);
    if (m == MAP_FAILED) { ::close(f->fd); return RFK_EIO; }
    f->map = static_cast<const unsigned char*>(m);
    const int rc = parse_header(f.get());
    if (rc != RFK_OK) {
        munmap(m, f->file_bytes);
        ::close(f->fd);
        return rc;
    }
    *out = f.release();
    return RFK_OK;
}

extern "C" int rfk_safetensors_close(rfk_safetensors* f) {
    if (!f) return RFK_OK;
    if (f->map) munmap(const_cast<unsigned char*>(f->map), f->file_bytes);
    if (f->fd >= 0) ::close(f->fd);
    delete f;
    return RFK_OK;
}

extern "C" int rfk_safetensors_count(const rfk_safetensors* f) { return f ? (int)f->entries.size() : 0; }

extern "C" int rfk_safetensors_entry(const rfk_safetensors* f, int index, rfk_tensor_info* info) {
    if (!f || !info || index < 0 || index >= (int)f->entries.size()) return RFK_EINVAL;
    fill(f, f->entries[(size_t)index], info);
    return RFK_OK;
}

extern "C" int rfk_safetensors_find(const rfk_safetensors* f, const char* name, rfk_tensor_info* info) {
    if (!f || !name || !info) return RFK_EINVAL;
    const auto it = f->by_name.find(name);
    if (it == f->by_name.end()) return RFK_ENOTFOUND;
    fill(f, f->entries[(size_t)it->second], info);
    return RFK_OK;
}

extern "C" size_t rfk_safetensors_data_bytes(const rfk_safetensors* f) { return f ? f->data_bytes : 0; }

extern "C" const char* rfk_safetensors_metadata(const rfk_safetensors* f, const char* key) {
    if (!f || !key) return nullptr;
    const auto it = f->metadata.find(key);
    return it == f->metadata.end() ? nullptr : it->second.c_str();
}

extern "C" int rfk_safetensors_upload(const rfk_safetensors* f, void* device_dst, rfk_stream_t stream) {
    if (!f || (!device_dst && f->data_bytes)) return RFK_EINVAL;
    if (f->data_bytes == 0) return RFK_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // Two pinned buffers: while one is on its way to the device the next chunk is read out of the page cache
    // into the other. A copy from the pageable mapping itself would be staged by the driver chunk by chunk,
    // without that overlap.
    constexpr size_t kChunk = 32u << 20;
    const size_t chunk = std::min(kChunk, f->data_bytes);
    unsigned char* pinned[2] = {nullptr, nullptr};
    cudaEvent_t done[2] = {nullptr, nullptr};
    cudaError_t e = cudaSuccess;
    for (int i = 0; i < 2 && e == cudaSuccess; ++i) {
        e = cudaMallocHost(reinterpret_cast<void**>(&pinned[i]), chunk);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&done[i], cudaEventDisableTiming);
    }
    const unsigned char* src = f->map + f->data_offset;
    size_t off = 0;
    for (int i = 0; e == cudaSuccess && off < f->data_bytes; ++i, off += chunk) {
        const int b = i & 1;
        const size_t n = std::min(chunk, f->data_bytes - off);
        if (i >= 2) e = cudaEventSynchronize(done[b]);  // the copy that last used this buffer
        if (e != cudaSuccess) break;
        std::memcpy(pinned[b], src + off, n);
        e = cudaMemcpyAsync(static_cast<unsigned char*>(device_dst) + off, pinned[b], n, cudaMemcpyHostToDevice, st);
        if (e == cudaSuccess) e = cudaEventRecord(done[b], st);
    }
    const cudaError_t es = cudaStreamSynchronize(st);  // also on the error path: the buffers are freed below
    if (e == cudaSuccess) e = es;
    for (int i = 0; i < 2; ++i) {
        if (done[i]) cudaEventDestroy(done[i]);
        if (pinned[i]) cudaFreeHost(pinned[i]);
    }
    return (int)e;
}

// ---------------------------------------------------------------- writers
namespace {

struct File {
    FILE* f;
    explicit File(const char* path) : f(std::fopen(path, "wb")) {}
    ~File() { if (f) std::fclose(f); }
    bool put(const void* p, size_t n) { return n == 0 || std::fwrite(p, 1, n, f) == n; }
    int finish() { const int rc = std::fclose(f); f = nullptr; return rc == 0 ? RFK_OK : RFK_EIO; }
};

void put_le(std::vector<unsigned char>& v, uint64_t x, int bytes) { for (int i = 0; i < bytes; ++i) v.push_back((unsigned char)(x >> (8 * i))); }
void put_be32(std::vector<unsigned char>& v, uint32_t x) { for (int i = 3; i >= 0; --i) v.push_back((unsigned char)(x >> (8 * i))); }
void put_str0(std::vector<unsigned char>& v, const char* s) { while (*s) v.push_back((unsigned char)*s++); v.push_back(0); }

std::string json_escape(const std::string& s) {
    std::string o;
    for (unsigned char c : s) {
        if (c == '"' || c == '\\') { o += '\\'; o += (char)c; }
        else if (c < 0x20) { char b[8]; std::snprintf(b, sizeof b, "\\u%04x", c); o += b; }
        else o += (char)c;
    }
    return o;
}

}  // namespace

extern "C" int rfk_safetensors_write(const char* path, int n, const char* const* names, const int* dtypes, const int* ndims,
                                     const int64_t* const* shapes, const void* const* data) {
    if (!path || n < 0 || (n && (!names || !dtypes || !ndims || !shapes || !data))) return RFK_EINVAL;
    std::string header = "{";
    std::vector<size_t> bytes((size_t)n);
    size_t off = 0;
    for (int i = 0; i < n; ++i) {
        const DtypeName* d = dtype_by_code(dtypes[i]);
        if (!d || !names[i] || ndims[i] < 0 || (ndims[i] && !shapes[i])) return RFK_EINVAL;
        size_t b = (size_t)d->bytes;
        std::string shape = "[";
        for (int k = 0; k < ndims[i]; ++k) {
            if (shapes[i][k] < 0) return RFK_EINVAL;
            b *= (size_t)shapes[i][k];
            shape += (k ? "," : "") + std::to_string(shapes[i][k]);
        }
        shape += "]";
        if (b && !data[i]) return RFK_EINVAL;
        bytes[(size_t)i] = b;
        header += std::string(i ? "," : "") + "\"" + json_escape(names[i]) + "\":{\"dtype\":\"" + d->name + "\",\"shape\":" + shape +
                  ",\"data_offsets\":[" + std::to_string(off) + "," + std::to_string(off + b) + "]}";
        off += b;
    }
    header += "}";
    while ((header.size() + 8) % 8) header += ' ';  // data section on an 8-byte boundary, as the format's writers do
    File out(path);
    if (!out.f) return RFK_EIO;
    std::vector<unsigned char> len;
    put_le(len, header.size(), 8);
    bool ok = out.put(len.data(), 8) && out.put(header.data(), header.size());
    for (int i = 0; ok && i < n; ++i) ok = out.put(data[i], bytes[(size_t)i]);
    const int rc = out.finish();
    return ok ? rc : RFK_EIO;
}

extern "C" int rfk_write_exr(const char* path, const float* data, int width, int height, int channels) {
    if (!path || !data || width <= 0 || height <= 0 || (channels != 1 && channels != 3 && channels != 4)) return RFK_EINVAL;
    // Channels are stored in alphabetical order of their names; source index of each stored channel:
    // RGB -> B, G, R; RGBA -> A, B, G, R; one channel -> Y.
    const char* names3[] = {"B", "G", "R"};
    const int src3[] = {2, 1, 0};
    const char* names4[] = {"A", "B", "G", "R"};
    const int src4[] = {3, 2, 1, 0};
    const char* names1[] = {"Y"};
    const int src1[] = {0};
    const char* const* names = channels == 1 ? names1 : channels == 3 ? names3 : names4;
    const int* src = channels == 1 ? src1 : channels == 3 ? src3 : src4;

    std::vector<unsigned char> h;
    put_le(h, 20000630u, 4);  // magic
    put_le(h, 2u, 4);         // version 2, scan lines, single part
    auto attr = [&](const char* name, const char* type, const std::vector<unsigned char>& value) {
        put_str0(h, name);
        put_str0(h, type);
        put_le(h, value.size(), 4);
        h.insert(h.end(), value.begin(), value.end());
    };
    std::vector<unsigned char> v;
    for (int c = 0; c < channels; ++c) {
        put_str0(v, names[c]);
        put_le(v, 2u, 4);       // FLOAT
        v.push_back(0);         // pLinear
        v.push_back(0); v.push_back(0); v.push_back(0);
        put_le(v, 1u, 4);       // x sampling
        put_le(v, 1u, 4);       // y sampling
    }
    v.push_back(0);
    attr("channels", "chlist", v);
    attr("compression", "compression", {0});
    v.clear();
    put_le(v, 0, 4); put_le(v, 0, 4); put_le(v, (uint32_t)(width - 1), 4); put_le(v, (uint32_t)(height - 1), 4);
    attr("dataWindow", "box2i", v);
    attr("displayWindow", "box2i", v);
    attr("lineOrder", "lineOrder", {0});  // increasing y
    const float one = 1.0f, zero2[2] = {0.0f, 0.0f};
    v.assign(reinterpret_cast<const unsigned char*>(&one), reinterpret_cast<const unsigned char*>(&one) + 4);
    attr("pixelAspectRatio", "float", v);
    v.assign(reinterpret_cast<const unsigned char*>(zero2), reinterpret_cast<const unsigned char*>(zero2) + 8);
    attr("screenWindowCenter", "v2f", v);
    v.assign(reinterpret_cast<const unsigned char*>(&one), reinterpret_cast<const unsigned char*>(&one) + 4);
    attr("screenWindowWidth", "float", v);
    h.push_back(0);  // end of header

    const size_t line_bytes = (size_t)width * channels * 4, block = 8 + line_bytes;
    const size_t table_at = h.size(), first = table_at + (size_t)height * 8;
    for (int y = 0; y < height; ++y) put_le(h, first + (size_t)y * block, 8);
    File out(path);
    if (!out.f) return RFK_EIO;
    bool ok = out.put(h.data(), h.size());
    std::vector<unsigned char> line;
    std::vector<float> plane((size_t)width);
    for (int y = 0; ok && y < height; ++y) {
        line.clear();
        put_le(line, (uint32_t)y, 4);
        put_le(line, line_bytes, 4);
        const float* row = data + (size_t)y * width * channels;
        for (int c = 0; c < channels; ++c) {
            for (int x = 0; x < width; ++x) plane[(size_t)x] = row[(size_t)x * channels + src[c]];
            const unsigned char* b = reinterpret_cast<const unsigned char*>(plane.data());  // little-endian host assumed (x86-64, aarch64)
            line.insert(line.end(), b, b + (size_t)width * 4);
        }
        ok = out.put(line.data(), line.size());
    }
    const int rc = out.finish();
    return ok ? rc : RFK_EIO;
}

extern "C" int rfk_write_png(const char* path, const unsigned char* data, int width, int height, int channels) {
    if (!path || !data || width <= 0 || height <= 0 || channels < 1 || channels > 4) return RFK_EINVAL;
    const unsigned char colour_type[] = {0, 0, 4, 2, 6};  // grey, grey + alpha, RGB, RGBA
    const size_t row = (size_t)width * channels;
    std::vector<unsigned char> raw((row + 1) * (size_t)height);
    for (int y = 0; y < height; ++y) {
        raw[(size_t)y * (row + 1)] = 0;  // filter type None
        std::memcpy(&raw[(size_t)y * (row + 1) + 1], data + (size_t)y * row, row);
    }
    uLongf zbytes = compressBound((uLong)raw.size());
    std::vector<unsigned char> z(zbytes);
    if (compress2(z.data(), &zbytes, raw.data(), (uLong)raw.size(), 6) != Z_OK) return RFK_EIO;
    std::vector<unsigned char> f = {0x89, 'P', 'N', 'G', 0x0D, 0x0A, 0x1A, 0x0A};
    auto chunk = [&](const char* type, const unsigned char* p, size_t n) {
        put_be32(f, (uint32_t)n);
        const size_t at = f.size();
        f.insert(f.end(), type, type + 4);
        f.insert(f.end(), p, p + n);
        put_be32(f, (uint32_t)crc32(0L, &f[at], (uInt)(n + 4)));
    };
    std::vector<unsigned char> ihdr;
    put_be32(ihdr, (uint32_t)width);
    put_be32(ihdr, (uint32_t)height);
    ihdr.push_back(8);
    ihdr.push_back(colour_type[channels]);
    ihdr.push_back(0); ihdr.push_back(0); ihdr.push_back(0);
    chunk("IHDR", ihdr.data(), ihdr.size());
    chunk("IDAT", z.data(), zbytes);
    chunk("IEND", nullptr, 0);
    File out(path);
    if (!out.f) return RFK_EIO;
    const bool ok = out.put(f.data(), f.size());
    const int rc = out.finish();
    return ok ? rc : RFK_EIO;
}

extern "C" int rfk_tonemap(const float* hdr, unsigned char* ldr, int width, int height, int channels) {
    if (!hdr || !ldr || width < 0 || height < 0 || channels < 1) return RFK_EINVAL;
    const size_t n = (size_t)width * height * channels;
    for (size_t i = 0; i < n; ++i) {
        float v = std::max(0.0f, hdr[i]);
        v = v / (v + 1.0f);
        v = std::pow(v, 1.0f / 2.2f);
        ldr[i] = (unsigned char)std::min(std::max(v * 255.0f, 0.0f), 255.0f);
    }
    return RFK_OK;
}
