#include "gguf.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cerrno>
#include <cstring>

namespace bc {

namespace {

// GGUF metadata value type ids.
enum : uint32_t { V_U8 = 0, V_I8, V_U16, V_I16, V_U32, V_I32, V_F32, V_BOOL, V_STRING, V_ARRAY, V_U64, V_I64, V_F64 };
constexpr uint32_t kMagic = 0x46554747u;  // "GGUF"
constexpr uint64_t kDefaultAlignment = 32;
constexpr uint32_t kMaxDims = 4;

size_t fixed_size(uint32_t type) {
    switch (type) {
        case V_U8: case V_I8: case V_BOOL: return 1;
        case V_U16: case V_I16: return 2;
        case V_U32: case V_I32: case V_F32: return 4;
        case V_U64: case V_I64: case V_F64: return 8;
        default: return 0;
    }
}

// A cursor that refuses to read past the end.
struct Reader {
    const uint8_t* bytes;
    size_t len;
    size_t pos = 0;
    size_t remaining() const { return len - pos; }
    bool take(size_t n, const uint8_t** out) {
        if (n > remaining()) return false;
        *out = bytes + pos;
        pos += n;
        return true;
    }
    bool u32(uint32_t* out) {
        const uint8_t* p;
        if (!take(4, &p)) return false;
        std::memcpy(out, p, 4);
        return true;
    }
    bool u64(uint64_t* out) {
        const uint8_t* p;
        if (!take(8, &p)) return false;
        std::memcpy(out, p, 8);
        return true;
    }
    bool string(uint64_t* start, uint64_t* n) {
        uint64_t count;
        if (!u64(&count)) return false;
        if (count > remaining()) return false;
        *start = pos;
        *n = count;
        pos += (size_t)count;
        return true;
    }
};

bool valid_utf8(const uint8_t* s, size_t n) {
    size_t i = 0;
    while (i < n) {
        uint8_t c = s[i];
        size_t extra;
        uint32_t cp;
        if (c < 0x80) { ++i; continue; }
        else if ((c & 0xe0) == 0xc0) { extra = 1; cp = c & 0x1f; if (cp < 2) return false; }
        else if ((c & 0xf0) == 0xe0) { extra = 2; cp = c & 0x0f; }
        else if ((c & 0xf8) == 0xf0) { extra = 3; cp = c & 0x07; }
        else return false;
        if (i + extra >= n) return false;
        for (size_t k = 1; k <= extra; ++k) {
            if ((s[i + k] & 0xc0) != 0x80) return false;
            cp = (cp << 6) | (s[i + k] & 0x3f);
        }
        if (extra == 2 && (cp < 0x800 || (cp >= 0xd800 && cp <= 0xdfff))) return false;
        if (extra == 3 && (cp < 0x10000 || cp > 0x10ffff)) return false;
        i += extra + 1;
    }
    return true;
}

bool read_value(Reader& r, uint32_t type, GgufValue* v) {
    v->type = type;
    if (type == V_STRING) return r.string(&v->start, &v->len);
    if (type == V_ARRAY) {
        uint32_t element;
        uint64_t count;
        if (!r.u32(&element) || !r.u64(&count)) return false;
        if (element > V_F64 || element == V_ARRAY) return false;
        size_t start = r.pos;
        if (element == V_STRING) {
            // Each string needs at least its 8-byte length.
            if (count > r.remaining() / 8) return false;
            for (uint64_t i = 0; i < count; ++i) {
                uint64_t s, n;
                if (!r.string(&s, &n)) return false;
            }
        } else {
            size_t size = fixed_size(element);
            if (count > SIZE_MAX / size) return false;
            const uint8_t* p;
            if (!r.take((size_t)count * size, &p)) return false;
        }
        v->element = element;
        v->count = count;
        v->start = start;
        v->len = r.pos - start;
        return true;
    }
    size_t size = fixed_size(type);
    if (size == 0) return false;
    const uint8_t* p;
    if (!r.take(size, &p)) return false;
    v->scalar_bits = 0;
    std::memcpy(&v->scalar_bits, p, size);
    return true;
}

// The value as a u32 when it is an integer that fits (lib.rs:255-270).
bool as_u32(uint32_t type, uint64_t bits, uint32_t* out) {
    int64_t s;
    switch (type) {
        case V_U8: *out = (uint8_t)bits; return true;
        case V_U16: *out = (uint16_t)bits; return true;
        case V_U32: *out = (uint32_t)bits; return true;
        case V_U64: if (bits > 0xffffffffull) return false; *out = (uint32_t)bits; return true;
        case V_I8: s = (int8_t)bits; break;
        case V_I16: s = (int16_t)bits; break;
        case V_I32: s = (int32_t)bits; break;
        case V_I64: s = (int64_t)bits; break;
        default: return false;
    }
    if (s < 0 || s > 0xffffffffll) return false;
    *out = (uint32_t)s;
    return true;
}

}  // namespace

bool type_block(uint32_t type, uint64_t* elements, uint64_t* bytes) {
    switch (type) {
        case T_F32: *elements = 1; *bytes = 4; return true;
        case T_F16: case T_BF16: *elements = 1; *bytes = 2; return true;
        case T_Q4_0: *elements = 32; *bytes = 18; return true;
        case T_Q8_0: *elements = 32; *bytes = 34; return true;
        case T_Q4K: *elements = 256; *bytes = 144; return true;
        case T_Q5K: *elements = 256; *bytes = 176; return true;
        case T_Q6K: *elements = 256; *bytes = 210; return true;
        default: return false;
    }
}

uint64_t type_row_bytes(uint32_t type, uint64_t n_cols) {
    uint64_t e = 1, b = 4;
    type_block(type, &e, &b);
    return n_cols / e * b;
}

Gguf::~Gguf() {
    if (mapping_) munmap(mapping_, mapping_len_);
}

bc_status Gguf::open(const char* path) {
    int fd = ::open(path, O_RDONLY);
    if (fd < 0) return fail(BC_ERR_IO, "cannot open %s: %s", path, strerror(errno));
    struct stat st;
    if (fstat(fd, &st) != 0) {
        ::close(fd);
        return fail(BC_ERR_IO, "cannot stat %s: %s", path, strerror(errno));
    }
    if (st.st_size == 0) {
        ::close(fd);
        return fail(BC_ERR_GGUF, "%s: not a GGUF file", path);
    }
    void* map = mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
    ::close(fd);
    if (map == MAP_FAILED) return fail(BC_ERR_IO, "cannot map %s: %s", path, strerror(errno));
    mapping_ = map;
    mapping_len_ = (size_t)st.st_size;
    bc_status status = parse((const uint8_t*)map, mapping_len_);
    if (status != BC_OK) {
        std::string why = last_error();
        return fail(status, "%s: %s", path, why.c_str());
    }
    return BC_OK;
}

bc_status Gguf::parse(const uint8_t* bytes, size_t len) {
    bytes_ = bytes;
    size_ = len;
    metadata_.clear();
    tensors_.clear();
    Reader r{bytes, len};
    uint32_t magic, version;
    uint64_t n_tensors, n_kv;
    if (!r.u32(&magic) || magic != kMagic) return fail(BC_ERR_GGUF, "not a GGUF file");
    if (!r.u32(&version) || !r.u64(&n_tensors) || !r.u64(&n_kv)) return fail(BC_ERR_GGUF, "truncated header");
    if (version != 2 && version != 3) return fail(BC_ERR_GGUF, "unsupported GGUF version %u", version);

    // Every entry needs at least a key length, a type and one byte of value.
    if (n_kv > r.remaining() / 13) return fail(BC_ERR_GGUF, "metadata count %llu exceeds the file", (unsigned long long)n_kv);
    for (uint64_t i = 0; i < n_kv; ++i) {
        uint64_t ks, kn;
        uint32_t type;
        GgufValue v;
        if (!r.string(&ks, &kn) || !valid_utf8(bytes + ks, (size_t)kn) || !r.u32(&type) || !read_value(r, type, &v))
            return fail(BC_ERR_GGUF, "malformed metadata entry %llu", (unsigned long long)i);
        std::string key((const char*)bytes + ks, (size_t)kn);
        if (!metadata_.emplace(key, v).second) return fail(BC_ERR_GGUF, "metadata key %s appears twice", key.c_str());
    }

    uint64_t alignment = kDefaultAlignment;
    auto al = metadata_.find("general.alignment");
    if (al != metadata_.end()) {
        uint32_t a = (uint32_t)al->second.scalar_bits;
        if (al->second.type != V_U32 || a == 0 || (a & (a - 1)) != 0) return fail(BC_ERR_GGUF, "general.alignment is not a power of two");
        alignment = a;
    }

    // Each header needs a name length, a dimension count, a type and an offset.
    if (n_tensors > r.remaining() / 24) return fail(BC_ERR_GGUF, "tensor count %llu exceeds the file", (unsigned long long)n_tensors);
    std::vector<GgufTensor> headers;
    headers.reserve((size_t)n_tensors);
    for (uint64_t i = 0; i < n_tensors; ++i) {
        uint64_t ns, nn;
        uint32_t n_dims;
        GgufTensor t;
        if (!r.string(&ns, &nn) || !valid_utf8(bytes + ns, (size_t)nn) || !r.u32(&n_dims))
            return fail(BC_ERR_GGUF, "malformed tensor header %llu", (unsigned long long)i);
        t.name.assign((const char*)bytes + ns, (size_t)nn);
        bool dims_ok = n_dims >= 1 && n_dims <= kMaxDims;
        if (dims_ok) {
            t.shape.resize(n_dims);
            for (uint32_t d = 0; d < n_dims; ++d)
                if (!r.u64(&t.shape[d])) return fail(BC_ERR_GGUF, "malformed tensor header %llu", (unsigned long long)i);
        }
        if (!r.u32(&t.type) || !r.u64(&t.offset)) return fail(BC_ERR_GGUF, "malformed tensor header %llu", (unsigned long long)i);
        if (!dims_ok) return fail(BC_ERR_GGUF, "tensor %s has %u dimensions", t.name.c_str(), n_dims);
        headers.push_back(std::move(t));
    }

    uint64_t header_end = r.pos;
    if (header_end > UINT64_MAX - alignment) return fail(BC_ERR_GGUF, "data section lies outside the file");
    uint64_t data_start = round_up(header_end, alignment);

    for (GgufTensor& t : headers) {
        uint64_t n_elements = 1;
        for (uint64_t d : t.shape) {
            if (d == 0 || n_elements > UINT64_MAX / d) return fail(BC_ERR_GGUF, "tensor %s has an invalid shape", t.name.c_str());
            n_elements *= d;
        }
        uint64_t block, block_bytes;
        if (!type_block(t.type, &block, &block_bytes)) return fail(BC_ERR_GGUF, "tensor %s has unsupported type %u", t.name.c_str(), t.type);
        if (t.shape[0] % block != 0)
            return fail(BC_ERR_GGUF, "tensor %s has rows of %llu elements, which blocks of %llu cannot divide", t.name.c_str(),
                        (unsigned long long)t.shape[0], (unsigned long long)block);
        uint64_t n_blocks = n_elements / block;
        if (n_blocks > UINT64_MAX / block_bytes) return fail(BC_ERR_GGUF, "tensor %s is too large", t.name.c_str());
        t.n_bytes = n_blocks * block_bytes;
        uint64_t relative = t.offset;
        if (relative > UINT64_MAX - data_start || data_start + relative > UINT64_MAX - t.n_bytes ||
            relative % alignment != 0 || data_start + relative + t.n_bytes > len)
            return fail(BC_ERR_GGUF, "tensor %s lies outside the file", t.name.c_str());
        t.offset = data_start + relative;
        std::string name = t.name;
        if (!tensors_.emplace(name, std::move(t)).second) return fail(BC_ERR_GGUF, "tensor %s appears twice", name.c_str());
    }
    return BC_OK;
}

bool Gguf::u32(const std::string& key, uint32_t* out) const {
    auto it = metadata_.find(key);
    if (it == metadata_.end()) return false;
    return as_u32(it->second.type, it->second.scalar_bits, out);
}

bool Gguf::f32(const std::string& key, float* out) const {
    auto it = metadata_.find(key);
    if (it == metadata_.end()) return false;
    if (it->second.type == V_F32) {
        uint32_t bits = (uint32_t)it->second.scalar_bits;
        std::memcpy(out, &bits, 4);
        return true;
    }
    if (it->second.type == V_F64) {
        double d;
        std::memcpy(&d, &it->second.scalar_bits, 8);
        *out = (float)d;
        return true;
    }
    return false;
}

bool Gguf::string(const std::string& key, std::string* out) const {
    auto it = metadata_.find(key);
    if (it == metadata_.end() || it->second.type != V_STRING) return false;
    out->assign((const char*)bytes_ + it->second.start, (size_t)it->second.len);
    return true;
}

bool Gguf::array_len(const std::string& key, uint64_t* out) const {
    auto it = metadata_.find(key);
    if (it == metadata_.end() || it->second.type != V_ARRAY) return false;
    *out = it->second.count;
    return true;
}

bool Gguf::array_u32(const std::string& key, uint64_t index, uint32_t* out) const {
    auto it = metadata_.find(key);
    if (it == metadata_.end() || it->second.type != V_ARRAY) return false;
    const GgufValue& v = it->second;
    if (index >= v.count) return false;
    size_t size = fixed_size(v.element);
    if (size == 0) return false;
    uint64_t bits = 0;
    std::memcpy(&bits, bytes_ + v.start + index * size, size);
    return as_u32(v.element, bits, out);
}

const GgufTensor* Gguf::tensor(const std::string& name) const {
    auto it = tensors_.find(name);
    return it == tensors_.end() ? nullptr : &it->second;
}

}  // namespace bc
