// GGUF writer for synthetic model files: a small library of its own (libbobcat_synth.so, plain
// C++), used by the tests and the benchmark to make their model files. It is not part of the
// product library and links nothing of it.
//
// The reference only reads GGUF; its tests and benchmarks use downloaded checkpoints. This writer
// produces files with the layout the reference's parser checks (crates/bobcat-gguf/src/lib.rs:
// 316-344, :693-751): magic, version 3, general.alignment 32, aligned tensor offsets, whole Q4_0
// blocks per row. Tensor values come from a counter-based generator keyed by (seed, tensor order,
// row, pair), so the bytes do not depend on how many threads fill the file.
//
// Q4_0 quantisation follows ggml's reference rounding (ggml/src/ggml-quants.c,
// quantize_row_q4_0_ref): per 32-element block the signed value of largest magnitude maps to -8,
// d = max / -8 stored as fp16, q = min(15, trunc(x / d + 8.5)).

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>
#include <cerrno>
#include <cmath>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include <algorithm>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <memory>

#include "synth_writer.h"

namespace {

// This library keeps its own failure message: it does not link against the CUDA library.
std::string& last_error() {
    thread_local std::string message;
    return message;
}

int32_t fail(int32_t status, const char* format, ...) __attribute__((format(printf, 2, 3)));
int32_t fail(int32_t status, const char* format, ...) {
    char buffer[512];
    va_list args;
    va_start(args, format);
    vsnprintf(buffer, sizeof buffer, format, args);
    va_end(args);
    last_error() = buffer;
    return status;
}

inline uint64_t round_up(uint64_t a, uint64_t b) { return (a + b - 1) / b * b; }

// Bytes of one row: F32 4 per element, Q4_0 18 per block of 32, Q8_0 34 per block of 32.
inline uint64_t type_row_bytes(uint32_t type, uint64_t n_cols) {
    if (type == BCS_Q4_0) return n_cols / 32 * 18;
    if (type == BCS_Q8_0) return n_cols / 32 * 34;
    return n_cols * 4;
}

constexpr uint64_t kAlignment = 32;

struct TensorSpec {
    std::string name;
    uint32_t type;
    std::vector<uint64_t> dims;
    int32_t init;
    float value;
    uint64_t n_rows, n_cols, row_bytes, offset;
};

void put_u32(std::vector<uint8_t>& b, uint32_t v) { b.insert(b.end(), (uint8_t*)&v, (uint8_t*)&v + 4); }
void put_u64(std::vector<uint8_t>& b, uint64_t v) { b.insert(b.end(), (uint8_t*)&v, (uint8_t*)&v + 8); }
void put_str(std::vector<uint8_t>& b, const std::string& s) {
    put_u64(b, s.size());
    b.insert(b.end(), s.begin(), s.end());
}

inline uint64_t mix64(uint64_t z) {
    z += 0x9e3779b97f4a7c15ull;
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    return z ^ (z >> 31);
}

// Two standard normal draws from one 64-bit hash (Box-Muller on two 24-bit uniforms in (0, 1)).
inline void normal_pair(uint64_t h, float* z0, float* z1) {
    float u1 = ((float)(h >> 40) + 0.5f) * (1.0f / 16777216.0f);
    float u2 = ((float)((h >> 16) & 0xffffffu) + 0.5f) * (1.0f / 16777216.0f);
    float r = sqrtf(-2.0f * logf(u1));
    float a = 6.28318530717958647692f * u2;
    *z0 = r * cosf(a);
    *z1 = r * sinf(a);
}

// f32 -> IEEE binary16, round to nearest even.
inline uint16_t f32_to_f16(float f) {
    uint32_t x;
    std::memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t mant = x & 0x007fffffu;
    int32_t exp = (int32_t)((x >> 23) & 0xff);
    if (exp == 255) return (uint16_t)(sign | 0x7c00u | (mant ? 0x200u : 0));
    exp = exp - 127 + 15;
    if (exp >= 31) return (uint16_t)(sign | 0x7c00u);
    if (exp <= 0) {
        if (exp < -10) return (uint16_t)sign;
        mant |= 0x00800000u;
        uint32_t shift = (uint32_t)(14 - exp);
        uint32_t half = mant >> shift;
        uint32_t rem = mant & ((1u << shift) - 1);
        uint32_t halfway = 1u << (shift - 1);
        if (rem > halfway || (rem == halfway && (half & 1))) ++half;
        return (uint16_t)(sign | half);
    }
    uint32_t half = ((uint32_t)exp << 10) | (mant >> 13);
    uint32_t rem = mant & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (half & 1))) ++half;
    return (uint16_t)(sign | half);
}

void quantize_row_q4_0(const float* x, uint8_t* out, uint64_t n_cols) {
    for (uint64_t b = 0; b < n_cols / 32; ++b) {
        const float* xb = x + 32 * b;
        uint8_t* ob = out + 18 * b;
        float amax = 0.f, max = 0.f;
        for (int j = 0; j < 32; ++j) {
            float v = xb[j];
            if (amax < fabsf(v)) {
                amax = fabsf(v);
                max = v;
            }
        }
        float d = max / -8.0f;
        float id = d != 0.f ? 1.0f / d : 0.f;
        uint16_t dh = f32_to_f16(d);
        std::memcpy(ob, &dh, 2);
        for (int j = 0; j < 16; ++j) {
            float x0 = xb[j] * id, x1 = xb[16 + j] * id;
            int q0 = (int)(int8_t)(x0 + 8.5f), q1 = (int)(int8_t)(x1 + 8.5f);
            if (q0 > 15) q0 = 15;
            if (q1 > 15) q1 = 15;
            ob[2 + j] = (uint8_t)(q0 | (q1 << 4));
        }
    }
}

// ggml's reference Q8_0 rounding (quantize_row_q8_0_ref): d = amax / 127 as fp16, q = round(x / d).
void quantize_row_q8_0(const float* x, uint8_t* out, uint64_t n_cols) {
    for (uint64_t b = 0; b < n_cols / 32; ++b) {
        const float* xb = x + 32 * b;
        uint8_t* ob = out + 34 * b;
        float amax = 0.f;
        for (int j = 0; j < 32; ++j) amax = std::max(amax, fabsf(xb[j]));
        float d = amax / 127.0f;
        float id = d != 0.f ? 1.0f / d : 0.f;
        uint16_t dh = f32_to_f16(d);
        std::memcpy(ob, &dh, 2);
        for (int j = 0; j < 32; ++j) ob[2 + j] = (uint8_t)(int8_t)roundf(xb[j] * id);
    }
}

void fill_row(const TensorSpec& t, uint64_t seed, uint64_t tensor_index, uint64_t row, float* scratch, uint8_t* out) {
    float* dst = t.type == BCS_F32 ? (float*)out : scratch;
    if (t.init == BCS_INIT_CONSTANT) {
        for (uint64_t i = 0; i < t.n_cols; ++i) dst[i] = t.value;
    } else {
        uint64_t key = mix64(mix64(seed ^ (tensor_index * 0xd1342543de82ef95ull)) ^ (row * 0x2545f4914f6cdd1dull));
        for (uint64_t i = 0; i < t.n_cols; i += 2) {
            float z0, z1;
            normal_pair(mix64(key + i / 2), &z0, &z1);
            dst[i] = z0 * t.value;
            if (i + 1 < t.n_cols) dst[i + 1] = z1 * t.value;
        }
        if (t.init == BCS_INIT_NEG_EXP_NORMAL)
            for (uint64_t i = 0; i < t.n_cols; ++i) dst[i] = -expf(dst[i]);
    }
    if (t.type == BCS_Q4_0) quantize_row_q4_0(scratch, out, t.n_cols);
    if (t.type == BCS_Q8_0) quantize_row_q8_0(scratch, out, t.n_cols);
}

}  // namespace

struct bcs_writer {
    std::string path;
    uint64_t seed = 0;
    std::vector<uint8_t> kv;
    uint64_t n_kv = 0;
    std::vector<TensorSpec> tensors;
};

extern "C" {

const char* bcs_last_error(void) { return last_error().c_str(); }

int32_t bcs_writer_new(const char* path, uint64_t seed, bcs_writer** out) {
    if (!path || !out) return fail(BCS_ERR_ARGUMENT, "path and out must be non-null");
    bcs_writer* w = new bcs_writer();
    w->path = path;
    w->seed = seed;
    *out = w;
    return BCS_OK;
}

int32_t bcs_writer_kv_u32(bcs_writer* w, const char* key, uint32_t value) {
    if (!w || !key) return fail(BCS_ERR_ARGUMENT, "writer and key must be non-null");
    put_str(w->kv, key);
    put_u32(w->kv, 4);
    put_u32(w->kv, value);
    ++w->n_kv;
    return BCS_OK;
}

int32_t bcs_writer_kv_f32(bcs_writer* w, const char* key, float value) {
    if (!w || !key) return fail(BCS_ERR_ARGUMENT, "writer and key must be non-null");
    put_str(w->kv, key);
    put_u32(w->kv, 6);
    uint32_t bits;
    std::memcpy(&bits, &value, 4);
    put_u32(w->kv, bits);
    ++w->n_kv;
    return BCS_OK;
}

int32_t bcs_writer_kv_str(bcs_writer* w, const char* key, const char* value) {
    if (!w || !key || !value) return fail(BCS_ERR_ARGUMENT, "writer, key and value must be non-null");
    put_str(w->kv, key);
    put_u32(w->kv, 8);
    put_str(w->kv, value);
    ++w->n_kv;
    return BCS_OK;
}

int32_t bcs_writer_kv_u32_array(bcs_writer* w, const char* key, const uint32_t* values, uint64_t n) {
    if (!w || !key || (!values && n)) return fail(BCS_ERR_ARGUMENT, "writer, key and values must be non-null");
    put_str(w->kv, key);
    put_u32(w->kv, 9);
    put_u32(w->kv, 4);
    put_u64(w->kv, n);
    for (uint64_t i = 0; i < n; ++i) put_u32(w->kv, values[i]);
    ++w->n_kv;
    return BCS_OK;
}

int32_t bcs_writer_tensor(bcs_writer* w, const char* name, int32_t type, const uint64_t* dims, uint32_t n_dims,
                                int32_t init, float value) {
    if (!w || !name || !dims) return fail(BCS_ERR_ARGUMENT, "writer, name and dims must be non-null");
    if (n_dims < 1 || n_dims > 4) return fail(BCS_ERR_ARGUMENT, "a tensor has 1 to 4 dimensions");
    if (type != BCS_F32 && type != BCS_Q4_0 && type != BCS_Q8_0) return fail(BCS_ERR_ARGUMENT, "the writer draws F32, Q4_0 and Q8_0 tensors");
    if (init < BCS_INIT_NORMAL || init > BCS_INIT_NEG_EXP_NORMAL) return fail(BCS_ERR_ARGUMENT, "unknown init kind");
    TensorSpec t;
    t.name = name;
    t.type = (uint32_t)type;
    t.dims.assign(dims, dims + n_dims);
    t.init = init;
    t.value = value;
    t.n_cols = dims[0];
    t.n_rows = 1;
    for (uint32_t d = 1; d < n_dims; ++d) t.n_rows *= dims[d];
    if (t.n_cols == 0 || t.n_rows == 0) return fail(BCS_ERR_ARGUMENT, "tensor %s has an empty dimension", name);
    if (type != BCS_F32 && t.n_cols % 32 != 0) return fail(BCS_ERR_ARGUMENT, "quantised rows hold whole blocks of 32");
    t.row_bytes = type_row_bytes(t.type, t.n_cols);
    t.offset = 0;
    w->tensors.push_back(std::move(t));
    return BCS_OK;
}

int32_t bcs_writer_finish(bcs_writer* w) {
    if (!w) return fail(BCS_ERR_ARGUMENT, "writer must be non-null");
    std::unique_ptr<bcs_writer> owner(w);

    std::vector<uint8_t> head;
    put_u32(head, 0x46554747u);
    put_u32(head, 3);
    put_u64(head, w->tensors.size());
    put_u64(head, w->n_kv + 1);
    put_str(head, "general.alignment");
    put_u32(head, 4);
    put_u32(head, (uint32_t)kAlignment);
    head.insert(head.end(), w->kv.begin(), w->kv.end());
    uint64_t relative = 0;
    for (TensorSpec& t : w->tensors) {
        t.offset = relative;
        relative = round_up(relative + t.n_rows * t.row_bytes, kAlignment);
        put_str(head, t.name);
        put_u32(head, (uint32_t)t.dims.size());
        for (uint64_t d : t.dims) put_u64(head, d);
        put_u32(head, t.type);
        put_u64(head, t.offset);
    }
    uint64_t data_start = round_up(head.size(), kAlignment);
    uint64_t total = data_start + relative;

    int fd = ::open(w->path.c_str(), O_RDWR | O_CREAT | O_TRUNC, 0644);
    if (fd < 0) return fail(BCS_ERR_IO, "cannot create %s: %s", w->path.c_str(), strerror(errno));
    if (ftruncate(fd, (off_t)total) != 0) {
        ::close(fd);
        return fail(BCS_ERR_IO, "cannot size %s: %s", w->path.c_str(), strerror(errno));
    }
    void* map = mmap(nullptr, (size_t)total, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
    ::close(fd);
    if (map == MAP_FAILED) return fail(BCS_ERR_IO, "cannot map %s: %s", w->path.c_str(), strerror(errno));
    uint8_t* base = (uint8_t*)map;
    std::memcpy(base, head.data(), head.size());

    // Work items are (tensor, run of rows); threads pull them from a shared counter.
    struct Item { uint32_t tensor; uint64_t row0, row1; };
    std::vector<Item> items;
    for (uint32_t ti = 0; ti < w->tensors.size(); ++ti) {
        const TensorSpec& t = w->tensors[ti];
        uint64_t rows_per = std::max<uint64_t>(1, (1u << 20) / std::max<uint64_t>(1, t.n_cols));
        for (uint64_t r = 0; r < t.n_rows; r += rows_per) items.push_back({ti, r, std::min(t.n_rows, r + rows_per)});
    }
    std::atomic<size_t> next{0};
    unsigned n_threads = std::max(1u, std::thread::hardware_concurrency());
    cpu_set_t set;
    if (sched_getaffinity(0, sizeof set, &set) == 0) n_threads = std::max(1, CPU_COUNT(&set));
    auto worker = [&]() {
        std::vector<float> scratch;
        for (;;) {
            size_t i = next.fetch_add(1);
            if (i >= items.size()) break;
            const Item& it = items[i];
            const TensorSpec& t = w->tensors[it.tensor];
            scratch.resize(t.n_cols);
            for (uint64_t r = it.row0; r < it.row1; ++r)
                fill_row(t, w->seed, it.tensor, r, scratch.data(), base + data_start + t.offset + r * t.row_bytes);
        }
    };
    std::vector<std::thread> threads;
    for (unsigned i = 1; i < n_threads; ++i) threads.emplace_back(worker);
    worker();
    for (std::thread& t : threads) t.join();
    munmap(map, (size_t)total);
    return BCS_OK;
}

}  // extern "C"
