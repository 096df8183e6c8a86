// TEST INFRASTRUCTURE — NOT PRODUCT CODE.
//
// CPU restatement of bobcat's scalar reference ops (crates/bobcat/src/scalar.rs), used only as the
// parity checker by the tests, the smoke check and the benchmark's CPU-baseline leg. Nothing in
// the shipped library includes or links this file.
//
// Every function keeps the accumulation width the reference uses on the same line: sums the
// reference carries in f64 are carried in f64 here, f32 sums stay f32, and the transcendental
// calls go to the same libm entry points (expf, powf, sinf, cosf, log1pf, sqrt). Compile without
// FMA contraction (-ffp-contract=off) so a*b+c rounds twice, as the reference's build does.
#pragma once

#include <cmath>
#include <cstddef>
#include <cstdint>
#include <cstring>
#include <vector>

namespace oracle {

// ggml tensor type ids the reference reads (crates/bobcat-gguf/src/lib.rs:126-152).
enum : uint32_t { T_F32 = 0, T_F16 = 1, T_Q4_0 = 2, T_Q8_0 = 8, T_Q6K = 14, T_BF16 = 30 };

// Elements and bytes of one block of `type` (crates/bobcat-gguf/src/lib.rs:156-166).
inline bool block_of(uint32_t type, size_t* elements, size_t* bytes) {
    switch (type) {
        case T_F32: *elements = 1; *bytes = 4; return true;
        case T_F16: case T_BF16: *elements = 1; *bytes = 2; return true;
        case T_Q4_0: *elements = 32; *bytes = 18; return true;
        case T_Q8_0: *elements = 32; *bytes = 34; return true;
        case T_Q6K: *elements = 256; *bytes = 210; return true;
        default: return false;
    }
}

// scalar.rs:28-31
inline size_t row_bytes(uint32_t type, size_t n_cols) {
    size_t e = 1, b = 4;
    block_of(type, &e, &b);
    return n_cols / e * b;
}

// IEEE binary16 -> binary32, exact (scalar.rs:18-20; the `half` crate's from_bits().to_f32()).
inline float f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {
            // Subnormal half: renormalise.
            int shift = 0;
            while ((man & 0x400u) == 0) { man <<= 1; ++shift; }
            man &= 0x3ffu;
            bits = sign | ((uint32_t)(127 - 15 - shift + 1) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7f800000u | (man << 13);
    } else {
        bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    std::memcpy(&f, &bits, 4);
    return f;
}

// scalar.rs:23-25
inline float bf16_to_f32(uint16_t h) {
    uint32_t bits = (uint32_t)h << 16;
    float f;
    std::memcpy(&f, &bits, 4);
    return f;
}

inline uint16_t le16(const uint8_t* p) { return (uint16_t)(p[0] | (p[1] << 8)); }

// scalar.rs:98-105 — fp16 scale, 16 bytes; low nibbles are elements 0..15, high nibbles 16..31,
// each offset by 8; one f32 multiply per element.
inline void dequantize_q4_0(const uint8_t* block, float* out) {
    float d = f16_to_f32(le16(block));
    for (int i = 0; i < 16; ++i) {
        uint8_t q = block[2 + i];
        out[i] = (float)((int16_t)(q & 0xf) - 8) * d;
        out[16 + i] = (float)((int16_t)(q >> 4) - 8) * d;
    }
}

// scalar.rs:108-113
inline void dequantize_q8_0(const uint8_t* block, float* out) {
    float d = f16_to_f32(le16(block));
    for (int i = 0; i < 32; ++i) out[i] = (float)(int8_t)block[2 + i] * d;
}

// scalar.rs:175-202 — a super-block of 256: 128 bytes of low 4-bit halves, 64 bytes of high 2-bit
// pairs, 16 int8 scales of 16-element blocks, then an fp16 d. Each half spreads 128 elements over
// 64 low bytes and 32 high bytes; value = (d * f32(scale)) * f32(quant - 32).
inline void dequantize_q6k(const uint8_t* block, float* out) {
    float d = f16_to_f32(le16(block + 208));
    for (int half = 0; half < 2; ++half) {
        const uint8_t* low = block + half * 64;
        const uint8_t* high = block + 128 + half * 32;
        const int8_t* scales = reinterpret_cast<const int8_t*>(block + 192 + half * 8);
        float* o = out + half * 128;
        for (int l = 0; l < 32; ++l) {
            int is = l / 16;
            auto quant = [&](uint8_t lo, int shift) { return (float)((int16_t)(lo | (((high[l] >> shift) & 3) << 4)) - 32); };
            auto scale = [&](int index) { return d * (float)scales[index]; };
            o[l] = scale(is) * quant(low[l] & 0xf, 0);
            o[l + 32] = scale(is + 2) * quant(low[l + 32] & 0xf, 2);
            o[l + 64] = scale(is + 4) * quant(low[l] >> 4, 4);
            o[l + 96] = scale(is + 6) * quant(low[l + 32] >> 4, 6);
        }
    }
}

// scalar.rs:59-82 — `n` elements of `type` from `bytes` into `out`.
inline void dequantize(uint32_t type, const uint8_t* bytes, size_t n, float* out) {
    switch (type) {
        case T_F32: std::memcpy(out, bytes, n * 4); break;
        case T_F16: for (size_t i = 0; i < n; ++i) out[i] = f16_to_f32(le16(bytes + 2 * i)); break;
        case T_BF16: for (size_t i = 0; i < n; ++i) out[i] = bf16_to_f32(le16(bytes + 2 * i)); break;
        case T_Q4_0: for (size_t b = 0; b < n / 32; ++b) dequantize_q4_0(bytes + 18 * b, out + 32 * b); break;
        case T_Q8_0: for (size_t b = 0; b < n / 32; ++b) dequantize_q8_0(bytes + 34 * b, out + 32 * b); break;
        case T_Q6K: for (size_t b = 0; b < n / 256; ++b) dequantize_q6k(bytes + 210 * b, out + 256 * b); break;
        default: break;
    }
}

// scalar.rs:292-304 — products and running sum in f64, one rounding to f32.
inline float dot(const float* a, const float* b, size_t n) {
    double sum = 0.0;
    for (size_t i = 0; i < n; ++i) sum += (double)a[i] * (double)b[i];
    return (float)sum;
}

// scalar.rs:206-209
inline void get_row(uint32_t type, const uint8_t* weights, size_t row, size_t n_cols, float* out) {
    size_t bytes = row_bytes(type, n_cols);
    dequantize(type, weights + row * bytes, n_cols, out);
}

// scalar.rs:213-220 — dequantise each row to f32, then `dot`. Rows are independent, so running
// them on several threads leaves every row's summation order, and so every result bit, unchanged.
inline void matvec(uint32_t type, const uint8_t* weights, const float* x, size_t n_cols, float* y,
                   size_t n_rows, int threads) {
    size_t bytes = row_bytes(type, n_cols);
#pragma omp parallel num_threads(threads) if (threads > 1)
    {
        std::vector<float> row(n_cols);
#pragma omp for schedule(static)
        for (long r = 0; r < (long)n_rows; ++r) {
            dequantize(type, weights + (size_t)r * bytes, n_cols, row.data());
            y[r] = dot(row.data(), x, n_cols);
        }
    }
}

// scalar.rs:240-249 — mean of squares in f64, reciprocal square root in f64, rounded to f32.
inline float rms_scale(const float* x, size_t n, float eps) {
    double sum = 0.0;
    for (size_t i = 0; i < n; ++i) sum += (double)x[i] * (double)x[i];
    double mean = sum / (double)n;
    return (float)(1.0 / std::sqrt(mean + (double)eps));
}

// scalar.rs:224-237 — note the order w * (x * scale).
inline void rms_norm(const float* x, const float* w, size_t n, float eps, float* out) {
    float scale = rms_scale(x, n, eps);
    for (size_t i = 0; i < n; ++i) out[i] = w[i] * (x[i] * scale);
}

// scalar.rs:253-266 — NeoX pairing (i, i + len/2); frequencies and angles in f32.
inline void rope_neox(float* vec, size_t len, uint32_t pos, float theta) {
    size_t half = len / 2;
    for (size_t i = 0; i < half; ++i) {
        float inv_freq = 1.0f / powf(theta, (float)(2 * i) / (float)len);
        float angle = (float)pos * inv_freq;
        float s = sinf(angle), c = cosf(angle);
        float a = vec[i], b = vec[i + half];
        vec[i] = a * c - b * s;
        vec[i + half] = b * c + a * s;
    }
}

// scalar.rs:269-271
inline float silu(float x) { return x / (1.0f + expf(-x)); }

// scalar.rs:274-289 — max in f32, exponentials in f32, their sum in f64, quotient rounded to f32.
inline void softmax(float* x, size_t n) {
    float max = -INFINITY;
    for (size_t i = 0; i < n; ++i) max = fmaxf(max, x[i]);
    double sum = 0.0;
    for (size_t i = 0; i < n; ++i) {
        x[i] = expf(x[i] - max);
        sum += (double)x[i];
    }
    for (size_t i = 0; i < n; ++i) x[i] = (float)((double)x[i] / sum);
}

}  // namespace oracle
