/*
 * TEST INFRASTRUCTURE — scalar C restatement of the CPU reference loops that the
 * reference's own op tests check its kernels against.  Never linked into the
 * product library.  Paths are relative to the reference root.
 *
 *   orc_rmsnorm_f32        tests/ops/test_reduce.cu:21-26
 *   orc_rmsnorm_bf16       tests/ops/test_reduce.cu:28-41   (x and w quantised to bf16, output rounded)
 *   orc_gated_f32          tests/ops/test_reduce.cu:47-62
 *   orc_gated_bf16         tests/ops/test_reduce.cu:64-87
 *   orc_relu2_f32          tests/ops/test_elementwise.cu:32-34
 *   orc_add_f32            tests/ops/test_elementwise.cu (operator+ on floats, :143)
 *   orc_embedding_u16      tests/ops/test_embedding.cu:22-31 (row copy, any 16-bit payload)
 *
 * Like the originals these work on float arrays; the *_bf16 forms round through
 * bf16 (round to nearest even) where the original calls __float2bfloat16_rn.
 */
#include <math.h>
#include <stdint.h>
#include <string.h>
#include <stddef.h>

static float bf16_round(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) {          /* NaN stays NaN */
        u |= 0x00400000u;
        u &= 0xffff0000u;
    } else {
        u += 0x7fffu + ((u >> 16) & 1u);            /* round to nearest, ties to even */
        u &= 0xffff0000u;
    }
    memcpy(&f, &u, 4);
    return f;
}

float orc_bf16_round(float f) { return bf16_round(f); }

static float silu(float z) { return z / (1.0f + expf(-z)); }

void orc_rmsnorm_f32(const float* x, float* y, const float* w, size_t rows, size_t n, float eps) {
    for (size_t r = 0; r < rows; ++r, x += n, y += n) {
        float acc = 0.f;
        for (size_t i = 0; i < n; ++i) acc += x[i] * x[i];
        const float scale = 1.0f / sqrtf(acc / (float)n + eps);
        for (size_t i = 0; i < n; ++i) y[i] = x[i] * scale * w[i];
    }
}

void orc_rmsnorm_bf16(const float* x, float* y, const float* w, size_t rows, size_t n, float eps) {
    for (size_t r = 0; r < rows; ++r, x += n, y += n) {
        float acc = 0.f;
        for (size_t i = 0; i < n; ++i) { const float q = bf16_round(x[i]); acc += q * q; }
        const float scale = 1.0f / sqrtf(acc / (float)n + eps);
        for (size_t i = 0; i < n; ++i) y[i] = bf16_round(bf16_round(x[i]) * scale * bf16_round(w[i]));
    }
}

void orc_gated_f32(const float* x, float* y, const float* w, const float* gate,
                   size_t rows, size_t cols, size_t group_size, float eps) {
    const size_t groups = cols / group_size;
    for (size_t r = 0; r < rows; ++r, x += cols, y += cols, gate += cols) {
        for (size_t g = 0; g < groups; ++g) {
            const size_t lo = g * group_size, hi = lo + group_size;
            float acc = 0.f;
            for (size_t i = lo; i < hi; ++i) { const float v = x[i] * silu(gate[i]); acc += v * v; }
            const float scale = 1.0f / sqrtf(acc / (float)group_size + eps);
            for (size_t i = lo; i < hi; ++i) y[i] = x[i] * silu(gate[i]) * scale * w[i];
        }
    }
}

void orc_gated_bf16(const float* x, float* y, const float* w, const float* gate,
                    size_t rows, size_t cols, size_t group_size, float eps) {
    const size_t groups = cols / group_size;
    for (size_t r = 0; r < rows; ++r, x += cols, y += cols, gate += cols) {
        for (size_t g = 0; g < groups; ++g) {
            const size_t lo = g * group_size, hi = lo + group_size;
            float acc = 0.f;
            for (size_t i = lo; i < hi; ++i) {
                const float v = bf16_round(x[i]) * silu(bf16_round(gate[i]));
                acc += v * v;
            }
            const float scale = 1.0f / sqrtf(acc / (float)group_size + eps);
            for (size_t i = lo; i < hi; ++i) {
                const float v = bf16_round(x[i]) * silu(bf16_round(gate[i]));
                y[i] = bf16_round(v * scale * bf16_round(w[i]));
            }
        }
    }
}

void orc_relu2_f32(const float* x, float* y, size_t n) {
    for (size_t i = 0; i < n; ++i) y[i] = x[i] > 0.f ? x[i] * x[i] : 0.f;
}

void orc_add_f32(const float* a, const float* b, float* y, size_t n) {
    for (size_t i = 0; i < n; ++i) y[i] = a[i] + b[i];
}

void orc_embedding_u16(const uint16_t* table, const int64_t* ids, uint16_t* out, size_t num_tokens, size_t hidden) {
    for (size_t t = 0; t < num_tokens; ++t)
        memcpy(out + t * hidden, table + (size_t)ids[t] * hidden, hidden * sizeof(uint16_t));
}
