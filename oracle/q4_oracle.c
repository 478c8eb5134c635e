/*
 * CPU oracle for the affine-Q4 projection path -- TEST INFRASTRUCTURE ONLY.
 * See q4_oracle.h for what this file is pinned to and who may call it.
 * Build: make -C oracle   (gcc -O3 -ffp-contract=off, so no product is fused into an add
 * behind the source's back and the fp32 sums below are exactly the ones written).
 */
#include "q4_oracle.h"

#include <math.h>
#include <pthread.h>
#include <stdlib.h>
#include <string.h>

/* ---- bf16 helpers: src/metal_runtime.rs:12128-12136, shaders/qwen38.metal:18-26 ---- */

uint16_t q4o_f32_to_bf16(float value) {
    uint32_t bits;
    memcpy(&bits, &value, 4);
    uint32_t rounded = bits + (0x7fffu + ((bits >> 16) & 1u));
    return (uint16_t)(rounded >> 16);
}

float q4o_bf16_to_f32(uint16_t v) {
    uint32_t bits = (uint32_t)v << 16;
    float out;
    memcpy(&out, &bits, 4);
    return out;
}

/* byte-wise little-endian loads, shaders/qwen38.metal:105-115 */
static inline uint32_t load_u32(const uint8_t *p) {
    return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24);
}
static inline uint16_t load_u16(const uint8_t *p) {
    return (uint16_t)((uint16_t)p[0] | ((uint16_t)p[1] << 8));
}

/* ---- packing: src/metal_runtime.rs:11962-11975 ---- */

void q4o_pack(const uint8_t *q, size_t count, uint32_t *words) {
    for (size_t w = 0; w < count / Q4O_PER_WORD; ++w) {
        uint32_t packed = 0;
        for (unsigned i = 0; i < Q4O_PER_WORD; ++i) {
            packed |= (uint32_t)(q[w * Q4O_PER_WORD + i] & 0xFu) << (i * 4u);
        }
        words[w] = packed;
    }
}

void q4o_unpack(const uint32_t *words, size_t word_count, uint8_t *q) {
    for (size_t w = 0; w < word_count; ++w) {
        for (unsigned i = 0; i < Q4O_PER_WORD; ++i) {
            q[w * Q4O_PER_WORD + i] = (uint8_t)((words[w] >> (i * 4u)) & 0xFu);
        }
    }
}

/* ---- quantiser (benchmark recipe) ---- */

static void quantize_group(const float *w, uint32_t *words, uint16_t *scale_out, uint16_t *bias_out) {
    float lo = w[0], hi = w[0];
    for (unsigned i = 1; i < Q4O_GROUP; ++i) {
        lo = w[i] < lo ? w[i] : lo;
        hi = w[i] > hi ? w[i] : hi;
    }
    float scale = (hi - lo) / 15.0f;
    float bias = lo;
    for (unsigned word = 0; word < Q4O_GROUP / Q4O_PER_WORD; ++word) {
        uint32_t packed = 0;
        for (unsigned i = 0; i < Q4O_PER_WORD; ++i) {
            float q = 0.0f;
            if (scale != 0.0f) {
                q = rintf((w[word * Q4O_PER_WORD + i] - bias) / scale); /* ties to even */
                q = q < 0.0f ? 0.0f : (q > 15.0f ? 15.0f : q);
            }
            packed |= (uint32_t)q << (i * 4u);
        }
        words[word] = packed;
    }
    *scale_out = q4o_f32_to_bf16(scale);
    *bias_out = q4o_f32_to_bf16(bias);
}

void q4o_quantize(const float *w, size_t rows, size_t cols, uint32_t *words, uint16_t *scales,
                  uint16_t *biases) {
    size_t groups = cols / Q4O_GROUP;
    for (size_t r = 0; r < rows; ++r) {
        for (size_t g = 0; g < groups; ++g) {
            quantize_group(w + r * cols + g * Q4O_GROUP, words + r * (cols / 8) + g * 8,
                           scales + r * groups + g, biases + r * groups + g);
        }
    }
}

/* ---- reference CPU form: src/metal_runtime.rs:11977-11997 ---- */

static void rows_dequant_f32(const float *x, size_t m, size_t k, const uint8_t *weights,
                             const uint8_t *scales, const uint8_t *biases, size_t n,
                             size_t row0, size_t row1, float *y) {
    size_t groups = k / Q4O_GROUP;
    for (size_t b = 0; b < m; ++b) {
        const float *xr = x + b * k;
        for (size_t row = row0; row < row1; ++row) {
            float total = 0.0f;
            for (size_t col = 0; col < k; ++col) {
                size_t p = row * groups + col / Q4O_GROUP;
                float scale = q4o_bf16_to_f32(load_u16(scales + 2 * p));
                float bias = q4o_bf16_to_f32(load_u16(biases + 2 * p));
                uint32_t word = load_u32(weights + 4 * (row * (k / 8) + col / 8));
                float weight = (float)((word >> ((col % 8) * 4)) & 0xFu) * scale + bias;
                total = total + xr[col] * weight;
            }
            y[b * n + row] = total;
        }
    }
}

void q4o_matmul_dequant_f32(const float *x, size_t m, size_t k, const uint8_t *weights,
                            const uint8_t *scales, const uint8_t *biases, size_t n, float *y) {
    rows_dequant_f32(x, m, k, weights, scales, biases, n, 0, n, y);
}

/* ---- kernel form: shaders/qwen38.metal:213-246 with helpers :28-43, :61-76 ---- */

static inline float word_dot(uint32_t packed, const float *x) {
    /* dot(values0, quantized0) + dot(values1, quantized1), shaders/qwen38.metal:28-43 */
    float d0 = x[0] * (float)(packed & 0xFu);
    d0 = d0 + x[1] * (float)((packed >> 4) & 0xFu);
    d0 = d0 + x[2] * (float)((packed >> 8) & 0xFu);
    d0 = d0 + x[3] * (float)((packed >> 12) & 0xFu);
    float d1 = x[4] * (float)((packed >> 16) & 0xFu);
    d1 = d1 + x[5] * (float)((packed >> 20) & 0xFu);
    d1 = d1 + x[6] * (float)((packed >> 24) & 0xFu);
    d1 = d1 + x[7] * (float)((packed >> 28) & 0xFu);
    return d0 + d1;
}

static void rows_factored_f32(const float *x, size_t m, size_t k, const uint8_t *weights,
                              const uint8_t *scales, const uint8_t *biases, size_t n,
                              size_t row0, size_t row1, float *y) {
    size_t groups = k / Q4O_GROUP;
    size_t words_per_row = k / 8;
    for (size_t b = 0; b < m; ++b) {
        const float *xr = x + b * k;
        for (size_t row = row0; row < row1; ++row) {
            float lanes[32];
            for (unsigned lane = 0; lane < 32; ++lane) {
                float sum = 0.0f;
                for (size_t group = lane; group < groups; group += 32) {
                    float scale = q4o_bf16_to_f32(load_u16(scales + 2 * (row * groups + group)));
                    float bias = q4o_bf16_to_f32(load_u16(biases + 2 * (row * groups + group)));
                    const uint8_t *wp = weights + 4 * (row * words_per_row + group * 8);
                    const float *xp = xr + group * Q4O_GROUP;
                    float dot_sum = 0.0f, input_sum = 0.0f;
                    for (unsigned word = 0; word < 8; ++word) {
                        const float *xw = xp + word * 8;
                        dot_sum += word_dot(load_u32(wp + 4 * word), xw);
                        input_sum += xw[0] + xw[1] + xw[2] + xw[3] + xw[4] + xw[5] + xw[6] + xw[7];
                    }
                    sum += dot_sum * scale + input_sum * bias;
                }
                lanes[lane] = sum;
            }
            /* simd_sum as an xor butterfly: the order of a warp __shfl_xor reduction */
            for (unsigned offset = 16; offset > 0; offset >>= 1) {
                float next[32];
                for (unsigned lane = 0; lane < 32; ++lane) next[lane] = lanes[lane] + lanes[lane ^ offset];
                memcpy(lanes, next, sizeof lanes);
            }
            y[b * n + row] = lanes[0];
        }
    }
}

void q4o_matmul_factored_f32(const float *x, size_t m, size_t k, const uint8_t *weights,
                             const uint8_t *scales, const uint8_t *biases, size_t n, float *y) {
    rows_factored_f32(x, m, k, weights, scales, biases, n, 0, n, y);
}

void q4o_matmul_f64(const float *x, size_t m, size_t k, const uint8_t *weights,
                    const uint8_t *scales, const uint8_t *biases, size_t n, double *y) {
    size_t groups = k / Q4O_GROUP;
    for (size_t b = 0; b < m; ++b) {
        for (size_t row = 0; row < n; ++row) {
            double total = 0.0;
            for (size_t col = 0; col < k; ++col) {
                size_t p = row * groups + col / Q4O_GROUP;
                double scale = q4o_bf16_to_f32(load_u16(scales + 2 * p));
                double bias = q4o_bf16_to_f32(load_u16(biases + 2 * p));
                uint32_t word = load_u32(weights + 4 * (row * (k / 8) + col / 8));
                double weight = (double)((word >> ((col % 8) * 4)) & 0xFu) * scale + bias;
                total += (double)x[b * k + col] * weight;
            }
            y[b * n + row] = total;
        }
    }
}

/* ---- 16-bit tile form: shaders/qwen38.metal:3806-3815, :4102-4125 (bf16 for half) ---- */

static void rows_bf16_tiles(const float *x, size_t m, size_t k, const uint8_t *weights,
                            const uint8_t *scales, const uint8_t *biases, size_t n, size_t row0,
                            size_t row1, float *y) {
    size_t groups = k / Q4O_GROUP;
    float *wrow = (float *)malloc(k * sizeof(float));
    float *xb = (float *)malloc(m * k * sizeof(float));
    for (size_t i = 0; i < m * k; ++i) xb[i] = q4o_bf16_to_f32(q4o_f32_to_bf16(x[i]));
    for (size_t row = row0; row < row1; ++row) {
        for (size_t col = 0; col < k; ++col) {
            size_t p = row * groups + col / Q4O_GROUP;
            float scale = q4o_bf16_to_f32(load_u16(scales + 2 * p));
            float bias = q4o_bf16_to_f32(load_u16(biases + 2 * p));
            uint32_t word = load_u32(weights + 4 * (row * (k / 8) + col / 8));
            float q = (float)((word >> ((col % 8) * 4)) & 0xFu);
            wrow[col] = q4o_bf16_to_f32(q4o_f32_to_bf16(q * scale + bias));
        }
        for (size_t b = 0; b < m; ++b) {
            const float *xr = xb + b * k;
            float total = 0.0f;
            for (size_t col = 0; col < k; ++col) total += xr[col] * wrow[col];
            y[b * n + row] = total;
        }
    }
    free(wrow);
    free(xb);
}

void q4o_matmul_bf16_tiles(const float *x, size_t m, size_t k, const uint8_t *weights,
                           const uint8_t *scales, const uint8_t *biases, size_t n, float *y) {
    rows_bf16_tiles(x, m, k, weights, scales, biases, n, 0, n, y);
}

/* ---- epilogue ops ---- */

void q4o_argmax_rows(const float *logits, size_t m, size_t n, uint32_t *tokens) {
    /* shaders/qwen38.metal:4213-4221: value > best, or equal with a lower index */
    for (size_t b = 0; b < m; ++b) {
        float best = -INFINITY;
        uint32_t best_index = 0;
        for (size_t i = 0; i < n; ++i) {
            float v = logits[b * n + i];
            if (v > best || (v == best && (uint32_t)i < best_index)) {
                best = v;
                best_index = (uint32_t)i;
            }
        }
        tokens[b] = best_index;
    }
}

void q4o_swiglu(const float *gate, const float *up, size_t count, float *out) {
    /* qwen38_silu(gate) * up with sigmoid = 1/(1+exp(-v)), shaders/qwen38.metal:4090-4096 */
    for (size_t i = 0; i < count; ++i) {
        float sig = 1.0f / (1.0f + expf(-gate[i]));
        out[i] = (gate[i] * sig) * up[i];
    }
}

void q4o_mlp(const float *x, size_t m, size_t k, const uint8_t *gate_w, const uint8_t *gate_s,
             const uint8_t *gate_b, const uint8_t *up_w, const uint8_t *up_s, const uint8_t *up_b,
             size_t inter, const uint8_t *down_w, const uint8_t *down_s, const uint8_t *down_b,
             size_t n, int form, float *y) {
    float *g = (float *)malloc(m * inter * sizeof(float));
    float *u = (float *)malloc(m * inter * sizeof(float));
    float *h = (float *)malloc(m * inter * sizeof(float));
    if (form == 0) {
        q4o_matmul_factored_f32(x, m, k, gate_w, gate_s, gate_b, inter, g);
        q4o_matmul_factored_f32(x, m, k, up_w, up_s, up_b, inter, u);
        q4o_swiglu(g, u, m * inter, h);
        q4o_matmul_factored_f32(h, m, inter, down_w, down_s, down_b, n, y);
    } else {
        q4o_matmul_bf16_tiles(x, m, k, gate_w, gate_s, gate_b, inter, g);
        q4o_matmul_bf16_tiles(x, m, k, up_w, up_s, up_b, inter, u);
        q4o_swiglu(g, u, m * inter, h);
        q4o_matmul_bf16_tiles(h, m, inter, down_w, down_s, down_b, n, y);
    }
    free(g);
    free(u);
    free(h);
}

void q4o_dequantize_row(const uint8_t *weights, const uint8_t *scales, const uint8_t *biases,
                        size_t k, size_t row, float *out) {
    size_t groups = k / Q4O_GROUP;
    for (size_t i = 0; i < k; ++i) {
        uint32_t word = load_u32(weights + 4 * (row * (k / 8) + i / 8));
        float q = (float)((word >> ((i % 8) * 4)) & 0xFu);
        size_t p = row * groups + i / Q4O_GROUP;
        out[i] = q * q4o_bf16_to_f32(load_u16(scales + 2 * p)) + q4o_bf16_to_f32(load_u16(biases + 2 * p));
    }
}

/* ---- threaded drivers (timed CPU baseline) ---- */

typedef void (*rows_fn)(const float *, size_t, size_t, const uint8_t *, const uint8_t *,
                        const uint8_t *, size_t, size_t, size_t, float *);
struct span {
    rows_fn fn;
    const float *x;
    size_t m, k;
    const uint8_t *w, *s, *b;
    size_t n, row0, row1;
    float *y;
};
static void *span_main(void *arg) {
    struct span *t = (struct span *)arg;
    t->fn(t->x, t->m, t->k, t->w, t->s, t->b, t->n, t->row0, t->row1, t->y);
    return NULL;
}
static void run_mt(rows_fn fn, const float *x, size_t m, size_t k, const uint8_t *w, const uint8_t *s,
                   const uint8_t *b, size_t n, float *y, int threads) {
    if (threads < 1) threads = 1;
    if ((size_t)threads > n) threads = (int)n;
    pthread_t *ids = (pthread_t *)malloc(sizeof(pthread_t) * (size_t)threads);
    struct span *spans = (struct span *)malloc(sizeof(struct span) * (size_t)threads);
    for (int t = 0; t < threads; ++t) {
        struct span sp = {fn, x, m, k, w, s, b, n, n * (size_t)t / (size_t)threads,
                          n * (size_t)(t + 1) / (size_t)threads, y};
        spans[t] = sp;
        pthread_create(&ids[t], NULL, span_main, &spans[t]);
    }
    for (int t = 0; t < threads; ++t) pthread_join(ids[t], NULL);
    free(ids);
    free(spans);
}

void q4o_matmul_factored_f32_mt(const float *x, size_t m, size_t k, const uint8_t *weights,
                                const uint8_t *scales, const uint8_t *biases, size_t n, float *y,
                                int threads) {
    run_mt(rows_factored_f32, x, m, k, weights, scales, biases, n, y, threads);
}

void q4o_matmul_bf16_tiles_mt(const float *x, size_t m, size_t k, const uint8_t *weights,
                              const uint8_t *scales, const uint8_t *biases, size_t n, float *y,
                              int threads) {
    run_mt(rows_bf16_tiles, x, m, k, weights, scales, biases, n, y, threads);
}

/* ---- seeded synthetic inputs ---- */

uint64_t q4o_splitmix64(uint64_t value) {
    /* src/native.rs:5293-5299 */
    value += 0x9e3779b97f4a7c15ull;
    uint64_t z = value;
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    return z ^ (z >> 31);
}

float q4o_synth_normal(uint64_t seed, uint64_t tensor, uint64_t index) {
    uint64_t base = q4o_splitmix64(seed ^ q4o_splitmix64(tensor));
    int32_t total = 0;
    for (uint64_t j = 0; j < 3; ++j) {
        uint64_t r = q4o_splitmix64(base ^ (index * 3u + j));
        total += (int32_t)(r & 0xffffu) + (int32_t)((r >> 16) & 0xffffu) +
                 (int32_t)((r >> 32) & 0xffffu) + (int32_t)((r >> 48) & 0xffffu);
    }
    return (float)(total - 6 * 65535) * (1.0f / 65536.0f);
}

void q4o_synth_q4_rows(uint64_t seed, uint64_t tensor, float sigma, size_t row0, size_t rows,
                       size_t k, uint32_t *words, uint16_t *scales, uint16_t *biases) {
    size_t groups = k / Q4O_GROUP;
    float w[Q4O_GROUP];
    for (size_t r = 0; r < rows; ++r) {
        for (size_t g = 0; g < groups; ++g) {
            uint64_t first = (uint64_t)(row0 + r) * k + g * Q4O_GROUP;
            for (unsigned i = 0; i < Q4O_GROUP; ++i) w[i] = sigma * q4o_synth_normal(seed, tensor, first + i);
            quantize_group(w, words + r * (k / 8) + g * 8, scales + r * groups + g, biases + r * groups + g);
        }
    }
}

void q4o_synth_bf16(uint64_t seed, uint64_t tensor, size_t count, uint16_t *out) {
    for (size_t i = 0; i < count; ++i) out[i] = q4o_f32_to_bf16(q4o_synth_normal(seed, tensor, i));
}
