/*
 * CPU oracle for the affine-Q4 projection path -- TEST INFRASTRUCTURE ONLY.
 *
 * This is a plain-C restatement of the arithmetic the reference (Fuxx-1/qwen38-metal)
 * performs on this path. It is a checker: only the tests, the smoke check and the
 * benchmark's CPU-baseline leg may link or call it; the product library never does.
 *
 * Pinning: the reference cannot be built or run outside macOS (Rust + Metal), and it
 * stores no literal output vectors for this path. The oracle is pinned to what the
 * reference's tests do hold: their deterministic fixture formulas, shape/alignment
 * matrix and tolerances (src/metal_runtime.rs:9332-10910), evaluated independently in
 * exact rational arithmetic and committed as fixtures (tests/golden/).
 *
 * Every function names the reference lines it follows (paths relative to the
 * reference repository root).
 */
#ifndef Q4_ORACLE_H
#define Q4_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define Q4O_GROUP 64u /* AFFINE_GROUP_SIZE, src/metal_runtime.rs (group of 64 inputs) */
#define Q4O_PER_WORD 8u /* VALUES_PER_PACKED_WORD: eight nibbles per little-endian u32 */

/* bf16 <-> f32. src/metal_runtime.rs:12128-12136, shaders/qwen38.metal:18-26 (RNE, no NaN case). */
uint16_t q4o_f32_to_bf16(float value);
float q4o_bf16_to_f32(uint16_t bits);

/* pack_q4, src/metal_runtime.rs:11962-11975: value i of a word sits at bits [4i, 4i+4). */
void q4o_pack(const uint8_t *q, size_t count, uint32_t *words);
/* inverse of q4o_pack; nibble order of shaders/qwen38.metal:28-43. */
void q4o_unpack(const uint32_t *words, size_t word_count, uint8_t *q);

/*
 * MLX-style affine quantisation of an fp32 [rows][cols] matrix, group of 64 along cols:
 * bias=min, scale=(max-min)/15, q=clamp(rint((w-bias)/scale),0,15) against the fp32
 * scale/bias; scale and bias are then stored as bf16 (RNE). max==min => scale=0, q=0.
 * (Benchmark recipe; the layout it produces is the one validated by
 * src/native.rs:5417-5471.)
 */
void q4o_quantize(const float *w, size_t rows, size_t cols, uint32_t *words,
                  uint16_t *scales, uint16_t *biases);

/*
 * cpu_q4_affine_matvec, src/metal_runtime.rs:11977-11997: w = q*scale + bias in fp32,
 * total += x*w sequentially over columns. x is [m][k], y is [m][n] row-major.
 * This is the reference's own CPU statement of the path.
 */
void q4o_matmul_dequant_f32(const float *x, size_t m, size_t k, const uint8_t *weights,
                            const uint8_t *scales, const uint8_t *biases, size_t n,
                            float *y);

/*
 * The kernel arithmetic, shaders/qwen38.metal:213-246 (qwen38_q4_affine_matvec_simd):
 * 32 lanes stride over the 64-groups; per group dot_sum = sum x*q and input_sum = sum x
 * are formed word by word (shaders/qwen38.metal:28-43, 61-76), then
 * sum += dot_sum*scale + input_sum*bias; the 32 lane sums are combined by an xor
 * butterfly (16, 8, 4, 2, 1), the order a warp shuffle reduction uses.
 * Pointers are byte pointers: any alignment is accepted
 * (shaders/qwen38.metal:105-115, byte-wise little-endian loads).
 */
void q4o_matmul_factored_f32(const float *x, size_t m, size_t k, const uint8_t *weights,
                             const uint8_t *scales, const uint8_t *biases, size_t n,
                             float *y);

/* Same sum with double accumulation of x*(q*scale+bias): separates order noise from error. */
void q4o_matmul_f64(const float *x, size_t m, size_t k, const uint8_t *weights,
                    const uint8_t *scales, const uint8_t *biases, size_t n, double *y);

/*
 * Dequantise-to-16-bit form of the matrix-core kernels, shaders/qwen38.metal:3806-3815 and
 * :4102-4125, with bf16 (RNE) in place of half: w = bf16(q*scale + bias), x = bf16(x),
 * fp32 accumulation in ascending k.
 */
void q4o_matmul_bf16_tiles(const float *x, size_t m, size_t k, const uint8_t *weights,
                           const uint8_t *scales, const uint8_t *biases, size_t n,
                           float *y);

/* qwen38_argmax_rows, shaders/qwen38.metal:4201-4245: greatest value, ties -> lowest index. */
void q4o_argmax_rows(const float *logits, size_t m, size_t n, uint32_t *tokens);

/* qwen38_swiglu_rows, shaders/qwen38.metal:4090-4096 and :4188-4198: g/(1+exp(-g)) * u. */
void q4o_swiglu(const float *gate, const float *up, size_t count, float *out);

/*
 * q4_affine_mlp_mapped_batch, src/metal_runtime.rs:4479-4689: gate,up -> swiglu -> down.
 * form: 0 = factored fp32 (decode chain), 1 = bf16 tiles with the intermediate rounded
 * to bf16 before the down projection (tensor-core chain).
 */
void q4o_mlp(const float *x, size_t m, size_t k, const uint8_t *gate_w, const uint8_t *gate_s,
             const uint8_t *gate_b, const uint8_t *up_w, const uint8_t *up_s,
             const uint8_t *up_b, size_t inter, const uint8_t *down_w, const uint8_t *down_s,
             const uint8_t *down_b, size_t n, int form, float *y);

/* dequantized_row, src/native.rs:4944-4987: one row of q*scale+bias in fp32. */
void q4o_dequantize_row(const uint8_t *weights, const uint8_t *scales, const uint8_t *biases,
                        size_t k, size_t row, float *out);

/* Row-parallel (pthreads) driver around q4o_matmul_factored_f32 for the timed CPU baseline. */
void q4o_matmul_factored_f32_mt(const float *x, size_t m, size_t k, const uint8_t *weights,
                                const uint8_t *scales, const uint8_t *biases, size_t n,
                                float *y, int threads);
void q4o_matmul_bf16_tiles_mt(const float *x, size_t m, size_t k, const uint8_t *weights,
                              const uint8_t *scales, const uint8_t *biases, size_t n,
                              float *y, int threads);

/*
 * Seeded synthetic inputs (the benchmark's stand-in for a checkpoint; not reference code).
 * value(seed, tensor, index) = (sum of twelve 16-bit uniforms - 6*65535) / 65536: an
 * integer-only Irwin-Hall normal, so a GPU twin can reproduce it bit for bit.
 * The twelve uniforms are the 16-bit fields of three splitmix64 outputs
 * (splitmix64 as in src/native.rs:5293-5299).
 */
uint64_t q4o_splitmix64(uint64_t x);
float q4o_synth_normal(uint64_t seed, uint64_t tensor, uint64_t index);
/* weights ~ sigma * normal, quantised per q4o_quantize, rows [row0,row0+rows) of an [.][k] tensor */
void q4o_synth_q4_rows(uint64_t seed, uint64_t tensor, float sigma, size_t row0, size_t rows,
                       size_t k, uint32_t *words, uint16_t *scales, uint16_t *biases);
/* activations: bf16(normal) returned as bf16 bits */
void q4o_synth_bf16(uint64_t seed, uint64_t tensor, size_t count, uint16_t *out);

#ifdef __cplusplus
}
#endif
#endif
