// Kernel-side parameter blocks and launcher prototypes shared between the .cu files and the
// host runtime (q4_runtime.cu). Plain C structs: no CUDA types beyond cudaStream_t/cudaError_t.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace q4 {

constexpr int kMaxJobs = 12;

// One projection of a grouped launch (the device image of a MappedQ4AffineJob,
// src/metal_runtime.rs:155-192 of the reference, with shard ids resolved to pointers).
struct GemvJob {
    const uint8_t *w;      // packed weights, [n][k/8] u32, any byte alignment
    const uint8_t *s;      // scales, [n][k/64] bf16
    const uint8_t *b;      // biases, [n][k/64] bf16
    float *out;            // [m][out_stride] fp32
    uint32_t n;            // output rows
    uint32_t out_stride;   // elements between activation rows of `out`
    uint32_t tile_begin;   // first 16-row tile of this job in the launch
    uint32_t w_misalign;   // (uintptr_t)w & 15
    // persistent decode kernel only: a tile of this job counts as `vcpt` >= cpt units when the launch's work is cut
    // into equal ranges -- the units past cpt are empty, so projections whose chunks cost more (weights at a byte
    // offset) get proportionally fewer real chunks per warp; unit_begin = first unit of the job
    uint32_t vcpt;
    uint32_t unit_begin;
};

struct GemvParams {
    GemvJob jobs[kMaxJobs];
    uint32_t n_jobs;
    const uint16_t *xp;    // prepared activation columns, [v_cols][kp] fp16 in fragment order, row-scaled
    const float *xsum;     // [kp/64][vpad] per-group column sums
    const float *row_inv;  // [m_rows] inverse of the power-of-two row scaling
    uint32_t v_cols;       // activation columns in use (m_rows, or 3*m_rows for fp32 input)
    uint32_t vpad;         // 4 * column tiles
    uint32_t m_rows;       // activation rows
    uint32_t x_is_f32;     // columns are hi/mid/lo splits of fp32 rows
    uint32_t accumulate;   // out += projection (residual form) instead of out = projection
    uint32_t k;            // input elements
    uint32_t kp;           // k rounded up to 128 (row stride of xp)
    uint32_t groups;       // k / 64
    uint32_t cpt;          // K-chunks (128 inputs) per tile = ceil(groups / 2)
    uint32_t workers;      // warps (= blocks) in the grid
    uint64_t units;        // tiles * cpt
    float *partials;       // [workers][2][column tiles][32][4] fp32 scratch for split tiles
    unsigned int *counters;  // [workers], zero between launches
    unsigned long long *trace;  // optional [workers][4] globaltimer stamps (start, first data, loop end, done); may be null
    // Row-sharded multi-GPU runs: mirror[job * kMaxPeers + r] is where rank r keeps the same output rows
    // (peer memory), or null; every result is stored there too. Null table on one GPU.
    float *const *mirror;
    uint32_t world, rank;
};

constexpr int kMaxPeers = 8;

// Short-batch kernel (q4_gemv_rows.cu): up to 16 activation rows, all tensors on 16-byte boundaries, K % 128 == 0.
struct RowsJob {
    const uint8_t *w, *s, *b;
    float *out;            // [m][out_stride] fp32
    uint32_t n;            // output rows
    uint32_t out_stride;
    uint32_t tile_begin;   // first 16-row tile of this job in the launch
    uint32_t pad;
};

struct RowsParams {
    RowsJob jobs[kMaxJobs];
    uint32_t n_jobs;
    uint32_t m;            // activation rows, 1..16
    const void *x;         // [m][k] bf16 or fp32, 16-byte aligned
    uint32_t x_is_f32;
    uint32_t k, groups, cpt;  // inputs, k / 64, k / 128
    uint32_t parts;        // runs the K range is cut into (q4k_rows_plan)
    uint32_t part_chunks;  // chunks of the longest run
    uint32_t tiles_per_warp;  // 1, or 2 (up to 8 rows): two tiles share the activation's fragments
    uint32_t tiles;        // 16-row tiles of all jobs
    uint32_t accumulate;
    float *partials;       // [parts][8 or 16][tiles * 16] fp32, used when parts > 1
    unsigned int *counters;  // [tiles], zero between launches
    unsigned long long *trace;  // optional [warps of the grid][4] globaltimer stamps (start, digits ready, first tile streamed, done)
};

}  // namespace q4

extern "C" {
cudaError_t q4k_prepare_x(const void *x, int x_is_f32, uint32_t m_rows, uint32_t k, uint32_t kp, uint32_t vpad,
                          uint16_t *xp, float *xsum, float *row_inv, cudaStream_t stream);
cudaError_t q4k_gemv(const q4::GemvParams *params, int column_tiles, int aligned, cudaStream_t stream);  // one warp per block
uint32_t q4k_gemv_occupancy(int column_tiles, int aligned);  // resident warps per SM, 0 on error

uint32_t q4k_rows_plan(uint32_t m, uint32_t k, uint32_t tiles, uint32_t sm_count, uint32_t *part_chunks, uint32_t *tiles_per_warp);  // parts, 0: unsupported
cudaError_t q4k_rows(const q4::RowsParams *params, uint32_t sm_count, cudaStream_t stream);

cudaError_t q4k_swiglu(const float *gate, const float *up, uint64_t count, float *out_f32, uint16_t *out_bf16,
                       cudaStream_t stream);
cudaError_t q4k_f32_to_bf16(const float *in, uint64_t count, uint16_t *out, cudaStream_t stream);
uint32_t q4k_argmax_parts(uint32_t n);
cudaError_t q4k_argmax_rows(const float *logits, uint32_t m, uint32_t n, uint32_t index_base, float *pv, uint32_t *pi,
                            uint32_t *tokens, float *values, cudaStream_t stream);
cudaError_t q4k_rms_unit_bf16(const float *in, uint32_t rows, uint32_t n, float eps, uint16_t *out, cudaStream_t stream);
cudaError_t q4k_dequantize_row(const uint8_t *w, const uint8_t *s, const uint8_t *b, uint32_t k, uint32_t row, float *out,
                               cudaStream_t stream);

cudaError_t q4k_gemm_prepare_x(const void *x, int x_is_f32, uint64_t elements, uint16_t *xp, cudaStream_t stream);
uint32_t q4k_gemm_tile_m(uint32_t m);
uint32_t q4k_gemm_k_splits(uint32_t m, uint32_t n, uint32_t k, uint32_t sm_count, uint32_t *split_blocks);
cudaError_t q4k_gemm_tc(const uint16_t *xp, uint32_t m, uint32_t k, const uint8_t *w, const uint8_t *s, const uint8_t *b,
                        uint32_t n, float *out, uint32_t out_stride, int accumulate, int *error_flag, uint32_t sm_count,
                        float *parts, cudaStream_t stream);

int q4k_gemm_pair_supported(const uint8_t *w_gate, const uint8_t *w_up);
cudaError_t q4k_gemm_tc_pair(const uint16_t *xp, uint32_t m, uint32_t k, const uint8_t *wg, const uint8_t *sg, const uint8_t *bg,
                             const uint8_t *wu, const uint8_t *su, const uint8_t *bu, uint32_t n, uint16_t *h_out, uint32_t h_stride,
                             int *error_flag, uint32_t sm_count, cudaStream_t stream);

cudaError_t q4k_synth_q4(uint64_t seed, uint64_t tensor, float sigma, uint64_t row0, uint64_t rows, uint32_t k,
                         uint8_t *w, uint8_t *s, uint8_t *b, cudaStream_t stream);
cudaError_t q4k_synth_bf16(uint64_t seed, uint64_t tensor, uint64_t count, uint16_t *out, cudaStream_t stream);
}
