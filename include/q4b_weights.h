/*
 * q4b_weights -- host side of the affine-Q4 projection path: the safetensors weight store and the
 * projection API the model code calls. C ABI over a C++ implementation that is itself a client of
 * q4b200.h (it uploads shards and launches projections only through those entry points).
 *
 * It replaces, in Fuxx-1/qwen38-metal (paths relative to that repository):
 *   MlxWeightStore / MlxTensor / open_mlx_safetensors_dir     src/model.rs:51-197, 312-459
 *   Q4AffineMatrix::{from_store, from_tensors}                src/native.rs:5383-5515
 *   NativeWeights::{open, q4_matrix, q4_affine_*_batch,
 *                   mapped_q4_jobs}                           src/native.rs:208-385
 *   dequantized_row                                           src/native.rs:4944-4987
 *
 * Not mirrored: the model manifest's geometry, model-type and MTP fields
 * (inspect_mlx_safetensors_dir, src/model.rs:199-298) -- they describe the transformer, not the
 * projection path. config.json is still required and its quantisation block is checked
 * (4-bit, affine, group size > 0), as the reference does before it opens any shard.
 *
 * Every function returns a q4b_status (q4b200.h); q4b_last_error() holds the message.
 */
#ifndef Q4B_WEIGHTS_H
#define Q4B_WEIGHTS_H

#include "q4b200.h"

#ifdef __cplusplus
extern "C" {
#endif

#define Q4B_MAX_TENSOR_RANK 8

/* MlxTensor, src/model.rs:58-65 */
typedef struct q4b_tensor_info {
    char dtype[16];                      /* safetensors dtype string, e.g. "U32", "BF16" */
    uint32_t rank;
    uint32_t shard_index;
    uint64_t shape[Q4B_MAX_TENSOR_RANK];
    uint64_t byte_offset;                /* from the start of the shard file: 8 + header length + data offset */
    uint64_t byte_len;
} q4b_tensor_info;

/* Q4AffineMatrix, src/native.rs:5383-5393. In a row-sharded view (q4b_weights_open_sharded) the three
 * tensors describe this rank's rows only: output_rows may then be 0, row_begin is the first global row
 * and total_rows the unsharded row count. */
typedef struct q4b_q4_matrix {
    q4b_tensor_info weight, scales, biases;
    uint64_t input_elements;             /* K = 8 * packed columns */
    uint64_t output_rows;                /* N (of this rank) */
    uint64_t row_begin;
    uint64_t total_rows;
} q4b_q4_matrix;

typedef struct q4b_store q4b_store;      /* MlxWeightStore */
typedef struct q4b_weights q4b_weights;  /* NativeWeights */

/* ---- weight store (host only; needs no GPU) ---- */

/* open_mlx_safetensors_dir, src/model.rs:136-197: reads config.json and model.safetensors.index.json,
 * groups the indexed tensors by shard file (shards are numbered in byte-wise name order), parses and
 * validates every shard header (length <= 128 MiB and <= file size - 8; dtype and shape present;
 * data offsets ordered and inside the data section), checks that every quantised ".weight" has both
 * or neither of ".scales"/".biases", and maps each shard read-only. Shard names that are absolute or
 * contain anything but plain components are refused. */
int q4b_store_open(const char *directory, q4b_store **out);
void q4b_store_close(q4b_store *store);
int q4b_store_tensor_count(const q4b_store *store, uint64_t *out);            /* MlxWeightStore::tensor_count */
int q4b_store_shard_count(const q4b_store *store, uint64_t *out);             /* ::shard_count */
int q4b_store_mapped_bytes(const q4b_store *store, uint64_t *out);            /* ::mapped_bytes */
int q4b_store_indexed_tensor_bytes(const q4b_store *store, uint64_t *out);    /* manifest.indexed_tensor_bytes */
int q4b_store_quantized_groups(const q4b_store *store, uint64_t *out);        /* manifest.quantized_tensor_groups */
int q4b_store_tensor(const q4b_store *store, const char *name, q4b_tensor_info *out);           /* ::tensor */
int q4b_store_tensor_name(const q4b_store *store, uint64_t index, const char **name);           /* names in sorted order */
int q4b_store_tensor_data(const q4b_store *store, const char *name, const void **data, uint64_t *len); /* ::tensor_data */
int q4b_store_shard_data(const q4b_store *store, uint64_t shard_index, const void **data, uint64_t *len); /* ::shard_data */
/* MlxWeightStore::tensor_values_f32, src/model.rs:87-112: BF16 or F32 tensors as fp32; `capacity` in elements. */
int q4b_store_tensor_values_f32(const q4b_store *store, const char *name, float *out, uint64_t capacity, uint64_t *count);

/* Q4AffineMatrix::from_store, src/native.rs:5396-5417 */
int q4b_store_q4_matrix(const q4b_store *store, const char *weight_name, q4b_q4_matrix *out);
/* Q4AffineMatrix::from_tensors, src/native.rs:5419-5471: weight U32 [N][K/8], K % 64 == 0, N > 0, exact byte
 * lengths; scales and biases BF16 [N][K/64]. */
int q4b_q4_matrix_from_tensors(const char *weight_name, const q4b_tensor_info *weight, const q4b_tensor_info *scales,
                               const q4b_tensor_info *biases, q4b_q4_matrix *out);

/* ---- weights resident in HBM ---- */

/* NativeWeights::open, src/native.rs:216-222 + MetalRuntime::map_weight_store, src/metal_runtime.rs:955-982:
 * opens the store and uploads every shard file byte for byte (one device allocation per shard, file offsets
 * kept, so a tensor misaligned in its file is misaligned in HBM). The host mappings stay open until close. */
int q4b_weights_open(q4b_runtime *rt, const char *directory, q4b_weights **out);
/* Row-sharded view for `world` GPUs: of every quantised projection this rank uploads rows
 * [floor(rank*N/world), floor((rank+1)*N/world)) of weight, scales and biases; all other tensors whole.
 * Each slice keeps its address modulo 16 from the file, so alignment-dependent kernel paths behave as they
 * would on the whole file. No reference counterpart (the reference runs on one GPU). */
int q4b_weights_open_sharded(q4b_runtime *rt, const char *directory, uint32_t rank, uint32_t world, q4b_weights **out);
void q4b_weights_close(q4b_weights *weights);
int q4b_weights_store(q4b_weights *weights, q4b_store **out);                 /* borrowed; closed with the weights */
int q4b_weights_shard_count(const q4b_weights *weights, uint64_t *out);       /* NativeWeights::mapped_shard_count */
int q4b_weights_device_bytes(const q4b_weights *weights, uint64_t *out);      /* bytes uploaded by this view */
int q4b_weights_q4_matrix(const q4b_weights *weights, const char *weight_name, q4b_q4_matrix *out); /* ::q4_matrix */
/* NativeWeights::mapped_q4_jobs, src/native.rs:325-382: checks K against every matrix, resolves the three
 * device shards and fills `aligned` from the device addresses (weights 4-byte, scales/biases 2-byte). */
int q4b_weights_jobs(const q4b_weights *weights, const q4b_q4_matrix *matrices, uint32_t n, uint64_t input_elements,
                     q4b_job *jobs);
/* NativeWeights::q4_affine_matvec_batch, src/native.rs:242-252: x fp32 [K]; outputs[j] fp32 [N_j]. */
int q4b_weights_matvec_batch(const q4b_weights *weights, const q4b_q4_matrix *matrices, uint32_t n, const float *x,
                             uint64_t x_len, float *const *outputs);
/* ::q4_affine_matmul_batch, src/native.rs:256-272: x fp32 [batch][K] row-major; outputs[j] fp32 [batch][N_j]. */
int q4b_weights_matmul_batch(const q4b_weights *weights, const q4b_q4_matrix *matrices, uint32_t n, const float *x,
                             uint64_t x_len, uint64_t batch_size, float *const *outputs);
/* ::q4_affine_argmax_batch, src/native.rs:276-292 */
int q4b_weights_argmax_batch(const q4b_weights *weights, const q4b_q4_matrix *matrix, const float *x, uint64_t x_len,
                             uint64_t batch_size, uint32_t *tokens);
/* ::q4_affine_mlp_batch, src/native.rs:296-323 */
int q4b_weights_mlp_batch(const q4b_weights *weights, const q4b_q4_matrix *gate, const q4b_q4_matrix *up,
                          const q4b_q4_matrix *down, const float *x, uint64_t x_len, uint64_t batch_size, float *out);
/* dequantized_row, src/native.rs:4944-4987 (embedding lookup): row `row` of the matrix as fp32 [K]; rows past
 * the end are Q4B_TOKEN_OUT_OF_RANGE. Runs on the GPU from the resident bytes. */
int q4b_weights_dequantized_row(const q4b_weights *weights, const q4b_q4_matrix *matrix, uint64_t row, float *out);

#ifdef __cplusplus
}
#endif
#endif
