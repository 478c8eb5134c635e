/*
 * q4b200 -- C ABI of the B200 (sm_100a) affine-Q4 projection library.
 *
 * This is the boundary a host program binds in place of the reference's Metal runtime
 * (Fuxx-1/qwen38-metal: src/metal.rs, the Q4 part of src/metal_runtime.rs, src/mps.rs).
 * Each entry point names the reference interface it replaces; paths are relative to the
 * reference repository root.
 *
 * Conventions
 *   - every function returns a q4b_status; outputs are untouched on error; nothing aborts
 *     and no exception crosses the boundary;
 *   - q4b_last_error() gives the message of the calling thread's last failed call;
 *   - host-pointer entry points are synchronous: results are in the caller's buffers on
 *     return. They serialise on an internal lock, as the reference's pooled entry points do
 *     (Mutex<Q4ActivationPool>, src/metal_runtime.rs:3627-3630), so one runtime may be
 *     shared by several host threads;
 *   - `_device` twins take device pointers and a cudaStream_t (passed as void*), enqueue
 *     work and return without synchronising. They use the runtime's scratch buffers: calls
 *     on one runtime must be ordered on the device (one stream, or events). Scratch grows on
 *     first use of a larger shape, so run a shape once before capturing it in a CUDA graph;
 *   - weights are uploaded byte for byte (no expansion, no repacking, file offsets kept), so
 *     a tensor that is misaligned in its safetensors shard is misaligned in HBM; the kernels
 *     take any byte alignment.
 *
 * Data format (MLX affine Q4, group 64): weights U32 [N][K/8], eight 4-bit values per
 * little-endian word, value i at bits [4i,4i+4); scales and biases BF16 [N][K/64];
 * w = scale*q + bias (src/native.rs:5417-5471, shaders/qwen38.metal:815-817).
 */
#ifndef Q4B200_H
#define Q4B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Mirrors MetalRuntimeError, src/metal_runtime.rs:9218-9257, plus CUDA-side codes. */
typedef enum q4b_status {
    Q4B_OK = 0,
    Q4B_NO_DEVICE = 1,              /* NoDevice */
    Q4B_EMPTY_BUFFER = 2,           /* EmptyBuffer */
    Q4B_POOL_POISONED = 3,          /* ActivationPoolPoisoned */
    Q4B_EMPTY_DIMENSION = 4,        /* EmptyDimension */
    Q4B_INPUT_NOT_GROUPED = 5,      /* InputNotGrouped{input_elements, group_size} */
    Q4B_WRONG_LENGTH = 6,           /* WrongLength{name, actual, expected} */
    Q4B_MISSING_SHARD = 7,          /* MissingMappedShard(index) */
    Q4B_INVALID_BUFFER_OFFSET = 8,  /* InvalidBufferOffset */
    Q4B_TENSOR_OUT_OF_RANGE = 9,    /* MappedTensorOutOfRange */
    Q4B_DIMENSION_OVERFLOW = 10,    /* DimensionOverflow(name) */
    Q4B_COMMAND_FAILED = 11,        /* CommandFailed: a kernel or copy reported an error */
    Q4B_CUDA_ERROR = 12,            /* Library/Function/Pipeline analogue: CUDA call failed */
    Q4B_INVALID_ARGUMENT = 13,      /* null pointer, unknown dtype, bad handle */
    Q4B_UNSUPPORTED = 14,           /* shape outside what this build handles */
    /* weight store and projection API (q4b_weights.h): ModelFormatError, src/model.rs:566-608, and the
     * projection-related variants of NativeError, src/native.rs:5518-5560 */
    Q4B_IO_ERROR = 15,                  /* ModelFormatError::Read */
    Q4B_JSON_ERROR = 16,                /* ::Json */
    Q4B_MISSING_QUANTIZATION = 17,      /* ::MissingQuantization */
    Q4B_UNSUPPORTED_QUANTIZATION = 18,  /* ::UnsupportedQuantization */
    Q4B_UNSAFE_SHARD_PATH = 19,         /* ::UnsafeShardPath */
    Q4B_INVALID_HEADER_LENGTH = 20,     /* ::InvalidHeaderLength */
    Q4B_MISSING_INDEXED_TENSOR = 21,    /* ::MissingIndexedTensor */
    Q4B_INVALID_TENSOR_OFFSETS = 22,    /* ::InvalidTensorOffsets */
    Q4B_INVALID_TENSOR_METADATA = 23,   /* ::InvalidTensorMetadata */
    Q4B_MISSING_TENSOR = 24,            /* ::MissingRuntimeTensor, NativeError::MissingTensor */
    Q4B_INVALID_RUNTIME_TENSOR = 25,    /* ::InvalidRuntimeTensor */
    Q4B_UNSUPPORTED_DTYPE = 26,         /* ::UnsupportedRuntimeDtype */
    Q4B_INCOMPLETE_AFFINE_GROUP = 27,   /* ::IncompleteAffineGroup */
    Q4B_NOT_QUANTIZED_WEIGHT = 28,      /* NativeError::NotQuantizedWeight */
    Q4B_INVALID_QUANTIZED_WEIGHT = 29,  /* NativeError::InvalidQuantizedWeight */
    Q4B_INVALID_AFFINE_TENSOR = 30,     /* NativeError::InvalidAffineTensor */
    Q4B_TENSOR_BYTE_LENGTH = 31,        /* NativeError::TensorByteLength */
    Q4B_INPUT_DIMENSION = 32,           /* NativeError::InputDimension */
    Q4B_INVALID_CONFIG = 33,            /* NativeError::InvalidConfig */
    Q4B_TOKEN_OUT_OF_RANGE = 34         /* NativeError::TokenOutOfRange */
} q4b_status;

typedef enum q4b_dtype {
    Q4B_F32 = 0,  /* the reference's activation type (device const float*, shaders/qwen38.metal:214) */
    Q4B_BF16 = 1  /* benchmarked activation type */
} q4b_dtype;

typedef struct q4b_runtime q4b_runtime; /* replaces MetalRuntime, src/metal_runtime.rs:79-153 */

/*
 * One projection: three (shard, byte offset) pairs and the row count.
 * Replaces MappedQ4AffineJob, src/metal_runtime.rs:155-192. `aligned` is the caller's hint
 * (weights 4-byte, scales/biases 2-byte aligned in the host mapping, src/native.rs:355-369);
 * the library derives the load path from device addresses and ignores the hint.
 */
typedef struct q4b_job {
    uint32_t weight_shard;
    uint32_t scale_shard;
    uint32_t bias_shard;
    int32_t aligned;
    uint64_t weight_offset;
    uint64_t scale_offset;
    uint64_t bias_offset;
    uint64_t output_rows;
} q4b_job;

/* ---- runtime ---- */

/* MetalRuntime::new, src/metal_runtime.rs:642-927. Options are latched from the environment
 * once, here (the reference reads QWEN38_* variables, :916-925): Q4B_FORCE_VARIANT. */
int q4b_runtime_create(int device_ordinal, q4b_runtime **out);
void q4b_runtime_destroy(q4b_runtime *rt);
/* Display impl of MetalRuntimeError, src/metal_runtime.rs:9259-9324 */
const char *q4b_last_error(void);
const char *q4b_status_name(int status);
int q4b_device_info(q4b_runtime *rt, int *sm_count, uint64_t *total_bytes, char *name, uint32_t name_len);

/* ---- weight shards ---- */

/* MetalRuntime::map_weight_store, src/metal_runtime.rs:955-982: one device allocation per
 * shard, bytes copied verbatim. An empty shard is Q4B_EMPTY_BUFFER (:964-966). */
int q4b_shard_upload(q4b_runtime *rt, const void *host_bytes, uint64_t bytes, uint32_t *shard_id);
/* Uninitialised device shard (for tensors generated in place). */
int q4b_shard_alloc(q4b_runtime *rt, uint64_t bytes, uint32_t *shard_id);
/* Copy into an existing shard (partial uploads, row slices). */
int q4b_shard_write(q4b_runtime *rt, uint32_t shard_id, uint64_t offset, const void *host_bytes, uint64_t bytes);
int q4b_shard_read(q4b_runtime *rt, uint32_t shard_id, uint64_t offset, void *host_bytes, uint64_t bytes);
/* Releases a shard's device memory (MappedWeightBuffers dropped, src/metal_runtime.rs:608-612). The id is not
 * reused; using it afterwards is Q4B_MISSING_SHARD. Waits for the device to go idle first. */
int q4b_shard_free(q4b_runtime *rt, uint32_t shard_id);
/* MappedWeightBuffers::shard_count, src/metal_runtime.rs:624-626 */
int q4b_shard_count(q4b_runtime *rt, uint32_t *count);
int q4b_shard_info(q4b_runtime *rt, uint32_t shard_id, void **device_ptr, uint64_t *bytes);
/* MappedWeightBuffers::offset_is_aligned, src/metal_runtime.rs:628-638, on the device address.
 * *aligned is 0 or 1. */
int q4b_offset_is_aligned(q4b_runtime *rt, uint32_t shard_id, uint64_t byte_offset, uint64_t alignment,
                          int *aligned);

/* ---- projections, host buffers (synchronous) ---- */

/* q4_affine_matvec_mapped_batch, src/metal_runtime.rs:3599-3678: several projections over one
 * activation of k elements; outputs[i] receives jobs[i].output_rows floats. */
int q4b_matvec_batch(q4b_runtime *rt, const void *x, int x_dtype, uint64_t k, const q4b_job *jobs,
                     uint32_t n_jobs, float *const *outputs);
/* q4_affine_matmul_mapped_batch, src/metal_runtime.rs:3683-3792: x is [m][k] row-major;
 * outputs[i] is [m][jobs[i].output_rows] row-major. Which kernel runs (the reference's dispatcher,
 * src/metal_runtime.rs:24-77, picks by m too): m = 1 the decode kernel; 2 <= m <= 16 the short-batch kernel when
 * k % 512 == 0 and all tensors are 16-byte aligned, else the general streaming kernel (m < 16); from there on the
 * tensor-core GEMM, which rounds activations and dequantised weights to bf16. q4b_describe_dispatch names the choice. */
int q4b_matmul_batch(q4b_runtime *rt, const void *x, int x_dtype, uint64_t m, uint64_t k, const q4b_job *jobs,
                     uint32_t n_jobs, float *const *outputs);
/* q4_affine_argmax_mapped_batch, src/metal_runtime.rs:3797-3891: tokens[m]; ties -> lowest index. */
int q4b_argmax_batch(q4b_runtime *rt, const void *x, int x_dtype, uint64_t m, uint64_t k, const q4b_job *job,
                     uint32_t *tokens);
/* q4_affine_mlp_mapped_batch, src/metal_runtime.rs:4479-4689: down(silu(gate x) * (up x));
 * gate and up have equal rows, down's input width is that row count; out is [m][down rows]. */
int q4b_mlp_batch(q4b_runtime *rt, const void *x, int x_dtype, uint64_t m, uint64_t k, const q4b_job *gate,
                  const q4b_job *up, const q4b_job *down, float *out);
/* encode_q4_affine_matmul_add, src/metal_runtime.rs:5644-5798: outputs[i] += projection
 * (residual form); outputs hold the residual on entry. */
int q4b_matmul_add_batch(q4b_runtime *rt, const void *x, int x_dtype, uint64_t m, uint64_t k, const q4b_job *jobs,
                         uint32_t n_jobs, float *const *outputs);
/* dequantized_row, src/native.rs:4944-4987 (embedding lookup): one row as fp32, on the device. */
int q4b_dequantize_row(q4b_runtime *rt, const q4b_job *job, uint64_t k, uint64_t row, float *out);

/* ---- device-resident twins (asynchronous, encode_q4_affine_* analogues,
 *      src/metal_runtime.rs:5476-6832) ---- */

#define Q4B_FLAG_ACCUMULATE 1u /* out += projection */
#define Q4B_FLAG_STREAM 2u     /* this call uses the streaming (decode) kernels whatever m is */
#define Q4B_FLAG_TENSOR 4u     /* this call uses the tensor-core GEMM whatever m is */

int q4b_matmul_batch_device(q4b_runtime *rt, const void *x_dev, int x_dtype, uint64_t m, uint64_t k,
                            const q4b_job *jobs, uint32_t n_jobs, float *const *outputs_dev, uint32_t flags,
                            void *stream);
/* q4_affine_mlp_mapped_batch on device buffers (src/metal_runtime.rs:4479-4689; fused 16-bit chain :4267-4474):
 * out_dev is [m][down rows] fp32. From the tensor-core hand-over on, gate and up run as one launch that applies the
 * SwiGLU in its epilogue and hands bf16 rows straight to the down projection. */
int q4b_mlp_batch_device(q4b_runtime *rt, const void *x_dev, int x_dtype, uint64_t m, uint64_t k, const q4b_job *gate,
                         const q4b_job *up, const q4b_job *down, float *out_dev, void *stream);
/* tokens_dev[m] (u32) and, if not null, values_dev[m] (the winning logits); token ids are
 * offset by index_base (row-sharded vocabularies). */
int q4b_argmax_batch_device(q4b_runtime *rt, const void *x_dev, int x_dtype, uint64_t m, uint64_t k,
                            const q4b_job *job, uint32_t index_base, uint32_t *tokens_dev, float *values_dev,
                            void *stream);
/* h = silu(gate)*up over `count` elements; either output may be null. */
int q4b_swiglu_device(q4b_runtime *rt, const float *gate_dev, const float *up_dev, uint64_t count,
                      float *out_f32_dev, uint16_t *out_bf16_dev, void *stream);
/* out = bf16(in / sqrt(mean(in^2) + eps)) per row of n elements (synthetic stack glue). */
int q4b_rms_unit_bf16_device(q4b_runtime *rt, const float *in_dev, uint32_t rows, uint32_t n, float eps,
                             uint16_t *out_bf16_dev, void *stream);

/* ---- persistent decode chain (decode_layers, src/metal_runtime.rs:2022-2081: a whole token in one submission) ---- */

#define Q4B_X_BF16 0u    /* activation = bf16 vector src0[k] */
#define Q4B_X_SWIGLU 1u  /* activation = bf16(silu(src0) * src1), fp32 vectors (qwen38_swiglu_rows) */
#define Q4B_X_RMS 2u     /* activation = bf16(v / sqrt(mean(v^2) + eps)), v = fp32 vector src0 (or a sum of vectors) */

/* One stage: build an activation of k elements from device vectors, then run n_jobs projections of it (M=1) into
 * outputs[i] (device, jobs[i].output_rows floats). Stages run in order; a stage may read what earlier stages wrote.
 * The chain is free to reorder work that nothing in it depends on: a projection whose output no later stage reads
 * (Q/K/V and the DeltaNet inputs of the reference's layer, src/metal_runtime.rs:3463-3517) may run while the next
 * stage is already in progress; every output is complete when the launch is. When a stage is the SwiGLU of two
 * whole outputs of the stage before it, those two projections are streamed row-interleaved and the SwiGLU is
 * applied as their rows finish (the fp32 outputs are still written). */
typedef struct q4b_stage {
    uint32_t x_kind;
    float eps;
    uint64_t k;
    const void *src0;
    const void *src1;
    void *x_bf16_out; /* optional: the bf16 activation that was built (k elements) */
    const q4b_job *jobs;
    uint32_t n_jobs;
    float *const *outputs;
    /* Sharded chains only, else null: peer_outputs[i * 8 + r] is where rank r keeps its copy of the output of job i
     * that this rank computes (peer memory opened with q4b_arena_open), or null when rank r does not need it. */
    float *const *peer_outputs;
    /* K-slice: the jobs' tensors have rows of k_total inputs (0: k) of which this stage multiplies inputs
     * [k_begin, k_begin + k) with its k-element activation; the tensors are read in place through strided rows.
     * k_begin must be a multiple of 64, k of 128, k_total of 512. */
    uint64_t k_total;
    uint64_t k_begin;
    /* Q4B_X_RMS only: src0 is the first of src_parts (0 = 1) fp32 vectors, src_part_stride bytes apart, that are
     * added in order before the norm (partial outputs of a projection cut along K, one per rank). */
    uint32_t src_parts;
    uint32_t reserved;
    uint64_t src_part_stride;
    void *sum_out; /* optional (Q4B_X_RMS): the summed fp32 vector (k elements) */
} q4b_stage;

/* The ranks of a sharded chain (one process per GPU). flags[r] and cand[r] are two small zeroed device arrays
 * (32 and 64 bytes, 8-byte aligned) living on rank r: entry [rank] is this GPU's own, the others are peer memory.
 * flags holds the 64-bit count of ranks that have arrived at cross-GPU barriers and, behind it, the count this
 * rank's earlier launches have used up; cand holds one (best logit, token id) pair per rank.
 * All ranks must run on GPUs with the same SM count. */
typedef struct q4b_peers {
    uint32_t world;
    uint32_t rank;
    void *flags[8];
    void *cand[8];
} q4b_peers;

/* Device memory that other processes on the same node may map: `handle` receives the 64-byte CUDA IPC handle to send
 * to them; q4b_arena_open maps a peer's arena here and enables peer access. Zero-filled on creation. */
int q4b_arena_create(q4b_runtime *rt, uint64_t bytes, void **device_ptr, uint8_t handle[64]);
int q4b_arena_open(q4b_runtime *rt, const uint8_t handle[64], void **peer_ptr);

typedef struct q4b_chain q4b_chain;

/* Compiles a list of stages into one cooperative kernel launch (one resident block per SM; barriers between
 * dependent stages, split into an arrival and a later wait with independent projections in between; next weights
 * requested before each wait). Requires k <= q4b_chain_max_k() except for a fused SwiGLU stage.
 * If logits is not null, the vocab floats there are reduced to *token_dev (+ index_base; ties to the lowest index)
 * and the winning value to *best_dev after the last stage.
 * With `peers` (every rank creates the same chain over its own slices) outputs with peer_outputs are also stored
 * into the other ranks' buffers, the barrier behind such a stage spans all ranks, `vocab`/`index_base` describe this
 * rank's slice and the token is the winner over all slices. All ranks must launch the chain the same number of
 * times. After a wait of a multi-rank chain has run out (Q4B_COMMAND_FAILED from q4b_device_status or
 * q4b_chain_run) the ranks' counters are out of step: q4b_chain_run[_device] then returns Q4B_POOL_POISONED until
 * the chain is destroyed, the arena zeroed on every rank and the chain created again. */
int q4b_chain_create(q4b_runtime *rt, const q4b_stage *stages, uint32_t n_stages, const float *logits, uint32_t vocab,
                     uint32_t index_base, uint32_t *token_dev, float *best_dev, const q4b_peers *peers, q4b_chain **out);
int q4b_chain_run_device(q4b_chain *chain, void *stream);
/* Host-buffer twin of the token step (src/native.rs:3250-3274, 2644-2652: host slice in, token out): copies the
 * first stage's bf16 activation (k elements) from x_host, runs the chain, returns the token id and, if best_host
 * is not null, the winning logit. Synchronous; serialises on the runtime lock. */
int q4b_chain_run(q4b_chain *chain, const void *x_host, uint32_t *token_host, float *best_host);
/* Polls after which a barrier wait of this chain gives up (default 2^21; each poll is one read of device memory). */
int q4b_chain_set_spin_limit(q4b_chain *chain, uint32_t polls);
void q4b_chain_destroy(q4b_chain *chain);
uint64_t q4b_chain_max_k(void);
int q4b_chain_phase_count(q4b_chain *chain, uint32_t *phases);
/* Per-block, per-phase timeline of the last run of a chain created while tracing was enabled (q4b_trace_enable):
 * eight device-clock stamps in ns per block and phase -- wait begun, wait over, activation rebuilt, warp 0 done with
 * its units, block arrived at the barrier, three unused; zero where a step does not exist. phase_info[p] (optional)
 * receives stage * 4 + role, role 0 = the stage's dependent projections, 1 = its deferred projections, 2 = deferred
 * projections of the stage before. */
int q4b_chain_trace_read(q4b_chain *chain, uint64_t *stamps, uint64_t capacity_words, uint32_t *blocks, uint32_t *phases,
                         uint32_t *phase_info, uint32_t phase_info_capacity);

/* ---- seeded synthetic tensors, generated in HBM (benchmark inputs) ---- */

int q4b_synth_q4_device(q4b_runtime *rt, uint64_t seed, uint64_t tensor, float sigma, uint64_t row0,
                        uint64_t rows, uint64_t k, const q4b_job *destination);
int q4b_synth_bf16_device(q4b_runtime *rt, uint64_t seed, uint64_t tensor, uint64_t count, uint16_t *out_dev,
                          void *stream);

/* ---- for callers that cannot allocate ---- */

/* No counterpart in the reference. One decode matvec (one projection, one bf16 activation row of k <= 32768
 * inputs, any byte alignment of the three tensors) that calls no cudaMalloc/cudaFree and no allocating library
 * routine: every scratch buffer lives in a static device array of about 1.1 MB that each GPU loading the library
 * holds until exit. For code that only receives pointers and a stream, or runs where allocator traffic is
 * forbidden. All pointers are device pointers on `device`; out_dev receives n floats. The tensors need no padding:
 * only 16-byte blocks that a tensor itself touches are read. The array is shared by all
 * calls on a device and keeps the last call's contents: calls that overlap on the GPU race on it, so order them.
 * The first call on a device also looks up the array's address and the kernel occupancy; make it outside any
 * stream capture. Shapes beyond the limits are rejected with Q4B_UNSUPPORTED.
 * q4b_noalloc_last_error() gives the message of the calling thread's last failed call. */
int q4b_matvec_noalloc(int device, const void *x_bf16_dev, uint64_t k, const void *weights_dev, const void *scales_dev,
                       const void *biases_dev, uint64_t n, float *out_dev, void *stream);
const char *q4b_noalloc_last_error(void);

/* ---- introspection ---- */

/* Name of the kernel variant the dispatcher would pick (tracing aid, cf. QWEN38_PAIR_TRACE). */
int q4b_describe_dispatch(q4b_runtime *rt, int x_dtype, uint64_t m, uint64_t k, const q4b_job *jobs,
                          uint32_t n_jobs, char *text, uint32_t text_len);
/* Per-kernel timing (the reference's QWEN38_BATCH_TIMING, src/metal_runtime.rs:2188-2245, uses
 * GPUStartTime/GPUEndTime; here a CUDA event pair is recorded around every projection-kernel launch,
 * on the stream it is launched on). q4b_profile_end synchronises, returns the number of timed
 * launches, the sum of their durations and the algorithmic bytes they moved (packed weights, scales,
 * biases, prepared activations, outputs) and the multiply-add work (2*m*n*k per projection), and stops recording. Not for use during graph capture. */
int q4b_profile_begin(q4b_runtime *rt);
int q4b_profile_end(q4b_runtime *rt, uint64_t *launches, double *total_ms, uint64_t *bytes, uint64_t *flops);
/* Synchronise the device and report asynchronous failures of `_device` calls: a CUDA error, or a kernel
 * that gave up on one of its bounded waits (CommandFailed, src/metal_runtime.rs:3661-3663). */
int q4b_device_status(q4b_runtime *rt);
/* Per-warp timeline of the last fast-variant projection launch (tracing aid): four device-clock stamps in
 * nanoseconds per warp -- start, first weights landed, last chunk done, results stored.
 * Not for use during graph capture. */
int q4b_trace_enable(q4b_runtime *rt, int on);
int q4b_trace_read(q4b_runtime *rt, uint64_t *stamps, uint32_t max_workers, uint32_t *workers);
/* Kernels launched by this runtime since creation (the benchmark's launch count). */
int q4b_launch_count(q4b_runtime *rt, uint64_t *launches);

#ifdef __cplusplus
}
#endif
#endif
