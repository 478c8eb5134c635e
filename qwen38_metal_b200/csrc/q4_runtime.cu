// Host runtime behind the C ABI (include/q4b200.h): shard table, validation, scratch pools,
// kernel selection and launch. It is the CUDA counterpart of the Q4 part of the reference's
// MetalRuntime (src/metal_runtime.rs:79-207, 929-982, 3523-4756, 5476-6922, 8831-9057).
// There is no CPU fallback: without a CUDA device every entry point fails with Q4B_NO_DEVICE.
#include "../../include/q4b200.h"

#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <algorithm>
#include <cstring>
#include <memory>
#include <mutex>
#include <new>
#include <string>
#include <vector>

#include "q4_kernels.h"
#include "q4_stack.h"

namespace {

thread_local std::string g_last_error;

int fail(int status, const char *fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    g_last_error = buf;
    return status;
}

}  // namespace

// lets the other translation units of the library (weight store) leave their message where q4b_last_error reads it
namespace q4 {
int set_error(int status, const char *message) {
    g_last_error = message;
    return status;
}
}  // namespace q4

namespace {

int fail_cuda(cudaError_t e, const char *what) {
    return fail(Q4B_CUDA_ERROR, "CUDA call failed in %s: %s", what, cudaGetErrorString(e));
}

#define Q4B_CUDA(call, what)                          \
    do {                                              \
        cudaError_t e__ = (call);                     \
        if (e__ != cudaSuccess) return fail_cuda(e__, what); \
    } while (0)

// Grow-only scratch buffer, power-of-two capacity: ensure_private_buffer /
// shared_reusable_buffer of the reference (src/metal_runtime.rs:8993-9057).
struct Pool {
    void *ptr = nullptr;
    size_t capacity = 0;
    cudaError_t ensure(size_t bytes) {
        if (bytes <= capacity) return cudaSuccess;
        size_t want = 256;
        while (want < bytes) want <<= 1;
        void *fresh = nullptr;
        cudaError_t e = cudaMalloc(&fresh, want);
        if (e != cudaSuccess) return e;
        if (ptr) cudaFree(ptr);
        ptr = fresh;
        capacity = want;
        return cudaSuccess;
    }
    void release() {
        if (ptr) cudaFree(ptr);
        ptr = nullptr;
        capacity = 0;
    }
};

// Grow-only pinned host buffer: results are downloaded here first and handed to the caller only after the device
// reported success, so that caller buffers stay untouched when a call fails.
struct HostPool {
    void *ptr = nullptr;
    size_t capacity = 0;
    cudaError_t ensure(size_t bytes) {
        if (bytes <= capacity) return cudaSuccess;
        size_t want = 4096;
        while (want < bytes) want <<= 1;
        void *fresh = nullptr;
        cudaError_t e = cudaHostAlloc(&fresh, want, cudaHostAllocDefault);
        if (e != cudaSuccess) return e;
        if (ptr) cudaFreeHost(ptr);
        ptr = fresh;
        capacity = want;
        return cudaSuccess;
    }
    void release() {
        if (ptr) cudaFreeHost(ptr);
        ptr = nullptr;
        capacity = 0;
    }
};

struct Shard {
    uint8_t *ptr = nullptr;
    uint64_t bytes = 0;
};

constexpr uint64_t kShardTailPad = 1024;  // prefetch and the unaligned window load may read a little past a tensor

struct Resolved {
    const uint8_t *w, *s, *b;
    uint32_t n;
};

}  // namespace

struct q4b_runtime {
    int device = 0;
    int sm_count = 0;
    uint64_t total_bytes = 0;
    char name[128] = {0};
    cudaStream_t stream = nullptr;
    std::recursive_mutex mu;  // host-side state (shard table, pools, counters); recursive: host entry points call the _device twins
    std::vector<Shard> shards;
    void *stage[2] = {nullptr, nullptr};  // pinned staging for uploads from pageable (mmap'd) memory
    cudaEvent_t stage_done[2] = {nullptr, nullptr};
    uint32_t gemv_ctas[3][2] = {{0, 0}, {0, 0}, {0, 0}};  // [column tiles][aligned] resident warps per SM
    uint32_t max_workers = 0;
    std::vector<void *> arenas, peer_arenas;
    Pool trace, gemm_x, gemm_parts, error_flag;
    uint32_t gemm_min_m = 16;  // activation rows from which the tensor-core GEMM takes over (when the short-batch kernel does not apply)
    uint32_t rows_max_m = 16;  // activation rows per launch of the short-batch kernel (0: never use it)
    uint32_t chain_offset_cost = 140;  // per cent: cost of a byte-offset projection's chunk against an aligned one (decode chain)
    uint32_t chain_defer_split = 50;   // per cent of a stage's deferred rows that run behind its own barrier (the rest behind the next one)
    uint32_t chain_spin_limit = 1u << 21;  // polls before a chain's barrier wait gives up
    // Deferred projections (run behind a barrier's arrival) are off unless asked for: measured on B200 the extra runs
    // of chunks they create cost more than the barrier time they cover.
    bool chain_no_fusion = false, chain_no_deferral = true;
    bool chain_no_handoff = false;     // keep a barrier between a projection and the RMS-norm that consumes it
    bool chain_split_tiles = true;     // a phase with fewer tiles than warps gives every tile the same number of warps
    uint32_t chain_flags = 0;
    bool chain_flags_set = false;      // Q4B_CHAIN_FLAGS was given: no per-chain default
    uint64_t failures = 0;             // bounded waits that ran out (finish() saw the error flag)
    uint64_t prof_flops = 0;
    bool tracing = false;
    uint32_t trace_workers = 0;
    Pool rows_partials, rows_counters;
    uint64_t rows_failures_seen = 0;  // rt->failures when the short-batch tile counters were last known to be zero
    Pool x_in, xp, xsum, row_inv, partials, counters, logits, amax_v, amax_i, tokens, gate, up, hidden;
    Pool outs[q4::kMaxJobs];
    HostPool results;  // staging for downloads (host-buffer entry points)
    // single decode launches (one activation row) run as a one-phase program of the persistent kernel
    Pool inline_partials, inline_state;  // split-tile slots; [0] barrier words, [64] launch count
    uint32_t inline_max_halfs = 0;       // longest activation the kernel's shared memory takes (0: path unavailable)
    uint64_t inline_failures_seen = 0;
    bool inline_off = false;
    bool mlp_unfused = false;            // Q4B_MLP_UNFUSED=1: never use the fused gate/up launch
    uint64_t launches = 0;
    std::string force_variant;
    // per-kernel timing window (q4b_profile_begin/end)
    bool profiling = false;
    std::vector<cudaEvent_t> prof_events;  // start/stop pairs
    size_t prof_used = 0;
    uint64_t prof_bytes = 0;
};

extern "C" uint32_t q4k_gemv_occupancy(int column_tiles, int aligned);

namespace {

struct DeviceGuard {
    int prev = -1;
    explicit DeviceGuard(int device) {
        cudaGetDevice(&prev);
        if (prev != device) cudaSetDevice(device);
        else prev = -1;
    }
    ~DeviceGuard() {
        if (prev >= 0) cudaSetDevice(prev);
    }
};

int check_rt(q4b_runtime *rt) {
    if (!rt) return fail(Q4B_INVALID_ARGUMENT, "runtime handle is null");
    return Q4B_OK;
}

// validate_mapped_q4_affine_shape, src/metal_runtime.rs:8854-8898, on shard ids
int resolve_job(q4b_runtime *rt, const q4b_job &job, uint64_t k, Resolved *out) {
    if (k == 0 || job.output_rows == 0) return fail(Q4B_EMPTY_DIMENSION, "matrix dimensions must be greater than zero");
    if (k % 64 != 0)
        return fail(Q4B_INPUT_NOT_GROUPED, "input dimension %llu is not divisible by affine group size 64",
                    (unsigned long long)k);
    const uint32_t ids[3] = {job.weight_shard, job.scale_shard, job.bias_shard};
    for (uint32_t id : ids) {
        if (id >= rt->shards.size() || rt->shards[id].ptr == nullptr)
            return fail(Q4B_MISSING_SHARD, "mapped safetensors shard %u is absent", id);
    }
    const Shard &ws = rt->shards[job.weight_shard], &ss = rt->shards[job.scale_shard], &bs = rt->shards[job.bias_shard];
    if (job.weight_offset > ws.bytes || job.scale_offset > ss.bytes || job.bias_offset > bs.bytes)
        return fail(Q4B_INVALID_BUFFER_OFFSET, "mapped tensor offset is outside its shard");
    if (job.output_rows > 0xffffffffull) return fail(Q4B_DIMENSION_OVERFLOW, "output rows exceeds runtime limits");
    if (k / 8 > 0xffffffffull) return fail(Q4B_DIMENSION_OVERFLOW, "words per row exceeds runtime limits");
    const uint64_t words = k / 8, groups = k / 64;
    if (job.output_rows > UINT64_MAX / 4 / words) return fail(Q4B_DIMENSION_OVERFLOW, "packed weight count exceeds runtime limits");
    const uint64_t weight_bytes = job.output_rows * words * 4;
    const uint64_t affine_bytes = job.output_rows * groups * 2;
    if (weight_bytes > ws.bytes - job.weight_offset || affine_bytes > ss.bytes - job.scale_offset ||
        affine_bytes > bs.bytes - job.bias_offset)
        return fail(Q4B_TENSOR_OUT_OF_RANGE, "mapped tensor range exceeds its safetensors shard");
    out->w = ws.ptr + job.weight_offset;
    out->s = ss.ptr + job.scale_offset;
    out->b = bs.ptr + job.bias_offset;
    out->n = (uint32_t)job.output_rows;
    return Q4B_OK;
}

int resolve_jobs(q4b_runtime *rt, const q4b_job *jobs, uint32_t n_jobs, uint64_t m, uint64_t k,
                 std::vector<Resolved> *out) {
    if (!jobs || n_jobs == 0 || m == 0 || k == 0)
        return fail(Q4B_EMPTY_DIMENSION, "matrix dimensions must be greater than zero");
    if (m > 0xffffffffull) return fail(Q4B_DIMENSION_OVERFLOW, "batch size exceeds runtime limits");
    out->resize(n_jobs);
    for (uint32_t i = 0; i < n_jobs; ++i) {
        int st = resolve_job(rt, jobs[i], k, &(*out)[i]);
        if (st != Q4B_OK) return st;
    }
    return Q4B_OK;
}

// the fast kernel variant copies parameters in 16-byte pieces of 8 groups
bool job_is_fast(const Resolved &r, uint32_t groups) {
    return (((uintptr_t)r.w | (uintptr_t)r.s | (uintptr_t)r.b) & 15u) == 0 && groups % 8u == 0;
}

int profile_open(q4b_runtime *rt, cudaStream_t stream) {
    if (!rt->profiling) return Q4B_OK;
    if (rt->prof_used + 2 > rt->prof_events.size()) {
        for (int i = 0; i < 2; ++i) {
            cudaEvent_t ev;
            Q4B_CUDA(cudaEventCreate(&ev), "cudaEventCreate");
            rt->prof_events.push_back(ev);
        }
    }
    Q4B_CUDA(cudaEventRecord(rt->prof_events[rt->prof_used], stream), "cudaEventRecord");
    return Q4B_OK;
}

int profile_close(q4b_runtime *rt, cudaStream_t stream, uint64_t bytes, uint64_t flops) {
    if (!rt->profiling) return Q4B_OK;
    Q4B_CUDA(cudaEventRecord(rt->prof_events[rt->prof_used + 1], stream), "cudaEventRecord");
    rt->prof_used += 2;
    rt->prof_bytes += bytes;
    rt->prof_flops += flops;
    return Q4B_OK;
}

// One activation row: the persistent kernel as a one-phase program in the kernel parameters -- the activation is built
// in shared memory by every block (no separate preparation kernel), projections are streamed on the integer
// tensor-core path, split tiles are combined through tagged slots. One launch per call.
int launch_single_row(q4b_runtime *rt, const void *x_dev, int x_dtype, uint32_t k, const Resolved *jobs, uint32_t n_jobs,
                      float *const *outs, cudaStream_t stream) {
    const uint32_t warps = q4k_stack_warps(), grid_warps = (uint32_t)rt->sm_count * warps;
    if (rt->inline_failures_seen != rt->failures) {
        // a kernel gave up on a wait since the last launch: its counters and tags may be anywhere
        Q4B_CUDA(cudaMemsetAsync(rt->inline_partials.ptr, 0, rt->inline_partials.capacity, stream), "decode launch repair");
        Q4B_CUDA(cudaMemsetAsync(rt->inline_state.ptr, 0, 256, stream), "decode launch repair");
        rt->inline_failures_seen = rt->failures;
    }
    q4::InlineProgram prog;
    memset(&prog, 0, sizeof prog);
    q4::StackPhase &P = prog.phase;
    P.k = k;
    P.kp = (k + 127u) & ~127u;
    P.groups = k / 64;
    P.cpt = (P.groups + 1u) / 2u;
    P.n_jobs = n_jobs;
    P.x_kind = x_dtype == Q4B_F32 ? q4::kRebuildF32 : q4::kRebuildBf16;
    P.src0 = x_dev;
    P.src_parts = 1;
    const uint32_t cpt = P.cpt;
    uint32_t tiles = 0;
    uint64_t units = 0, bytes = 0, rows = 0;
    for (uint32_t i = 0; i < n_jobs; ++i) {
        q4::StackJob &j = prog.jobs[i];
        j.w[0] = j.w[1] = jobs[i].w;
        j.s[0] = j.s[1] = jobs[i].s;
        j.b[0] = j.b[1] = jobs[i].b;
        j.out[0] = j.out[1] = outs[i];
        j.n = jobs[i].n;
        j.rows_per_tile = 16;
        j.b_row_offset = 8;
        j.w_stride = k / 2;
        j.p_stride = (k / 64) * 2;
        j.tile_begin = tiles;
        j.vcpt = cpt;
        j.unit_begin = (uint32_t)units;
        const uint32_t job_tiles = (jobs[i].n + 15u) / 16u;
        tiles += job_tiles;
        units += (uint64_t)job_tiles * cpt;
        bytes += (uint64_t)jobs[i].n * (k / 2 + (uint64_t)P.groups * 4) + (uint64_t)jobs[i].n * 4;
        rows += jobs[i].n;
    }
    if (units > 0xffffffffull) return fail(Q4B_UNSUPPORTED, "launch is too large");
    P.tiles = tiles;
    P.units = units;
    // few tiles: every tile in equal parts, one per warp, a block on one part of sixteen tiles (it then builds only that
    // slice of the activation); many tiles: equal runs of units
    const uint32_t min_chunks = (cpt + 31u) / 32u;
    const uint32_t tile_groups = (tiles + warps - 1u) / warps;
    uint32_t parts = tile_groups <= (uint32_t)rt->sm_count ? (uint32_t)rt->sm_count / tile_groups : 0u;
    if (parts > cpt / min_chunks) parts = cpt / min_chunks;
    if (parts > 32u) parts = 32u;
    uint64_t workers = grid_warps;
    if (parts >= 1u && (uint64_t)tiles * parts * 100u >= (uint64_t)grid_warps * 70u) {
        workers = (uint64_t)tiles * parts;
        P.kparts = parts;
        P.sliced = parts > 1u ? 1u : 0u;
    } else {
        if (workers > units / min_chunks) workers = units / min_chunks;
        if (workers == 0) workers = 1;
    }
    P.workers = (uint32_t)workers;
    q4::StackParams &sp = prog.params;
    sp.halfs[0] = P.kp;
    if (P.sliced) {
        uint32_t chunks = 0;
        for (uint32_t part = 0; part < P.kparts; ++part) {
            const uint32_t lo = (cpt * part / P.kparts) & ~3u, hi = cpt * (part + 1u) / P.kparts;
            chunks = hi - lo > chunks ? hi - lo : chunks;
        }
        sp.halfs[0] = (chunks + 1u) * 128u;
    }
    sp.local_bar = (unsigned int *)rt->inline_state.ptr;
    sp.launch_seq = (unsigned int *)rt->inline_state.ptr + 64;
    sp.error_flag = (int *)rt->error_flag.ptr;
    sp.partials = (uint4 *)rt->inline_partials.ptr;
    sp.max_workers = grid_warps;
    sp.spin_limit = rt->chain_spin_limit;
    sp.flags = rt->chain_flags;
    sp.long_rebuild = (uint32_t)q4k_stack_phase_is_long(&prog.phase);
    if (int st = profile_open(rt, stream)) return st;
    Q4B_CUDA(q4k_stack_launch_inline(&prog, rt->sm_count, stream), "decode launch");
    rt->launches++;
    return profile_close(rt, stream, bytes + (uint64_t)k * (x_dtype == Q4B_F32 ? 4 : 2), 2ull * rows * k);
}

// One streaming launch: up to kMaxJobs projections, up to 8 bf16 (2 fp32) activation rows.
int launch_streaming(q4b_runtime *rt, const void *x_dev, int x_dtype, uint32_t m, uint32_t k, const Resolved *jobs,
                     uint32_t n_jobs, float *const *outs, const uint32_t *out_strides, uint32_t flags,
                     cudaStream_t stream) {
    const bool f32 = x_dtype == Q4B_F32;
    const uint32_t v_cols = m * (f32 ? 3u : 1u);
    const int nt = v_cols <= 4 ? 1 : 2;
    const uint32_t vpad = 4u * nt;
    const uint32_t groups = k / 64;
    const uint32_t kp = (k + 127u) & ~127u;
    Q4B_CUDA(rt->xp.ensure((size_t)v_cols * kp * 2 + 1024), "activation scratch");  // + over-read slack
    Q4B_CUDA(rt->xsum.ensure((size_t)(kp / 64) * vpad * 4 + 1024), "activation sum scratch");
    Q4B_CUDA(rt->row_inv.ensure(256), "row scale scratch");
    Q4B_CUDA(q4k_prepare_x(x_dev, f32 ? 1 : 0, m, k, kp, vpad, (uint16_t *)rt->xp.ptr, (float *)rt->xsum.ptr,
                           (float *)rt->row_inv.ptr, stream),
             "q4_prepare_x launch");
    rt->launches++;

    // Jobs that meet the fast variant's conditions (all three tensors on 16-byte boundaries, K % 512 == 0)
    // go in one launch, the rest in a second launch of the general (byte-addressed) variant.
    for (int fast = 1; fast >= 0; --fast) {
        q4::GemvParams p;
        memset(&p, 0, sizeof p);
        uint32_t tiles = 0, count = 0;
        uint64_t prof_bytes = 0, prof_rows = 0;
        for (uint32_t i = 0; i < n_jobs; ++i) {
            if ((job_is_fast(jobs[i], groups) ? 1 : 0) != fast) continue;
            q4::GemvJob &j = p.jobs[count++];
            j.w = jobs[i].w;
            j.s = jobs[i].s;
            j.b = jobs[i].b;
            j.out = outs[i];
            j.n = jobs[i].n;
            j.out_stride = out_strides ? out_strides[i] : jobs[i].n;
            j.tile_begin = tiles;
            j.w_misalign = (uint32_t)((uintptr_t)jobs[i].w & 15u);
            tiles += (jobs[i].n + 15u) / 16u;
            prof_bytes += (uint64_t)jobs[i].n * (k / 2 + (uint64_t)groups * 4) + (uint64_t)m * jobs[i].n * 4;
            prof_rows += jobs[i].n;
        }
        if (count == 0) continue;
        p.n_jobs = count;
        p.xp = (const uint16_t *)rt->xp.ptr;
        p.xsum = (const float *)rt->xsum.ptr;
        p.row_inv = (const float *)rt->row_inv.ptr;
        p.kp = kp;
        p.v_cols = v_cols;
        p.vpad = vpad;
        p.m_rows = m;
        p.x_is_f32 = f32 ? 1u : 0u;
        p.accumulate = (flags & Q4B_FLAG_ACCUMULATE) ? 1u : 0u;
        p.k = k;
        p.groups = groups;
        p.cpt = (groups + 1u) / 2u;
        p.units = (uint64_t)tiles * p.cpt;
        // one warp per block, every SM filled to the variant's occupancy; never more warps than units, so
        // every worker owns at least one unit (the split-tile arrival count relies on it)
        uint64_t workers = (uint64_t)rt->sm_count * rt->gemv_ctas[nt][fast];
        // at most 32 warps share a tile: the warp that combines a split tile reads their partials four at a time
        const uint64_t min_chunks = (p.cpt + 31u) / 32u;
        if (workers > p.units / min_chunks) workers = p.units / min_chunks;
        if (workers == 0) workers = 1;
        p.workers = (uint32_t)workers;
        p.partials = (float *)rt->partials.ptr;
        p.counters = (unsigned int *)rt->counters.ptr;
        p.trace = rt->tracing ? (unsigned long long *)rt->trace.ptr : nullptr;
        if (rt->tracing) rt->trace_workers = p.workers;
        if (int st = profile_open(rt, stream)) return st;
        Q4B_CUDA(q4k_gemv(&p, nt, fast, stream), "q4_gemv launch");
        rt->launches++;
        if (int st = profile_close(rt, stream, prof_bytes + (uint64_t)v_cols * kp * 2 + (uint64_t)(kp / 64) * vpad * 4, 2ull * m * prof_rows * k)) return st;
    }
    return Q4B_OK;
}

// Tensor-core path: activations to bf16 once, then one tcgen05 GEMM launch per projection.
int enqueue_gemm(q4b_runtime *rt, const void *x_dev, int x_dtype, uint64_t m, uint64_t k, const std::vector<Resolved> &jobs,
                 float *const *outs, uint32_t flags, cudaStream_t stream) {
    Q4B_CUDA(rt->gemm_x.ensure((size_t)m * k * 2), "activation scratch");
    Q4B_CUDA(q4k_gemm_prepare_x(x_dev, x_dtype == Q4B_F32 ? 1 : 0, m * k, (uint16_t *)rt->gemm_x.ptr, stream),
             "q4_gemm_prepare_x launch");
    rt->launches++;
    for (size_t i = 0; i < jobs.size(); ++i) {
        uint32_t split_blocks = 0;
        const uint32_t splits = q4k_gemm_k_splits((uint32_t)m, jobs[i].n, (uint32_t)k, (uint32_t)rt->sm_count, &split_blocks);
        if (splits > 1) Q4B_CUDA(rt->gemm_parts.ensure((size_t)splits * m * jobs[i].n * 4), "partial output scratch");
        if (int st = profile_open(rt, stream)) return st;
        Q4B_CUDA(q4k_gemm_tc((const uint16_t *)rt->gemm_x.ptr, (uint32_t)m, (uint32_t)k, jobs[i].w, jobs[i].s, jobs[i].b, jobs[i].n,
                             outs[i], jobs[i].n, (flags & Q4B_FLAG_ACCUMULATE) ? 1 : 0, (int *)rt->error_flag.ptr,
                             (uint32_t)rt->sm_count, (float *)rt->gemm_parts.ptr, stream),
                 "q4_gemm_tc launch");
        rt->launches++;
        const uint64_t bytes = (uint64_t)jobs[i].n * (k / 2 + (k / 64) * 4) + m * k * 2 + m * jobs[i].n * 4;
        if (int st = profile_close(rt, stream, bytes, 2ull * m * jobs[i].n * k)) return st;
    }
    return Q4B_OK;
}

// Short batches on the integer tensor-core path (q4_gemv_rows.cu). Returns -1 when the call does not meet the kernel's
// conditions (the caller falls back to the general streaming kernel), else a status.
int launch_rows(q4b_runtime *rt, const void *x_dev, int x_dtype, uint32_t m, uint32_t k, const Resolved *jobs, uint32_t n_jobs,
                float *const *outs, uint32_t flags, cudaStream_t stream) {
    if (m < 1 || m > 16 || k % 512u != 0 || ((uintptr_t)x_dev & 15u)) return -1;
    uint32_t tiles = 0;
    for (uint32_t i = 0; i < n_jobs; ++i) {
        if ((((uintptr_t)jobs[i].w | (uintptr_t)jobs[i].s | (uintptr_t)jobs[i].b) & 15u) != 0 || jobs[i].n == 0) return -1;
        tiles += (jobs[i].n + 15u) / 16u;
    }
    uint32_t part_chunks = 0, tiles_per_warp = 1;
    const uint32_t parts = q4k_rows_plan(m, k, tiles, (uint32_t)rt->sm_count, &part_chunks, &tiles_per_warp);
    if (parts == 0) return -1;
    q4::RowsParams p;
    memset(&p, 0, sizeof p);
    uint64_t prof_bytes = 0, prof_rows = 0;
    uint32_t t0 = 0;
    for (uint32_t i = 0; i < n_jobs; ++i) {
        q4::RowsJob &j = p.jobs[i];
        j.w = jobs[i].w;
        j.s = jobs[i].s;
        j.b = jobs[i].b;
        j.out = outs[i];
        j.n = jobs[i].n;
        j.out_stride = jobs[i].n;
        j.tile_begin = t0;
        t0 += (jobs[i].n + 15u) / 16u;
        prof_bytes += (uint64_t)jobs[i].n * (k / 2 + (uint64_t)(k / 64) * 4) + (uint64_t)m * jobs[i].n * 4;
        prof_rows += jobs[i].n;
    }
    p.n_jobs = n_jobs;
    p.m = m;
    p.x = x_dev;
    p.x_is_f32 = x_dtype == Q4B_F32 ? 1u : 0u;
    p.k = k;
    p.groups = k / 64u;
    p.cpt = k / 128u;
    p.parts = parts;
    p.part_chunks = part_chunks;
    p.tiles_per_warp = tiles_per_warp;
    p.tiles = tiles;
    p.accumulate = (flags & Q4B_FLAG_ACCUMULATE) ? 1u : 0u;
    if (parts > 1) {
        const size_t mp = m <= 8 ? 8 : 16;
        Q4B_CUDA(rt->rows_partials.ensure((size_t)parts * mp * tiles * 16 * 4), "partial sum scratch");
        const size_t had = rt->rows_counters.capacity;
        Q4B_CUDA(rt->rows_counters.ensure((size_t)tiles * 4), "tile counter scratch");
        // the counters are put back to zero by the kernel itself; after a failed command on this runtime (a launch may
        // have been cut short) and for a fresh buffer they are cleared here
        if (rt->rows_counters.capacity != had || rt->rows_failures_seen != rt->failures) {
            Q4B_CUDA(cudaMemsetAsync(rt->rows_counters.ptr, 0, rt->rows_counters.capacity, stream), "tile counter reset");
            rt->rows_failures_seen = rt->failures;
        }
        p.partials = (float *)rt->rows_partials.ptr;
        p.counters = (unsigned int *)rt->rows_counters.ptr;
    }
    const uint32_t grid_warps = ((uint32_t)rt->sm_count / parts) * parts * 16u;
    if (rt->tracing && grid_warps <= rt->max_workers) {
        p.trace = (unsigned long long *)rt->trace.ptr;
        rt->trace_workers = grid_warps;
    }
    if (int st = profile_open(rt, stream)) return st;
    Q4B_CUDA(q4k_rows(&p, (uint32_t)rt->sm_count, stream), "q4_rows launch");
    rt->launches++;
    return profile_close(rt, stream, prof_bytes + (uint64_t)m * k * (x_dtype == Q4B_F32 ? 4 : 2), 2ull * m * prof_rows * k);
}

// Any m, any number of jobs: the short-batch kernel up to rows_max_m rows where it applies, the tensor-core GEMM from
// gemm_min_m rows, else launches the streaming kernel accepts.
int enqueue_matmul(q4b_runtime *rt, const void *x_dev, int x_dtype, uint64_t m, uint64_t k,
                   const std::vector<Resolved> &jobs, float *const *outs, uint32_t flags, cudaStream_t stream) {
    const bool want_tensor = (flags & Q4B_FLAG_TENSOR) != 0, want_stream = (flags & Q4B_FLAG_STREAM) != 0;
    const size_t esize = x_dtype == Q4B_F32 ? 4 : 2;
    // Short batches (2 .. rows_max_m rows; any m when the caller asks for the streaming form) run on the integer
    // tensor-core kernel when every launch of the call meets its conditions.
    bool rows = !want_tensor && m >= 2 && rt->rows_max_m >= 2 && (want_stream || m <= rt->rows_max_m) && k % 512 == 0 &&
                ((uintptr_t)x_dev & 15u) == 0;
    for (size_t j = 0; j < jobs.size() && rows; ++j)
        rows = (((uintptr_t)jobs[j].w | (uintptr_t)jobs[j].s | (uintptr_t)jobs[j].b) & 15u) == 0 && jobs[j].n != 0;
    for (size_t j0 = 0; j0 < jobs.size() && rows; j0 += q4::kMaxJobs) {
        uint32_t tiles = 0, part_chunks = 0, tw = 1;
        for (size_t j = j0; j < jobs.size() && j < j0 + q4::kMaxJobs; ++j) tiles += (jobs[j].n + 15u) / 16u;
        const uint32_t full = (uint32_t)(m < rt->rows_max_m ? m : rt->rows_max_m), rest = (uint32_t)(m % rt->rows_max_m);
        rows = q4k_rows_plan(full, (uint32_t)k, tiles, (uint32_t)rt->sm_count, &part_chunks, &tw) != 0 &&
               (m <= rt->rows_max_m || rest == 0 || q4k_rows_plan(rest, (uint32_t)k, tiles, (uint32_t)rt->sm_count, &part_chunks, &tw) != 0);
    }
    if (rows) {
        for (uint64_t m0 = 0; m0 < m; m0 += rt->rows_max_m) {
            const uint32_t mb = (uint32_t)((m - m0) < rt->rows_max_m ? (m - m0) : rt->rows_max_m);
            const uint8_t *xb = (const uint8_t *)x_dev + m0 * k * esize;
            for (size_t j0 = 0; j0 < jobs.size(); j0 += q4::kMaxJobs) {
                const uint32_t nj = (uint32_t)((jobs.size() - j0) < (size_t)q4::kMaxJobs ? (jobs.size() - j0) : (size_t)q4::kMaxJobs);
                float *o[q4::kMaxJobs];
                for (uint32_t i = 0; i < nj; ++i) o[i] = outs[j0 + i] + m0 * jobs[j0 + i].n;
                const int st = launch_rows(rt, xb, x_dtype, mb, (uint32_t)k, &jobs[j0], nj, o, flags, stream);
                if (st == -1) return fail(Q4B_CUDA_ERROR, "short-batch launch refused a call its conditions admit");
                if (st != Q4B_OK) return st;
            }
        }
        return Q4B_OK;
    }
    if (want_tensor || (!want_stream && m >= rt->gemm_min_m)) return enqueue_gemm(rt, x_dev, x_dtype, m, k, jobs, outs, flags, stream);
    if (m == 1 && !(flags & Q4B_FLAG_ACCUMULATE) && rt->inline_max_halfs && k % 512 == 0 && k <= rt->inline_max_halfs && k <= q4k_stack_max_k()) {
        for (size_t j0 = 0; j0 < jobs.size(); j0 += q4::kMaxJobs) {
            const uint32_t nj = (uint32_t)((jobs.size() - j0) < (size_t)q4::kMaxJobs ? (jobs.size() - j0) : (size_t)q4::kMaxJobs);
            if (int st = launch_single_row(rt, x_dev, x_dtype, (uint32_t)k, &jobs[j0], nj, outs + j0, stream)) return st;
        }
        return Q4B_OK;
    }
    const uint32_t rows_per_launch = x_dtype == Q4B_F32 ? 2u : 8u;
    for (uint64_t m0 = 0; m0 < m; m0 += rows_per_launch) {
        const uint32_t mb = (uint32_t)((m - m0) < rows_per_launch ? (m - m0) : rows_per_launch);
        const uint8_t *xb = (const uint8_t *)x_dev + m0 * k * esize;
        for (size_t j0 = 0; j0 < jobs.size(); j0 += q4::kMaxJobs) {
            const uint32_t nj = (uint32_t)((jobs.size() - j0) < (size_t)q4::kMaxJobs ? (jobs.size() - j0) : (size_t)q4::kMaxJobs);
            float *o[q4::kMaxJobs];
            for (uint32_t i = 0; i < nj; ++i) o[i] = outs[j0 + i] + m0 * jobs[j0 + i].n;
            int st = launch_streaming(rt, xb, x_dtype, mb, (uint32_t)k, &jobs[j0], nj, o, nullptr, flags, stream);
            if (st != Q4B_OK) return st;
        }
    }
    return Q4B_OK;
}

int check_dtype(int x_dtype) {
    if (x_dtype != Q4B_F32 && x_dtype != Q4B_BF16) return fail(Q4B_INVALID_ARGUMENT, "unknown activation dtype %d", x_dtype);
    return Q4B_OK;
}

int finish(q4b_runtime *rt, cudaStream_t stream) {
    cudaError_t e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) return fail(Q4B_COMMAND_FAILED, "CUDA command failed: %s", cudaGetErrorString(e));
    int flag = 0;
    e = cudaMemcpy(&flag, rt->error_flag.ptr, sizeof flag, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return fail(Q4B_COMMAND_FAILED, "CUDA command failed: %s", cudaGetErrorString(e));
    if (flag) {
        cudaMemset(rt->error_flag.ptr, 0, sizeof flag);
        rt->failures++;
        return fail(Q4B_COMMAND_FAILED, "a kernel gave up on a bounded wait (pipeline stalled); results are invalid");
    }
    return Q4B_OK;
}

}  // namespace

// ------------------------------------------------------------------------------------------
// runtime
// ------------------------------------------------------------------------------------------

extern "C" int q4b_runtime_create(int device_ordinal, q4b_runtime **out) {
    if (!out) return fail(Q4B_INVALID_ARGUMENT, "output handle pointer is null");
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0) {
        cudaGetLastError();
        return fail(Q4B_NO_DEVICE, "no CUDA device is available");
    }
    if (device_ordinal < 0 || device_ordinal >= count)
        return fail(Q4B_NO_DEVICE, "CUDA device %d is not available (%d visible)", device_ordinal, count);
    DeviceGuard guard(device_ordinal);
    cudaDeviceProp prop;
    Q4B_CUDA(cudaGetDeviceProperties(&prop, device_ordinal), "cudaGetDeviceProperties");
    if (prop.major != 10)
        return fail(Q4B_NO_DEVICE, "device %d is sm_%d%d; this library is built for sm_100a only", device_ordinal,
                    prop.major, prop.minor);
    q4b_runtime *rt = new (std::nothrow) q4b_runtime();
    if (!rt) return fail(Q4B_CUDA_ERROR, "out of host memory");
    rt->device = device_ordinal;
    rt->sm_count = prop.multiProcessorCount;
    rt->total_bytes = prop.totalGlobalMem;
    snprintf(rt->name, sizeof rt->name, "%s", prop.name);
    if (const char *cost = getenv("Q4B_CHAIN_OFFSET_COST")) {
        const long v = strtol(cost, nullptr, 10);
        if (v >= 100 && v <= 300) rt->chain_offset_cost = (uint32_t)v;
    }
    if (const char *split = getenv("Q4B_CHAIN_DEFER_SPLIT")) {
        const long v = strtol(split, nullptr, 10);
        if (v >= 0 && v <= 100) rt->chain_defer_split = (uint32_t)v;
    }
    if (const char *mode = getenv("Q4B_CHAIN_SPLIT")) rt->chain_split_tiles = strcmp(mode, "equal") != 0;
    if (const char *fl = getenv("Q4B_CHAIN_FLAGS")) {
        rt->chain_flags = (uint32_t)strtol(fl, nullptr, 10);
        rt->chain_flags_set = true;
    }
    if (const char *plain = getenv("Q4B_CHAIN_PLAIN")) rt->chain_no_fusion = strtol(plain, nullptr, 10) != 0;  // no gate/up fusion
    if (const char *hand = getenv("Q4B_CHAIN_HANDOFF")) rt->chain_no_handoff = strtol(hand, nullptr, 10) == 0;
    if (const char *defer = getenv("Q4B_CHAIN_DEFER")) rt->chain_no_deferral = strtol(defer, nullptr, 10) == 0;
    if (const char *force = getenv("Q4B_FORCE_VARIANT")) rt->force_variant = force;
    if (const char *rm = getenv("Q4B_ROWS_MAX_M")) {
        const long v = strtol(rm, nullptr, 10);
        if (v >= 0 && v <= 16) rt->rows_max_m = (uint32_t)v;
    }
    if (rt->force_variant == "stream") rt->gemm_min_m = 0xffffffffu;   // never use the tensor-core GEMM
    if (rt->force_variant == "tensor") rt->gemm_min_m = 1;            // always use it
    if (const char *min_m = getenv("Q4B_GEMM_MIN_M")) {
        long v = strtol(min_m, nullptr, 10);
        if (v > 0) rt->gemm_min_m = (uint32_t)v;
    }
    e = cudaStreamCreateWithFlags(&rt->stream, cudaStreamNonBlocking);
    if (e != cudaSuccess) {
        delete rt;
        return fail_cuda(e, "cudaStreamCreate");
    }
    uint32_t max_ctas = 1;
    for (int nt = 1; nt <= 2; ++nt)
        for (int al = 0; al < 2; ++al) {
            uint32_t occ = q4k_gemv_occupancy(nt, al);
            if (occ == 0) {
                cudaStreamDestroy(rt->stream);
                delete rt;
                return fail(Q4B_CUDA_ERROR, "streaming kernel cannot be resident on this device (sm_100a image missing?)");
            }
            rt->gemv_ctas[nt][al] = occ;
            max_ctas = occ > max_ctas ? occ : max_ctas;
        }
    rt->max_workers = (uint32_t)rt->sm_count * max_ctas;
    // split-tile scratch: [workers][2 slots][2 column tiles][32 lanes][4 floats] and one counter per worker
    e = rt->partials.ensure((size_t)rt->max_workers * 2 * 2 * 32 * 16);
    if (e == cudaSuccess) e = rt->counters.ensure((size_t)rt->max_workers * 4);
    if (e == cudaSuccess) e = cudaMemset(rt->counters.ptr, 0, rt->counters.capacity);
    if (e == cudaSuccess) e = rt->error_flag.ensure(256);
    if (e == cudaSuccess) e = cudaMemset(rt->error_flag.ptr, 0, rt->error_flag.capacity);
    if (const char *unf = getenv("Q4B_MLP_UNFUSED")) rt->mlp_unfused = strtol(unf, nullptr, 10) != 0;
    if (const char *off = getenv("Q4B_NO_INLINE")) rt->inline_off = strtol(off, nullptr, 10) != 0;
    if (e == cudaSuccess && !rt->inline_off) {
        // the largest activation for which the one-phase kernel is resident: try the chain's limit, then half of it
        for (uint32_t halfs : {q4k_stack_max_k(), q4k_stack_max_k() / 2u, 8192u, 4096u}) {
            if (q4k_stack_inline_supported(halfs)) {
                rt->inline_max_halfs = halfs;
                break;
            }
        }
        if (rt->inline_max_halfs) {
            e = rt->inline_partials.ensure((size_t)rt->sm_count * q4k_stack_warps() * 32 * sizeof(uint4));
            if (e == cudaSuccess) e = cudaMemset(rt->inline_partials.ptr, 0, rt->inline_partials.capacity);
            if (e == cudaSuccess) e = rt->inline_state.ensure(1024);
            if (e == cudaSuccess) e = cudaMemset(rt->inline_state.ptr, 0, rt->inline_state.capacity);
        }
    }
    if (e != cudaSuccess) {
        q4b_runtime_destroy(rt);
        return fail_cuda(e, "scratch allocation");
    }
    *out = rt;
    return Q4B_OK;
}

extern "C" void q4b_runtime_destroy(q4b_runtime *rt) {
    if (!rt) return;
    DeviceGuard guard(rt->device);
    cudaDeviceSynchronize();
    for (Shard &s : rt->shards)
        if (s.ptr) cudaFree(s.ptr);
    for (void *p : rt->peer_arenas) cudaIpcCloseMemHandle(p);
    for (void *p : rt->arenas) cudaFree(p);
    Pool *pools[] = {&rt->rows_partials, &rt->rows_counters, &rt->gemm_x, &rt->gemm_parts, &rt->error_flag, &rt->trace, &rt->x_in, &rt->xp, &rt->xsum, &rt->row_inv, &rt->partials, &rt->counters, &rt->logits, &rt->amax_v,
                     &rt->amax_i, &rt->tokens, &rt->gate, &rt->up, &rt->hidden};
    for (Pool *p : pools) p->release();
    for (Pool &p : rt->outs) p.release();
    rt->inline_partials.release();
    rt->inline_state.release();
    rt->results.release();
    for (cudaEvent_t ev : rt->prof_events) cudaEventDestroy(ev);
    for (int i = 0; i < 2; ++i) {
        if (rt->stage[i]) cudaFreeHost(rt->stage[i]);
        if (rt->stage_done[i]) cudaEventDestroy(rt->stage_done[i]);
    }
    if (rt->stream) cudaStreamDestroy(rt->stream);
    delete rt;
}

extern "C" const char *q4b_last_error(void) { return g_last_error.c_str(); }

extern "C" const char *q4b_status_name(int status) {
    switch (status) {
        case Q4B_OK: return "Ok";
        case Q4B_NO_DEVICE: return "NoDevice";
        case Q4B_EMPTY_BUFFER: return "EmptyBuffer";
        case Q4B_POOL_POISONED: return "ActivationPoolPoisoned";
        case Q4B_EMPTY_DIMENSION: return "EmptyDimension";
        case Q4B_INPUT_NOT_GROUPED: return "InputNotGrouped";
        case Q4B_WRONG_LENGTH: return "WrongLength";
        case Q4B_MISSING_SHARD: return "MissingMappedShard";
        case Q4B_INVALID_BUFFER_OFFSET: return "InvalidBufferOffset";
        case Q4B_TENSOR_OUT_OF_RANGE: return "MappedTensorOutOfRange";
        case Q4B_DIMENSION_OVERFLOW: return "DimensionOverflow";
        case Q4B_COMMAND_FAILED: return "CommandFailed";
        case Q4B_CUDA_ERROR: return "CudaError";
        case Q4B_INVALID_ARGUMENT: return "InvalidArgument";
        case Q4B_UNSUPPORTED: return "Unsupported";
        case Q4B_IO_ERROR: return "Read";
        case Q4B_JSON_ERROR: return "Json";
        case Q4B_MISSING_QUANTIZATION: return "MissingQuantization";
        case Q4B_UNSUPPORTED_QUANTIZATION: return "UnsupportedQuantization";
        case Q4B_UNSAFE_SHARD_PATH: return "UnsafeShardPath";
        case Q4B_INVALID_HEADER_LENGTH: return "InvalidHeaderLength";
        case Q4B_MISSING_INDEXED_TENSOR: return "MissingIndexedTensor";
        case Q4B_INVALID_TENSOR_OFFSETS: return "InvalidTensorOffsets";
        case Q4B_INVALID_TENSOR_METADATA: return "InvalidTensorMetadata";
        case Q4B_MISSING_TENSOR: return "MissingTensor";
        case Q4B_INVALID_RUNTIME_TENSOR: return "InvalidRuntimeTensor";
        case Q4B_UNSUPPORTED_DTYPE: return "UnsupportedRuntimeDtype";
        case Q4B_INCOMPLETE_AFFINE_GROUP: return "IncompleteAffineGroup";
        case Q4B_NOT_QUANTIZED_WEIGHT: return "NotQuantizedWeight";
        case Q4B_INVALID_QUANTIZED_WEIGHT: return "InvalidQuantizedWeight";
        case Q4B_INVALID_AFFINE_TENSOR: return "InvalidAffineTensor";
        case Q4B_TENSOR_BYTE_LENGTH: return "TensorByteLength";
        case Q4B_INPUT_DIMENSION: return "InputDimension";
        case Q4B_INVALID_CONFIG: return "InvalidConfig";
        case Q4B_TOKEN_OUT_OF_RANGE: return "TokenOutOfRange";
        default: return "Unknown";
    }
}

extern "C" int q4b_device_info(q4b_runtime *rt, int *sm_count, uint64_t *total_bytes, char *name, uint32_t name_len) {
    if (int st = check_rt(rt)) return st;
    if (sm_count) *sm_count = rt->sm_count;
    if (total_bytes) *total_bytes = rt->total_bytes;
    if (name && name_len) snprintf(name, name_len, "%s", rt->name);
    return Q4B_OK;
}

// ------------------------------------------------------------------------------------------
// shards
// ------------------------------------------------------------------------------------------

static int shard_new(q4b_runtime *rt, uint64_t bytes, uint32_t *shard_id) {
    if (int st = check_rt(rt)) return st;
    if (!shard_id) return fail(Q4B_INVALID_ARGUMENT, "shard id pointer is null");
    if (bytes == 0) return fail(Q4B_EMPTY_BUFFER, "CUDA buffers cannot be empty");
    void *p = nullptr;
    Q4B_CUDA(cudaMalloc(&p, bytes + kShardTailPad), "shard allocation");
    Q4B_CUDA(cudaMemset((uint8_t *)p + bytes, 0, kShardTailPad), "shard tail clear");
    Shard s;
    s.ptr = (uint8_t *)p;
    s.bytes = bytes;
    rt->shards.push_back(s);
    *shard_id = (uint32_t)(rt->shards.size() - 1);
    return Q4B_OK;
}

// Host-to-device copy of a large pageable range (a mapped safetensors file): the range is moved through two
// pinned staging buffers so that the host-side copy (and the page faults behind it) of one piece overlaps the DMA
// of the previous one. Small copies go straight through cudaMemcpy.
constexpr size_t kStageBytes = 16u << 20;

static cudaError_t staged_h2d(q4b_runtime *rt, uint8_t *dst, const uint8_t *src, uint64_t bytes) {
    if (bytes <= kStageBytes / 2) return cudaMemcpy(dst, src, bytes, cudaMemcpyHostToDevice);
    for (int i = 0; i < 2; ++i) {
        if (!rt->stage[i]) {
            cudaError_t e = cudaHostAlloc(&rt->stage[i], kStageBytes, cudaHostAllocDefault);
            if (e != cudaSuccess) {
                rt->stage[i] = nullptr;
                cudaGetLastError();
                return cudaMemcpy(dst, src, bytes, cudaMemcpyHostToDevice);  // no pinned memory to be had: plain copy
            }
            e = cudaEventCreateWithFlags(&rt->stage_done[i], cudaEventDisableTiming);
            if (e != cudaSuccess) return e;
        }
    }
    uint64_t done = 0;
    int slot = 0;
    bool used[2] = {false, false};
    while (done < bytes) {
        const uint64_t n = bytes - done < kStageBytes ? bytes - done : kStageBytes;
        if (used[slot]) {
            cudaError_t e = cudaEventSynchronize(rt->stage_done[slot]);
            if (e != cudaSuccess) return e;
        }
        memcpy(rt->stage[slot], src + done, n);
        cudaError_t e = cudaMemcpyAsync(dst + done, rt->stage[slot], n, cudaMemcpyHostToDevice, rt->stream);
        if (e == cudaSuccess) e = cudaEventRecord(rt->stage_done[slot], rt->stream);
        if (e != cudaSuccess) return e;
        used[slot] = true;
        done += n;
        slot ^= 1;
    }
    return cudaStreamSynchronize(rt->stream);
}

extern "C" int q4b_shard_upload(q4b_runtime *rt, const void *host_bytes, uint64_t bytes, uint32_t *shard_id) {
    if (int st = check_rt(rt)) return st;
    if (!host_bytes && bytes) return fail(Q4B_INVALID_ARGUMENT, "host pointer is null");
    std::lock_guard<std::recursive_mutex> lock(rt->mu);
    DeviceGuard guard(rt->device);
    uint32_t id = 0;
    if (int st = shard_new(rt, bytes, &id)) return st;
    cudaError_t e = staged_h2d(rt, rt->shards[id].ptr, (const uint8_t *)host_bytes, bytes);
    if (e != cudaSuccess) {
        cudaFree(rt->shards[id].ptr);
        rt->shards.pop_back();
        return fail_cuda(e, "shard upload");
    }
    *shard_id = id;
    return Q4B_OK;
}

// MappedWeightBuffers going out of scope in the reference: the device copy is released; the id stays taken and
// later use of it reports Q4B_MISSING_SHARD.
extern "C" int q4b_shard_free(q4b_runtime *rt, uint32_t shard_id) {
    if (int st = check_rt(rt)) return st;
    std::lock_guard<std::recursive_mutex> lock(rt->mu);
    DeviceGuard guard(rt->device);
    if (shard_id >= rt->shards.size() || !rt->shards[shard_id].ptr)
        return fail(Q4B_MISSING_SHARD, "mapped safetensors shard %u is absent", shard_id);
    Q4B_CUDA(cudaDeviceSynchronize(), "device synchronize");
    cudaFree(rt->shards[shard_id].ptr);
    rt->shards[shard_id].ptr = nullptr;
    rt->shards[shard_id].bytes = 0;
    return Q4B_OK;
}

extern "C" int q4b_shard_alloc(q4b_runtime *rt, uint64_t bytes, uint32_t *shard_id) {
    if (int st = check_rt(rt)) return st;
    std::lock_guard<std::recursive_mutex> lock(rt->mu);
    DeviceGuard guard(rt->device);
    return shard_new(rt, bytes, shard_id);
}

static int shard_range(q4b_runtime *rt, uint32_t shard_id, uint64_t offset, uint64_t bytes) {
    if (shard_id >= rt->shards.size() || !rt->shards[shard_id].ptr)
        return fail(Q4B_MISSING_SHARD, "mapped safetensors shard %u is absent", shard_id);
    if (offset > rt->shards[shard_id].bytes) return fail(Q4B_INVALID_BUFFER_OFFSET, "mapped tensor offset is outside its shard");
    if (bytes > rt->shards[shard_id].bytes - offset)
        return fail(Q4B_TENSOR_OUT_OF_RANGE, "mapped tensor range exceeds its safetensors shard");
    return Q4B_OK;
}

extern "C" int q4b_shard_write(q4b_runtime *rt, uint32_t shard_id, uint64_t offset, const void *host_bytes,
                               uint64_t bytes) {
    if (int st = check_rt(rt)) return st;
    std::lock_guard<std::recursive_mutex> lock(rt->mu);
    DeviceGuard guard(rt->device);
    if (int st = shard_range(rt, shard_id, offset, bytes)) return st;
    if (bytes == 0) return Q4B_OK;
    if (!host_bytes) return fail(Q4B_INVALID_ARGUMENT, "host pointer is null");
    Q4B_CUDA(staged_h2d(rt, rt->shards[shard_id].ptr + offset, (const uint8_t *)host_bytes, bytes), "shard write");
    return Q4B_OK;
}

extern "C" int q4b_shard_read(q4b_runtime *rt, uint32_t shard_id, uint64_t offset, void *host_bytes, uint64_t bytes) {
    if (int st = check_rt(rt)) return st;
    std::lock_guard<std::recursive_mutex> lock(rt->mu);
    DeviceGuard guard(rt->device);
    if (int st = shard_range(rt, shard_id, offset, bytes)) return st;
    if (bytes == 0) return Q4B_OK;
    if (!host_bytes) return fail(Q4B_INVALID_ARGUMENT, "host pointer is null");
    Q4B_CUDA(cudaDeviceSynchronize(), "device synchronize");
    Q4B_CUDA(cudaMemcpy(host_bytes, rt->shards[shard_id].ptr + offset, bytes, cudaMemcpyDeviceToHost), "shard read");
    return Q4B_OK;
}

extern "C" int q4b_shard_count(q4b_runtime *rt, uint32_t *count) {
    if (int st = check_rt(rt)) return st;
    if (!count) return fail(Q4B_INVALID_ARGUMENT, "count pointer is null");
    std::lock_guard<std::recursive_mutex> lock(rt->mu);
    *count = (uint32_t)rt->shards.size();
    return Q4B_OK;
}

extern "C" int q4b_shard_info(q4b_runtime *rt, uint32_t shard_id, void **device_ptr, uint64_t *bytes) {
    if (int st = check_rt(rt)) return st;
    std::lock_guard<std::recursive_mutex> lock(rt->mu);
    if (int st = shard_range(rt, shard_id, 0, 0)) return st;
    if (device_ptr) *device_ptr = rt->shards[shard_id].ptr;
    if (bytes) *bytes = rt->shards[shard_id].bytes;
    return Q4B_OK;
}

extern "C" int q4b_offset_is_aligned(q4b_runtime *rt, uint32_t shard_id, uint64_t byte_offset, uint64_t alignment,
                                     int *aligned) {
    if (int st = check_rt(rt)) return st;
    if (!aligned || alignment == 0) return fail(Q4B_INVALID_ARGUMENT, "alignment must be positive and the result pointer non-null");
    std::lock_guard<std::recursive_mutex> lock(rt->mu);
    if (int st = shard_range(rt, shard_id, 0, 0)) return st;
    *aligned = (((uintptr_t)rt->shards[shard_id].ptr + byte_offset) % alignment) == 0 ? 1 : 0;
    return Q4B_OK;
}

// ------------------------------------------------------------------------------------------
// device-resident entry points
// ------------------------------------------------------------------------------------------

extern "C" int q4b_matmul_batch_device(q4b_runtime *rt, const void *x_dev, int x_dtype, uint64_t m, uint64_t k,
                                       const q4b_job *jobs, uint32_t n_jobs, float *const *outputs_dev,
                                       uint32_t flags, void *stream) {
    if (int st = check_rt(rt)) return st;
    if (int st = check_dtype(x_dtype)) return st;
    if (!x_dev || !outputs_dev) return fail(Q4B_INVALID_ARGUMENT, "activation or output pointer is null");
    if ((uintptr_t)x_dev & 15u) return fail(Q4B_INVALID_ARGUMENT, "device activations must be 16-byte aligned");
    std::lock_guard<std::recursive_mutex> lock(rt->mu);
    DeviceGuard guard(rt->device);
    std::vector<Resolved> resolved;
    if (int st = resolve_jobs(rt, jobs, n_jobs, m, k, &resolved)) return st;
    for (uint32_t i = 0; i < n_jobs; ++i)
        if (!outputs_dev[i]) return fail(Q4B_INVALID_ARGUMENT, "output pointer %u is null", i);
    return enqueue_matmul(rt, x_dev, x_dtype, m, k, resolved, outputs_dev, flags, (cudaStream_t)stream);
}

extern "C" int q4b_argmax_batch_device(q4b_runtime *rt, const void *x_dev, int x_dtype, uint64_t m, uint64_t k,
                                       const q4b_job *job, uint32_t index_base, uint32_t *tokens_dev,
                                       float *values_dev, void *stream) {
    if (int st = check_rt(rt)) return st;
    if (int st = check_dtype(x_dtype)) return st;
    if (!x_dev || !tokens_dev || !job) return fail(Q4B_INVALID_ARGUMENT, "activation, job or token pointer is null");
    std::lock_guard<std::recursive_mutex> lock(rt->mu);
    DeviceGuard guard(rt->device);
    std::vector<Resolved> resolved;
    if (int st = resolve_jobs(rt, job, 1, m, k, &resolved)) return st;
    const uint32_t n = resolved[0].n;
    const uint32_t parts = q4k_argmax_parts(n);
    Q4B_CUDA(rt->logits.ensure((size_t)m * n * 4), "logit scratch");
    Q4B_CUDA(rt->amax_v.ensure((size_t)m * parts * 4), "argmax scratch");
    Q4B_CUDA(rt->amax_i.ensure((size_t)m * parts * 4), "argmax scratch");
    float *logits = (float *)rt->logits.ptr;
    if (int st = enqueue_matmul(rt, x_dev, x_dtype, m, k, resolved, &logits, 0, (cudaStream_t)stream)) return st;
    Q4B_CUDA(q4k_argmax_rows(logits, (uint32_t)m, n, index_base, (float *)rt->amax_v.ptr, (uint32_t *)rt->amax_i.ptr,
                             tokens_dev, values_dev, (cudaStream_t)stream),
             "argmax launch");
    rt->launches += 2;
    return Q4B_OK;
}

extern "C" int q4b_swiglu_device(q4b_runtime *rt, const float *gate_dev, const float *up_dev, uint64_t count,
                                 float *out_f32_dev, uint16_t *out_bf16_dev, void *stream) {
    if (int st = check_rt(rt)) return st;
    if (!gate_dev || !up_dev || (!out_f32_dev && !out_bf16_dev)) return fail(Q4B_INVALID_ARGUMENT, "swiglu pointer is null");
    if (count == 0) return fail(Q4B_EMPTY_DIMENSION, "matrix dimensions must be greater than zero");
    std::lock_guard<std::recursive_mutex> lock(rt->mu);
    DeviceGuard guard(rt->device);
    Q4B_CUDA(q4k_swiglu(gate_dev, up_dev, count, out_f32_dev, out_bf16_dev, (cudaStream_t)stream), "swiglu launch");
    rt->launches++;
    return Q4B_OK;
}

extern "C" int q4b_rms_unit_bf16_device(q4b_runtime *rt, const float *in_dev, uint32_t rows, uint32_t n, float eps,
                                        uint16_t *out_bf16_dev, void *stream) {
    if (int st = check_rt(rt)) return st;
    if (!in_dev || !out_bf16_dev) return fail(Q4B_INVALID_ARGUMENT, "rms pointer is null");
    if (rows == 0 || n == 0) return fail(Q4B_EMPTY_DIMENSION, "matrix dimensions must be greater than zero");
    std::lock_guard<std::recursive_mutex> lock(rt->mu);
    DeviceGuard guard(rt->device);
    Q4B_CUDA(q4k_rms_unit_bf16(in_dev, rows, n, eps, out_bf16_dev, (cudaStream_t)stream), "rms launch");
    rt->launches++;
    return Q4B_OK;
}

// ------------------------------------------------------------------------------------------
// host-buffer entry points
// ------------------------------------------------------------------------------------------

static int host_matmul(q4b_runtime *rt, const void *x, int x_dtype, uint64_t m, uint64_t k, const q4b_job *jobs,
                       uint32_t n_jobs, float *const *outputs, uint32_t flags) {
    if (int st = check_rt(rt)) return st;
    if (int st = check_dtype(x_dtype)) return st;
    if (!x || !outputs) return fail(Q4B_INVALID_ARGUMENT, "activation or output pointer is null");
    std::lock_guard<std::recursive_mutex> lock(rt->mu);
    DeviceGuard guard(rt->device);
    std::vector<Resolved> resolved;
    if (int st = resolve_jobs(rt, jobs, n_jobs, m, k, &resolved)) return st;
    for (uint32_t i = 0; i < n_jobs; ++i)
        if (!outputs[i]) return fail(Q4B_INVALID_ARGUMENT, "output pointer %u is null", i);
    const size_t esize = x_dtype == Q4B_F32 ? 4 : 2;
    Q4B_CUDA(rt->x_in.ensure((size_t)m * k * esize), "activation buffer");
    // one device buffer holds every job's [m][n] output, 256-byte aligned slices
    std::vector<size_t> offs(n_jobs);
    size_t total = 0;
    for (uint32_t i = 0; i < n_jobs; ++i) {
        offs[i] = total;
        total += (((size_t)m * resolved[i].n * 4) + 255) & ~(size_t)255;
    }
    Q4B_CUDA(rt->outs[0].ensure(total), "output buffer");
    cudaStream_t s = rt->stream;
    Q4B_CUDA(cudaMemcpyAsync(rt->x_in.ptr, x, (size_t)m * k * esize, cudaMemcpyHostToDevice, s), "activation upload");
    std::vector<float *> outs_dev(n_jobs);
    for (uint32_t i = 0; i < n_jobs; ++i) {
        outs_dev[i] = (float *)((uint8_t *)rt->outs[0].ptr + offs[i]);
        if (flags & Q4B_FLAG_ACCUMULATE)
            Q4B_CUDA(cudaMemcpyAsync(outs_dev[i], outputs[i], (size_t)m * resolved[i].n * 4, cudaMemcpyHostToDevice, s),
                     "residual upload");
    }
    if (int st = enqueue_matmul(rt, rt->x_in.ptr, x_dtype, m, k, resolved, outs_dev.data(), flags, s)) {
        cudaStreamSynchronize(s);
        return st;
    }
    // results are downloaded into the runtime's staging buffer and copied to the caller only after the device
    // reported success: caller buffers stay untouched on failure
    Q4B_CUDA(rt->results.ensure(total), "result staging");
    for (uint32_t i = 0; i < n_jobs; ++i)
        Q4B_CUDA(cudaMemcpyAsync((uint8_t *)rt->results.ptr + offs[i], outs_dev[i], (size_t)m * resolved[i].n * 4, cudaMemcpyDeviceToHost, s),
                 "result download");
    if (int st = finish(rt, s)) return st;
    for (uint32_t i = 0; i < n_jobs; ++i) memcpy(outputs[i], (uint8_t *)rt->results.ptr + offs[i], (size_t)m * resolved[i].n * 4);
    return Q4B_OK;
}

extern "C" int q4b_matvec_batch(q4b_runtime *rt, const void *x, int x_dtype, uint64_t k, const q4b_job *jobs,
                                uint32_t n_jobs, float *const *outputs) {
    return host_matmul(rt, x, x_dtype, 1, k, jobs, n_jobs, outputs, 0);
}

extern "C" int q4b_matmul_batch(q4b_runtime *rt, const void *x, int x_dtype, uint64_t m, uint64_t k,
                                const q4b_job *jobs, uint32_t n_jobs, float *const *outputs) {
    return host_matmul(rt, x, x_dtype, m, k, jobs, n_jobs, outputs, 0);
}

extern "C" int q4b_matmul_add_batch(q4b_runtime *rt, const void *x, int x_dtype, uint64_t m, uint64_t k,
                                    const q4b_job *jobs, uint32_t n_jobs, float *const *outputs) {
    return host_matmul(rt, x, x_dtype, m, k, jobs, n_jobs, outputs, Q4B_FLAG_ACCUMULATE);
}

extern "C" int q4b_argmax_batch(q4b_runtime *rt, const void *x, int x_dtype, uint64_t m, uint64_t k,
                                const q4b_job *job, uint32_t *tokens) {
    if (int st = check_rt(rt)) return st;
    if (int st = check_dtype(x_dtype)) return st;
    if (!x || !tokens || !job) return fail(Q4B_INVALID_ARGUMENT, "activation, job or token pointer is null");
    if (m == 0 || k == 0) return fail(Q4B_EMPTY_DIMENSION, "matrix dimensions must be greater than zero");
    std::lock_guard<std::recursive_mutex> lock(rt->mu);
    DeviceGuard guard(rt->device);
    const size_t esize = x_dtype == Q4B_F32 ? 4 : 2;
    Q4B_CUDA(rt->x_in.ensure((size_t)m * k * esize), "activation buffer");
    Q4B_CUDA(rt->tokens.ensure((size_t)m * 4), "token buffer");
    cudaStream_t s = rt->stream;
    Q4B_CUDA(cudaMemcpyAsync(rt->x_in.ptr, x, (size_t)m * k * esize, cudaMemcpyHostToDevice, s), "activation upload");
    if (int st = q4b_argmax_batch_device(rt, rt->x_in.ptr, x_dtype, m, k, job, 0, (uint32_t *)rt->tokens.ptr, nullptr, s)) {
        cudaStreamSynchronize(s);
        return st;
    }
    std::vector<uint32_t> staged(m);
    Q4B_CUDA(cudaMemcpyAsync(staged.data(), rt->tokens.ptr, (size_t)m * 4, cudaMemcpyDeviceToHost, s), "token download");
    if (int st = finish(rt, s)) return st;
    memcpy(tokens, staged.data(), (size_t)m * 4);
    return Q4B_OK;
}

// down(silu(gate x) * (up x)) on device buffers. From gemm_min_m activation rows on, and when gate and up sit at the same
// offset from a 16-byte boundary, the front half is ONE tensor-core launch whose epilogue applies the SwiGLU and
// writes the hidden rows as bf16 in the layout the down projection's GEMM reads -- no fp32 [m][inter] buffers, no
// separate SwiGLU or conversion pass (the reference keeps this chain in 16-bit intermediates under one fence,
// src/metal_runtime.rs:4267-4474). Otherwise: two projections, the SwiGLU kernel, the down projection.
extern "C" int q4b_mlp_batch_device(q4b_runtime *rt, const void *x_dev, int x_dtype, uint64_t m, uint64_t k, const q4b_job *gate,
                                    const q4b_job *up, const q4b_job *down, float *out_dev, void *stream) {
    if (int st = check_rt(rt)) return st;
    if (int st = check_dtype(x_dtype)) return st;
    if (!x_dev || !out_dev || !gate || !up || !down) return fail(Q4B_INVALID_ARGUMENT, "activation, job or output pointer is null");
    if (m == 0 || k == 0) return fail(Q4B_EMPTY_DIMENSION, "matrix dimensions must be greater than zero");
    // gate and up must agree (src/metal_runtime.rs:4511-4517)
    if (gate->output_rows != up->output_rows)
        return fail(Q4B_WRONG_LENGTH, "up projection rows has %llu elements, expected %llu",
                    (unsigned long long)up->output_rows, (unsigned long long)gate->output_rows);
    std::lock_guard<std::recursive_mutex> lock(rt->mu);
    DeviceGuard guard(rt->device);
    cudaStream_t s = (cudaStream_t)stream;
    const uint64_t inter = gate->output_rows;
    std::vector<Resolved> gu, dn;
    const q4b_job pair[2] = {*gate, *up};
    if (int st = resolve_jobs(rt, pair, 2, m, k, &gu)) return st;
    if (int st = resolve_jobs(rt, down, 1, m, inter, &dn)) return st;
    const bool fused = m >= rt->gemm_min_m && !rt->mlp_unfused && inter % 64 == 0 && q4k_gemm_pair_supported(gu[0].w, gu[1].w);
    if (fused) {
        Q4B_CUDA(rt->gemm_x.ensure((size_t)m * k * 2), "activation scratch");
        Q4B_CUDA(rt->hidden.ensure((size_t)m * inter * 2), "hidden buffer");
        Q4B_CUDA(q4k_gemm_prepare_x(x_dev, x_dtype == Q4B_F32 ? 1 : 0, m * k, (uint16_t *)rt->gemm_x.ptr, s), "q4_gemm_prepare_x launch");
        if (int st = profile_open(rt, s)) return st;
        Q4B_CUDA(q4k_gemm_tc_pair((const uint16_t *)rt->gemm_x.ptr, (uint32_t)m, (uint32_t)k, gu[0].w, gu[0].s, gu[0].b, gu[1].w, gu[1].s,
                                  gu[1].b, (uint32_t)inter, (uint16_t *)rt->hidden.ptr, (uint32_t)inter, (int *)rt->error_flag.ptr,
                                  (uint32_t)rt->sm_count, s),
                 "q4_gemm_tc pair launch");
        if (int st = profile_close(rt, s, 2 * inter * (k / 2 + (k / 64) * 4) + m * k * 2 + m * inter * 2, 4ull * m * inter * k)) return st;
        uint32_t split_blocks = 0;
        const uint32_t splits = q4k_gemm_k_splits((uint32_t)m, dn[0].n, (uint32_t)inter, (uint32_t)rt->sm_count, &split_blocks);
        if (splits > 1) Q4B_CUDA(rt->gemm_parts.ensure((size_t)splits * m * dn[0].n * 4), "partial output scratch");
        if (int st = profile_open(rt, s)) return st;
        Q4B_CUDA(q4k_gemm_tc((const uint16_t *)rt->hidden.ptr, (uint32_t)m, (uint32_t)inter, dn[0].w, dn[0].s, dn[0].b, dn[0].n, out_dev,
                             dn[0].n, 0, (int *)rt->error_flag.ptr, (uint32_t)rt->sm_count, (float *)rt->gemm_parts.ptr, s),
                 "q4_gemm_tc launch");
        rt->launches += 3;
        return profile_close(rt, s, (uint64_t)dn[0].n * (inter / 2 + (inter / 64) * 4) + m * inter * 2 + m * dn[0].n * 4, 2ull * m * dn[0].n * inter);
    }
    Q4B_CUDA(rt->gate.ensure((size_t)m * inter * 4), "gate buffer");
    Q4B_CUDA(rt->up.ensure((size_t)m * inter * 4), "up buffer");
    Q4B_CUDA(rt->hidden.ensure((size_t)m * inter * 4), "hidden buffer");
    float *gu_out[2] = {(float *)rt->gate.ptr, (float *)rt->up.ptr};
    if (int st = enqueue_matmul(rt, x_dev, x_dtype, m, k, gu, gu_out, 0, s)) return st;
    Q4B_CUDA(q4k_swiglu(gu_out[0], gu_out[1], m * inter, (float *)rt->hidden.ptr, nullptr, s), "swiglu launch");
    rt->launches++;
    // the intermediate stays fp32 (the decode chain of the reference, src/metal_runtime.rs:4616-4645)
    return enqueue_matmul(rt, rt->hidden.ptr, Q4B_F32, m, inter, dn, &out_dev, 0, s);
}

extern "C" int q4b_mlp_batch(q4b_runtime *rt, const void *x, int x_dtype, uint64_t m, uint64_t k, const q4b_job *gate,
                             const q4b_job *up, const q4b_job *down, float *out) {
    if (int st = check_rt(rt)) return st;
    if (int st = check_dtype(x_dtype)) return st;
    if (!x || !out || !gate || !up || !down) return fail(Q4B_INVALID_ARGUMENT, "activation, job or output pointer is null");
    if (m == 0 || k == 0) return fail(Q4B_EMPTY_DIMENSION, "matrix dimensions must be greater than zero");
    std::lock_guard<std::recursive_mutex> lock(rt->mu);
    DeviceGuard guard(rt->device);
    const size_t esize = x_dtype == Q4B_F32 ? 4 : 2;
    const uint64_t rows = down->output_rows;
    if (rows == 0 || rows > 0xffffffffull) return fail(Q4B_EMPTY_DIMENSION, "matrix dimensions must be greater than zero");
    Q4B_CUDA(rt->x_in.ensure((size_t)m * k * esize), "activation buffer");
    Q4B_CUDA(rt->outs[0].ensure((size_t)m * rows * 4), "output buffer");
    cudaStream_t s = rt->stream;
    Q4B_CUDA(cudaMemcpyAsync(rt->x_in.ptr, x, (size_t)m * k * esize, cudaMemcpyHostToDevice, s), "activation upload");
    float *dn_out = (float *)rt->outs[0].ptr;
    if (int st = q4b_mlp_batch_device(rt, rt->x_in.ptr, x_dtype, m, k, gate, up, down, dn_out, s)) {
        cudaStreamSynchronize(s);
        return st;
    }
    Q4B_CUDA(rt->results.ensure((size_t)m * rows * 4), "result staging");
    Q4B_CUDA(cudaMemcpyAsync(rt->results.ptr, dn_out, (size_t)m * rows * 4, cudaMemcpyDeviceToHost, s), "result download");
    if (int fst = finish(rt, s)) return fst;
    memcpy(out, rt->results.ptr, (size_t)m * rows * 4);
    return Q4B_OK;
}

extern "C" int q4b_dequantize_row(q4b_runtime *rt, const q4b_job *job, uint64_t k, uint64_t row, float *out) {
    if (int st = check_rt(rt)) return st;
    if (!job || !out) return fail(Q4B_INVALID_ARGUMENT, "job or output pointer is null");
    std::lock_guard<std::recursive_mutex> lock(rt->mu);
    DeviceGuard guard(rt->device);
    Resolved r;
    if (int st = resolve_job(rt, *job, k, &r)) return st;
    if (row >= r.n) return fail(Q4B_WRONG_LENGTH, "row has %llu elements, expected %u", (unsigned long long)row, r.n);
    Q4B_CUDA(rt->outs[0].ensure((size_t)k * 4), "output buffer");
    cudaStream_t s = rt->stream;
    Q4B_CUDA(q4k_dequantize_row(r.w, r.s, r.b, (uint32_t)k, (uint32_t)row, (float *)rt->outs[0].ptr, s), "dequantize launch");
    rt->launches++;
    Q4B_CUDA(rt->results.ensure((size_t)k * 4), "result staging");
    Q4B_CUDA(cudaMemcpyAsync(rt->results.ptr, rt->outs[0].ptr, (size_t)k * 4, cudaMemcpyDeviceToHost, s), "result download");
    if (int st = finish(rt, s)) return st;
    memcpy(out, rt->results.ptr, (size_t)k * 4);
    return Q4B_OK;
}

// ------------------------------------------------------------------------------------------
// persistent decode chain
// ------------------------------------------------------------------------------------------

struct q4b_chain {
    q4b_runtime *rt = nullptr;
    q4::StackParams params;               // kernel arguments (device pointers)
    std::vector<void *> owned;            // device allocations of this chain
    void *reset_region = nullptr;         // local arrival counter + running maxima: zeroed before every launch
    size_t reset_bytes = 0;
    uint32_t n_phases = 0, n_stages = 0;
    void *first_x = nullptr;              // first stage's bf16 activation (host twin of run copies into it)
    uint64_t first_x_bytes = 0;
    uint32_t *token = nullptr;
    float *best = nullptr;
    bool multi_rank = false;
    uint64_t failures_seen = 0;           // rt->failures when the chain was created / last repaired
    std::vector<uint32_t> phase_stage;    // stage each phase belongs to (trace read-out)
    std::vector<uint32_t> phase_role;     // 0 main, 1 deferred jobs of the same stage, 2 deferred jobs of the stage before
};

extern "C" int q4b_arena_create(q4b_runtime *rt, uint64_t bytes, void **device_ptr, uint8_t handle[64]) {
    if (int st = check_rt(rt)) return st;
    if (!device_ptr || !handle) return fail(Q4B_INVALID_ARGUMENT, "output pointer is null");
    if (bytes == 0) return fail(Q4B_EMPTY_BUFFER, "CUDA buffers cannot be empty");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    std::lock_guard<std::recursive_mutex> lock(rt->mu);
    DeviceGuard guard(rt->device);
    void *p = nullptr;
    Q4B_CUDA(cudaMalloc(&p, bytes), "arena allocation");
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaMemset(p, 0, bytes);
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) {
        cudaFree(p);
        return fail_cuda(e, "arena export");
    }
    memcpy(handle, &h, 64);
    rt->arenas.push_back(p);
    *device_ptr = p;
    return Q4B_OK;
}

extern "C" int q4b_arena_open(q4b_runtime *rt, const uint8_t handle[64], void **peer_ptr) {
    if (int st = check_rt(rt)) return st;
    if (!peer_ptr || !handle) return fail(Q4B_INVALID_ARGUMENT, "output pointer is null");
    std::lock_guard<std::recursive_mutex> lock(rt->mu);
    DeviceGuard guard(rt->device);
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, 64);
    void *p = nullptr;
    Q4B_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess), "arena import");
    rt->peer_arenas.push_back(p);
    *peer_ptr = p;
    return Q4B_OK;
}

extern "C" uint64_t q4b_chain_max_k(void) { return q4k_stack_max_k(); }

namespace {

struct ByteRange {
    uintptr_t lo, hi;
    bool overlaps(uintptr_t a, uintptr_t b) const { return a < hi && lo < b; }
};

// what one stage reads to build its activation
void stage_sources(const q4b_stage &S, std::vector<ByteRange> *out) {
    const uintptr_t s0 = (uintptr_t)S.src0, s1 = (uintptr_t)S.src1;
    if (S.x_kind == Q4B_X_BF16) out->push_back({s0, s0 + S.k * 2});
    if (S.x_kind == Q4B_X_SWIGLU) {
        out->push_back({s0, s0 + S.k * 4});
        out->push_back({s1, s1 + S.k * 4});
    }
    if (S.x_kind == Q4B_X_RMS) {
        const uint64_t parts = S.src_parts ? S.src_parts : 1;
        out->push_back({s0, s0 + (parts - 1) * S.src_part_stride + S.k * 4});
    }
}

struct ChainBuild {
    std::vector<void *> owned;
    ~ChainBuild() {
        for (void *p : owned) cudaFree(p);
    }
    cudaError_t alloc(void **p, size_t bytes, bool zero) {
        cudaError_t e = cudaMalloc(p, bytes ? bytes : 16);
        if (e != cudaSuccess) return e;
        owned.push_back(*p);
        return zero ? cudaMemset(*p, 0, bytes ? bytes : 16) : cudaSuccess;
    }
};

}  // namespace

extern "C" int q4b_chain_create(q4b_runtime *rt, const q4b_stage *stages, uint32_t n_stages, const float *logits, uint32_t vocab,
                                uint32_t index_base, uint32_t *token_dev, float *best_dev, const q4b_peers *peers, q4b_chain **out) {
    if (int st = check_rt(rt)) return st;
    if (!stages || n_stages == 0 || !out) return fail(Q4B_INVALID_ARGUMENT, "stage list or output handle is null");
    if (logits && (!token_dev || vocab == 0)) return fail(Q4B_INVALID_ARGUMENT, "token pointer is null or vocabulary empty");
    if (peers && (peers->world < 2 || peers->world > (uint32_t)q4::kMaxPeers || peers->rank >= peers->world))
        return fail(Q4B_INVALID_ARGUMENT, "a multi-rank chain needs 2..%d ranks and a rank below the world size", q4::kMaxPeers);
    std::lock_guard<std::recursive_mutex> lock(rt->mu);
    DeviceGuard guard(rt->device);
    const uint32_t warps = q4k_stack_warps();
    const uint32_t grid_warps = (uint32_t)rt->sm_count * warps;

    // ---- validate and resolve every stage ----
    struct StageJobs {
        std::vector<Resolved> res;
        uint32_t k, k_total, k_begin;
        int pair_a = -1, pair_b = -1;  // jobs fused with the SwiGLU of the next stage
        std::vector<int> deferred;     // jobs nothing later reads
        // Tagged hand-off to the next stage (its RMS-norm source is this job's output): 0 none, 1 through a buffer of
        // the chain (one GPU, or an output that stays local), 2 through the ranks' exchange arenas
        int ll_job = -1, ll_mode = 0;
        bool plain_consumed = false;   // a later stage reads an output of this stage as plain floats: needs a barrier
    };
    std::vector<StageJobs> sj(n_stages);
    uint32_t halfs[2] = {0, 0};
    for (uint32_t si = 0; si < n_stages; ++si) {
        const q4b_stage &S = stages[si];
        if (S.x_kind > Q4B_X_RMS) return fail(Q4B_INVALID_ARGUMENT, "unknown activation kind %u in stage %u", S.x_kind, si);
        if (!S.src0 || (S.x_kind == Q4B_X_SWIGLU && !S.src1) || !S.outputs || !S.jobs || S.n_jobs == 0)
            return fail(Q4B_INVALID_ARGUMENT, "stage %u has a null pointer or no projection", si);
        if (((uintptr_t)S.src0 | (uintptr_t)S.src1) & 15u) return fail(Q4B_INVALID_ARGUMENT, "stage %u: source vectors must be 16-byte aligned", si);
        if (S.n_jobs > (uint32_t)q4::kMaxJobs) return fail(Q4B_UNSUPPORTED, "stage %u has more than %d projections", si, q4::kMaxJobs);
        const uint64_t k_total = S.k_total ? S.k_total : S.k;
        if (S.k == 0 || S.k % 128 != 0 || k_total % 512 != 0 || S.k_begin % 64 != 0 || S.k_begin + S.k > k_total)
            return fail(Q4B_UNSUPPORTED, "stage %u: the decode chain needs k %% 128 == 0, a row length that is a multiple of 512 and a slice inside the row", si);
        if (S.x_kind != Q4B_X_SWIGLU && S.k > q4k_stack_max_k())
            return fail(Q4B_UNSUPPORTED, "stage %u: k exceeds %u", si, q4k_stack_max_k());
        if (S.x_kind == Q4B_X_RMS && S.src_parts > 1 && (S.src_part_stride % 16 != 0 || S.src_part_stride < S.k * 4))
            return fail(Q4B_INVALID_ARGUMENT, "stage %u: partial vectors must be 16-byte aligned and must not overlap", si);
        if (int st = resolve_jobs(rt, S.jobs, S.n_jobs, 1, k_total, &sj[si].res)) return st;
        for (uint32_t i = 0; i < S.n_jobs; ++i)
            if (!S.outputs[i]) return fail(Q4B_INVALID_ARGUMENT, "stage %u output %u is null", si, i);
        sj[si].k = (uint32_t)S.k;
        sj[si].k_total = (uint32_t)k_total;
        sj[si].k_begin = (uint32_t)S.k_begin;
    }
    if (n_stages * 3u >= q4::kMaxPhases) return fail(Q4B_UNSUPPORTED, "the decode chain takes fewer than %u stages", q4::kMaxPhases / 3u);

    auto has_peer_out = [&](uint32_t si, uint32_t i) {
        if (!peers || !stages[si].peer_outputs) return false;
        for (uint32_t r = 0; r < peers->world; ++r)
            if (r != peers->rank && stages[si].peer_outputs[(size_t)i * 8 + r]) return true;
        return false;
    };

    ChainBuild build;
    std::vector<q4::StackPhase> phases;
    std::vector<q4::StackJob> jobs;
    std::vector<uint32_t> phase_stage, phase_role;
    std::vector<std::pair<size_t, size_t>> pair_fixups;  // (job index, pair ordinal): h buffer and amax word assigned below
    std::vector<std::pair<size_t, uint32_t>> ll_fixups;  // (job index, stage): tagged hand-off buffers assigned below
    std::vector<uint32_t> pair_k;
    std::vector<uint32_t> pair_of_stage;
    std::vector<std::vector<ByteRange>> reads(n_stages);
    for (uint32_t si = 0; si < n_stages; ++si) stage_sources(stages[si], &reads[si]);
    // Two activation buffers (stages alternate between them, so that deferred projections can still read the previous
    // activation) when shared memory allows, else one buffer and no deferral: the plan is made twice if need be.
    bool single_buffer = rt->chain_no_deferral;
    for (int attempt = 0;; ++attempt) {
    phases.clear();
    jobs.clear();
    phase_stage.clear();
    phase_role.clear();
    pair_fixups.clear();
    ll_fixups.clear();
    pair_k.clear();
    pair_of_stage.assign(n_stages, 0xffffffffu);
    for (StageJobs &J : sj) {
        J.pair_a = J.pair_b = -1;
        J.deferred.clear();
        J.ll_job = -1;
        J.ll_mode = 0;
        J.plain_consumed = false;
    }
    // ---- fusion and deferral ----
    for (uint32_t si = 0; si + 1 < n_stages; ++si) {
        const q4b_stage &S = stages[si], &N = stages[si + 1];
        // gate/up pair: the next stage is the SwiGLU of two of this stage's outputs, whole
        if (N.x_kind == Q4B_X_SWIGLU && !rt->chain_no_fusion) {
            int ga = -1, ub = -1;
            for (uint32_t i = 0; i < S.n_jobs; ++i) {
                if ((const void *)S.outputs[i] == N.src0) ga = (int)i;
                if ((const void *)S.outputs[i] == N.src1) ub = (int)i;
            }
            if (ga >= 0 && ub >= 0 && ga != ub && sj[si].res[ga].n == N.k && sj[si].res[ub].n == N.k && !has_peer_out(si, ga) &&
                !has_peer_out(si, ub)) {
                sj[si].pair_a = ga;
                sj[si].pair_b = ub;
            }
        }
        // tagged hand-off: the next stage is the RMS-norm of this stage's output (one job, whole) or of the ranks'
        // partial outputs of it (arena slots wide enough for two tagged copies: 16 bytes per element)
        if (N.x_kind == Q4B_X_RMS && !rt->chain_no_handoff) {
            const uint64_t parts = N.src_parts ? N.src_parts : 1;
            for (uint32_t i = 0; i < S.n_jobs; ++i) {
                if (sj[si].res[i].n != N.k) continue;
                if (parts == 1 && (const void *)S.outputs[i] == N.src0 && !has_peer_out(si, i)) {
                    sj[si].ll_job = (int)i;
                    sj[si].ll_mode = 1;
                } else if (peers && parts == peers->world && has_peer_out(si, i) && N.src_part_stride >= 16 * N.k &&
                           (uintptr_t)S.outputs[i] == (uintptr_t)N.src0 + (uint64_t)peers->rank * N.src_part_stride) {
                    sj[si].ll_job = (int)i;
                    sj[si].ll_mode = 2;
                }
            }
        }
        // which outputs does a later stage (or the token reduction) read as plain floats? The fused SwiGLU and the tagged
        // hand-off are served by tags, everything else needs this stage's barrier
        for (uint32_t i = 0; i < S.n_jobs; ++i) {
            const uintptr_t lo = (uintptr_t)S.outputs[i], hi = lo + (uint64_t)sj[si].res[i].n * 4;
            if (logits && ByteRange{(uintptr_t)logits, (uintptr_t)logits + (uint64_t)vocab * 4}.overlaps(lo, hi)) sj[si].plain_consumed = true;
            for (uint32_t later = si + 1; later < n_stages; ++later) {
                const bool served_by_tags = later == si + 1 && (((int)i == sj[si].pair_a || (int)i == sj[si].pair_b) || (int)i == sj[si].ll_job);
                if (!served_by_tags)
                    for (const ByteRange &r : reads[later]) sj[si].plain_consumed = sj[si].plain_consumed || r.overlaps(lo, hi);
                // a stage that writes the same buffer again ends this value's life (layers reuse their buffers)
                bool rewritten = false;
                for (uint32_t j = 0; j < stages[later].n_jobs; ++j) {
                    const uintptr_t wlo = (uintptr_t)stages[later].outputs[j], whi = wlo + (uint64_t)sj[later].res[j].n * 4;
                    rewritten = rewritten || (wlo <= lo && hi <= whi);
                }
                if (rewritten) break;
            }
        }
        // deferral: outputs that no later stage (and not the token reduction) reads
        if (single_buffer) continue;
        for (uint32_t i = 0; i < S.n_jobs; ++i) {
            if ((int)i == sj[si].pair_a || (int)i == sj[si].pair_b || has_peer_out(si, i)) continue;
            const uintptr_t lo = (uintptr_t)S.outputs[i], hi = lo + (uint64_t)sj[si].res[i].n * 4;
            bool read_later = logits && ByteRange{(uintptr_t)logits, (uintptr_t)logits + (uint64_t)vocab * 4}.overlaps(lo, hi);
            for (uint32_t later = si + 1; later < n_stages && !read_later; ++later)
                for (const ByteRange &r : reads[later]) read_later = read_later || r.overlaps(lo, hi);
            if (!read_later) sj[si].deferred.push_back((int)i);
        }
        if (sj[si].deferred.size() == S.n_jobs) sj[si].deferred.clear();  // a stage keeps at least one job in its main phase
    }
    for (uint32_t si = 0; si < n_stages; ++si) {
        const bool fused = si > 0 && sj[si - 1].pair_a >= 0;
        if (stages[si].x_kind == Q4B_X_SWIGLU && !fused && stages[si].k > q4k_stack_max_k())
            return fail(Q4B_UNSUPPORTED, "stage %u: a SwiGLU stage that cannot be fused with the projections before it needs k <= %u", si, q4k_stack_max_k());
    }

    // ---- phases ----
    auto add_phase = [&](uint32_t si, uint32_t role, const std::vector<int> &list, bool with_pair) -> int {
        const q4b_stage &S = stages[si];
        const StageJobs &J = sj[si];
        q4::StackPhase P;
        memset(&P, 0, sizeof P);
        P.job_begin = (uint32_t)jobs.size();
        P.k = J.k;
        P.kp = (J.k + 127u) & ~127u;
        P.groups = J.k / 64;
        P.cpt = (P.groups + 1u) / 2u;
        P.x_buf = single_buffer ? 0u : (si & 1u);
        P.slot_set = (uint32_t)(phases.size() % q4::kPartialSets);
        const uint32_t cpt = P.cpt;
        const uint32_t extra = rt->chain_offset_cost - 100u;  // per cent a byte-offset chunk costs more than an aligned one
        uint32_t tiles = 0, vcpt_max = cpt;
        uint64_t units = 0;
        auto push = [&](const Resolved &a, const Resolved &b, float *out_a, float *out_b, bool pair, uint32_t stage_job) -> int {
            q4::StackJob j;
            memset(&j, 0, sizeof j);
            const Resolved *side[2] = {&a, &b};
            for (int sdx = 0; sdx < 2; ++sdx) {
                j.w[sdx] = side[sdx]->w + J.k_begin / 2;
                j.s[sdx] = side[sdx]->s + (J.k_begin / 64) * 2;
                j.b[sdx] = side[sdx]->b + (J.k_begin / 64) * 2;
            }
            j.out[0] = out_a;
            j.out[1] = out_b;
            j.n = a.n;
            j.rows_per_tile = pair ? 8u : 16u;
            j.b_row_offset = pair ? 0u : 8u;
            j.w_stride = J.k_total / 2;
            j.p_stride = (J.k_total / 64) * 2;
            j.tile_begin = tiles;
            j.pair = pair ? 1u : 0u;
            const uint32_t off_sides = (((uintptr_t)j.w[0] & 15u) ? 1u : 0u) + (((uintptr_t)j.w[1] & 15u) ? 1u : 0u);
            j.vcpt = (cpt * (200u + extra * off_sides) + 100u) / 200u;
            if (units > 0xffffffffull) return fail(Q4B_UNSUPPORTED, "stage %u is too large for the decode chain", si);
            j.unit_begin = (uint32_t)units;
            const uint32_t job_tiles = (a.n + j.rows_per_tile - 1u) / j.rows_per_tile;
            tiles += job_tiles;
            units += (uint64_t)job_tiles * j.vcpt;
            vcpt_max = j.vcpt > vcpt_max ? j.vcpt : vcpt_max;
            if (!pair && (int)stage_job == J.ll_job && role == 0) {
                j.has_ll = 1;
                ll_fixups.push_back({jobs.size(), si});
                if (J.ll_mode == 2) j.out[0] = j.out[1] = nullptr;  // the arena slots hold tagged words, not floats
            } else if (!pair && has_peer_out(si, stage_job)) {
                j.has_peers = 1;
                for (uint32_t r = 0; r < peers->world; ++r)
                    j.peer_out[r] = r == peers->rank ? nullptr : S.peer_outputs[(size_t)stage_job * 8 + r];
            }
            jobs.push_back(j);
            return Q4B_OK;
        };
        if (with_pair) {
            pair_fixups.push_back({jobs.size(), pair_k.size()});
            pair_of_stage[si] = (uint32_t)pair_k.size();
            pair_k.push_back(J.res[J.pair_a].n);
            if (int st = push(J.res[J.pair_a], J.res[J.pair_b], S.outputs[J.pair_a], S.outputs[J.pair_b], true, 0)) return st;
        }
        for (int i : list)
            if (int st = push(J.res[i], J.res[i], S.outputs[i], S.outputs[i], false, (uint32_t)i)) return st;
        P.n_jobs = (uint32_t)jobs.size() - P.job_begin;
        uint64_t workers = grid_warps;
        // at most 32 warps share a tile: the warp that combines a split tile reads their partials four at a time
        const uint64_t min_chunks = (vcpt_max + 31u) / 32u;
        P.tiles = tiles;
        const uint32_t tile_groups = (tiles + warps - 1u) / warps;  // blocks that hold every tile once, one tile per warp
        uint32_t best_parts = tile_groups <= (uint32_t)rt->sm_count ? (uint32_t)rt->sm_count / tile_groups : 0u;
        if (best_parts > cpt / (uint32_t)min_chunks) best_parts = cpt / (uint32_t)min_chunks;
        if (best_parts > 32u) best_parts = 32u;
        // (worth it only while it keeps at least 85 % of the warps busy; else the plain equal split of units)
        if (rt->chain_split_tiles && best_parts >= 1u && (uint64_t)tiles * best_parts * 100u >= (uint64_t)grid_warps * 85u) {
            // Fewer tiles than warps: every tile is cut into the same number of equal parts, one per warp, so a warp
            // has exactly one run of chunks (one pipeline ramp, at most one partial-sum exchange) per phase. The equal
            // split of units yields this when all tiles count the same and the warps are a multiple of the tiles. With
            // more than one part the phase is K-major: a block takes one part of sixteen tiles and only rebuilds and
            // holds that slice of the activation.
            uint32_t parts = (uint32_t)rt->sm_count / tile_groups;
            if (parts > cpt / (uint32_t)min_chunks) parts = cpt / (uint32_t)min_chunks;
            if (parts > 32u) parts = 32u;
            if (parts == 0) parts = 1;
            units = 0;
            for (uint32_t i = P.job_begin; i < jobs.size(); ++i) {
                jobs[i].vcpt = cpt;
                jobs[i].unit_begin = (uint32_t)units;
                units += (uint64_t)((jobs[i].n + jobs[i].rows_per_tile - 1u) / jobs[i].rows_per_tile) * cpt;
            }
            workers = (uint64_t)tiles * parts;
            P.kparts = parts;
            // only the stage's own dependent phase rebuilds the buffer, and it may keep a slice only when no deferred
            // phase (whose parts differ) reads the same buffer later
            P.sliced = (parts > 1u && role == 0 && J.deferred.empty()) ? 1u : 0u;
        } else {
            if (workers > units / min_chunks) workers = units / min_chunks;
            if (workers == 0) workers = 1;
        }
        P.units = units;
        P.workers = (uint32_t)workers;
        phases.push_back(P);
        phase_stage.push_back(si);
        phase_role.push_back(role);
        return Q4B_OK;
    };

    std::vector<int> carried;  // deferred jobs of the previous stage that run behind this stage's arrival
    uint32_t carried_stage = 0;
    bool any_global = false;
    uint32_t prev_arrive = q4::kSyncNone;
    for (uint32_t si = 0; si < n_stages; ++si) {
        const q4b_stage &S = stages[si];
        const StageJobs &J = sj[si];
        std::vector<int> main_list;
        for (uint32_t i = 0; i < S.n_jobs; ++i) {
            const bool is_def = std::find(J.deferred.begin(), J.deferred.end(), (int)i) != J.deferred.end();
            if (!is_def && (int)i != J.pair_a && (int)i != J.pair_b) main_list.push_back((int)i);
        }
        if (int st = add_phase(si, 0, main_list, J.pair_a >= 0)) return st;
        q4::StackPhase &M = phases.back();
        // the main phase waits for the stage before it and rebuilds the activation
        M.wait_kind = si > 0 ? prev_arrive : (uint32_t)q4::kSyncNone;
        const bool fused_in = si > 0 && sj[si - 1].pair_a >= 0;
        M.x_kind = fused_in ? q4::kRebuildH : S.x_kind == Q4B_X_BF16 ? q4::kRebuildBf16 : S.x_kind == Q4B_X_SWIGLU ? q4::kRebuildSwiglu : q4::kRebuildRms;
        M.src0 = S.src0;
        M.src1 = S.src1;
        M.src_parts = S.src_parts ? S.src_parts : 1u;
        M.src_part_stride = (uint32_t)S.src_part_stride;
        M.eps = S.eps;
        M.x_bf16_out = (uint16_t *)S.x_bf16_out;
        M.sum_out = (float *)S.sum_out;
        bool global = false;
        for (uint32_t i = 0; i < S.n_jobs; ++i) global = global || (has_peer_out(si, i) && (int)i != J.ll_job);
        // the last stage's arrival publishes the logits; without a token reduction only peers would need it
        const bool last = si + 1 == n_stages;
        M.arrive_kind = global ? q4::kSyncGlobal : (last && !logits) ? q4::kSyncNone : q4::kSyncLocal;
        // the next stages poll the tags of what they read (hidden vector of a fused pair, hand-off of a projection)
        // instead of waiting at a barrier -- unless something of this stage is consumed through plain memory
        if (!last && !global && !J.plain_consumed && (J.ll_job >= 0 || J.pair_a >= 0)) M.arrive_kind = q4::kSyncNone;
        prev_arrive = M.arrive_kind;
        any_global = any_global || global;
        // behind this stage's arrival: the carried half of the previous stage's deferred jobs, then the first part of
        // this stage's own
        if (!carried.empty()) {
            if (int st = add_phase(carried_stage, 2, carried, false)) return st;
            carried.clear();
        }
        if (!J.deferred.empty()) {
            std::vector<int> now = J.deferred, later;
            if (si + 2 < n_stages) {
                // split by rows (all of a stage's jobs share k); the share that stays is rt->chain_defer_split per cent
                uint64_t total = 0, run = 0;
                for (int i : J.deferred) total += J.res[i].n;
                now.clear();
                for (int i : J.deferred) {
                    if (run * 100 < total * rt->chain_defer_split || now.empty()) now.push_back(i);
                    else later.push_back(i);
                    run += J.res[i].n;
                }
            }
            if (int st = add_phase(si, 1, now, false)) return st;
            carried = later;
            carried_stage = si;
        }
    }
    (void)any_global;
    // what each activation buffer has to hold: the whole activation, or the longest slice of a K-major phase (from a
    // multiple of four chunks, plus the chunk that is read ahead)
    halfs[0] = halfs[1] = 0;
    for (const q4::StackPhase &P : phases) {
        uint32_t chunks = P.kp / 128u;
        if (P.kparts > 1u && P.sliced) {
            chunks = 0;
            for (uint32_t part = 0; part < P.kparts; ++part) {
                const uint32_t lo = (P.cpt * part / P.kparts) & ~3u, hi = P.cpt * (part + 1u) / P.kparts;
                chunks = hi - lo > chunks ? hi - lo : chunks;
            }
            chunks += 1u;
        }
        halfs[P.x_buf] = chunks * 128u > halfs[P.x_buf] ? chunks * 128u : halfs[P.x_buf];
    }
    if (q4k_stack_supported(halfs[0], halfs[1])) break;
    if (single_buffer || attempt > 0)
        return fail(Q4B_UNSUPPORTED, "the decode chain kernel cannot be resident with an activation of %u inputs on this device", halfs[0]);
    single_buffer = true;
    }
    const size_t n_pairs = pair_k.size();

    // ---- device memory of the chain ----
    q4b_chain *c = new (std::nothrow) q4b_chain();
    if (!c) return fail(Q4B_CUDA_ERROR, "out of host memory");
    std::unique_ptr<q4b_chain> guard_chain(c);
    uint8_t *reset = nullptr, *hbuf = nullptr;
    const size_t reset_bytes = 256;
    size_t h_total = 0;
    std::vector<size_t> h_off(n_pairs);
    for (size_t i = 0; i < n_pairs; ++i) {
        h_off[i] = h_total;
        h_total += ((size_t)pair_k[i] * 4 + 255) & ~(size_t)255;  // one {two bf16 values, tag} word per two rows
    }
    cudaError_t e = build.alloc((void **)&reset, reset_bytes, true);
    if (e == cudaSuccess) e = build.alloc((void **)&hbuf, h_total + 256, true);
    if (e != cudaSuccess) return fail_cuda(e, "decode chain allocation");
    for (auto &fx : pair_fixups) jobs[fx.first].h_out = (unsigned long long *)(hbuf + h_off[fx.second]);
    // tagged hand-offs: where the producer stores its {value, tag} words and what the consumer's rebuild polls
    {
        size_t ll_total = 0;
        for (auto &fx : ll_fixups)
            if (sj[fx.second].ll_mode == 1) ll_total += ((size_t)jobs[fx.first].n * 8 + 255) & ~(size_t)255;
        uint8_t *llbuf = nullptr;
        if (ll_total) {
            e = build.alloc((void **)&llbuf, ll_total, true);
            if (e != cudaSuccess) return fail_cuda(e, "decode chain allocation");
        }
        size_t ll_used = 0;
        uint32_t arena_handoffs = 0;
        for (auto &fx : ll_fixups) {
            const uint32_t si = fx.second;
            q4::StackJob &j = jobs[fx.first];
            size_t producer = 0, consumer = 0;
            for (size_t pi = 0; pi < phases.size(); ++pi) {
                if (phase_role[pi] != 0) continue;
                if (phase_stage[pi] == si) producer = pi;
                if (phase_stage[pi] == si + 1) consumer = pi;
            }
            q4::StackPhase &C = phases[consumer];
            C.src_tagged = 1;
            C.src_tag_phase = (uint32_t)producer;
            if (sj[si].ll_mode == 1) {
                j.ll_out[0] = (unsigned long long *)(llbuf + ll_used);
                C.src0 = llbuf + ll_used;
                C.src_parts = 1;
                C.src_part_stride = 0;
                ll_used += ((size_t)j.n * 8 + 255) & ~(size_t)255;
            } else {
                // two copies per arena slot, used alternately by successive hand-offs: a rank may be one hand-off ahead
                // of the slowest reader of the previous one, never two
                const size_t copy = (size_t)(arena_handoffs++ & 1u) * j.n * 8;
                const q4b_stage &S = stages[si];
                for (uint32_t r = 0; r < peers->world; ++r) {
                    uint8_t *slot = r == peers->rank ? (uint8_t *)S.outputs[sj[si].ll_job] : (uint8_t *)S.peer_outputs[(size_t)sj[si].ll_job * 8 + r];
                    j.ll_out[r] = slot ? (unsigned long long *)(slot + copy) : nullptr;
                }
                C.src0 = (const uint8_t *)stages[si + 1].src0 + copy;
            }
        }
    }
    for (size_t pi = 0; pi < phases.size(); ++pi) {
        if (phases[pi].x_kind != q4::kRebuildH) continue;
        const uint32_t pr = pair_of_stage[phase_stage[pi] - 1];
        phases[pi].src0 = hbuf + h_off[pr];
        phases[pi].src1 = nullptr;
        phases[pi].src_tagged = 1;
        for (size_t pj = 0; pj < pi; ++pj)
            if (phase_role[pj] == 0 && phase_stage[pj] == phase_stage[pi] - 1) phases[pi].src_tag_phase = (uint32_t)pj;
    }
    void *phases_dev = nullptr, *jobs_dev = nullptr, *partials = nullptr, *counters = nullptr, *aux = nullptr, *peers_dev = nullptr, *trace = nullptr;
    e = build.alloc(&phases_dev, phases.size() * sizeof(q4::StackPhase), false);
    if (e == cudaSuccess) e = cudaMemcpy(phases_dev, phases.data(), phases.size() * sizeof(q4::StackPhase), cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = build.alloc(&jobs_dev, jobs.size() * sizeof(q4::StackJob), false);
    if (e == cudaSuccess) e = cudaMemcpy(jobs_dev, jobs.data(), jobs.size() * sizeof(q4::StackJob), cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = build.alloc(&partials, (size_t)q4::kPartialSets * grid_warps * 32 * sizeof(uint4), true);
    if (e == cudaSuccess) e = build.alloc(&counters, 256, true);
    if (e == cudaSuccess) e = build.alloc(&aux, (size_t)rt->sm_count * 8, true);
    if (e == cudaSuccess && rt->tracing) e = build.alloc(&trace, (size_t)rt->sm_count * phases.size() * q4::kTraceStamps * 8, true);
    if (e == cudaSuccess && peers) {
        q4::StackPeers pimage;
        memset(&pimage, 0, sizeof pimage);
        pimage.world = peers->world;
        pimage.rank = peers->rank;
        pimage.flag_local = (unsigned long long *)peers->flags[peers->rank];
        pimage.consumed = pimage.flag_local + 1;
        pimage.cand_local = (float2 *)peers->cand[peers->rank];
        for (uint32_t r = 0; r < peers->world; ++r) {
            if (!peers->flags[r] || !peers->cand[r]) return fail(Q4B_INVALID_ARGUMENT, "peer table entry %u is null", r);
            pimage.flag_peer[r] = (unsigned long long *)peers->flags[r];
            pimage.cand_peer[r] = (float2 *)peers->cand[r];
        }
        e = build.alloc(&peers_dev, sizeof pimage, false);
        if (e == cudaSuccess) e = cudaMemcpy(peers_dev, &pimage, sizeof pimage, cudaMemcpyHostToDevice);
    }
    if (e != cudaSuccess) return fail_cuda(e, "decode chain allocation");

    q4::StackParams &sp = c->params;
    memset(&sp, 0, sizeof sp);
    sp.phases = (const q4::StackPhase *)phases_dev;
    sp.jobs = (const q4::StackJob *)jobs_dev;
    sp.n_phases = (uint32_t)phases.size();
    sp.halfs[0] = halfs[0];
    sp.halfs[1] = halfs[1];
    for (const q4::StackPhase &P : phases) sp.long_rebuild |= (uint32_t)q4k_stack_phase_is_long(&P);
    sp.local_bar = (unsigned int *)reset;
    sp.error_flag = (int *)rt->error_flag.ptr;
    sp.partials = (uint4 *)partials;
    sp.launch_seq = (unsigned int *)counters;
    sp.max_workers = grid_warps;
    sp.spin_limit = rt->chain_spin_limit;
    sp.flags = rt->chain_flags;
    // Across GPUs the last blocks of a phase rebuild first and request their next weights afterwards (measured: +2 % at
    // 2 and 4 ranks, where the block everyone waits for also waits for the other ranks; -0.7 % on one GPU, so not there)
    if (!rt->chain_flags_set && peers_dev) sp.flags = q4::kFlagLateSkipsRequest | (16u << 8);
    sp.logits = logits;
    sp.vocab = vocab;
    sp.index_base = index_base;
    sp.part_val = (float *)aux;
    sp.part_idx = (uint32_t *)((uint8_t *)aux + (size_t)rt->sm_count * 4);
    sp.token = token_dev;
    sp.best = best_dev;
    sp.peers = (const q4::StackPeers *)peers_dev;
    sp.trace = (unsigned long long *)trace;
    c->rt = rt;
    c->reset_region = reset;
    c->reset_bytes = reset_bytes;
    c->n_phases = sp.n_phases;
    c->n_stages = n_stages;
    c->token = token_dev;
    c->best = best_dev;
    c->multi_rank = peers != nullptr;
    c->failures_seen = rt->failures;
    c->phase_stage = phase_stage;
    c->phase_role = phase_role;
    if (stages[0].x_kind == Q4B_X_BF16) {
        c->first_x = const_cast<void *>(stages[0].src0);
        c->first_x_bytes = stages[0].k * 2;
    }
    c->owned.swap(build.owned);
    *out = guard_chain.release();
    return Q4B_OK;
}

extern "C" int q4b_chain_set_spin_limit(q4b_chain *chain, uint32_t polls) {
    if (!chain || !chain->rt) return fail(Q4B_INVALID_ARGUMENT, "chain handle is null");
    if (polls == 0) return fail(Q4B_INVALID_ARGUMENT, "the poll limit must be positive");
    chain->params.spin_limit = polls;
    return Q4B_OK;
}

extern "C" int q4b_chain_run_device(q4b_chain *chain, void *stream) {
    if (!chain || !chain->rt) return fail(Q4B_INVALID_ARGUMENT, "chain handle is null");
    q4b_runtime *rt = chain->rt;
    std::lock_guard<std::recursive_mutex> lock(rt->mu);
    DeviceGuard guard(rt->device);
    if (chain->failures_seen != rt->failures) {
        // a bounded wait ran out on this runtime since the chain last ran. The counters of a multi-rank chain live
        // on several GPUs and are out of step now; a single-GPU chain only needs the tags of its split-tile slots and its counters cleared (the launch that gave up did not put them back).
        if (chain->multi_rank)
            return fail(Q4B_POOL_POISONED, "a kernel gave up on a bounded wait: destroy this multi-rank chain, zero the arena on every rank and create it again");
        Q4B_CUDA(cudaMemsetAsync(chain->params.partials, 0, (size_t)q4::kPartialSets * chain->params.max_workers * 32 * sizeof(uint4), (cudaStream_t)stream),
                 "decode chain repair");
        Q4B_CUDA(cudaMemsetAsync(chain->reset_region, 0, chain->reset_bytes, (cudaStream_t)stream), "decode chain repair");
        chain->failures_seen = rt->failures;
    }
    Q4B_CUDA(q4k_stack_launch(&chain->params, rt->sm_count, (cudaStream_t)stream), "decode chain launch");
    rt->launches++;
    return Q4B_OK;
}

// Host-buffer twin: the reference's token step takes a host slice and returns a token (src/native.rs:3250-3274,
// 2644-2652). Copies the first stage's bf16 activation in, runs the chain, copies the token (and winning logit) out.
extern "C" int q4b_chain_run(q4b_chain *chain, const void *x_host, uint32_t *token_host, float *best_host) {
    if (!chain || !chain->rt) return fail(Q4B_INVALID_ARGUMENT, "chain handle is null");
    if (!x_host || !token_host) return fail(Q4B_INVALID_ARGUMENT, "activation or token pointer is null");
    if (!chain->first_x || !chain->token) return fail(Q4B_UNSUPPORTED, "the chain's first stage does not take a bf16 vector, or it produces no token");
    q4b_runtime *rt = chain->rt;
    std::lock_guard<std::recursive_mutex> lock(rt->mu);
    DeviceGuard guard(rt->device);
    cudaStream_t s = rt->stream;
    Q4B_CUDA(cudaMemcpyAsync(chain->first_x, x_host, chain->first_x_bytes, cudaMemcpyHostToDevice, s), "activation upload");
    if (int st = q4b_chain_run_device(chain, s)) {
        cudaStreamSynchronize(s);
        return st;
    }
    // token, logit and the error flag come back through one pinned staging block and ONE synchronisation (three
    // downloads into pageable memory would each wait for the stream)
    Q4B_CUDA(rt->results.ensure(64), "result staging");
    uint8_t *h = (uint8_t *)rt->results.ptr;
    Q4B_CUDA(cudaMemcpyAsync(h, chain->token, 4, cudaMemcpyDeviceToHost, s), "token download");
    if (best_host && chain->best) Q4B_CUDA(cudaMemcpyAsync(h + 4, chain->best, 4, cudaMemcpyDeviceToHost, s), "logit download");
    Q4B_CUDA(cudaMemcpyAsync(h + 8, rt->error_flag.ptr, 4, cudaMemcpyDeviceToHost, s), "status download");
    const cudaError_t e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) return fail(Q4B_COMMAND_FAILED, "CUDA command failed: %s", cudaGetErrorString(e));
    int flag = 0;
    memcpy(&flag, h + 8, 4);
    if (flag) {
        cudaMemset(rt->error_flag.ptr, 0, sizeof flag);
        rt->failures++;
        return fail(Q4B_COMMAND_FAILED, "a kernel gave up on a bounded wait (pipeline stalled); results are invalid");
    }
    memcpy(token_host, h, 4);
    if (best_host && chain->best) memcpy(best_host, h + 4, 4);
    return Q4B_OK;
}

extern "C" int q4b_chain_phase_count(q4b_chain *chain, uint32_t *phases) {
    if (!chain || !phases) return fail(Q4B_INVALID_ARGUMENT, "chain handle or output pointer is null");
    *phases = chain->n_phases;
    return Q4B_OK;
}

extern "C" int q4b_chain_trace_read(q4b_chain *chain, uint64_t *stamps, uint64_t capacity_words, uint32_t *blocks, uint32_t *phases,
                                    uint32_t *phase_info, uint32_t phase_info_capacity) {
    if (!chain || !chain->rt || !stamps || !blocks || !phases) return fail(Q4B_INVALID_ARGUMENT, "chain handle or output pointer is null");
    if (!chain->params.trace) return fail(Q4B_UNSUPPORTED, "the chain was created without tracing (q4b_trace_enable before q4b_chain_create)");
    DeviceGuard guard(chain->rt->device);
    const uint64_t words = (uint64_t)chain->rt->sm_count * chain->n_phases * q4::kTraceStamps;
    if (capacity_words < words) return fail(Q4B_WRONG_LENGTH, "trace buffer has %llu elements, expected %llu", (unsigned long long)capacity_words, (unsigned long long)words);
    Q4B_CUDA(cudaDeviceSynchronize(), "device synchronize");
    Q4B_CUDA(cudaMemcpy(stamps, chain->params.trace, words * 8, cudaMemcpyDeviceToHost), "trace download");
    *blocks = (uint32_t)chain->rt->sm_count;
    *phases = chain->n_phases;
    if (phase_info) {
        for (uint32_t i = 0; i < chain->n_phases && i < phase_info_capacity; ++i) phase_info[i] = chain->phase_stage[i] * 4u + chain->phase_role[i];
    }
    return Q4B_OK;
}

extern "C" void q4b_chain_destroy(q4b_chain *chain) {
    if (!chain) return;
    if (chain->rt) {
        DeviceGuard guard(chain->rt->device);
        cudaDeviceSynchronize();
        for (void *p : chain->owned) cudaFree(p);
    }
    delete chain;
}

// ------------------------------------------------------------------------------------------
// synthetic tensors, introspection
// ------------------------------------------------------------------------------------------

extern "C" int q4b_synth_q4_device(q4b_runtime *rt, uint64_t seed, uint64_t tensor, float sigma, uint64_t row0,
                                   uint64_t rows, uint64_t k, const q4b_job *destination) {
    if (int st = check_rt(rt)) return st;
    if (!destination) return fail(Q4B_INVALID_ARGUMENT, "destination job is null");
    std::lock_guard<std::recursive_mutex> lock(rt->mu);
    DeviceGuard guard(rt->device);
    Resolved r;
    q4b_job job = *destination;
    job.output_rows = rows;
    if (int st = resolve_job(rt, job, k, &r)) return st;
    Q4B_CUDA(q4k_synth_q4(seed, tensor, sigma, row0, rows, (uint32_t)k, (uint8_t *)r.w, (uint8_t *)r.s, (uint8_t *)r.b,
                          rt->stream),
             "synthetic weight launch");
    return finish(rt, rt->stream);
}

extern "C" int q4b_synth_bf16_device(q4b_runtime *rt, uint64_t seed, uint64_t tensor, uint64_t count,
                                     uint16_t *out_dev, void *stream) {
    if (int st = check_rt(rt)) return st;
    if (!out_dev) return fail(Q4B_INVALID_ARGUMENT, "output pointer is null");
    DeviceGuard guard(rt->device);
    Q4B_CUDA(q4k_synth_bf16(seed, tensor, count, out_dev, (cudaStream_t)stream), "synthetic activation launch");
    return Q4B_OK;
}

extern "C" int q4b_describe_dispatch(q4b_runtime *rt, int x_dtype, uint64_t m, uint64_t k, const q4b_job *jobs,
                                     uint32_t n_jobs, char *text, uint32_t text_len) {
    if (int st = check_rt(rt)) return st;
    if (int st = check_dtype(x_dtype)) return st;
    if (!text || text_len == 0) return fail(Q4B_INVALID_ARGUMENT, "text buffer is null");
    std::lock_guard<std::recursive_mutex> lock(rt->mu);
    std::vector<Resolved> resolved;
    if (int st = resolve_jobs(rt, jobs, n_jobs, m, k, &resolved)) return st;
    uint32_t fast = 0;
    for (const Resolved &r : resolved) fast += job_is_fast(r, (uint32_t)(k / 64)) ? 1u : 0u;
    if (m == 1 && rt->inline_max_halfs && k % 512 == 0 && k <= rt->inline_max_halfs && k <= q4k_stack_max_k()) {
        snprintf(text, text_len, "single_row_i8 one-phase persistent launch, jobs=%u (byte-addressed %u)", n_jobs, n_jobs - fast);
        return Q4B_OK;
    }
    if (m >= 2 && m <= rt->rows_max_m && fast == n_jobs && k % 512 == 0) {
        uint32_t tiles = 0, part_chunks = 0, tw = 1;
        for (const Resolved &r : resolved) tiles += (r.n + 15u) / 16u;
        const uint32_t mb = (uint32_t)(m < rt->rows_max_m ? m : rt->rows_max_m);
        const uint32_t parts = q4k_rows_plan(mb, (uint32_t)k, tiles, (uint32_t)rt->sm_count, &part_chunks, &tw);
        if (parts) {
            snprintf(text, text_len, "rows_i8 (short batch, integer tensor cores) rows_per_launch=%u k_parts=%u chunks_per_part=%u tiles_per_warp=%u jobs=%u (a 16-byte aligned activation is assumed)",
                     mb, parts, part_chunks, tw, n_jobs);
            return Q4B_OK;
        }
    }
    if (m >= rt->gemm_min_m) {
        snprintf(text, text_len, "tensor_core_gemm (tcgen05) tile_m=%u jobs=%u", q4k_gemm_tile_m((uint32_t)m), n_jobs);
        return Q4B_OK;
    }
    const uint32_t rows = x_dtype == Q4B_F32 ? 2u : 8u;
    const uint32_t mb = (uint32_t)(m < rows ? m : rows);
    const uint32_t v = mb * (x_dtype == Q4B_F32 ? 3u : 1u);
    snprintf(text, text_len, "stream_mma column_tiles=%d fast_jobs=%u byte_addressed_jobs=%u row_blocks=%llu", v <= 4 ? 1 : 2, fast,
             n_jobs - fast, (unsigned long long)((m + rows - 1) / rows));
    return Q4B_OK;
}

extern "C" int q4b_profile_begin(q4b_runtime *rt) {
    if (int st = check_rt(rt)) return st;
    rt->profiling = true;
    rt->prof_used = 0;
    rt->prof_bytes = 0;
    rt->prof_flops = 0;
    return Q4B_OK;
}

extern "C" int q4b_profile_end(q4b_runtime *rt, uint64_t *launches, double *total_ms, uint64_t *bytes, uint64_t *flops) {
    if (int st = check_rt(rt)) return st;
    DeviceGuard guard(rt->device);
    rt->profiling = false;
    double total = 0.0;
    for (size_t i = 0; i + 1 < rt->prof_used; i += 2) {
        Q4B_CUDA(cudaEventSynchronize(rt->prof_events[i + 1]), "cudaEventSynchronize");
        float ms = 0.f;
        Q4B_CUDA(cudaEventElapsedTime(&ms, rt->prof_events[i], rt->prof_events[i + 1]), "cudaEventElapsedTime");
        total += ms;
    }
    if (launches) *launches = rt->prof_used / 2;
    if (total_ms) *total_ms = total;
    if (bytes) *bytes = rt->prof_bytes;
    if (flops) *flops = rt->prof_flops;
    rt->prof_used = 0;
    return Q4B_OK;
}

extern "C" int q4b_trace_enable(q4b_runtime *rt, int on) {
    if (int st = check_rt(rt)) return st;
    DeviceGuard guard(rt->device);
    if (on) {
        Q4B_CUDA(rt->trace.ensure((size_t)rt->max_workers * 4 * 8), "trace buffer");
        Q4B_CUDA(cudaMemset(rt->trace.ptr, 0, rt->trace.capacity), "trace clear");
    }
    rt->tracing = on != 0;
    return Q4B_OK;
}

extern "C" int q4b_trace_read(q4b_runtime *rt, uint64_t *stamps, uint32_t max_workers, uint32_t *workers) {
    if (int st = check_rt(rt)) return st;
    if (!stamps || !workers) return fail(Q4B_INVALID_ARGUMENT, "trace output pointer is null");
    DeviceGuard guard(rt->device);
    Q4B_CUDA(cudaDeviceSynchronize(), "device synchronize");
    uint32_t n = rt->trace_workers < max_workers ? rt->trace_workers : max_workers;
    if (n && rt->trace.ptr) Q4B_CUDA(cudaMemcpy(stamps, rt->trace.ptr, (size_t)n * 32, cudaMemcpyDeviceToHost), "trace download");
    *workers = n;
    return Q4B_OK;
}

extern "C" int q4b_device_status(q4b_runtime *rt) {
    if (int st = check_rt(rt)) return st;
    DeviceGuard guard(rt->device);
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return fail(Q4B_COMMAND_FAILED, "CUDA command failed: %s", cudaGetErrorString(e));
    return finish(rt, rt->stream);
}

extern "C" int q4b_launch_count(q4b_runtime *rt, uint64_t *launches) {
    if (int st = check_rt(rt)) return st;
    if (!launches) return fail(Q4B_INVALID_ARGUMENT, "launch count pointer is null");
    *launches = rt->launches;
    return Q4B_OK;
}
