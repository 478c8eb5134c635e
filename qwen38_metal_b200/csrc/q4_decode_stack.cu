// Persistent decode kernel: a whole token's chain of grouped Q4 projections in ONE cooperative launch.
//
// The reference encodes a token as one command buffer of many dispatches (decode_layers,
// src/metal_runtime.rs:2022-2081; encode_decode_linear_layer :3301-3520). On B200 a launch per projection group
// leaves the memory system idle for longer than a group takes to stream (launch gap, the first-data latency of
// every kernel, the tail of its slowest warp). Here one block per SM stays resident for the whole token:
//   for every stage:  build the activation in shared memory from the previous stage's outputs
//                     (bf16 vector | SwiGLU of two vectors | weightless RMS-norm of a vector),
//                     stream this block's share of the stage's projections (same arithmetic and work split as the
//                     single-launch kernels in q4_gemv.cu),
//                     start the async copies of the next stage's first weights, then cross a grid barrier.
// Weights do not depend on earlier results, so the copies issued before the barrier keep HBM busy while the
// barrier and the activation rebuild run. After the last stage the blocks reduce the logits to a token id.
// Every block computes the activation itself (identical code, identical result); nothing but outputs crosses SMs.
//
// All waits are bounded: a barrier that does not complete within its limit raises the error flag and the block
// leaves the kernel.
#include <cooperative_groups.h>

#include <cstring>

#include "q4_gemv_core.cuh"

namespace q4 {

constexpr int kStackRingBytes = kStages * kStageBytesAligned + 2 * 1024;  // weight ring + two parameter stages of 2 windows
constexpr int kStackMaxIters = 5;                                        // activation blocks of 8 per thread
constexpr uint32_t kBarrierSpinLimit = 1u << 21;

struct StackStage {
    GemvParams gemv;        // jobs, k, kp, groups, cpt, units, workers, partials, counters (xp/xsum/row_inv unused)
    uint32_t x_kind;        // 0: bf16 vector src0; 1: bf16(silu(src0) * src1), fp32 inputs; 2: bf16(src0 / rms(src0)), fp32 input
    float eps;
    const void *src0, *src1;
    uint16_t *x_bf16_out;   // optional: block 0 stores the bf16 activation it built (next token's input, inspection)
};

// Cross-GPU part of a row-sharded chain. Every rank runs the same chain on its row slices; outputs that feed a
// later stage are stored into every rank's buffers, and each grid barrier also waits for the other ranks.
struct StackPeers {
    uint32_t world, rank;
    unsigned long long *arrivals_local;            // barrier arrivals of all blocks of all ranks, in this GPU's memory
    unsigned long long *arrivals_peer[kMaxPeers];  // the same counter on every rank (every block adds to all of them)
    float2 *cand_local;                    // [kMaxPeers] (best logit, token id) candidates, in this GPU's memory
    float2 *cand_peer[kMaxPeers];
};

struct StackParams {
    const StackStage *stages;
    uint32_t n_stages;
    uint32_t x_halfs;       // capacity of the shared activation buffer in fp16 elements (largest kp)
    unsigned int *barrier;  // [0] arrivals of all blocks at all barriers of this launch; zero at launch
    int *error_flag;
    const float *logits;    // output of the last stage to reduce, or null
    uint32_t vocab, index_base;
    float *part_val;        // [gridDim.x]
    uint32_t *part_idx;     // [gridDim.x]
    uint32_t *token;
    float *best;
    const StackPeers *peers;    // null on one GPU
    unsigned int epoch;         // with peers: barrier generations consumed by earlier launches (flags only grow)
    unsigned long long *trace;  // optional [blocks][n_stages][4] device-clock stamps (stage start, activation built, work done, barrier passed)
};

__device__ __forceinline__ unsigned long long stack_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void lds_v4_keep(uint4 &v, uint32_t addr, bool pred) {
    asm volatile("{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %5, 0;\n\t@q ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n\t}"
                 : "+r"(v.x), "+r"(v.y), "+r"(v.z), "+r"(v.w)
                 : "r"(addr), "r"((uint32_t)pred)
                 : "memory");
}
__device__ __forceinline__ void lds_f32_keep(float &v, uint32_t addr, bool pred) {
    asm volatile("{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %2, 0;\n\t@q ld.shared.f32 %0, [%1];\n\t}" : "+f"(v) : "r"(addr), "r"((uint32_t)pred) : "memory");
}

// Grid-wide barrier with a bounded wait; with peers it is also a barrier across the GPUs of the chain.
// Generations only grow (`generation` starts at the launch's epoch), so nothing has to be reset between launches.
// Returns false when it gave up (error flag raised).
//
// Across GPUs every block announces itself directly in every rank's memory: after a system-scope fence behind its peer
// stores it adds one to an arrival counter on each rank (remote reductions over NVLink, sent back to back) and then
// polls the counter in its own GPU's memory until all blocks of all ranks have arrived `generation` times. There is no
// gather-then-forward step: the critical path is one fence, one NVLink hop and a local poll. All ranks run the same
// number of blocks. A rank that runs ahead into its next barrier only adds arrivals that the others wait for anyway.
__device__ __forceinline__ bool grid_barrier(unsigned int *bar, uint32_t &generation, int *error_flag, const StackPeers *peers) {
    __syncthreads();
    int ok = 1;
    ++generation;
    if (threadIdx.x == 0) {
        if (peers) {
            __threadfence_system();  // this block's stores (peer stores included) are visible before its arrival counts
            for (uint32_t r = 0; r < peers->world; ++r)
                asm volatile("red.relaxed.sys.global.add.u64 [%0], %1;" ::"l"(peers->arrivals_peer[r]), "l"(1ull) : "memory");
            const unsigned long long target = (unsigned long long)generation * gridDim.x * peers->world;
            uint32_t spins = 0;
            while (true) {
                unsigned long long seen;
                asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(seen) : "l"(peers->arrivals_local) : "memory");
                if (seen >= target) break;
                if (++spins > kBarrierSpinLimit || *reinterpret_cast<volatile int *>(error_flag)) {
                    *error_flag = 1;
                    ok = 0;
                    break;
                }
                __nanosleep(20);
            }
        } else {
            // one GPU: every block adds to one counter (zero at launch) and polls it until all blocks have arrived
            // `generation` times -- no last-arriver hop
            __threadfence();
            atomicAdd(&bar[0], 1u);
            const unsigned int target = generation * gridDim.x;
            uint32_t spins = 0;
            while (true) {
                unsigned int seen;
                asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(bar) : "memory");
                if (seen >= target) break;
                if (++spins > kBarrierSpinLimit || *reinterpret_cast<volatile int *>(error_flag)) {
                    *error_flag = 1;
                    ok = 0;
                    break;
                }
                __nanosleep(20);
            }
        }
        // the acquire loads above order this block's later reads behind the arrivals they observed
        __threadfence();
    }
    return __syncthreads_and(ok) != 0;
}

// deterministic block-wide sum / max through shared memory (same order on every block)
template <int WARPS>
__device__ __forceinline__ float block_sum(float v, float *red) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    __syncthreads();
    if ((threadIdx.x & 31u) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for (int i = 0; i < WARPS; ++i) total += red[i];
    return total;
}
template <int WARPS>
__device__ __forceinline__ uint32_t block_max_u32(uint32_t v, uint32_t *red) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v = max(v, __shfl_xor_sync(0xffffffffu, v, off));
    __syncthreads();
    if ((threadIdx.x & 31u) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    uint32_t total = 0;
#pragma unroll
    for (int i = 0; i < WARPS; ++i) total = max(total, red[i]);
    return total;
}

// Build the stage's activation in shared memory: fp16 after an exact power-of-two scaling, fragment order,
// per-group sums, and the inverse scale. Ends with a block barrier.
template <int WARPS>
__device__ __forceinline__ void build_activation(const StackStage &S, uint8_t *xp_smem, float *xsum_smem, float *inv_smem,
                                                 float *red) {
    constexpr uint32_t T = WARPS * 32;
    const uint32_t k = S.gemv.k, kp = S.gemv.kp;
    const uint32_t blocks = k / 8, blocks_p = kp / 8;
    float v[kStackMaxIters][8];
    float ss = 0.f;
#pragma unroll
    for (int it = 0; it < kStackMaxIters; ++it) {
        const uint32_t b = threadIdx.x + it * T;
#pragma unroll
        for (int i = 0; i < 8; ++i) v[it][i] = 0.f;
        if (b < blocks) {
            if (S.x_kind == 0) {
                const uint4 raw = __ldcg(reinterpret_cast<const uint4 *>(static_cast<const uint16_t *>(S.src0) + b * 8));
                const uint32_t r[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    v[it][2 * i] = bf16_bits_to_float(r[i] & 0xffffu);
                    v[it][2 * i + 1] = bf16_bits_to_float(r[i] >> 16);
                }
            } else {
                const float4 *p0 = reinterpret_cast<const float4 *>(static_cast<const float *>(S.src0) + b * 8);
                const float4 a0 = __ldcg(p0), a1 = __ldcg(p0 + 1);
                const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
                if (S.x_kind == 1) {
                    const float4 *p1 = reinterpret_cast<const float4 *>(static_cast<const float *>(S.src1) + b * 8);
                    const float4 u0 = __ldcg(p1), u1 = __ldcg(p1 + 1);
                    const float u[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        // qwen38_swiglu_rows with the hardware exponential and reciprocal (as Metal's fast math does): every
                        // block evaluates all of it, so the full-precision forms were most of this stage's rebuild time;
                        // the result is rounded to bf16 right away
                        const float h = __fdividef(a[i], 1.0f + __expf(-a[i])) * u[i];
                        v[it][i] = bf16_bits_to_float(float_to_bf16_bits(h));
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        v[it][i] = a[i];
                        ss += a[i] * a[i];
                    }
                }
            }
        }
    }
    if (S.x_kind == 2) {
        const float inv = rsqrtf(block_sum<WARPS>(ss, red) / (float)k + S.eps);
#pragma unroll
        for (int it = 0; it < kStackMaxIters; ++it)
#pragma unroll
            for (int i = 0; i < 8; ++i) v[it][i] = bf16_bits_to_float(float_to_bf16_bits(v[it][i] * inv));
    }
    uint32_t amax = 0;
#pragma unroll
    for (int it = 0; it < kStackMaxIters; ++it)
#pragma unroll
        for (int i = 0; i < 8; ++i) amax = max(amax, __float_as_uint(v[it][i]) & 0x7fffffffu);
    amax = block_max_u32<WARPS>(amax, reinterpret_cast<uint32_t *>(red));
    int e = 14 - ((int)((amax >> 23) & 0xffu) - 127);
    e = amax == 0 ? 0 : max(-100, min(100, e));
    const float scale = __uint_as_float((uint32_t)(e + 127) << 23);
    if (threadIdx.x == 0) *inv_smem = __uint_as_float((uint32_t)(127 - e) << 23);
#pragma unroll
    for (int it = 0; it < kStackMaxIters; ++it) {
        const uint32_t b = threadIdx.x + it * T;
        uint32_t bits[8];
        float sum = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const __half h = __float2half_rn(v[it][i] * scale);
            bits[i] = (uint32_t)__half_as_ushort(h);
            sum += __half2float(h);
        }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        sum += __shfl_xor_sync(0xffffffffu, sum, 4);
        if (b < blocks_p) {
            uint4 out;
            out.x = bits[0] | (bits[4] << 16);
            out.y = bits[1] | (bits[5] << 16);
            out.z = bits[2] | (bits[6] << 16);
            out.w = bits[3] | (bits[7] << 16);
            *reinterpret_cast<uint4 *>(xp_smem + b * 16) = out;
            if ((threadIdx.x & 7u) == 0) xsum_smem[b / 8] = sum;
            if (blockIdx.x == 0 && S.x_bf16_out && b < blocks) {
                uint4 plain;
                uint32_t bb[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) bb[i] = float_to_bf16_bits(v[it][i]);
                plain.x = bb[0] | (bb[1] << 16);
                plain.y = bb[2] | (bb[3] << 16);
                plain.z = bb[4] | (bb[5] << 16);
                plain.w = bb[6] | (bb[7] << 16);
                *reinterpret_cast<uint4 *>(S.x_bf16_out + b * 8) = plain;
            }
        }
    }
    __syncthreads();
}

// One contiguous run of chunks of one tile, as seen by one lane.
struct Segment {
    uint32_t tile, c0, c1, cbase, job_index;
    uint32_t c0v, c1v;               // the run in the job's virtual chunk numbering (c0, c1 are clamped to real chunks)
    uint32_t mis_w, mis_s, mis_b;   // byte misalignment (address & 15) of the job's three tensors
    uint32_t pmis;                   // misalignment of the parameter array this lane copies
    const uint8_t *wa, *wb, *pp;     // cursors at chunk cbase (weights: this lane's aligned window)
};

__device__ __forceinline__ void segment_setup(const GemvParams &P, uint64_t u, uint64_t u1, uint32_t &job_index, uint32_t lane,
                                              Segment &sg) {
    const uint32_t g = lane >> 2, t = lane & 3u, cpt = P.cpt;
    while (job_index + 1 < P.n_jobs && u >= P.jobs[job_index + 1].unit_begin) ++job_index;
    sg.job_index = job_index;
    const GemvJob &job = P.jobs[job_index];
    const uint32_t rel = (uint32_t)(u - job.unit_begin), vcpt = job.vcpt;
    const uint32_t tile_local = rel / vcpt;
    sg.tile = job.tile_begin + tile_local;
    sg.c0v = rel - tile_local * vcpt;
    const uint64_t left = u1 - u;
    sg.c1v = (left < (uint64_t)(vcpt - sg.c0v)) ? sg.c0v + (uint32_t)left : vcpt;
    sg.c0 = sg.c0v < cpt ? sg.c0v : cpt;
    sg.c1 = sg.c1v < cpt ? sg.c1v : cpt;
    sg.cbase = sg.c0 & ~3u;
    sg.mis_w = job.w_misalign;
    sg.mis_s = (uint32_t)((uintptr_t)job.s & 15u);
    sg.mis_b = (uint32_t)((uintptr_t)job.b & 15u);
    const uint32_t row0 = (sg.tile - job.tile_begin) * 16u, prow = lane & 15u;
    uint32_t row_a = row0 + g, row_b = row0 + g + 8u, row_p = row0 + prow;
    row_a = row_a < job.n ? row_a : job.n - 1u;  // rows past N read a valid row and are never stored
    row_b = row_b < job.n ? row_b : job.n - 1u;
    row_p = row_p < job.n ? row_p : job.n - 1u;
    const uint64_t row_bytes = (uint64_t)P.k >> 1;
    sg.wa = job.w + (uint64_t)row_a * row_bytes + t * 16u + sg.cbase * 64u - sg.mis_w;
    sg.wb = job.w + (uint64_t)row_b * row_bytes + t * 16u + sg.cbase * 64u - sg.mis_w;
    const bool is_bias = (lane >> 4) != 0;
    sg.pmis = is_bias ? sg.mis_b : sg.mis_s;
    sg.pp = (is_bias ? job.b : job.s) + ((uint64_t)row_p * P.groups) * 2u + sg.cbase * 4u - sg.pmis;
}

// Async copies of the first two groups of four chunks. With misaligned weights the chunk after the segment is
// copied as well: the last lane of a quad completes its 16 bytes from the next chunk's first window.
__device__ __forceinline__ void segment_prologue(const Segment &sg, uint32_t ring, uint32_t pring, uint32_t lane) {
    const uint32_t wend = sg.c1 + ((sg.mis_w && sg.c1 > sg.c0) ? 1u : 0u);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
#pragma unroll
        for (int s = 0; s < 4; ++s) {
            const uint32_t c = sg.cbase + 4 * h + s;
            const uint32_t stage = ring + (4 * h + s) * kStageBytesAligned + lane * 16u;
            const bool in = c >= sg.c0 && c < wend;
            cp_async_16_pred(stage, sg.wa + (4 * h + s) * 64, in);
            cp_async_16_pred(stage + 512u, sg.wb + (4 * h + s) * 64, in);
        }
        const bool pin = sg.cbase + 4 * h < sg.c1;
        cp_async_16_pred(pring + h * 1024u + lane * 16u, sg.pp + h * 16, pin);
        cp_async_16_pred(pring + h * 1024u + 512u + lane * 16u, sg.pp + h * 16 + 16, pin && sg.pmis != 0);
        cp_async_commit();
    }
}

template <int WARPS>
__global__ void __launch_bounds__(WARPS * 32, 1) q4_stack_kernel(const __grid_constant__ StackParams sp) {
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const uint32_t g = lane >> 2, t = lane & 3u;
    const uint32_t worker = blockIdx.x * WARPS + warp;
    uint8_t *xp_smem = smem + WARPS * kStackRingBytes;
    float *xsum_smem = reinterpret_cast<float *>(xp_smem + sp.x_halfs * 2);
    float *inv_smem = xsum_smem + sp.x_halfs / 64;
    float *red = inv_smem + 4;
    const uint32_t ring = (uint32_t)__cvta_generic_to_shared(smem) + warp * kStackRingBytes;
    const uint32_t pring = ring + kStages * kStageBytesAligned;
    const uint32_t xp_addr = (uint32_t)__cvta_generic_to_shared(xp_smem) + t * 64u;
    const uint32_t xsum_addr = (uint32_t)__cvta_generic_to_shared(xsum_smem) + (t >> 1) * 4u;
    // one activation row: MMA column 0 carries group A (lanes g==0, t<2), column 4 group B (lanes g==4, t>=2)
    const bool has_x = (g == 0 && t < 2u) || (g == 4 && t >= 2u);
    const bool has_sum = (t & 1u) == 0;  // lanes whose MMA result columns include column 0 / 4
    const uint32_t half_sel = (t >> 1) ? 0x3244u : 0x1044u;
    const Magic mg = make_magic();
    uint4 xf[2][1][4];
#pragma unroll
    for (int b = 0; b < 2; ++b)
#pragma unroll
        for (int w = 0; w < 4; ++w) xf[b][0][w] = make_uint4(0, 0, 0, 0);

    uint32_t generation = sp.peers ? sp.epoch : 0;
    bool prefetched = false;
    Segment sg;
    uint32_t job_index = 0;

    for (uint32_t st = 0; st < sp.n_stages; ++st) {
        const StackStage &S = sp.stages[st];
        const GemvParams &P = S.gemv;
        unsigned long long *tr = sp.trace ? sp.trace + ((size_t)blockIdx.x * sp.n_stages + st) * 4 : nullptr;
        if (tr && threadIdx.x == 0) tr[0] = stack_ns();
        build_activation<WARPS>(S, xp_smem, xsum_smem, inv_smem, red);
        if (tr && threadIdx.x == 0) tr[1] = stack_ns();

        if (worker < P.workers) {
            const Q4Split split{P.units, P.cpt, P.workers};
            uint64_t u = q4_split_begin(split, worker);
            const uint64_t u1 = q4_split_begin(split, worker + 1);
            bool first = true;
            if (!prefetched) job_index = 0;
            while (u < u1) {
                if (!(first && prefetched)) {
                    segment_setup(P, u, u1, job_index, lane, sg);
                    segment_prologue(sg, ring, pring, lane);
                }
                first = false;
                const uint32_t c0 = sg.c0, c1 = sg.c1;
                const uint32_t mis_w = sg.mis_w, mis_s = sg.mis_s, mis_b = sg.mis_b;
                const uint32_t wend = c1 + ((mis_w && c1 > c0) ? 1u : 0u);
                const uint8_t *wa = sg.wa, *wb = sg.wb, *pp = sg.pp;
                uint32_t xa = xp_addr + sg.cbase * 256u;           // this lane's fragment of chunk cbase
                uint32_t xs = xsum_addr + sg.cbase * 8u;           // group sum of this lane's group in chunk cbase
                float acc[1][4] = {{0.f, 0.f, 0.f, 0.f}};
                if (c0 & 1u) {
#pragma unroll
                    for (int w = 0; w < 4; ++w) lds_v4_keep(xf[1][0][w], xa + (c0 - sg.cbase) * 256u + w * 16u, has_x);
                } else {
#pragma unroll
                    for (int w = 0; w < 4; ++w) lds_v4_keep(xf[0][0][w], xa + (c0 - sg.cbase) * 256u + w * 16u, has_x);
                }

                uint32_t half = 0;
                for (uint32_t cg = sg.cbase; cg < c1; cg += 4) {
                    const uint32_t stage0 = ring + half * (4 * kStageBytesAligned) + lane * 16u;
                    const uint32_t other0 = ring + (half ^ 1u) * (4 * kStageBytesAligned) + lane * 16u;
                    const uint32_t pstage = pring + half * 1024u;
                    cp_async_wait<1>();  // this half's group has landed; the other half's may be pending
                    __syncwarp();        // parameters (and neighbouring weight windows) were copied by other lanes
                    uint4 psa = lds_v4(pstage + g * 16u), psb = lds_v4(pstage + (g + 8u) * 16u);
                    uint4 pba = lds_v4(pstage + 256u + g * 16u), pbb = lds_v4(pstage + 256u + (g + 8u) * 16u);
                    if (mis_s) {
                        psa = realign_16(psa, lds_v4(pstage + 512u + g * 16u), mis_s);
                        psb = realign_16(psb, lds_v4(pstage + 512u + (g + 8u) * 16u), mis_s);
                    }
                    if (mis_b) {
                        pba = realign_16(pba, lds_v4(pstage + 768u + g * 16u), mis_b);
                        pbb = realign_16(pbb, lds_v4(pstage + 768u + (g + 8u) * 16u), mis_b);
                    }
                    const uint32_t wsa[4] = {psa.x, psa.y, psa.z, psa.w}, wsb[4] = {psb.x, psb.y, psb.z, psb.w};
                    const uint32_t wba[4] = {pba.x, pba.y, pba.z, pba.w}, wbb[4] = {pbb.x, pbb.y, pbb.z, pbb.w};
#pragma unroll
                    for (int s = 0; s < 4; ++s) {
                        const uint32_t c = cg + s;
                        if (c >= c0 && c < c1) {
                            const int b = s & 1;
                            const uint32_t stage = stage0 + s * kStageBytesAligned;
                            uint4 cwa = lds_v4(stage), cwb = lds_v4(stage + 512u);
                            if (mis_w) {
                                // the 16 bytes end in the next window: the next lane's slot, or for the quad's last
                                // lane the first window of the next chunk (next stage; after the fourth chunk of a
                                // half that is the other half, which must have landed)
                                uint32_t next = stage + 16u;
                                if (s == 3) {
                                    cp_async_wait<0>();
                                    __syncwarp();
                                    if (t == 3u) next = other0 - 48u;
                                } else if (t == 3u) {
                                    next = stage + kStageBytesAligned - 48u;
                                }
                                cwa = realign_16(cwa, lds_v4(next), mis_w);
                                cwb = realign_16(cwb, lds_v4(next + 512u), mis_w);
                            }
#pragma unroll
                            for (int w = 0; w < 4; ++w) lds_v4_keep(xf[b ^ 1][0][w], xa + (s + 1) * 256u + w * 16u, has_x);
                            float xsv = 0.f;
                            lds_f32_keep(xsv, xs + s * 8u, has_sum);
                            float d[1][4];
                            chunk_mma<1>(cwa, cwb, xf[b], mg, d);
                            const float sa = param_of(wsa[s], half_sel), sb = param_of(wsb[s], half_sel);
                            const float ba = param_of(wba[s], half_sel), bb = param_of(wbb[s], half_sel);
                            acc[0][0] = fmaf(d[0][0], sa, fmaf(xsv, ba, acc[0][0]));
                            acc[0][2] = fmaf(d[0][2], sb, fmaf(xsv, bb, acc[0][2]));
                        }
                    }
                    __syncwarp();  // every lane is done with this half before it is refilled
#pragma unroll
                    for (int s = 0; s < 4; ++s) {
                        const bool more = cg + 8 + s < wend;
                        cp_async_16_pred(stage0 + s * kStageBytesAligned, wa + (8 + s) * 64, more);
                        cp_async_16_pred(stage0 + s * kStageBytesAligned + 512u, wb + (8 + s) * 64, more);
                    }
                    cp_async_16_pred(pstage + lane * 16u, pp + 32, cg + 8 < c1);
                    cp_async_16_pred(pstage + 512u + lane * 16u, pp + 48, cg + 8 < c1 && sg.pmis != 0);
                    cp_async_commit();
                    wa += 4 * 64;
                    wb += 4 * 64;
                    pp += 16;
                    xa += 4 * 256u;
                    xs += 4 * 8u;
                    half ^= 1u;
                }
                cp_async_wait<0>();
                __syncwarp();
                {
                    const GemvJob &job = P.jobs[sg.job_index];
                    finish_tile<1>(P, inv_smem, split, worker, sg.tile, sg.c0v == 0 && sg.c1v == job.vcpt, acc, lane, g, t, sg.job_index,
                                   (uint64_t)job.unit_begin + (uint64_t)(sg.tile - job.tile_begin) * job.vcpt, job.vcpt);
                }
                u += sg.c1v - sg.c0v;
            }
        }

        // weights of the next stage's first segment start streaming before the barrier
        prefetched = false;
        if (st + 1 < sp.n_stages) {
            const GemvParams &N = sp.stages[st + 1].gemv;
            if (worker < N.workers) {
                const Q4Split nsplit{N.units, N.cpt, N.workers};
                const uint64_t nu = q4_split_begin(nsplit, worker), nu1 = q4_split_begin(nsplit, worker + 1);
                if (nu < nu1) {
                    job_index = 0;
                    segment_setup(N, nu, nu1, job_index, lane, sg);
                    segment_prologue(sg, ring, pring, lane);
                    prefetched = true;
                }
            }
        }
        if (tr) {
            __syncthreads();
            if (threadIdx.x == 0) tr[2] = stack_ns();
        }
        if (!grid_barrier(sp.barrier, generation, sp.error_flag, sp.peers)) return;
        if (tr && threadIdx.x == 0) tr[3] = stack_ns();
    }

    // ---- logits -> token: per-block candidates, barrier, block 0 picks (ties to the lowest index) ----
    if (sp.logits) {
        const uint32_t per = (sp.vocab + gridDim.x - 1) / gridDim.x;
        const uint32_t lo = blockIdx.x * per, hi = min(sp.vocab, lo + per);
        float bv = -INFINITY;
        uint32_t bi = 0xffffffffu;
        for (uint32_t i = lo + threadIdx.x; i < hi; i += WARPS * 32) {
            const float v = __ldcg(sp.logits + i);
            if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
        }
        float *rv = red;
        uint32_t *ri = reinterpret_cast<uint32_t *>(red) + 32;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
            const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, off);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        __syncthreads();
        if (lane == 0) { rv[warp] = bv; ri[warp] = bi; }
        __syncthreads();
        if (threadIdx.x == 0) {
            for (int i = 1; i < WARPS; ++i)
                if (rv[i] > bv || (rv[i] == bv && ri[i] < bi)) { bv = rv[i]; bi = ri[i]; }
            sp.part_val[blockIdx.x] = bv;
            sp.part_idx[blockIdx.x] = bi;
        }
        if (!grid_barrier(sp.barrier, generation, sp.error_flag, sp.peers)) return;
        if (blockIdx.x == 0 && threadIdx.x == 0) {
            float fv = -INFINITY;
            uint32_t fi = 0xffffffffu;
            for (uint32_t i = 0; i < gridDim.x; ++i) {
                const float v = __ldcg(sp.part_val + i);
                const uint32_t ix = __ldcg(sp.part_idx + i);
                if (v > fv || (v == fv && ix < fi)) { fv = v; fi = ix; }
            }
            const uint32_t mine = (fi == 0xffffffffu ? 0u : fi) + sp.index_base;
            if (!sp.peers) {
                *sp.token = mine;
                if (sp.best) *sp.best = fv;
            } else {
                // candidates of every vocabulary slice go to every rank; the barrier below publishes them
                const float2 c = make_float2(fv, __uint_as_float(mine));
                for (uint32_t r = 0; r < sp.peers->world; ++r) sp.peers->cand_peer[r][sp.peers->rank] = c;
            }
        }
        if (sp.peers) {
            if (!grid_barrier(sp.barrier, generation, sp.error_flag, sp.peers)) return;
            if (blockIdx.x == 0 && threadIdx.x == 0) {
                float fv = -INFINITY;
                uint32_t fi = 0xffffffffu;
                for (uint32_t r = 0; r < sp.peers->world; ++r) {
                    const float2 c = __ldcg(sp.peers->cand_local + r);
                    const uint32_t ix = __float_as_uint(c.y);
                    if (c.x > fv || (c.x == fv && ix < fi)) { fv = c.x; fi = ix; }
                }
                *sp.token = fi;
                if (sp.best) *sp.best = fv;
            }
        }
    }
}

}  // namespace q4

// ---------------------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------------------

namespace {
constexpr int kStackWarps = 16;

size_t stack_smem_bytes(uint32_t x_halfs) {
    return (size_t)kStackWarps * q4::kStackRingBytes + (size_t)x_halfs * 2 + (size_t)(x_halfs / 64) * 4 + 16 + 64 * 4 + 128;
}
}  // namespace

extern "C" size_t q4k_stack_peers_bytes(void) { return sizeof(q4::StackPeers); }
extern "C" void q4k_stack_fill_peers(void *image, uint32_t world, uint32_t rank, void *const *flags, void *const *cand) {
    q4::StackPeers *p = static_cast<q4::StackPeers *>(image);
    memset(p, 0, sizeof *p);
    p->world = world;
    p->rank = rank;
    p->arrivals_local = static_cast<unsigned long long *>(flags[rank]);
    p->cand_local = static_cast<float2 *>(cand[rank]);
    for (uint32_t r = 0; r < world; ++r) {
        p->arrivals_peer[r] = static_cast<unsigned long long *>(flags[r]);
        p->cand_peer[r] = static_cast<float2 *>(cand[r]);
    }
}
extern "C" size_t q4k_stack_stage_bytes(void) { return sizeof(q4::StackStage); }
extern "C" uint32_t q4k_stack_warps(void) { return kStackWarps; }
extern "C" uint32_t q4k_stack_max_k(void) { return q4::kStackMaxIters * kStackWarps * 32 * 8; }

// Fills one stage image (host memory) for upload; `gemv` carries jobs and shape, workers/partials/counters included.
extern "C" void q4k_stack_fill_stage(void *stage_image, const q4::GemvParams *gemv, uint32_t x_kind, float eps, const void *src0,
                                     const void *src1, uint16_t *x_bf16_out) {
    q4::StackStage *s = static_cast<q4::StackStage *>(stage_image);
    s->gemv = *gemv;
    s->x_kind = x_kind;
    s->eps = eps;
    s->src0 = src0;
    s->src1 = src1;
    s->x_bf16_out = x_bf16_out;
}

// 0 when the kernel cannot be made resident with one block per SM for this activation size
extern "C" int q4k_stack_supported(uint32_t x_halfs, int sm_count) {
    const size_t smem = stack_smem_bytes(x_halfs);
    if (cudaFuncSetAttribute(q4::q4_stack_kernel<kStackWarps>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    int blocks = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, q4::q4_stack_kernel<kStackWarps>, kStackWarps * 32, smem) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    (void)sm_count;
    return blocks >= 1 ? 1 : 0;
}

extern "C" cudaError_t q4k_stack_launch(const void *stages_dev, uint32_t n_stages, uint32_t x_halfs, unsigned int *barrier,
                                        int *error_flag, const float *logits, uint32_t vocab, uint32_t index_base, float *part_val,
                                        uint32_t *part_idx, uint32_t *token, float *best, unsigned long long *trace, const void *peers,
                                        unsigned int epoch, int sm_count, cudaStream_t stream) {
    q4::StackParams sp;
    sp.stages = static_cast<const q4::StackStage *>(stages_dev);
    sp.n_stages = n_stages;
    sp.x_halfs = x_halfs;
    sp.barrier = barrier;
    sp.error_flag = error_flag;
    sp.logits = logits;
    sp.vocab = vocab;
    sp.index_base = index_base;
    sp.part_val = part_val;
    sp.part_idx = part_idx;
    sp.token = token;
    sp.best = best;
    sp.trace = trace;
    sp.peers = static_cast<const q4::StackPeers *>(peers);
    sp.epoch = epoch;
    cudaError_t e = cudaSuccess;
    if (!peers) {  // with peers generations only grow; on one GPU the two words restart at zero
        e = cudaMemsetAsync(barrier, 0, 8, stream);
        if (e != cudaSuccess) return e;
    }
    void *args[] = {&sp};
    return cudaLaunchCooperativeKernel(reinterpret_cast<void *>(q4::q4_stack_kernel<kStackWarps>), dim3(sm_count), dim3(kStackWarps * 32),
                                       args, stack_smem_bytes(x_halfs), stream);
}
