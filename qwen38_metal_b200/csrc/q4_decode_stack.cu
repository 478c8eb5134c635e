// Persistent decode kernel: a whole token's chain of grouped Q4 projections in ONE cooperative launch.
//
// The reference encodes a token as one command buffer of many dispatches (decode_layers,
// src/metal_runtime.rs:2022-2081; encode_decode_linear_layer :3301-3520). On B200 a launch per projection group
// leaves the memory system idle for longer than a group takes to stream (launch gap, the first-data latency of
// every kernel, the tail of its slowest warp). Here one block per SM stays resident for the whole token and walks a
// list of phases (q4_stack.h):
//   [wait for the previous barrier, rebuild the activation in shared memory]
//   stream this warp's share of the phase's projections (the arithmetic of the single-launch kernels, q4_gemv.cu)
//   [arrive at the next barrier]
// Arrival and wait are separate steps. Projections that feed nothing downstream (Q/K/V, the DeltaNet inputs) are
// placed between them, reading the previous activation from a second shared-memory buffer, so the weight stream
// continues while the barrier completes. The first weights of every phase are requested before the wait that
// precedes it: weights do not depend on earlier results.
//
// Fusions: a gate/up pair is streamed as tiles of 8 gate rows + the same 8 up rows, so a lane ends up with both sums
// of a row and stores bf16(silu(gate)*up) (qwen38_swiglu_rows, shaders/qwen38.metal:4188-4198) plus a running
// maximum; the next phase then only converts 2 bytes per input instead of evaluating the whole vector in every block.
// Across GPUs the down projection is cut along K (each rank consumes the slice of the hidden vector it produced) and
// the partial outputs are pushed to every rank with peer stores; the rebuild of the next activation adds them in rank
// order. One cross-GPU barrier per layer: blocks arrive on a counter in their own GPU's memory, the last of them
// forwards one arrival per rank over NVLink, waiters poll their own memory.
//
// All waits are bounded: a barrier that does not complete within the chain's poll limit raises the error flag and the
// block leaves the kernel.
#include <cooperative_groups.h>

#include <cstring>

#include "q4_gemv_core.cuh"
#include "q4_stack.h"

namespace q4 {

constexpr int kStackRingBytes = kStages * kStageBytesAligned + 2 * 1024;  // weight ring + two parameter stages of 2 windows
constexpr int kStackMaxIters = 5;                                        // activation blocks of 8 per thread (register-held rebuilds)
constexpr int kXChunkBytes = 384;                                        // activation of one chunk: three digit planes of 128 bytes
constexpr int kXSlack = kXChunkBytes;                                    // the fragment of the chunk after the last one is read ahead

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
__device__ __forceinline__ void prefetch_l2(const void *p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }
__device__ __forceinline__ void prefetch_l1(const void *p) { asm volatile("prefetch.global.L1 [%0];" ::"l"(p)); }

// ---------------------------------------------------------------------------------------------------------
// Barriers. Every block arrives exactly once per barrier and every block makes the same sequence of arrivals, so
// the targets are plain multiples: after its n-th arrival a block waits for n * gridDim.x arrivals on the counter in
// its own GPU's memory (zero at launch), or for n * world arrivals of whole ranks on the cross-GPU word (which only
// grows; `gbase` is what earlier launches left there).
// ---------------------------------------------------------------------------------------------------------
struct SyncState {
    uint32_t local_gen;   // arrivals this block has made on the local counter
    uint32_t global_gen;  // of those, arrivals at cross-GPU barriers
    const unsigned long long *gbase;  // shared memory: what earlier launches left on the cross-GPU word
};

// Called by every warp once it has finished the phase's units. The warp's results are ordered before the arrival by
// a fence (system scope when it stored into other GPUs' memory); the last warp of the block arrives for the block,
// and the block that completes the local count of a cross-GPU barrier forwards one arrival to every rank.
template <int WARPS>
__device__ __forceinline__ void phase_arrive(const StackParams &sp, uint32_t kind, const SyncState &ss, uint32_t *arrive_smem,
                                             bool stored_to_peers, uint32_t lane, unsigned long long *tr) {
    if (stored_to_peers) __threadfence_system();
    else if (sp.flags & kFlagWarpFenceGpu) __threadfence();
    else __threadfence_block();  // the block's last warp fences at device scope for everyone it has seen arrive
    __syncwarp();
    if (lane != 0) return;
    const uint32_t before = atomicAdd(arrive_smem, 1u);
    if (before != WARPS - 1) return;
    *reinterpret_cast<volatile uint32_t *>(arrive_smem) = 0;  // the next arrival follows a block barrier
    __threadfence();
    const unsigned int target = (ss.local_gen + 1u) * gridDim.x;
    const unsigned int seen = atomicAdd(sp.local_bar, 1u);
    if (tr) tr[4] = stack_ns();
    if (kind == kSyncGlobal && seen + 1u == target) {
        // every block of this GPU has arrived (each behind its own fence): tell all ranks, this one included
        __threadfence_system();
        const StackPeers *peers = sp.peers;
        for (uint32_t r = 0; r < peers->world; ++r)
            asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(peers->flag_peer[r]), "l"(1ull) : "memory");
    }
}

// Block-wide wait for the latest arrival; false when it gave up (error flag raised).
__device__ __forceinline__ bool phase_wait(const StackParams &sp, uint32_t kind, const SyncState &ss) {
    int ok = 1;
    if (threadIdx.x == 0) {
        uint32_t spins = 0;
        if (*reinterpret_cast<volatile int *>(sp.error_flag)) {
            ok = 0;  // somebody has already given up: leave instead of working on invalid data
        } else if (kind == kSyncGlobal) {
            const unsigned long long target = *ss.gbase + (unsigned long long)ss.global_gen * sp.peers->world;
            while (true) {
                unsigned long long seen;
                asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(seen) : "l"(sp.peers->flag_local) : "memory");
                if (seen >= target) break;
                if (++spins > sp.spin_limit || *reinterpret_cast<volatile int *>(sp.error_flag)) {
                    *sp.error_flag = 1;
                    ok = 0;
                    break;
                }
                __nanosleep(20);
            }
        } else {
            const unsigned int target = ss.local_gen * gridDim.x;
            while (true) {
                unsigned int seen;
                asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(sp.local_bar) : "memory");
                if (seen >= target) break;
                if (++spins > sp.spin_limit || *reinterpret_cast<volatile int *>(sp.error_flag)) {
                    *sp.error_flag = 1;
                    ok = 0;
                    break;
                }
                __nanosleep(20);
            }
        }
        __threadfence();
    }
    return __syncthreads_and(ok) != 0;
}

// ---------------------------------------------------------------------------------------------------------
// Activation rebuilds: fp16 after an exact power-of-two scaling, fragment order (k0,k4,k1,k5,k2,k6,k3,k7 inside each
// block of 8), per-group sums, and the inverse scale. Each ends with a block barrier.
// ---------------------------------------------------------------------------------------------------------
struct XBuf {
    uint8_t *xp;   // fp16 fragments
    float *xsum;   // per-group sums
    float *inv;    // inverse of the power-of-two scaling
};

// x' is stored as three signed 8-bit digits, x' = d0 + 256 d1 + 65536 d2 with every digit in [-128, 127], one 128-byte
// plane per digit and chunk. Inside a plane the byte order is the one the tensor-core B fragment of the integer MMA
// (m16n8k32) wants, given that lane t of a quad feeds its own 32 consecutive nibbles of a weight row as A operand:
// byte [t][r][i] (t: quad lane, r: one of the 8 B registers of the chunk's four MMAs, i: byte) holds input
//   k = 32 t + 16 (r >> 2) + 8 (r & 1) + ((r >> 1) & 1) + 2 i.
// One thread converts 8 consecutive inputs (k = 8b .. 8b+7): the even ones fill register r, the odd ones r + 2.
__device__ __forceinline__ void emit_block(const float (&v)[8], float scale, uint32_t b, bool in_range, const XBuf &X) {
    int xi[8];
    int sum = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        xi[i] = __float2int_rn(v[i] * scale);
        sum += xi[i];
    }
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    sum += __shfl_xor_sync(0xffffffffu, sum, 4);
    // Signed digits from one addition: x' + 128 (1 + 256 + 65536) has the plain bytes d0 + 128, d1 + 128, d2 + 128
    // (x' lies within +-2^22, so the sum is positive and below 2^24), and flipping bit 7 of a byte subtracts the 128.
    uint32_t z[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) z[i] = ((uint32_t)xi[i] + 0x00808080u) ^ 0x00808080u;
    // plane c of the even inputs: byte c of z[0], z[2], z[4], z[6]; of the odd inputs: of z[1], z[3], z[5], z[7]
    uint32_t even[3], odd[3];
#pragma unroll
    for (int c = 0; c < 3; ++c) {
        const uint32_t sel = (uint32_t)c | ((4u + (uint32_t)c) << 4);
        even[c] = __byte_perm(__byte_perm(z[0], z[2], sel), __byte_perm(z[4], z[6], sel), 0x5410u);
        odd[c] = __byte_perm(__byte_perm(z[1], z[3], sel), __byte_perm(z[5], z[7], sel), 0x5410u);
    }
    if (in_range) {
        const uint32_t chunk = b >> 4, bb = b & 15u;
        const uint32_t r = ((bb & 2u) << 1) | (bb & 1u);  // inputs 8 (bb & 3) + {0,2,4,6}: register r, the odd ones r + 2
        uint8_t *dst = X.xp + (size_t)chunk * kXChunkBytes + (bb >> 2) * 32u + r * 4u;
#pragma unroll
        for (int c = 0; c < 3; ++c) {
            *reinterpret_cast<uint32_t *>(dst + c * 128) = even[c];
            *reinterpret_cast<uint32_t *>(dst + c * 128 + 8) = odd[c];
        }
        if ((threadIdx.x & 7u) == 0) X.xsum[b / 8] = (float)sum;
    }
}

__device__ __forceinline__ uint4 pack_bf16x8(const float (&v)[8]) {
    uint32_t bb[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) bb[i] = float_to_bf16_bits(v[i]);
    uint4 plain;
    plain.x = bb[0] | (bb[1] << 16);
    plain.y = bb[2] | (bb[3] << 16);
    plain.z = bb[4] | (bb[5] << 16);
    plain.w = bb[6] | (bb[7] << 16);
    return plain;
}

// sum and maximum over the block in one exchange, the same order on every block
template <int WARPS>
__device__ __forceinline__ void block_sum_max(float &sum, uint32_t &mx, float *red) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        sum += __shfl_xor_sync(0xffffffffu, sum, off);
        mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    }
    __syncthreads();
    if ((threadIdx.x & 31u) == 0) {
        red[threadIdx.x >> 5] = sum;
        reinterpret_cast<uint32_t *>(red)[32 + (threadIdx.x >> 5)] = mx;
    }
    __syncthreads();
    float total = 0.f;
    uint32_t top = 0;
#pragma unroll
    for (int i = 0; i < WARPS; ++i) {
        total += red[i];
        top = max(top, reinterpret_cast<uint32_t *>(red)[32 + i]);
    }
    sum = total;
    mx = top;
}

// Tagged vectors hold an fp32 value per 8-byte {value, tag} word; a block of 8 values is four 16-byte loads. The two
// helpers below poll until every word of the wanted blocks carries `tag`. The wait is bounded; when it runs out the
// error flag is raised and whatever was read is used (every block leaves at its next wait).
__device__ __forceinline__ bool tagged_block_load(const uint4 *p0, uint32_t tag, uint4 (&q)[4]) {
#pragma unroll
    for (int i = 0; i < 4; ++i)
        asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(q[i].x), "=r"(q[i].y), "=r"(q[i].z), "=r"(q[i].w) : "l"(p0 + i) : "memory");
    bool ok = true;
#pragma unroll
    for (int i = 0; i < 4; ++i) ok = ok && q[i].y == tag && q[i].w == tag;
    return ok;
}

__device__ __forceinline__ bool tagged_wait_expired(const StackParams &sp, uint32_t &spins) {
    if (++spins > sp.spin_limit || *reinterpret_cast<volatile int *>(sp.error_flag)) {
        *sp.error_flag = 1;
        return true;
    }
    __nanosleep(40);
    return false;
}

// One block of 8 (if `have`), added to acc.
__device__ __forceinline__ void add_tagged_block(const StackParams &sp, const uint8_t *vector, uint32_t b, bool have, uint32_t tag, float (&acc)[8]) {
    if (!have) return;
    const uint4 *p0 = reinterpret_cast<const uint4 *>(vector + (size_t)b * 64);
    uint4 q[4];
    uint32_t spins = 0;
    while (!tagged_block_load(p0, tag, q))
        if (tagged_wait_expired(sp, spins)) break;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        acc[2 * i] += __uint_as_float(q[i].x);
        acc[2 * i + 1] += __uint_as_float(q[i].z);
    }
}

// Two blocks of 8 polled together: the loads of both are in flight at once, so a poll costs one round trip to L2
// instead of two. The second block is optional.
__device__ __forceinline__ void add_tagged_pair(const StackParams &sp, const uint8_t *vector, uint32_t b0, uint32_t b1, bool have1, uint32_t tag,
                                                float (&acc0)[8], float (&acc1)[8]) {
    if (!have1) {
        add_tagged_block(sp, vector, b0, true, tag, acc0);
        return;
    }
    const uint4 *p0 = reinterpret_cast<const uint4 *>(vector + (size_t)b0 * 64);
    const uint4 *p1 = reinterpret_cast<const uint4 *>(vector + (size_t)b1 * 64);
    uint4 q0[4], q1[4];
    uint32_t spins = 0;
    while (true) {
#pragma unroll
        for (int i = 0; i < 4; ++i)
            asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(q0[i].x), "=r"(q0[i].y), "=r"(q0[i].z), "=r"(q0[i].w) : "l"(p0 + i) : "memory");
#pragma unroll
        for (int i = 0; i < 4; ++i)
            asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(q1[i].x), "=r"(q1[i].y), "=r"(q1[i].z), "=r"(q1[i].w) : "l"(p1 + i) : "memory");
        bool ok = true;
#pragma unroll
        for (int i = 0; i < 4; ++i) ok = ok && q0[i].y == tag && q0[i].w == tag && q1[i].y == tag && q1[i].w == tag;
        if (ok) break;
        if (tagged_wait_expired(sp, spins)) break;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        acc0[2 * i] += __uint_as_float(q0[i].x);
        acc0[2 * i + 1] += __uint_as_float(q0[i].z);
        acc1[2 * i] += __uint_as_float(q1[i].x);
        acc1[2 * i + 1] += __uint_as_float(q1[i].z);
    }
}

// bf16 vector | fp32 vector | bf16(silu(gate)*up) of two fp32 vectors | weightless RMS-norm of an fp32 vector given as
// the sum of src_parts vectors (plain, or tagged words that are polled) | the hidden vector as a fused gate/up
// epilogue left it (tagged pairs of bf16 values, polled; only this SM's slice is read and scaled by the slice's own
// maximum). Values are held in registers between the reduction and the conversion.
// [b_lo, b_hi): the 8-input blocks this SM holds (all of them, or the slice of a K-major phase; b_lo is a multiple of
// 64 and X is offset so that block b_lo lands at the start of the buffer); [o_lo, o_hi): blocks this SM writes to the
// optional bf16 copy.
// ITERS: blocks of 8 a thread may hold (the caller picks the small instance when the vector is short: fewer registers
// are live, and the polls of a thread's two blocks go out together).
template <int WARPS, int ITERS>
__device__ __forceinline__ void rebuild_general(const StackParams &sp, const StackPhase &P, const XBuf &X, float *red, uint32_t b_lo, uint32_t b_hi,
                                                uint32_t o_lo, uint32_t o_hi, uint32_t src_tag, unsigned long long *tr) {
    constexpr uint32_t T = WARPS * 32;
    const uint32_t k = P.k;
    const uint32_t blocks = k / 8, blocks_p = P.kp / 8;
    float v[ITERS][8];
    float ss = 0.f;
    uint32_t amax = 0;
    // (The partial vectors of several ranks are read part after part by every block. Adding them up once per GPU and
    // sharing the sum was tried and is slower at 2, 4 and 8 ranks: it makes every block wait for every other block's
    // arrival at the rebuild, which a direct read does not.)
    const uint32_t n_parts = P.src_parts;
    const uint8_t *src_base = reinterpret_cast<const uint8_t *>(P.src0);
    // a block reads the slice it holds (all of the vector unless the phase is K-major) and scales it by the slice's own
    // maximum; only the RMS-norm needs the whole vector (its sum of squares)
    const bool whole = P.x_kind == kRebuildRms;
    const uint32_t base = whole ? 0u : b_lo, limit = whole ? blocks_p : b_hi;
#pragma unroll
    for (int it = 0; it < ITERS; ++it)
#pragma unroll
        for (int i = 0; i < 8; ++i) v[it][i] = 0.f;
    bool polled = false;
    if (ITERS == 2 && P.x_kind == kRebuildRms && P.src_tagged) {
        polled = true;
        if (threadIdx.x < blocks) {
            for (uint32_t part = 0; part < n_parts; ++part)
                add_tagged_pair(sp, src_base + (size_t)part * P.src_part_stride, threadIdx.x, threadIdx.x + T, threadIdx.x + T < blocks, src_tag, v[0],
                                v[ITERS - 1]);
        }
    }
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
        const uint32_t b = base + threadIdx.x + it * T;
        if (base + it * T >= limit) continue;  // (uniform) nothing left for any thread
        if (b < blocks && b < limit) {
            if (P.x_kind == kRebuildH) {
                // four {two bf16 values, tag} words per block of 8: wait (bounded) for the epilogues that produce them
                const uint4 *p0 = reinterpret_cast<const uint4 *>(static_cast<const uint8_t *>(P.src0) + (size_t)b * 32);
                uint4 q[2];
                uint32_t spins = 0;
                while (true) {
                    bool ok = true;
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(q[i].x), "=r"(q[i].y), "=r"(q[i].z), "=r"(q[i].w) : "l"(p0 + i) : "memory");
                        ok = ok && q[i].y == src_tag && q[i].w == src_tag;
                    }
                    if (ok) break;
                    if (++spins > sp.spin_limit || *reinterpret_cast<volatile int *>(sp.error_flag)) {
                        *sp.error_flag = 1;
                        break;
                    }
                    __nanosleep(40);
                }
                const uint32_t r[4] = {q[0].x, q[0].z, q[1].x, q[1].z};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    v[it][2 * i] = bf16_bits_to_float(r[i] & 0xffffu);
                    v[it][2 * i + 1] = bf16_bits_to_float(r[i] >> 16);
                }
            } else if (P.x_kind == kRebuildBf16) {
                const uint4 raw = __ldcg(reinterpret_cast<const uint4 *>(static_cast<const uint16_t *>(P.src0) + (size_t)b * 8));
                const uint32_t r[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    v[it][2 * i] = bf16_bits_to_float(r[i] & 0xffffu);
                    v[it][2 * i + 1] = bf16_bits_to_float(r[i] >> 16);
                }
            } else if (P.x_kind == kRebuildF32) {
                const float4 *p0 = reinterpret_cast<const float4 *>(static_cast<const float *>(P.src0) + (size_t)b * 8);
                const float4 a0 = __ldcg(p0), a1 = __ldcg(p0 + 1);
                v[it][0] = a0.x; v[it][1] = a0.y; v[it][2] = a0.z; v[it][3] = a0.w;
                v[it][4] = a1.x; v[it][5] = a1.y; v[it][6] = a1.z; v[it][7] = a1.w;
            } else if (P.x_kind == kRebuildSwiglu) {
                const float4 *p0 = reinterpret_cast<const float4 *>(static_cast<const float *>(P.src0) + (size_t)b * 8);
                const float4 *p1 = reinterpret_cast<const float4 *>(static_cast<const float *>(P.src1) + (size_t)b * 8);
                const float4 a0 = __ldcg(p0), a1 = __ldcg(p0 + 1), u0 = __ldcg(p1), u1 = __ldcg(p1 + 1);
                const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
                const float u[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float h = (a[i] * (1.0f / (1.0f + expf(-a[i])))) * u[i];  // qwen38_swiglu_rows
                    v[it][i] = bf16_bits_to_float(float_to_bf16_bits(h));
                }
            } else {
                for (uint32_t part = 0; part < n_parts && !polled; ++part) {
                    const uint8_t *vector = src_base + (size_t)part * P.src_part_stride;
                    if (P.src_tagged) {
                        add_tagged_block(sp, vector, b, true, src_tag, v[it]);
                    } else {
                        const float4 *p0 = reinterpret_cast<const float4 *>(vector + (size_t)b * 32);
                        const float4 a0 = __ldcg(p0), a1 = __ldcg(p0 + 1);
                        v[it][0] += a0.x; v[it][1] += a0.y; v[it][2] += a0.z; v[it][3] += a0.w;
                        v[it][4] += a1.x; v[it][5] += a1.y; v[it][6] += a1.z; v[it][7] += a1.w;
                    }
                }
                if (blockIdx.x == 0 && P.sum_out) {
                    float4 *dst = reinterpret_cast<float4 *>(P.sum_out + (size_t)b * 8);
                    dst[0] = make_float4(v[it][0], v[it][1], v[it][2], v[it][3]);
                    dst[1] = make_float4(v[it][4], v[it][5], v[it][6], v[it][7]);
                }
#pragma unroll
                for (int i = 0; i < 8; ++i) ss += v[it][i] * v[it][i];
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) amax = max(amax, __float_as_uint(v[it][i]) & 0x7fffffffu);
        }
    }
    if (tr) tr[7] = stack_ns();  // thread 0 has its source values
    block_sum_max<WARPS>(ss, amax, red);
    if (P.x_kind == kRebuildRms) {
        const float inv = rsqrtf(ss / (float)k + P.eps);
        // rounding is monotonic, so the largest rounded magnitude is the rounded largest magnitude
        amax = float_to_bf16_bits(__uint_as_float(amax) * inv) << 16;
#pragma unroll
        for (int it = 0; it < ITERS; ++it) {
            if (base + it * T >= limit) continue;
#pragma unroll
            for (int i = 0; i < 8; ++i) v[it][i] = bf16_bits_to_float(float_to_bf16_bits(v[it][i] * inv));
        }
    }
    const int e = scale_exponent(amax);
    const float scale = __uint_as_float((uint32_t)(e + 127) << 23);
    if (threadIdx.x == 0) *X.inv = __uint_as_float((uint32_t)(127 - e) << 23);
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
        const uint32_t b = base + threadIdx.x + it * T;
        if (base + it * T >= limit) continue;
        emit_block(v[it], scale, b, b >= b_lo && b < b_hi, X);
        if (P.x_bf16_out && b >= o_lo && b < o_hi && b < blocks) *reinterpret_cast<uint4 *>(P.x_bf16_out + (size_t)b * 8) = pack_bf16x8(v[it]);
    }
    __syncthreads();
}

// ---------------------------------------------------------------------------------------------------------
// Work: one contiguous run of chunks of one tile, as seen by one lane.
// ---------------------------------------------------------------------------------------------------------
struct Segment {
    uint32_t job;                   // index into the chain's job array
    uint32_t tile_local, tile_row;  // tile within the job, its first side-a row
    uint32_t c0, c1, cbase;         // real chunks [c0, c1); cbase = c0 rounded down to four
    uint32_t c0v, c1v;              // the run in the job's virtual chunk numbering
    uint32_t mis_wa, mis_wb;        // byte misalignment (address & 15) of the two sides' weights
    uint32_t mis_p;                 // and of their scale / bias arrays, four bits each: scales a, scales b, biases a, biases b
    uint32_t pmis;                  // misalignment of the parameter row this lane copies
    const uint8_t *wa, *wb, *pp;    // cursors at chunk cbase (this lane's aligned window)
};

__device__ __forceinline__ void segment_setup(const StackPhase &P, const StackJob *jobs, uint32_t u, uint32_t u1, uint32_t &job_rel,
                                              uint32_t lane, Segment &sg) {
    const uint32_t g = lane >> 2, t = lane & 3u, cpt = P.cpt;
    while (job_rel + 1 < P.n_jobs && u >= jobs[P.job_begin + job_rel + 1].unit_begin) ++job_rel;
    sg.job = P.job_begin + job_rel;
    const StackJob &J = jobs[sg.job];
    const uint32_t rel = u - J.unit_begin, vcpt = J.vcpt;
    sg.tile_local = rel / vcpt;
    sg.tile_row = sg.tile_local * J.rows_per_tile;
    sg.c0v = rel - sg.tile_local * vcpt;
    const uint32_t left = u1 - u;
    sg.c1v = (left < vcpt - sg.c0v) ? sg.c0v + left : vcpt;
    sg.c0 = sg.c0v < cpt ? sg.c0v : cpt;
    sg.c1 = sg.c1v < cpt ? sg.c1v : cpt;
    sg.cbase = sg.c0 & ~3u;
    sg.mis_wa = (uint32_t)((uintptr_t)J.w[0] & 15u);
    sg.mis_wb = (uint32_t)((uintptr_t)J.w[1] & 15u);
    sg.mis_p = (uint32_t)((uintptr_t)J.s[0] & 15u) | ((uint32_t)((uintptr_t)J.s[1] & 15u) << 4) |
               ((uint32_t)((uintptr_t)J.b[0] & 15u) << 8) | ((uint32_t)((uintptr_t)J.b[1] & 15u) << 12);
    const uint32_t last = J.n - 1u;
    uint32_t row_a = sg.tile_row + g, row_b = sg.tile_row + g + J.b_row_offset;
    row_a = row_a < last ? row_a : last;  // rows past N read a valid row and are never stored
    row_b = row_b < last ? row_b : last;
    sg.wa = J.w[0] + (uint64_t)row_a * J.w_stride + t * 16u + sg.cbase * 64u - sg.mis_wa;
    sg.wb = J.w[1] + (uint64_t)row_b * J.w_stride + t * 16u + sg.cbase * 64u - sg.mis_wb;
    // parameter copies: lane l moves 16 bytes of tile row (l & 15) of array (l >> 4: scales, biases)
    const uint32_t prow = lane & 15u, side = prow >> 3;
    uint32_t row_p = sg.tile_row + (prow & 7u) + (side ? J.b_row_offset : 0u);
    row_p = row_p < last ? row_p : last;
    const uint8_t *pbase = (lane >> 4) ? J.b[side] : J.s[side];
    sg.pmis = (uint32_t)((uintptr_t)pbase & 15u);
    sg.pp = pbase + (uint64_t)row_p * J.p_stride + sg.cbase * 4u - sg.pmis;
}

// Async copies of the first two groups of four chunks. With misaligned weights the chunk after the segment is
// copied as well: the last lane of a quad completes its 16 bytes from the next chunk's first window.
__device__ __forceinline__ void segment_prologue(const Segment &sg, uint32_t ring, uint32_t pring, uint32_t lane) {
    const uint32_t live = sg.c1 > sg.c0 ? 1u : 0u;
    const uint32_t wend_a = sg.c1 + (sg.mis_wa ? live : 0u), wend_b = sg.c1 + (sg.mis_wb ? live : 0u);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
#pragma unroll
        for (int s = 0; s < 4; ++s) {
            const uint32_t c = sg.cbase + 4 * h + s;
            const uint32_t stage = ring + (4 * h + s) * kStageBytesAligned + lane * 16u;
            cp_async_16_pred(stage, sg.wa + (4 * h + s) * 64, c >= sg.c0 && c < wend_a);
            cp_async_16_pred(stage + 512u, sg.wb + (4 * h + s) * 64, c >= sg.c0 && c < wend_b);
        }
        const bool pin = sg.cbase + 4 * h < sg.c1;
        cp_async_16_pred(pring + h * 1024u + lane * 16u, sg.pp + h * 16, pin);
        cp_async_16_pred(pring + h * 1024u + 512u + lane * 16u, sg.pp + h * 16 + 16, pin && sg.pmis != 0);
        cp_async_commit();
    }
}

// What is needed to finish a tile after the lane's cursors have moved on to the next run of chunks.
struct TileEnd {
    uint32_t job, tile_local, tile_row, c0v, c1v;
};

// End of a tile for one activation row. A lane holds two sums: side a (tile row g) and side b. A whole tile is stored
// at once. A tile split between warps is owned by the warp that computed its first chunks (the last thing that warp
// does in the phase, while the other contributors met the tile at the start of their ranges): every other contributor
// posts its sums in its partial slot as 8-byte {value, tag} words -- value and tag travel in one store, so no fence and
// no counter are needed -- and the owner adds them to its own in worker order once their tags show this launch and
// phase. The wait for a late contributor is bounded. Returns true when this warp stored into other GPUs' memory.
__device__ __forceinline__ bool finish_tile_m1(const StackParams &sp, const StackPhase &P, const StackJob &J, uint32_t worker,
                                               const TileEnd &te, float acc_a, float acc_b, uint32_t tag, uint32_t lane, uint32_t g,
                                               uint32_t t) {
    const bool whole = te.c0v == 0 && te.c1v == J.vcpt;
    if (!whole) {
        const Q4Split split{P.units, P.cpt, P.workers};
        const uint64_t u0 = (uint64_t)J.unit_begin + (uint64_t)te.tile_local * J.vcpt;
        uint32_t first, last;
        q4_split_span_contributors(split, u0, J.vcpt, &first, &last);
        uint4 *slots = sp.partials + (size_t)P.slot_set * sp.max_workers * 32u;
        if (worker != first) {
            uint4 *dst = slots + (size_t)worker * 32u + lane;
            asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(dst), "r"(__float_as_uint(acc_a)), "r"(tag),
                         "r"(__float_as_uint(acc_b)), "r"(tag)
                         : "memory");
            return false;
        }
        // the other contributors' sums, four slots at a time (independent loads in flight), added in worker order
        for (uint32_t w0 = first + 1; w0 <= last; w0 += 4) {
            uint4 pv[4];
            uint32_t spins = 0;
            while (true) {
                bool ok = true;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const uint32_t w = w0 + i <= last ? w0 + i : last;
                    const uint4 *src = slots + (size_t)w * 32u + lane;
                    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(pv[i].x), "=r"(pv[i].y), "=r"(pv[i].z), "=r"(pv[i].w) : "l"(src) : "memory");
                    ok = ok && pv[i].y == tag && pv[i].w == tag;
                }
                if (__all_sync(0xffffffffu, ok)) break;
                if (++spins > sp.spin_limit || *reinterpret_cast<volatile int *>(sp.error_flag)) {
                    *sp.error_flag = 1;  // the next barrier wait of every block sees it and leaves
                    return false;
                }
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                if (w0 + i <= last) {
                    acc_a += __uint_as_float(pv[i].x);
                    acc_b += __uint_as_float(pv[i].z);
                }
            }
        }
    }
    // a row's sum is spread over the four lanes of its quad: digits (0,1) and digit 2 of group A in lanes 0 and 1,
    // those of group B in lanes 2 and 3
    acc_a += __shfl_xor_sync(0xffffffffu, acc_a, 1);
    acc_b += __shfl_xor_sync(0xffffffffu, acc_b, 1);
    const float ya = acc_a + __shfl_xor_sync(0xffffffffu, acc_a, 2);
    const float yb = acc_b + __shfl_xor_sync(0xffffffffu, acc_b, 2);
    const uint32_t row_a = te.tile_row + g, row_b = row_a + J.b_row_offset;
    if (J.pair) {
        const bool valid = t == 0 && row_a < J.n;
        const float h = (ya * (1.0f / (1.0f + expf(-ya)))) * yb;  // qwen38_swiglu_rows, shaders/qwen38.metal:4188-4198
        const uint32_t hb = valid ? float_to_bf16_bits(h) : 0u;
        // rows come in pairs: the lane of the even row stores both bf16 values and the tag as one 8-byte word
        const uint32_t hb_next = __shfl_down_sync(0xffffffffu, hb, 4);
        if (valid) {
            if ((g & 1u) == 0)
                asm volatile("st.volatile.global.v2.u32 [%0], {%1,%2};" ::"l"(J.h_out + (row_a >> 1)), "r"(hb | (hb_next << 16)), "r"(tag) : "memory");
            if (J.out[0]) J.out[0][row_a] = ya;
            if (J.out[1]) J.out[1][row_a] = yb;
        }
        return false;
    }
    if (t != 0) return J.has_peers != 0;
    if (J.out[0]) {
        if (row_a < J.n) J.out[0][row_a] = ya;
        if (row_b < J.n) J.out[0][row_b] = yb;
    }
    if (J.has_ll) {
#pragma unroll
        for (int r = 0; r < kMaxPeers; ++r) {
            unsigned long long *dst = J.ll_out[r];
            if (dst) {
                if (row_a < J.n) asm volatile("st.volatile.global.v2.u32 [%0], {%1,%2};" ::"l"(dst + row_a), "r"(__float_as_uint(ya)), "r"(tag) : "memory");
                if (row_b < J.n) asm volatile("st.volatile.global.v2.u32 [%0], {%1,%2};" ::"l"(dst + row_b), "r"(__float_as_uint(yb)), "r"(tag) : "memory");
            }
        }
    }
    if (J.has_peers) {
        // the other ranks' copies of this output (peer stores over NVLink)
#pragma unroll
        for (int r = 0; r < kMaxPeers; ++r) {
            float *peer = J.peer_out[r];
            if (peer) {
                if (row_a < J.n) peer[row_a] = ya;
                if (row_b < J.n) peer[row_b] = yb;
            }
        }
    }
    return J.has_peers != 0;
}

// The worker number of a warp in a phase (0xffffffff: none) -- see StackPhase::kparts.
__device__ __forceinline__ uint32_t phase_worker(const StackPhase &P, uint32_t warp, uint32_t warps) {
    if (P.kparts <= 1u) return blockIdx.x * warps + warp;
    const uint32_t tile = (blockIdx.x / P.kparts) * warps + warp;
    return tile < P.tiles ? tile * P.kparts + blockIdx.x % P.kparts : 0xffffffffu;
}

// One chunk on the integer tensor-core path: d = sum over the chunk of q * digit for rows g (d[0], d[1]) and g+8 (d[2],
// d[3]) and the lane's two result columns. A packed word becomes two byte registers with three logic instructions
// (even nibbles: w & 0x0f0f0f0f, odd nibbles: (w >> 4) & 0x0f0f0f0f); the products are exact integers.
__device__ __forceinline__ void chunk_mma_i8(const uint4 &cwa, const uint4 &cwb, const uint4 (&xr)[2], int (&d)[4]) {
    const uint32_t wa[4] = {cwa.x, cwa.y, cwa.z, cwa.w}, wb[4] = {cwb.x, cwb.y, cwb.z, cwb.w};
    const uint32_t m = 0x0f0f0f0fu;
    uint32_t la[4], ha[4], lb[4], hb[4];
#pragma unroll
    for (int w = 0; w < 4; ++w) {
        la[w] = wa[w] & m;
        ha[w] = (wa[w] >> 4) & m;
        lb[w] = wb[w] & m;
        hb[w] = (wb[w] >> 4) & m;
    }
    d[0] = d[1] = d[2] = d[3] = 0;
    mma_u8s8_16832(d, la[0], lb[0], la[1], lb[1], xr[0].x, xr[0].y);
    mma_u8s8_16832(d, ha[0], hb[0], ha[1], hb[1], xr[0].z, xr[0].w);
    mma_u8s8_16832(d, la[2], lb[2], la[3], lb[3], xr[1].x, xr[1].y);
    mma_u8s8_16832(d, ha[2], hb[2], ha[3], hb[3], xr[1].z, xr[1].w);
}

// LONG: the instance that can rebuild vectors of more than two blocks of 8 per thread (an unsliced hidden vector,
// K > 8192). Its 40 value registers push the streaming loop into spills (128 registers, 90 bytes of spill stores);
// chains that never need it (params.long_rebuild == 0) run the other instance: 122 registers, no spills.
template <int WARPS, bool LONG>
__device__ __forceinline__ void stack_body(const StackParams &sp) {
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const uint32_t g = lane >> 2, t = lane & 3u;
    // shared memory: per-warp rings | activation buffer 0 | activation buffer 1 | group sums 0 | group sums 1 | misc
    uint8_t *xp0 = smem + WARPS * kStackRingBytes;
    uint8_t *xp1 = xp0 + sp.halfs[0] * 3 + kXSlack;
    float *xsum0 = reinterpret_cast<float *>(xp1 + sp.halfs[1] * 3 + kXSlack);
    float *xsum1 = xsum0 + sp.halfs[0] / 64 + 4;
    float *misc = xsum1 + sp.halfs[1] / 64 + 4;
    uint32_t *arrive_smem = reinterpret_cast<uint32_t *>(misc + 2);
    uint32_t *units_done_smem = reinterpret_cast<uint32_t *>(misc + 70);  // warps of this block through with a phase, running count
    float *red = misc + 4;
    const uint32_t ring = (uint32_t)__cvta_generic_to_shared(smem) + warp * kStackRingBytes;
    const uint32_t pring = ring + kStages * kStageBytesAligned;
    // One activation row as three digit columns per affine group: MMA columns 0,1,2 carry the digits of group A (fed by
    // lanes g = 0,1,2 with t < 2, which hold group A's k slots), columns 4,5,6 those of group B (lanes g = 4,5,6, t >= 2);
    // every other B lane supplies zeros. A lane's results are columns 2t and 2t+1.
    const bool has_x = (g & 3u) < 3u && ((g < 4u) == (t < 2u));
    const bool has_sum = (t & 1u) == 0;  // lanes whose result columns include digit 0 of a group (column 0 / 4)
    const uint32_t half_sel = (t >> 1) ? 0x3244u : 0x1044u;
    uint4 xf[2][2];  // B registers of the chunk in use and the next one
#pragma unroll
    for (int b = 0; b < 2; ++b) xf[b][0] = xf[b][1] = make_uint4(0, 0, 0, 0);

    unsigned long long *gbase_smem = reinterpret_cast<unsigned long long *>(misc + 68);
    SyncState sync{0u, 0u, gbase_smem};
    bool prefetched = false;
    Segment sg;
    uint32_t job_rel = 0;
    // Weights of a phase's first run of chunks depend on nothing, so they are requested as soon as the ring is free:
    // at the very start of the kernel for the first phase, and for every later phase once the warp has delivered the
    // results of the phase before and arrived at its barrier.
    auto request_phase = [&](uint32_t next) {
        prefetched = false;
        if (next < sp.n_phases) {
            const StackPhase &N = sp.phases[next];
            const uint32_t nworker = phase_worker(N, warp, WARPS);
            if (nworker < N.workers) {
                const Q4Split nsplit{N.units, N.cpt, N.workers};
                const uint32_t nu = (uint32_t)q4_split_begin(nsplit, nworker), nu1 = (uint32_t)q4_split_begin(nsplit, nworker + 1);
                if (nu < nu1) {
                    job_rel = 0;
                    segment_setup(N, sp.jobs, nu, nu1, job_rel, lane, sg);
                    segment_prologue(sg, ring, pring, lane);
                    prefetched = true;
                }
            }
        }
    };
    request_phase(0);
    if (threadIdx.x == 0) {
        *arrive_smem = 0;
        *units_done_smem = 0;
        *gbase_smem = sp.peers ? *reinterpret_cast<volatile unsigned long long *>(sp.peers->consumed) : 0ull;
        reinterpret_cast<uint32_t *>(misc)[3] = *reinterpret_cast<volatile unsigned int *>(sp.launch_seq);
    }
    __syncthreads();
    // tags of the split-tile partial slots: unique per launch and phase, never zero
    const uint32_t tag_base = reinterpret_cast<uint32_t *>(misc)[3] * kMaxPhases + 1u;

    for (uint32_t ph = 0; ph < sp.n_phases; ++ph) {
        const StackPhase &P = sp.phases[ph];
        // trace slot of this block and phase for lane 0 of any warp, null otherwise
        auto trace_slot = [&]() -> unsigned long long * {
            return (sp.trace && lane == 0) ? sp.trace + ((size_t)blockIdx.x * sp.n_phases + ph) * kTraceStamps : nullptr;
        };
        const bool second = P.x_buf != 0;
        const uint32_t worker = phase_worker(P, warp, WARPS);
        // chunks of the activation this SM holds: all, or the run of its part (K-major phases), from a multiple of four
        uint32_t c_lo = 0, c_hi = P.kp / 128u;
        if (P.kparts > 1u && P.sliced) {
            const uint32_t part = blockIdx.x % P.kparts;
            c_lo = P.cpt * part / P.kparts;
            c_hi = P.cpt * (part + 1u) / P.kparts;
        }
        const uint32_t cs4 = c_lo & ~3u;
        // pointers such that chunk cs4 lands at the start of the buffer
        const XBuf X{(second ? xp1 : xp0) - (size_t)cs4 * kXChunkBytes, (second ? xsum1 : xsum0) - (size_t)cs4 * 2u, misc + (second ? 1 : 0)};
        // Descriptors ahead: the phase after the next one into L2, the next one (whose first run of chunks every warp
        // sets up at the end of this phase, a chain of dependent loads) into this SM's L1.
        if (warp == 1) {
            if (ph + 2 < sp.n_phases) {
                const StackPhase &N2 = sp.phases[ph + 2];
                if (lane == 0) prefetch_l2(&N2);
                const uint32_t lines = (N2.n_jobs * (uint32_t)sizeof(StackJob) + 127u) / 128u;
                if (lane >= 1 && lane <= lines) prefetch_l2(reinterpret_cast<const uint8_t *>(sp.jobs + N2.job_begin) + (lane - 1u) * 128u);
            }
            if (ph + 1 < sp.n_phases) {
                const StackPhase &N1 = sp.phases[ph + 1];
                if (lane < 2) prefetch_l1(reinterpret_cast<const uint8_t *>(&N1) + lane * 128u);
                const uint32_t lines = (N1.n_jobs * (uint32_t)sizeof(StackJob) + 127u) / 128u;
                if (lane >= 2 && lane < 2u + lines) prefetch_l1(reinterpret_cast<const uint8_t *>(sp.jobs + N1.job_begin) + (lane - 2u) * 128u);
            }
        }
        if (P.wait_kind != kSyncNone || P.x_kind != kRebuildNone) {
            if (sp.trace && threadIdx.x == 0) trace_slot()[0] = stack_ns();
            if (P.wait_kind != kSyncNone) {
                if (!phase_wait(sp, P.wait_kind, sync)) return;
            } else {
                __syncthreads();  // everyone is done with the buffer that is about to be rewritten
            }
            if (sp.trace && threadIdx.x == 0) trace_slot()[1] = stack_ns();
            // the bf16 copy of the activation is written by block 0, or by the first kparts blocks (one part each)
            const bool writes = blockIdx.x < ((P.kparts > 1u && P.sliced) ? P.kparts : 1u);
            const uint32_t o_lo = writes ? c_lo * 16u : 0u, o_hi = writes ? c_hi * 16u : 0u;
            if (P.x_kind != kRebuildNone) {
                unsigned long long *tr = (sp.trace && threadIdx.x == 0) ? trace_slot() : nullptr;
                const uint32_t held = P.x_kind == kRebuildRms ? P.kp / 8u : c_hi * 16u - cs4 * 16u;
                if (held <= 2u * WARPS * 32u) {
                    rebuild_general<WARPS, 2>(sp, P, X, red, cs4 * 16u, c_hi * 16u, o_lo, o_hi, tag_base + P.src_tag_phase, tr);
                } else if constexpr (LONG) {
                    rebuild_general<WARPS, kStackMaxIters>(sp, P, X, red, cs4 * 16u, c_hi * 16u, o_lo, o_hi, tag_base + P.src_tag_phase, tr);
                } else {
                    if (threadIdx.x == 0) *sp.error_flag = 1;  // the host picked the wrong instance: report, compute nothing
                    __syncthreads();
                }
            }
            if (sp.trace && threadIdx.x == 0) trace_slot()[2] = stack_ns();
        }

        bool stored_to_peers = false;
        uint32_t blocks_done = 0;
        uint32_t u = 0, u1 = 0;  // this warp's units of the phase (a phase has fewer than 2^32)
        if (worker < P.workers) {
            const Q4Split split{P.units, P.cpt, P.workers};
            u = (uint32_t)q4_split_begin(split, worker);
            u1 = (uint32_t)q4_split_begin(split, worker + 1);
        }
        bool more = u < u1;
        if (more && !prefetched) {
            job_rel = 0;
            segment_setup(P, sp.jobs, u, u1, job_rel, lane, sg);
            segment_prologue(sg, ring, pring, lane);
        }
        const uint32_t xp_addr = (uint32_t)__cvta_generic_to_shared(X.xp) + (g & 3u) * 128u + t * 32u;
        const uint32_t xsum_addr = (uint32_t)__cvta_generic_to_shared(X.xsum) + (t >> 1) * 4u;
        while (more) {
            {
                const uint32_t c0 = sg.c0, c1 = sg.c1;
                const uint32_t mis_wa = sg.mis_wa, mis_wb = sg.mis_wb;
                const bool mis_any = (mis_wa | mis_wb) != 0;
                const uint32_t live = c1 > c0 ? 1u : 0u;
                const uint32_t wend_a = c1 + (mis_wa ? live : 0u), wend_b = c1 + (mis_wb ? live : 0u);
                const uint8_t *wa = sg.wa, *wb = sg.wb, *pp = sg.pp;
                uint32_t xa = xp_addr + sg.cbase * kXChunkBytes;  // this lane's fragment of chunk cbase
                uint32_t xs = xsum_addr + sg.cbase * 8u;  // group sum of this lane's group in chunk cbase
                float acc[4] = {0.f, 0.f, 0.f, 0.f};
                if (c0 & 1u) {
                    lds_v4_keep(xf[1][0], xa + (c0 - sg.cbase) * kXChunkBytes, has_x);
                    lds_v4_keep(xf[1][1], xa + (c0 - sg.cbase) * kXChunkBytes + 16u, has_x);
                } else {
                    lds_v4_keep(xf[0][0], xa + (c0 - sg.cbase) * kXChunkBytes, has_x);
                    lds_v4_keep(xf[0][1], xa + (c0 - sg.cbase) * kXChunkBytes + 16u, has_x);
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
                    if (sg.mis_p) {
                        const uint32_t mp = sg.mis_p;
                        if (mp & 0x000fu) psa = realign_16(psa, lds_v4(pstage + 512u + g * 16u), mp & 15u);
                        if (mp & 0x00f0u) psb = realign_16(psb, lds_v4(pstage + 512u + (g + 8u) * 16u), (mp >> 4) & 15u);
                        if (mp & 0x0f00u) pba = realign_16(pba, lds_v4(pstage + 768u + g * 16u), (mp >> 8) & 15u);
                        if (mp & 0xf000u) pbb = realign_16(pbb, lds_v4(pstage + 768u + (g + 8u) * 16u), (mp >> 12) & 15u);
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
                            if (mis_any) {
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
                                if (mis_wa) cwa = realign_16(cwa, lds_v4(next), mis_wa);
                                if (mis_wb) cwb = realign_16(cwb, lds_v4(next + 512u), mis_wb);
                            }
                            lds_v4_keep(xf[b ^ 1][0], xa + (s + 1) * kXChunkBytes, has_x);
                            lds_v4_keep(xf[b ^ 1][1], xa + (s + 1) * kXChunkBytes + 16u, has_x);
                            float xsv = 0.f;
                            lds_f32_keep(xsv, xs + s * 8u, has_sum);
                            int d[4];
                            chunk_mma_i8(cwa, cwb, xf[b], d);
                            const float sa = param_of(wsa[s], half_sel), sb = param_of(wsb[s], half_sel);
                            const float ba = param_of(wba[s], half_sel), bb = param_of(wbb[s], half_sel);
                            // per result column: the digit's integer sum times the group's scale; the bias term rides
                            // on digit 0 (weight 1)
                            acc[0] = fmaf(small_int_to_float(d[0]), sa, fmaf(xsv, ba, acc[0]));
                            acc[1] = fmaf(small_int_to_float(d[1]), sa, acc[1]);
                            acc[2] = fmaf(small_int_to_float(d[2]), sb, fmaf(xsv, bb, acc[2]));
                            acc[3] = fmaf(small_int_to_float(d[3]), sb, acc[3]);
                        }
                    }
                    __syncwarp();  // every lane is done with this half before it is refilled
#pragma unroll
                    for (int s = 0; s < 4; ++s) {
                        cp_async_16_pred(stage0 + s * kStageBytesAligned, wa + (8 + s) * 64, cg + 8 + s < wend_a);
                        cp_async_16_pred(stage0 + s * kStageBytesAligned + 512u, wb + (8 + s) * 64, cg + 8 + s < wend_b);
                    }
                    cp_async_16_pred(pstage + lane * 16u, pp + 32, cg + 8 < c1);
                    cp_async_16_pred(pstage + 512u + lane * 16u, pp + 48, cg + 8 < c1 && sg.pmis != 0);
                    cp_async_commit();
                    wa += 4 * 64;
                    wb += 4 * 64;
                    pp += 16;
                    xa += 4 * kXChunkBytes;
                    xs += 4 * 8u;
                    half ^= 1u;
                }
                cp_async_wait<0>();
                __syncwarp();
                // the ring is free: within a phase the next run of chunks is requested before this tile is finished, so
                // that the finish (a round trip to the other contributors' slots for a split tile) overlaps the load
                // latency. After the last run the order is the other way round: results and arrival first -- other
                // blocks wait for them -- then the next phase's first weights (pushing 8 KB per warp into a memory
                // system that every warp floods at the same moment takes a few microseconds).
                const TileEnd te{sg.job, sg.tile_local, sg.tile_row, sg.c0v, sg.c1v};
                u += sg.c1v - sg.c0v;
                more = u < u1;
                // (a hint, read while the last tile is being finished: how many blocks are through with this phase)
                if (!more && (sp.flags & kFlagLateSkipsRequest)) blocks_done = *reinterpret_cast<volatile unsigned int *>(sp.local_bar + kProgressWord);
                if (more) {
                    segment_setup(P, sp.jobs, u, u1, job_rel, lane, sg);
                    segment_prologue(sg, ring, pring, lane);
                }
                // digits back together: a lane's columns are digits (0, 1) of its group for even t, (2, none) for odd t
                const float w0 = (t & 1u) ? 65536.f : 1.f, w1 = (t & 1u) ? 0.f : 256.f;
                // ... and the power-of-two scaling of this SM's activation undone (exact) before sums of different SMs meet:
                // the slices of a K-major phase are scaled independently
                const float inv = *X.inv;
                const float part_a = fmaf(acc[1], w1, acc[0] * w0) * inv, part_b = fmaf(acc[3], w1, acc[2] * w0) * inv;
                stored_to_peers |= finish_tile_m1(sp, P, sp.jobs[te.job], worker, te, part_a, part_b, tag_base + ph, lane, g, t);
            }
        }
        if (sp.trace && threadIdx.x == 0) trace_slot()[3] = stack_ns();
        if (sp.trace && lane == 0) {
            atomicMax(trace_slot() + 6, stack_ns());  // the block's last warp
            if (warp == 0) {
                uint32_t smid;
                asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
                trace_slot()[5] = smid;
            }
        }

        if (P.arrive_kind != kSyncNone) {
            phase_arrive<WARPS>(sp, P.arrive_kind, sync, arrive_smem, stored_to_peers, lane, trace_slot());
            ++sync.local_gen;
            if (P.arrive_kind == kSyncGlobal) ++sync.global_gen;
        }
        // The next phase's first weights: requested now when nothing stands between this phase and the next one's
        // units; after the rebuild when there is one (kFlagRequestAfterRebuild) -- the polls and shared-memory stores
        // of a rebuild queue behind the copies a warp has in flight, which costs the last block to finish (the one
        // all others are waiting for) several microseconds per phase.
        //
        // kFlagLateSkipsRequest does that only for the warps that finish when nearly every block is through with the
        // phase: the blocks that are waiting anyway keep filling their rings during the wait. Blocks count themselves
        // in one word (the last warp of a block adds one per phase); the count is a hint and orders nothing.
        bool request_later = (sp.flags & kFlagRequestAfterRebuild) != 0;
        if (sp.flags & kFlagLateSkipsRequest) {
            if (lane == 0) {
                const uint32_t through = atomicAdd(units_done_smem, 1u) + 1u;
                if (through % WARPS == 0) atomicAdd(sp.local_bar + kProgressWord, 1u);
            }
            const uint32_t margin = (sp.flags >> 8) & 0xffu;
            request_later = blocks_done >= ph * gridDim.x + gridDim.x - margin && blocks_done < (ph + 1u) * gridDim.x + gridDim.x;
        }
        if (request_later && ph + 1u < sp.n_phases && sp.phases[ph + 1u].x_kind != kRebuildNone)
            prefetched = false;  // (the phase's own start requests them)
        else
            request_phase(ph + 1u);
    }

    // ---- logits -> token: per-block candidates, barrier, block 0 picks (ties to the lowest index) ----
    if (sp.logits) {
        const uint32_t last_kind = sp.phases[sp.n_phases - 1].arrive_kind;  // the last phase arrived for the logits
        if (!phase_wait(sp, last_kind, sync)) return;
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
        phase_arrive<WARPS>(sp, kSyncLocal, sync, arrive_smem, false, lane, nullptr);
        ++sync.local_gen;
        if (!phase_wait(sp, kSyncLocal, sync)) return;
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
            phase_arrive<WARPS>(sp, kSyncGlobal, sync, arrive_smem, blockIdx.x == 0 && warp == 0, lane, nullptr);
            ++sync.local_gen;
            ++sync.global_gen;
            if (!phase_wait(sp, kSyncGlobal, sync)) return;
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
    // End of the launch. Every block counts itself out; the block that counts last -- every other block has finished,
    // and every block read the launch count before it did anything -- puts the words back that the next launch expects:
    // barrier counters to zero, the launch count (tags of partial slots and hand-offs) one further,
    // the cross-GPU arrivals this launch used up. So no memset precedes a launch. (A launch that gave up on a wait
    // leaves them inconsistent; the host repairs them before the next launch.)
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const unsigned int done = atomicAdd(sp.local_bar + 1, 1u);
        if (done + 1u == gridDim.x) {
            __threadfence();
            sp.local_bar[0] = 0;
            sp.local_bar[1] = 0;
            sp.local_bar[kProgressWord] = 0;
            if (sp.peers) *sp.peers->consumed = *gbase_smem + (unsigned long long)sync.global_gen * sp.peers->world;
            *sp.launch_seq = reinterpret_cast<uint32_t *>(misc)[3] + 1u;
        }
    }
}

template <int WARPS, bool LONG>
__global__ void __launch_bounds__(WARPS * 32, 1) q4_stack_kernel(const __grid_constant__ StackParams sp) {
    stack_body<WARPS, LONG>(sp);
}

// The same kernel for a program of ONE phase that travels in the kernel parameters: a single grouped decode launch
// (q4b_matvec_batch and friends) builds its activation, streams its projections and stores its results in one launch,
// without a device-side program or a host-to-device copy in front of it.
template <int WARPS, bool LONG>
__global__ void __launch_bounds__(WARPS * 32, 1) q4_stack_inline_kernel(const __grid_constant__ InlineProgram prog) {
    StackParams sp = prog.params;
    sp.phases = &prog.phase;
    sp.jobs = prog.jobs;
    sp.n_phases = 1;
    stack_body<WARPS, LONG>(sp);
}

}  // namespace q4

// ---------------------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------------------

namespace {
constexpr int kStackWarps = 16;
}  // namespace

extern "C" uint32_t q4k_stack_warps(void) { return kStackWarps; }

// 1 when a phase's rebuild holds more than two blocks of 8 inputs per thread, i.e. needs the kernel instance with the
// long rebuild (the device applies the same rule to pick the rebuild)
extern "C" int q4k_stack_phase_is_long(const q4::StackPhase *P) {
    if (P->x_kind == q4::kRebuildNone) return 0;
    uint32_t held = P->kp / 8u;
    if (P->x_kind != q4::kRebuildRms) {
        held = 0;
        const uint32_t parts = (P->kparts > 1u && P->sliced) ? P->kparts : 1u;
        for (uint32_t part = 0; part < parts; ++part) {
            uint32_t c_lo = 0, c_hi = P->kp / 128u;
            if (parts > 1u) {
                c_lo = P->cpt * part / parts;
                c_hi = P->cpt * (part + 1u) / parts;
            }
            const uint32_t blocks = (c_hi - (c_lo & ~3u)) * 16u;
            held = blocks > held ? blocks : held;
        }
    }
    return held > 2u * kStackWarps * 32u ? 1 : 0;
}
extern "C" uint32_t q4k_stack_max_k(void) { return q4::kStackMaxIters * kStackWarps * 32 * 8; }

extern "C" size_t q4k_stack_smem_bytes(uint32_t halfs0, uint32_t halfs1) {
    return (size_t)kStackWarps * q4::kStackRingBytes + (size_t)(halfs0 + halfs1) * 3 + 2 * q4::kXSlack +
           (size_t)(halfs0 / 64 + halfs1 / 64 + 8) * 4 + 4 * 4 + 64 * 4 + 32 + 128;
}

// 0 when the kernel cannot be made resident with one block per SM for these activation sizes
template <typename Kernel>
static int stack_resident(Kernel kernel, size_t smem) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    int blocks = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, kernel, kStackWarps * 32, smem) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return blocks >= 1 ? 1 : 0;
}

extern "C" int q4k_stack_supported(uint32_t halfs0, uint32_t halfs1) {
    const size_t smem = q4k_stack_smem_bytes(halfs0, halfs1);
    return stack_resident(q4::q4_stack_kernel<kStackWarps, false>, smem) && stack_resident(q4::q4_stack_kernel<kStackWarps, true>, smem);
}

extern "C" cudaError_t q4k_stack_launch(const q4::StackParams *params, int sm_count, cudaStream_t stream) {
    q4::StackParams sp = *params;
    void *args[] = {&sp};
    void *kernel = sp.long_rebuild ? reinterpret_cast<void *>(q4::q4_stack_kernel<kStackWarps, true>)
                                   : reinterpret_cast<void *>(q4::q4_stack_kernel<kStackWarps, false>);
    return cudaLaunchCooperativeKernel(kernel, dim3(sm_count), dim3(kStackWarps * 32), args, q4k_stack_smem_bytes(sp.halfs[0], sp.halfs[1]), stream);
}

extern "C" int q4k_stack_inline_supported(uint32_t halfs) {
    const size_t smem = q4k_stack_smem_bytes(halfs, 0);
    return stack_resident(q4::q4_stack_inline_kernel<kStackWarps, false>, smem) && stack_resident(q4::q4_stack_inline_kernel<kStackWarps, true>, smem);
}

extern "C" cudaError_t q4k_stack_launch_inline(const q4::InlineProgram *program, int sm_count, cudaStream_t stream) {
    q4::InlineProgram prog = *program;
    void *args[] = {&prog};
    void *kernel = prog.params.long_rebuild ? reinterpret_cast<void *>(q4::q4_stack_inline_kernel<kStackWarps, true>)
                                            : reinterpret_cast<void *>(q4::q4_stack_inline_kernel<kStackWarps, false>);
    return cudaLaunchCooperativeKernel(kernel, dim3(sm_count), dim3(kStackWarps * 32), args, q4k_stack_smem_bytes(prog.params.halfs[0], 0), stream);
}
