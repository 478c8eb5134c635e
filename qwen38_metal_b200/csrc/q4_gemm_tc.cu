// Prefill affine-Q4 GEMM on the 5th-generation tensor cores (tcgen05 + TMEM), sm_100a.
//
// Replaces the reference's prompt path: qwen38_q4_affine_matmul_simdgroup / _simdgroup_wide
// (shaders/qwen38.metal:3769-3966), and the dequantise-whole-matrix + MPS FP16 GEMM route
// (qwen38_q4_affine_dequantize_f16, shaders/qwen38.metal:4102-4164; src/mps.rs:93-104;
// src/metal_runtime.rs:3897-4047). Arithmetic is that path's: w = 16bit(q*scale + bias), products of
// 16-bit operands, fp32 accumulation -- with bf16 where the reference uses half. No dequantised copy of the
// matrix is ever written to HBM: tiles are expanded in shared memory right before the MMA reads them.
//
// Orientation: the weight tile is the MMA's A operand (128 rows = UMMA M), the activation tile the B operand
// (up to 256 activation rows = UMMA N), so D[n][m] lands in TMEM with one weight row per lane and the epilogue
// writes out[m][n] with the lanes of a warp on consecutive n (coalesced). K advances 64 per stage = one affine
// group, so a producer thread needs one scale and one bias per stage.
//
// Warp roles in a block of 23 warps (one block per SM, persistent over output tiles):
//   warp 0      one thread issues TMA loads of activation tiles (bf16, 128-byte swizzle)
//   warp 1      allocates TMEM; one thread issues tcgen05.mma and commits to mbarriers
//   warps 2-5   epilogue: tcgen05.ld the fp32 accumulators, store to global (two accumulators alternate)
//   warp 6      one thread issues TMA loads of packed weight tiles (128 rows x 128 bytes = four K stages) into a
//               staging ring, when the weights are 16-byte aligned; whole 128-byte lines per row keep DRAM pages
//               and L2 sectors fully used and take the fetch latency off the dequantising warps. Weights at other
//               alignments are fetched by the dequantising threads themselves, a few stages ahead, into registers.
//   warps 7-22  dequantise: packed words (from the staging ring) -> bf16 pairs -> swizzled K-major tile in shared
//               memory; four threads per weight row, two packed words each per stage. Sixteen warps, because a
//               stage's work per warp is a short dependent chain (wait, read, convert, store, fence, arrive) and
//               only other warps can fill its latencies.
// Every wait is bounded: a wait that runs out sets an error flag, the block drains and frees its TMEM.
#include <cuda.h>

#include <cstring>

#include "q4_kernels.h"

#include "q4_device.cuh"

namespace q4 {

constexpr int kProducerWarps = 16;
constexpr int kFirstProducerWarp = 7;
constexpr int kGemmThreads = (kFirstProducerWarp + kProducerWarps) * 32;
constexpr int kTileN = 128;              // weight rows per tile (UMMA M)
constexpr int kTileK = 64;               // inputs per stage: one affine group, 128 bytes of bf16
constexpr uint32_t kThreadsPerRow = kProducerWarps * 32 / kTileN;  // 4
constexpr uint32_t kWordsPerThread = 8 / kThreadsPerRow;        // packed words of a row's stage per thread
static_assert(kThreadsPerRow == 4 && kWordsPerThread == 2, "the producer indexing below assumes four threads per row");
constexpr uint32_t kATileBytes = kTileN * kTileK * 2;  // 16 KB
constexpr uint32_t kSpinLimit = 1u << 24;
// Packed weights are staged in shared memory by TMA, a few K stages of all 128 rows at a time:
//   16-byte aligned tensors: 128-byte rows (four stages), 128-byte swizzle, so the 16-byte reads of a warp spread
//                            over all banks;
//   any other alignment:     the tensor map starts at the address rounded down to 16 bytes and a tile holds an
//                            80-byte window per row (two stages plus the misalignment), unswizzled; readers take
//                            two 16-byte pieces and funnel-shift (the byte-addressed twin of the aligned read).
constexpr uint32_t kWAlignedStages = 4, kWAlignedPitch = 128, kWAlignedBytes = kTileN * kWAlignedPitch;  // 16 KB
constexpr uint32_t kWWindowStages = 2, kWWindowPitch = 80, kWWindowBytes = kTileN * kWWindowPitch;       // 10 KB
constexpr uint32_t kParamPeriod = 8;     // K stages whose scales (or biases) one 16-byte load covers

struct GemmParams {
    const uint8_t *w, *s, *b;  // packed weights, scales, biases (any byte alignment)
    float *out;                // [m][out_stride]
    uint32_t n, m, k;          // weight rows, activation rows, inputs
    uint32_t out_stride;
    uint32_t tiles_n, tiles_m;
    uint32_t w_misalign;       // (uintptr_t)w & 15
    uint32_t accumulate;       // out += result
    // With fewer output tiles than SMs the K range is cut into k_splits parts (each a multiple of eight stages) that
    // different blocks work on; part s writes its partial sums to out + s * split_stride and a second kernel adds the
    // parts in order (same result on every run).
    uint32_t k_splits, split_blocks;  // parts, K stages per part
    uint64_t split_stride;            // floats between the partial outputs of consecutive parts
    int *error_flag;           // set non-zero when a bounded wait runs out
    // Pair mode (fused MLP front half, src/metal_runtime.rs:4267-4474): every work item multiplies the same activation
    // tile with 128 rows of the gate tensor (w, s, b; accumulator 0) and then with the same 128 rows of the up tensor
    // (w2, s2, b2; accumulator 1); the epilogue holds both sums of an element in one thread and stores
    // bf16(silu(gate) * up) (qwen38_swiglu_rows, shaders/qwen38.metal:4188-4198) as h_out[m][h_stride], in the
    // element order of a prepared activation, i.e. ready to be the B operand of the down projection's GEMM.
    const uint8_t *w2, *s2, *b2;
    uint16_t *h_out;
    uint32_t h_stride;
    uint32_t pair;
};

// ---- PTX wrappers ---------------------------------------------------------------------------------

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait. Returns false (and raises the block's abort flag) when the limit is reached or another
// role has already given up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
    for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spin & 255u) == 255u && *abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int32_t x, int32_t y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y)
        : "memory");
}

__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc(uint32_t smem_result, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}

// D[tmem] (+)= A[smem] * B[smem], 128 x N x 16, bf16 inputs, fp32 accumulate
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// arrive on an mbarrier once every MMA issued so far by this thread has completed
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// 32 lanes x 32 consecutive fp32 columns of TMEM -> 32 registers per thread
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
// 32 lanes x 16 consecutive fp32 columns
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major bf16 tile with 128-byte swizzle: rows are 128 bytes, groups
// of 8 rows (1024 bytes) follow each other (stride byte offset 1024), descriptor version 1 (Blackwell).
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t smem_addr) {
    uint64_t d = (uint64_t)((smem_addr & 0x3ffffu) >> 4);
    d |= (uint64_t)1 << 16;            // leading byte offset: unused with swizzled K-major layouts
    d |= (uint64_t)(1024 >> 4) << 32;  // stride byte offset
    d |= (uint64_t)1 << 46;            // descriptor version
    d |= (uint64_t)2 << 61;            // 128-byte swizzle
    return d;
}

// two nibbles -> bf16x2 of q*scale + bias (one rounding): 0x4300|q is bf16 128+q, minus 128 is exact
__device__ __forceinline__ uint32_t dequant_pair(uint32_t v, uint32_t scale2, uint32_t bias2) {
    uint32_t biased = (v & 0x000f000fu) | 0x43004300u, q, out;
    asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(q) : "r"(biased), "r"(0x43004300u));
    asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(out) : "r"(q), "r"(scale2), "r"(bias2));
    return out;
}

// ---- activation preparation: bf16, each block of 8 inputs reordered k0,k4,k1,k5,k2,k6,k3,k7 (the order the
// nibble extraction yields), so weights and activations agree on k inside every MMA ----------------------------
__global__ void __launch_bounds__(256) q4_gemm_prepare_x_kernel(const void *__restrict__ x, int x_is_f32, uint64_t blocks,
                                                               uint16_t *__restrict__ xp) {
    uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= blocks) return;
    uint32_t bits[8];
    if (x_is_f32) {
        const float4 *src = reinterpret_cast<const float4 *>(static_cast<const float *>(x) + i * 8);
        float4 lo = src[0], hi = src[1];
        const float v[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) bits[j] = float_to_bf16_bits(v[j]);
    } else {
        uint4 raw = *reinterpret_cast<const uint4 *>(static_cast<const uint16_t *>(x) + i * 8);
        const uint32_t r[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            bits[2 * j] = r[j] & 0xffffu;
            bits[2 * j + 1] = r[j] >> 16;
        }
    }
    uint4 out;
    out.x = bits[0] | (bits[4] << 16);
    out.y = bits[1] | (bits[5] << 16);
    out.z = bits[2] | (bits[6] << 16);
    out.w = bits[3] | (bits[7] << 16);
    *reinterpret_cast<uint4 *>(xp + i * 8) = out;
}

// ---- the GEMM ------------------------------------------------------------------------------------------------

template <int BN>
struct GemmSmem {
    // more stages where the activation tile is small: a stage's round trip (free -> TMA fetch -> MMA -> free) is
    // set by the fetch latency, whatever the tile size
    static constexpr uint32_t kStages = BN >= 128 ? 4 : (BN == 64 ? 6 : 8);
    static constexpr uint32_t kBTileBytes = BN * kTileK * 2;
    static constexpr uint32_t kStageBytes = kATileBytes + kBTileBytes;
    static constexpr uint32_t kWBufs = BN >= 256 ? 2 : 4;  // staged packed-weight tiles in flight
    static constexpr uint32_t kWStageOffset = kStages * kStageBytes;
    static constexpr uint32_t kWRingBytes = kWBufs * kWAlignedBytes;
    static constexpr uint32_t kWWindowBufs = kWRingBytes / kWWindowBytes;  // 3 or 6 tiles of the window form
    static constexpr uint32_t kBarrierOffset = kWStageOffset + kWRingBytes;
    static constexpr uint32_t kTotal = kBarrierOffset + 384 + 1024;  // barriers + slack for 1024-byte alignment
};

template <int BN>
__global__ void __launch_bounds__(kGemmThreads, 1) q4_gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_x,
                                                                    const __grid_constant__ CUtensorMap tmap_w,
                                                                    const __grid_constant__ CUtensorMap tmap_w2,
                                                                    const __grid_constant__ GemmParams p) {
    extern __shared__ uint8_t gemm_smem_raw[];
    using L = GemmSmem<BN>;
    const uint32_t smem_base = ((uint32_t)__cvta_generic_to_shared(gemm_smem_raw) + 1023u) & ~1023u;
    const uint32_t bars = smem_base + L::kBarrierOffset;
    // barrier slots (8 bytes each): full_x[8] full_w[8] empty[8] acc_full[2] acc_empty[2], the TMEM base and the
    // abort flag, staged_full[6] staged_empty[6]
    constexpr uint32_t kGemmStages = L::kStages;
    auto full_x = [&](uint32_t s) { return bars + 8u * s; };
    auto full_w = [&](uint32_t s) { return bars + 64u + 8u * s; };
    auto empty = [&](uint32_t s) { return bars + 128u + 8u * s; };
    auto acc_full = [&](uint32_t a) { return bars + 192u + 8u * a; };
    auto acc_empty = [&](uint32_t a) { return bars + 208u + 8u * a; };
    auto staged_full = [&](uint32_t b) { return bars + 240u + 8u * b; };
    auto staged_empty = [&](uint32_t b) { return bars + 288u + 8u * b; };
    // geometry of the staged weight tiles for this launch
    const bool windowed = p.w_misalign != 0;
    const uint32_t w_bufs = windowed ? L::kWWindowBufs : L::kWBufs;
    const uint32_t w_stages = windowed ? kWWindowStages : kWAlignedStages;
    const uint32_t w_bytes = windowed ? kWWindowBytes : kWAlignedBytes;
    uint8_t *smem_generic = gemm_smem_raw + (smem_base - (uint32_t)__cvta_generic_to_shared(gemm_smem_raw));
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem_generic + L::kBarrierOffset + 224);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem_generic + L::kBarrierOffset + 232);

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    constexpr uint32_t kTmemCols = 2 * BN < 32 ? 32 : 2 * BN;  // two accumulators; power of two >= 32

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < kGemmStages; ++s) {
            mbar_init(full_x(s), 1);
            mbar_init(full_w(s), kProducerWarps);   // one arrival per producer warp
            mbar_init(empty(s), 1);    // tcgen05.commit
        }
        for (uint32_t a = 0; a < 2; ++a) {
            mbar_init(acc_full(a), 1);
            mbar_init(acc_empty(a), 4);  // one arrival per epilogue warp
        }
        for (uint32_t b = 0; b < 6; ++b) {
            mbar_init(staged_full(b), 1);
            mbar_init(staged_empty(b), kProducerWarps);  // one arrival per producer warp
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc(bars + 224u, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const uint32_t k_blocks_all = p.k / kTileK;
    const uint32_t out_tiles = p.tiles_n * p.tiles_m;
    const uint32_t total_tiles = out_tiles * p.k_splits;  // work items: (K part, output tile), parts outermost
    // K stages [kb_lo, kb_lo + k_blocks) of work item `item`
    auto part_of = [&](uint32_t item) { return item / out_tiles; };
    auto stages_of = [&](uint32_t item) {
        const uint32_t lo = part_of(item) * p.split_blocks;
        return k_blocks_all - lo < p.split_blocks ? k_blocks_all - lo : p.split_blocks;
    };
    const uint32_t subs = p.pair ? 2u : 1u;  // weight tiles per work item (pair mode: gate rows, then the same up rows)

    if (warp == 0) {
        // ---- TMA producer: activation tiles ----
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (uint32_t item = blockIdx.x; item < total_tiles && ok; item += gridDim.x) {
                const uint32_t tile = item % out_tiles, kb_lo = part_of(item) * p.split_blocks, k_blocks = stages_of(item);
                const uint32_t m0 = (tile % p.tiles_m) * BN;
                for (uint32_t kbs = 0; kbs < k_blocks * subs; ++kbs, ++it) {
                    const uint32_t kb = kbs < k_blocks ? kbs : kbs - k_blocks;
                    const uint32_t s = it % kGemmStages, ph = (it / kGemmStages) & 1u;
                    if (!mbar_wait(empty(s), ph ^ 1u, abort_flag)) { ok = false; break; }
                    mbar_expect_tx(full_x(s), L::kBTileBytes);
                    tma_load_2d(smem_base + s * L::kStageBytes + kATileBytes, &tmap_x, full_x(s), (int32_t)((kb_lo + kb) * kTileK), (int32_t)m0);
                }
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer ----
        if (lane == 0) {
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(kTileN >> 4) << 24);
            uint32_t it = 0, tcount = 0;
            bool ok = true;
            for (uint32_t item = blockIdx.x; item < total_tiles && ok; item += gridDim.x, ++tcount) {
                const uint32_t k_blocks = stages_of(item);
                // one accumulator per work item, two alternating; in pair mode an item takes both (gate, up) and
                // the barriers of accumulator 0 stand for the pair
                const uint32_t acc = p.pair ? 0u : (tcount & 1u), aph = p.pair ? (tcount & 1u) : ((tcount >> 1) & 1u);
                if (!mbar_wait(acc_empty(acc), aph ^ 1u, abort_flag)) { ok = false; break; }
                tc_fence_after();
                for (uint32_t kbs = 0; kbs < k_blocks * subs; ++kbs, ++it) {
                    const uint32_t sub = kbs < k_blocks ? 0u : 1u, kb = kbs - sub * k_blocks;
                    const uint32_t d_tmem = tmem_base + (acc + sub) * BN;
                    const uint32_t s = it % kGemmStages, ph = (it / kGemmStages) & 1u;
                    if (!mbar_wait(full_x(s), ph, abort_flag) || !mbar_wait(full_w(s), ph, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = smem_base + s * L::kStageBytes, b_addr = a_addr + kATileBytes;
                    const uint64_t adesc = smem_desc_sw128(a_addr), bdesc = smem_desc_sw128(b_addr);
#pragma unroll
                    for (uint32_t k16 = 0; k16 < kTileK / 16; ++k16) {
                        // 16 inputs = 32 bytes further along K inside the 128-byte rows: +2 in 16-byte units
                        umma_bf16(d_tmem, adesc + 2u * k16, bdesc + 2u * k16, idesc, (kb | k16) != 0 ? 1u : 0u);
                    }
                    umma_commit(empty(s));  // frees the stage once these MMAs have read it
                }
                if (ok) umma_commit(acc_full(acc));
            }
        }
    } else if (warp == 6) {
        // ---- TMA producer: packed weight tiles ----
        if (lane == 0) {
            uint32_t wb = 0, ph = 0;
            bool ok = true;
            for (uint32_t item = blockIdx.x; item < total_tiles && ok; item += gridDim.x) {
                const uint32_t tile = item % out_tiles, kb_lo = part_of(item) * p.split_blocks;
                const uint32_t w_tiles = (stages_of(item) + w_stages - 1) / w_stages;
                const uint32_t n0 = (tile / p.tiles_m) * kTileN;
                for (uint32_t wts = 0; wts < w_tiles * subs && ok; ++wts) {
                    const uint32_t sub = wts < w_tiles ? 0u : 1u, wt = wts - sub * w_tiles;
                    if (!mbar_wait(staged_empty(wb), ph ^ 1u, abort_flag)) { ok = false; break; }
                    mbar_expect_tx(staged_full(wb), w_bytes);
                    // x is a byte offset from the (rounded-down) tensor base: a multiple of 16 in both forms
                    tma_load_2d(smem_base + L::kWStageOffset + wb * w_bytes, sub ? &tmap_w2 : &tmap_w, staged_full(wb),
                                (int32_t)((kb_lo + wt * w_stages) * 32u), (int32_t)n0);
                    if (++wb == w_bufs) {
                        wb = 0;
                        ph ^= 1u;
                    }
                }
            }
        }
    } else if (warp < 6) {
        // ---- epilogue: TMEM -> registers -> global ----
        const uint32_t quarter = warp & 3u;  // a warp may touch TMEM lanes 32*(warp%4) .. +31
        uint32_t tcount = 0;
        bool ok = true;
        for (uint32_t item = blockIdx.x; item < total_tiles && ok; item += gridDim.x, ++tcount) {
            const uint32_t tile = item % out_tiles;
            float *const out = p.out + (uint64_t)part_of(item) * p.split_stride;
            const uint32_t acc = p.pair ? 0u : (tcount & 1u), aph = p.pair ? (tcount & 1u) : ((tcount >> 1) & 1u);
            const uint32_t n0 = (tile / p.tiles_m) * kTileN, m0 = (tile % p.tiles_m) * BN;
            if (!mbar_wait(acc_full(acc), aph, abort_flag)) { ok = false; break; }
            tc_fence_after();
            const uint32_t n = n0 + quarter * 32u + lane;
            if (p.pair) {
                // gate sums in accumulator 0, up sums in accumulator 1, the same lane (row) and column (activation row):
                // h = bf16(silu(gate) * up), stored where the down projection's GEMM expects input n of activation row m
                // (inside each block of 8 inputs the order is k0,k4,k1,k5,k2,k6,k3,k7)
                const uint32_t pos = (n & ~7u) | ((n & 3u) << 1) | ((n >> 2) & 1u);
#pragma unroll 1
                for (uint32_t c0 = 0; c0 < BN; c0 += 16) {
                    uint32_t r[16], u[16];
                    tmem_ld_32x16(tmem_base + ((quarter * 32u) << 16) + c0, r);
                    tmem_ld_32x16(tmem_base + ((quarter * 32u) << 16) + BN + c0, u);
                    tmem_ld_wait();
                    if (n < p.n) {
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const uint32_t m = m0 + c0 + i;
                            if (m < p.m) {
                                // hardware exponential and reciprocal (as Metal's fast math in the reference's kernel):
                                // their error is far below the bf16 rounding that follows, and this epilogue runs
                                // while the tensor cores wait for the accumulators
                                const float g = __uint_as_float(r[i]);
                                const float h = __fdividef(g, 1.0f + __expf(-g)) * __uint_as_float(u[i]);
                                p.h_out[(uint64_t)m * p.h_stride + pos] = (uint16_t)float_to_bf16_bits(h);
                            }
                        }
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(acc_empty(acc));
                continue;
            }
#pragma unroll 1
            for (uint32_t c0 = 0; c0 < BN; c0 += 32) {
                uint32_t r[32];
                tmem_ld_32x32(tmem_base + ((quarter * 32u) << 16) + acc * BN + c0, r);
                tmem_ld_wait();
                if (n < p.n) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const uint32_t m = m0 + c0 + i;
                        if (m < p.m) {
                            float *dst = out + (uint64_t)m * p.out_stride + n;
                            float v = __uint_as_float(r[i]);
                            if (p.accumulate) v += *dst;
                            *dst = v;
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty(acc));
        }
    } else {
        // ---- dequantise producers: 512 threads, four per weight row, two packed words each ----
        const uint32_t pid = threadIdx.x - kFirstProducerWarp * 32;
        const uint32_t row = pid >> 2, part = pid & 3u;
        const uint32_t groups = p.k / 64;
        uint32_t s = 0, ph = 0;      // stage ring position
        uint32_t wb = 0, wph = 0;    // staging ring position
        bool ok = true;
        for (uint32_t item = blockIdx.x; item < total_tiles && ok; item += gridDim.x) {
            const uint32_t tile = item % out_tiles, kb_lo = part_of(item) * p.split_blocks, k_blocks = stages_of(item);
            const uint32_t n0 = (tile / p.tiles_m) * kTileN;
            uint32_t grow = n0 + row;
            grow = grow < p.n ? grow : p.n - 1u;  // rows past N take a valid row's parameters and are never stored
            for (uint32_t sub = 0; sub < subs && ok; ++sub) {
            const uint8_t *srow = (sub ? p.s2 : p.s) + ((uint64_t)grow * groups + kb_lo) * 2u, *brow = (sub ? p.b2 : p.b) + ((uint64_t)grow * groups + kb_lo) * 2u;
            // Scales and biases of eight stages come in one 16-byte load each (any byte alignment), one period ahead,
            // so that no load is waited for in the stage loop.
            auto params = [&](const uint8_t *base, uint32_t kb) {
                const uint8_t *q = base + 2u * kb;
                return ldg_stream_v4_unaligned(q, (uint32_t)(reinterpret_cast<uintptr_t>(q) & 15u));
            };
            uint4 sc_next = params(srow, 0), bi_next = params(brow, 0);
            for (uint32_t kb0 = 0; kb0 < k_blocks && ok; kb0 += kParamPeriod) {
                const uint4 sc8 = sc_next, bi8 = bi_next;
                if (kb0 + kParamPeriod < k_blocks) {
                    sc_next = params(srow, kb0 + kParamPeriod);
                    bi_next = params(brow, kb0 + kParamPeriod);
                }
                const uint32_t scw[4] = {sc8.x, sc8.y, sc8.z, sc8.w}, biw[4] = {bi8.x, bi8.y, bi8.z, bi8.w};
#pragma unroll
                for (uint32_t j = 0; j < kParamPeriod; ++j) {
                    const uint32_t kb = kb0 + j;
                    if (kb >= k_blocks) break;
                    const uint32_t jj = windowed ? (j % kWWindowStages) : (j % kWAlignedStages);  // stage inside the staged tile
                    if (jj == 0 && !mbar_wait(staged_full(wb), wph, abort_flag)) { ok = false; break; }
                    const uint32_t staged = smem_base + L::kWStageOffset + wb * w_bytes;
                    uint32_t words[kWordsPerThread];  // this thread's 8 bytes: 16 of the row's 64 weights
                    if (!windowed) {
                        const uint32_t chunk = 2u * jj + (part >> 1);
                        const uint2 v = lds_v2(staged + row * kWAlignedPitch + ((chunk ^ (row & 7u)) << 4) + (part & 1u) * 8u);
                        words[0] = v.x;
                        words[1] = v.y;
                    } else {
                        const uint32_t at = staged + row * kWWindowPitch + jj * 32u + (part >> 1) * 16u;
                        const uint4 v = realign_16(lds_v4(at), lds_v4(at + 16u), p.w_misalign);
                        words[0] = (part & 1u) ? v.z : v.x;
                        words[1] = (part & 1u) ? v.w : v.y;
                    }
                    // both halves of the register get the stage's bf16 parameter
                    const uint32_t sel = (j & 1u) ? 0x3232u : 0x1010u;
                    const uint32_t sc = __byte_perm(scw[j >> 1], 0u, sel), bi = __byte_perm(biw[j >> 1], 0u, sel);
                    if (!mbar_wait(empty(s), ph ^ 1u, abort_flag)) { ok = false; break; }
                    const uint32_t a_row = smem_base + s * L::kStageBytes + row * 128u;
#pragma unroll
                    for (uint32_t wi = 0; wi < kWordsPerThread; ++wi) {
                        const uint32_t wv = words[wi];
                        const uint32_t o0 = dequant_pair(wv, sc, bi), o1 = dequant_pair(wv >> 4, sc, bi);
                        const uint32_t o2 = dequant_pair(wv >> 8, sc, bi), o3 = dequant_pair(wv >> 12, sc, bi);
                        const uint32_t chunk = part * kWordsPerThread + wi;  // 16-byte piece of the 128-byte row
                        const uint32_t dst = a_row + ((chunk ^ (row & 7u)) << 4);  // 128-byte swizzle
                        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dst), "r"(o0), "r"(o1), "r"(o2), "r"(o3) : "memory");
                    }
                    fence_async_smem();  // the tensor core reads shared memory through the async proxy
                    __syncwarp();
                    if (lane == 0) mbar_arrive(full_w(s));
                    if (++s == kGemmStages) {
                        s = 0;
                        ph ^= 1u;
                    }
                    if (jj == w_stages - 1u || kb + 1u == k_blocks) {
                        // the warp's reads of the staged tile are complete (their values were consumed above)
                        if (lane == 0) mbar_arrive(staged_empty(wb));
                        if (++wb == w_bufs) {
                            wb = 0;
                            wph ^= 1u;
                        }
                    }
                }
            }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
    if (threadIdx.x == 0 && *abort_flag && p.error_flag) *p.error_flag = 1;
}

// out[m][n] (+)= part[0][m][n] + part[1][m][n] + ... in that order (the second step of a launch cut along K)
__global__ void __launch_bounds__(256) q4_gemm_sum_parts_kernel(const float *__restrict__ parts, uint64_t split_stride, uint32_t k_splits,
                                                               uint64_t elements, float *__restrict__ out, int accumulate) {
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= elements) return;
    float acc = accumulate ? out[i] : 0.f;
    for (uint32_t s = 0; s < k_splits; ++s) acc += __ldcg(parts + (uint64_t)s * split_stride + i);
    out[i] = acc;
}

}  // namespace q4

// ---------------------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------------------

extern "C" cudaError_t q4k_gemm_prepare_x(const void *x, int x_is_f32, uint64_t elements, uint16_t *xp, cudaStream_t stream) {
    const uint64_t blocks = elements / 8;
    q4::q4_gemm_prepare_x_kernel<<<(uint32_t)((blocks + 255) / 256), 256, 0, stream>>>(x, x_is_f32, blocks, xp);
    return cudaGetLastError();
}

namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
    return fn;
}

template <int BN>
cudaError_t launch_gemm(const CUtensorMap &map, const CUtensorMap &wmap, const CUtensorMap &wmap2, const q4::GemmParams &p, uint32_t ctas,
                        cudaStream_t stream) {
    cudaError_t e = cudaFuncSetAttribute(q4::q4_gemm_tc_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)q4::GemmSmem<BN>::kTotal);
    if (e != cudaSuccess) return e;
    q4::q4_gemm_tc_kernel<BN><<<ctas, q4::kGemmThreads, q4::GemmSmem<BN>::kTotal, stream>>>(map, wmap, wmap2, p);
    return cudaGetLastError();
}

}  // namespace

// activation rows per tile the kernel would use for m rows
extern "C" uint32_t q4k_gemm_tile_m(uint32_t m) {
    if (m > 128) return 256;
    if (m > 64) return 128;
    if (m > 32) return 64;
    if (m > 16) return 32;
    return 16;
}

// How many parts the K range of an m x n x k projection is cut into (1: not cut), every part at least 32 stages long
// and a multiple of eight stages. Two cases: the output tiles fill less than half of the SMs (as many parts as fit), or
// the last of several rounds of tiles would leave many SMs idle (2 to 4 parts, the fewest that bring the rounds to
// 85 % occupancy; the extra pass over the partial outputs costs less than the idle round).
extern "C" uint32_t q4k_gemm_k_splits(uint32_t m, uint32_t n, uint32_t k, uint32_t sm_count, uint32_t *split_blocks) {
    const uint32_t bn = q4k_gemm_tile_m(m);
    const uint32_t tiles = ((n + q4::kTileN - 1) / q4::kTileN) * ((m + bn - 1) / bn);
    const uint32_t k_blocks = k / q4::kTileK;
    const uint32_t longest = k_blocks / 32;  // most parts the K range allows
    uint32_t splits = 1;
    if (tiles * 2 <= sm_count) {
        splits = sm_count / tiles;
    } else {
        auto fill = [&](uint32_t s) {
            const uint32_t items = tiles * s, rounds = (items + sm_count - 1) / sm_count;
            return (double)items / ((double)rounds * sm_count);
        };
        if (fill(1) < 0.85) {
            double best = fill(1);
            for (uint32_t s = 2; s <= 4 && s <= longest; ++s) {
                if (fill(s) > best + 0.05) {
                    best = fill(s);
                    splits = s;
                    if (best >= 0.85) break;
                }
            }
        }
    }
    if (splits > longest) splits = longest;
    if (splits < 2) {
        *split_blocks = k_blocks;
        return 1;
    }
    const uint32_t per = ((k_blocks + splits - 1) / splits + 7u) & ~7u;
    *split_blocks = per;
    return (k_blocks + per - 1) / per;
}

namespace {

// packed weights as a byte matrix [n][k/2] from the tensor's address rounded down to 16 bytes (TMA needs that;
// the row pitch k/2 is a multiple of 32): 128-byte swizzled rows when the tensor is aligned, 80-byte windows else.
// The matrix is declared 16 bytes wider than k/2 in the window form so the last window of a row is in range; the
// extra bytes are the next row's first bytes or, after the last row, the padding every shard carries.
bool encode_weight_map(EncodeTiledFn encode, CUtensorMap *wmap, const uint8_t *w, uint32_t n, uint32_t k) {
    const uint32_t w_mis = (uint32_t)((uintptr_t)w & 15u);
    const cuuint64_t wdims[2] = {(cuuint64_t)k / 2 + (w_mis ? 16u : 0u), n};
    const cuuint64_t wstrides[1] = {(cuuint64_t)k / 2};
    const cuuint32_t wbox[2] = {w_mis ? q4::kWWindowPitch : q4::kWAlignedPitch, (cuuint32_t)q4::kTileN};
    const cuuint32_t estr[2] = {1, 1};
    return encode(wmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t *>(w - w_mis), wdims, wstrides, wbox, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, w_mis ? CU_TENSOR_MAP_SWIZZLE_NONE : CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool encode_activation_map(EncodeTiledFn encode, CUtensorMap *map, const uint16_t *xp, uint32_t m, uint32_t k, uint32_t bn) {
    const cuuint64_t dims[2] = {k, m};
    const cuuint64_t strides[1] = {(cuuint64_t)k * 2};
    const cuuint32_t box[2] = {(cuuint32_t)q4::kTileK, bn};
    const cuuint32_t estr[2] = {1, 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<uint16_t *>(xp), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

cudaError_t launch_by_tile(uint32_t bn, const CUtensorMap &map, const CUtensorMap &wmap, const CUtensorMap &wmap2, const q4::GemmParams &p,
                           uint32_t ctas, cudaStream_t stream) {
    switch (bn) {
        case 256: return launch_gemm<256>(map, wmap, wmap2, p, ctas, stream);
        case 128: return launch_gemm<128>(map, wmap, wmap2, p, ctas, stream);
        case 64: return launch_gemm<64>(map, wmap, wmap2, p, ctas, stream);
        case 32: return launch_gemm<32>(map, wmap, wmap2, p, ctas, stream);
        default: return launch_gemm<16>(map, wmap, wmap2, p, ctas, stream);
    }
}

}  // namespace

// xp: prepared activations [m][k] bf16 (q4k_gemm_prepare_x), 16-byte aligned. One projection per launch. `parts`:
// scratch for m * out_stride * q4k_gemm_k_splits(...) floats when that is more than one, else unused.
extern "C" cudaError_t q4k_gemm_tc(const uint16_t *xp, uint32_t m, uint32_t k, const uint8_t *w, const uint8_t *s, const uint8_t *b,
                                   uint32_t n, float *out, uint32_t out_stride, int accumulate, int *error_flag, uint32_t sm_count,
                                   float *parts, cudaStream_t stream) {
    EncodeTiledFn encode = encode_tiled_fn();
    if (!encode) return cudaErrorNotSupported;
    const uint32_t bn = q4k_gemm_tile_m(m);
    CUtensorMap map, wmap;
    if (!encode_activation_map(encode, &map, xp, m, k, bn) || !encode_weight_map(encode, &wmap, w, n, k)) return cudaErrorInvalidValue;
    q4::GemmParams p;
    memset(&p, 0, sizeof p);
    p.w = w;
    p.s = s;
    p.b = b;
    p.out = out;
    p.n = n;
    p.m = m;
    p.k = k;
    p.out_stride = out_stride;
    p.tiles_n = (n + q4::kTileN - 1) / q4::kTileN;
    p.tiles_m = (m + bn - 1) / bn;
    p.w_misalign = (uint32_t)((uintptr_t)w & 15u);
    p.accumulate = accumulate ? 1u : 0u;
    p.error_flag = error_flag;
    p.k_splits = q4k_gemm_k_splits(m, n, k, sm_count, &p.split_blocks);
    p.split_stride = 0;
    if (p.k_splits > 1) {
        if (!parts) return cudaErrorInvalidValue;
        p.out = parts;
        p.out_stride = out_stride;
        p.split_stride = (uint64_t)m * out_stride;
        p.accumulate = 0;
    }
    const uint32_t tiles = p.tiles_n * p.tiles_m * p.k_splits;
    const uint32_t ctas = tiles < sm_count ? tiles : sm_count;
    const cudaError_t launched = launch_by_tile(bn, map, wmap, wmap, p, ctas, stream);
    if (launched != cudaSuccess || p.k_splits == 1) return launched;
    const uint64_t elements = (uint64_t)m * out_stride;
    q4::q4_gemm_sum_parts_kernel<<<(uint32_t)((elements + 255) / 256), 256, 0, stream>>>(parts, p.split_stride, p.k_splits, elements, out,
                                                                                  accumulate ? 1 : 0);
    return cudaGetLastError();
}

// 1 when the gate and up tensors can share one pair launch: the staged weight tiles of a launch have one geometry, so
// both tensors must sit at the same offset from a 16-byte boundary
extern "C" int q4k_gemm_pair_supported(const uint8_t *w_gate, const uint8_t *w_up) {
    return (((uintptr_t)w_gate ^ (uintptr_t)w_up) & 15u) == 0 ? 1 : 0;
}

// Fused front half of the MLP: h[m][n] = bf16(silu(x gate^T) * (x up^T)) in one launch, written as the prepared
// activation of the down projection (h_stride elements between activation rows, 16-byte aligned rows).
extern "C" cudaError_t q4k_gemm_tc_pair(const uint16_t *xp, uint32_t m, uint32_t k, const uint8_t *wg, const uint8_t *sg, const uint8_t *bg,
                                        const uint8_t *wu, const uint8_t *su, const uint8_t *bu, uint32_t n, uint16_t *h_out,
                                        uint32_t h_stride, int *error_flag, uint32_t sm_count, cudaStream_t stream) {
    EncodeTiledFn encode = encode_tiled_fn();
    if (!encode) return cudaErrorNotSupported;
    if (!q4k_gemm_pair_supported(wg, wu)) return cudaErrorNotSupported;
    const uint32_t bn = q4k_gemm_tile_m(m);
    CUtensorMap map, wmap, wmap2;
    if (!encode_activation_map(encode, &map, xp, m, k, bn) || !encode_weight_map(encode, &wmap, wg, n, k) ||
        !encode_weight_map(encode, &wmap2, wu, n, k))
        return cudaErrorInvalidValue;
    q4::GemmParams p;
    memset(&p, 0, sizeof p);
    p.w = wg;
    p.s = sg;
    p.b = bg;
    p.w2 = wu;
    p.s2 = su;
    p.b2 = bu;
    p.h_out = h_out;
    p.h_stride = h_stride;
    p.pair = 1;
    p.n = n;
    p.m = m;
    p.k = k;
    p.tiles_n = (n + q4::kTileN - 1) / q4::kTileN;
    p.tiles_m = (m + bn - 1) / bn;
    p.w_misalign = (uint32_t)((uintptr_t)wg & 15u);
    p.error_flag = error_flag;
    p.k_splits = 1;
    p.split_blocks = k / q4::kTileK;
    const uint32_t tiles = p.tiles_n * p.tiles_m;
    return launch_by_tile(bn, map, wmap, wmap2, p, tiles < sm_count ? tiles : sm_count, stream);
}
