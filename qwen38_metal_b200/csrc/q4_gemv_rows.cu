// Short batches (2..16 activation rows) of MLX affine-Q4 projections on the integer tensor-core path: the shape of the
// reference's batched kernels (qwen38_q4_affine_matvec_batch2/4/8, shaders/qwen38.metal:213-246 applied per row),
// HBM-bound on B200 because every packed weight is read once for all rows.
//
// Arithmetic. Every activation row is held as 23-bit fixed point after an exact power-of-two scaling,
// x' = d0 + 256 d1 + 65536 d2 with signed 8-bit digits. A packed weight word becomes two byte registers (even and odd
// nibbles) and is the A operand of mma.sync.m16n8k32.s32.u8.s8 as it is; the B operand holds one digit of eight
// activation rows, so one MMA returns, for 16 weight rows and 8 activation rows, the exact integer sum of
// q * digit over 32 inputs. An affine group (64 inputs) is two MMAs per digit; its three integer sums are
// put together (q0 + 256 q1 + 65536 q2, the group's exact integer dot product, rounded to fp32 once) and scaled with the
// group's bf16 scale in fp32; the bias term is bias * (sum of x' over the group). Products and group sums are exact; the
// approximations are the fixed-point step of the activation and fp32 rounding of the per-group terms, as in the reference.
//
// Work. The K range is cut into `parts` runs of 128-input chunks. A block holds the digits of ONE part for all rows
// in shared memory (converted by the block itself from the caller's bf16 or fp32 rows; the power-of-two scale is the
// part's own and is undone, exactly, before partial sums of different parts meet) and its 16 warps walk 16-row tiles
// of that part, each with a private ring of eight 1 KB cp.async stages. Partial sums go to scratch; the LAST part to
// finish a tile (one counter per tile, put back to zero by that warp) adds all parts in part order -- the result does
// not depend on which part came last -- and stores the tile. No block ever waits for another one.
#include "q4_decomp.h"
#include "q4_device.cuh"
#include "q4_kernels.h"

namespace q4 {

constexpr int kRowsWarps = 16;
constexpr int kRowsStageBytes = 1024;  // one chunk of one tile: 16 weight rows x 64 packed bytes
constexpr int kRowsPerThread = 8;      // blocks of 8 inputs a thread converts at most (bounds a part: rows x chunks <= 256)

// A warp walks TW tiles at a time (1 or 2): with two, the B fragments (activation digits) are read from shared memory
// once for 32 weight rows. The ring of a warp is 8 KB either way: 8 stages of one chunk, or 4 stages of a chunk of both
// tiles. Scales and biases travel per four chunks (16 rows x 2 arrays x 16 bytes per tile): three such stages cover
// the 7 chunks a one-tile warp is ahead, two the 3 chunks of a two-tile warp.
__host__ __device__ constexpr uint32_t rows_stages(uint32_t tw) { return 8u / tw; }
__host__ __device__ constexpr uint32_t rows_param_stages(uint32_t tw) { return tw == 1u ? 3u : 2u; }
__host__ __device__ constexpr uint32_t rows_ring_bytes(uint32_t tw) { return 8u * kRowsStageBytes + rows_param_stages(tw) * 512u * tw; }

// Shared memory of one chunk's digits: [group 2][digit 3][activation row MP][64 bytes]. The 64 bytes of a (group, digit,
// row) hold the 64 inputs of the group in the order lane t of a quad wants them as B registers of the group's two MMAs:
// byte 16 t + 8 j + 4 odd + i  <->  input 16 t + 8 j + 2 i + odd   (t: quad lane, j: MMA of the group, i: byte).
__host__ __device__ constexpr uint32_t rows_chunk_bytes(uint32_t mp) { return 2u * 3u * mp * 64u; }

__host__ __device__ inline size_t rows_smem_bytes(uint32_t mp, uint32_t part_chunks, uint32_t tw) {
    return (size_t)kRowsWarps * rows_ring_bytes(tw) + (size_t)part_chunks * rows_chunk_bytes(mp) +
           (size_t)part_chunks * 2u * mp * 4u + 2u * mp * 4u + 64u;
}

__device__ __forceinline__ unsigned long long rows_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

template <int NB, int TW>
__global__ void __launch_bounds__(kRowsWarps * 32, 1) q4_rows_kernel(const __grid_constant__ RowsParams p) {
    constexpr uint32_t MP = 8 * NB;
    constexpr uint32_t T = kRowsWarps * 32;
    constexpr uint32_t S = rows_stages(TW), PS = rows_param_stages(TW);
    constexpr uint32_t kStage = kRowsStageBytes * TW, kParamStage = 512u * TW;
    // stages requested before the activation is converted, the rest right after (measured: one is best up to 8 rows,
    // all of them for 16, whose conversion is twice as long)
    constexpr uint32_t kEarly = NB == 1 ? 1u : S - 1u;
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const uint32_t g = lane >> 2, t = lane & 3u;
    const uint32_t part = blockIdx.x % p.parts, gi = blockIdx.x / p.parts, blocks_per_part = gridDim.x / p.parts;
    // parts begin at multiples of four chunks (K % 512 == 0): parameters are copied in 16-byte pieces of eight groups
    const uint32_t c_lo = q4_rows_part_begin(p.cpt, p.parts, part), c_hi = q4_rows_part_begin(p.cpt, p.parts, part + 1u), nch = c_hi - c_lo;
    uint8_t *xdig = smem + kRowsWarps * rows_ring_bytes(TW);
    float *xsum = reinterpret_cast<float *>(xdig + (size_t)p.part_chunks * rows_chunk_bytes(MP));
    uint32_t *amax_s = reinterpret_cast<uint32_t *>(xsum + (size_t)p.part_chunks * 2u * MP);
    float *inv_s = reinterpret_cast<float *>(amax_s + MP);
    const uint32_t ring = (uint32_t)__cvta_generic_to_shared(smem) + warp * rows_ring_bytes(TW);
    const uint32_t pring = ring + S * kStage;

    // ---- an item's weights (TW tiles): lane l copies 16 bytes of row l >> 2 (and of the row eight further down) per
    // chunk and tile. The four 16-byte quarters of a row are stored with quarter q at q ^ (2 * bit 1 of the row), so
    // that the 8-byte reads below (lane (g, t): bytes 8 t.. of a group) touch every bank once per half-warp.
    const uint32_t cr = lane >> 2, cq = lane & 3u;
    const uint32_t copy_off = 16u * (cr * 4u + (cq ^ (2u * ((cr >> 1) & 1u))));
    const uint64_t row_bytes = (uint64_t)p.k >> 1;
    const uint8_t *wa[TW], *wb[TW], *pw[TW];
    const RowsJob *job[TW];
    uint32_t row0[TW];
    bool tile_live[TW];
#pragma unroll
    for (int w = 0; w < TW; ++w) {
        wa[w] = wb[w] = pw[w] = nullptr;
        job[w] = nullptr;
        row0[w] = 0;
        tile_live[w] = false;
    }
    // chunks are requested in order: wa, wb and pw walk along with the next chunk to request
    auto issue_chunk = [&](uint32_t c) {  // chunk c of the part (absolute index), into its ring stage
        const uint32_t rel = c - c_lo;
        const uint32_t stage = ring + (rel % S) * kStage;
        const bool pred = c < c_hi;
#pragma unroll
        for (int w = 0; w < TW; ++w) {
            cp_async_16_pred(stage + w * kRowsStageBytes + copy_off, wa[w], pred);
            cp_async_16_pred(stage + w * kRowsStageBytes + 512u + copy_off, wb[w], pred);
            wa[w] += 64;
            wb[w] += 64;
        }
        // every fourth chunk: lane l copies the scales (l < 16) or biases of row l & 15 for the next eight groups
        if ((rel & 3u) == 0) {
#pragma unroll
            for (int w = 0; w < TW; ++w) {
                cp_async_16_pred(pring + ((rel >> 2) % PS) * kParamStage + w * 512u + lane * 16u, pw[w], pred);
                pw[w] += 16;
            }
        }
    };
    // item i of a part = tiles TW * i .. TW * i + TW - 1 (a tile past the last one repeats the last: computed, never stored)
    const uint32_t items = (p.tiles + TW - 1) / TW;
    auto open_item = [&](uint32_t it) {
#pragma unroll
        for (int w = 0; w < TW; ++w) {
            const uint32_t want = it * TW + w;
            tile_live[w] = want < p.tiles;
            const uint32_t tile = tile_live[w] ? want : p.tiles - 1u;
            uint32_t ji = 0;
            while (ji + 1 < p.n_jobs && tile >= p.jobs[ji + 1].tile_begin) ++ji;
            job[w] = &p.jobs[ji];
            row0[w] = (tile - job[w]->tile_begin) * 16u;
            const uint32_t n = job[w]->n;
            const uint32_t ra = min(row0[w] + cr, n - 1u), rb = min(row0[w] + 8u + cr, n - 1u);  // rows past n: read a valid row
            wa[w] = job[w]->w + (uint64_t)ra * row_bytes + cq * 16u + (size_t)c_lo * 64u;
            wb[w] = job[w]->w + (uint64_t)rb * row_bytes + cq * 16u + (size_t)c_lo * 64u;
            const uint32_t rp = min(row0[w] + (lane & 15u), n - 1u);
            pw[w] = ((lane >> 4) ? job[w]->b : job[w]->s) + ((size_t)rp * p.groups) * 2u + (size_t)c_lo * 4u;
        }
    };
    auto prologue = [&](uint32_t first, uint32_t end) {  // the chunks [first, end) of the S - 1 a warp is ahead
#pragma unroll
        for (uint32_t i = 0; i < S - 1; ++i) {
            if (i < first || i >= end) continue;
            issue_chunk(c_lo + i);
            cp_async_commit();
        }
    };
    unsigned long long *tr = (p.trace && lane == 0) ? p.trace + ((size_t)blockIdx.x * kRowsWarps + warp) * 4 : nullptr;
    if (tr) tr[0] = rows_ns();
    bool first_tile = true;
    uint32_t item = gi * kRowsWarps + warp;

    // ---- the part's digits for every row ----
    const uint32_t span8 = nch * 16u;  // blocks of 8 inputs per row in this part
    if (threadIdx.x < MP) amax_s[threadIdx.x] = 0;
    __syncthreads();
    // Every thread holds its blocks of 8 inputs (at most kRowsPerThread) in registers between the maximum and the
    // conversion, and all of its loads are in flight at once: one round trip to L2 instead of one per block.
    uint4 raw[kRowsPerThread][2];
    const uint32_t total8 = p.m * span8, padded8 = MP * span8;  // rows past m are zero-filled
#pragma unroll
    for (int i = 0; i < kRowsPerThread; ++i) {
        const uint32_t idx = threadIdx.x + i * T;
        raw[i][0] = raw[i][1] = make_uint4(0, 0, 0, 0);
        if (idx < total8) {
            const uint32_t mrow = idx / span8, b8 = idx - mrow * span8;
            const size_t at = (size_t)mrow * p.k + (size_t)c_lo * 128u + (size_t)b8 * 8u;
            if (p.x_is_f32) {
                const uint4 *src = reinterpret_cast<const uint4 *>(static_cast<const float *>(p.x) + at);
                raw[i][0] = __ldg(src);
                raw[i][1] = __ldg(src + 1);
            } else {
                raw[i][0] = __ldg(reinterpret_cast<const uint4 *>(static_cast<const uint16_t *>(p.x) + at));
            }
        }
    }
    // the first weights travel while the block converts the activation -- requested once every warp of the block has
    // its activation loads out: those would otherwise queue behind 7 KB of copies per warp
    __syncthreads();
    if (item < items) {
        open_item(item);
        prologue(0, kEarly);
    }
    auto unpack8 = [&](const uint4 (&r)[2], float (&v)[8]) {
        if (p.x_is_f32) {
            v[0] = __uint_as_float(r[0].x); v[1] = __uint_as_float(r[0].y); v[2] = __uint_as_float(r[0].z); v[3] = __uint_as_float(r[0].w);
            v[4] = __uint_as_float(r[1].x); v[5] = __uint_as_float(r[1].y); v[6] = __uint_as_float(r[1].z); v[7] = __uint_as_float(r[1].w);
        } else {
            const uint32_t w[4] = {r[0].x, r[0].y, r[0].z, r[0].w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                v[2 * j] = bf16_bits_to_float(w[j] & 0xffffu);
                v[2 * j + 1] = bf16_bits_to_float(w[j] >> 16);
            }
        }
    };
    // (span8 is a multiple of 16, so the 16 lanes of a half-warp always look at the same row: one atomic per half-warp)
#pragma unroll
    for (int i = 0; i < kRowsPerThread; ++i) {
        if ((uint32_t)i * T >= total8) continue;  // (uniform)
        const uint32_t idx = threadIdx.x + i * T;
        float v[8];
        unpack8(raw[i], v);
        uint32_t mx = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) mx = max(mx, __float_as_uint(v[j]) & 0x7fffffffu);
#pragma unroll
        for (int off = 8; off > 0; off >>= 1) mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, off));
        if ((lane & 15u) == 0 && idx < total8) atomicMax(&amax_s[idx / span8], mx);
    }
    __syncthreads();
    if (threadIdx.x < MP) {
        const int e = scale_exponent(amax_s[threadIdx.x]);
        inv_s[threadIdx.x] = __uint_as_float((uint32_t)(127 - e) << 23);
    }
#pragma unroll
    for (int i = 0; i < kRowsPerThread; ++i) {
        if ((uint32_t)i * T >= padded8) continue;  // (uniform)
        const uint32_t idx = threadIdx.x + i * T;
        const bool live = idx < padded8;
        const uint32_t mrow = live ? idx / span8 : 0u, b8 = live ? idx - mrow * span8 : 0u;
        if (mrow >= p.m) {
            // (uniform per warp: a row's blocks are a multiple of 64) rows past m hold zeros
            if (live) {
                const uint32_t chunk = b8 >> 4, grp = (b8 >> 3) & 1u, b = b8 & 7u;
                uint8_t *dst = xdig + (size_t)chunk * rows_chunk_bytes(MP) + (size_t)grp * 3u * MP * 64u + (size_t)mrow * 64u + 16u * (b >> 1) + 8u * (b & 1u);
#pragma unroll
                for (int d = 0; d < 3; ++d) *reinterpret_cast<uint2 *>(dst + (size_t)d * MP * 64u) = make_uint2(0u, 0u);
                if (b == 0) xsum[(chunk * 2u + grp) * MP + mrow] = 0.f;
            }
            continue;
        }
        float v[8];
        unpack8(raw[i], v);
        const float scale = __uint_as_float((uint32_t)(scale_exponent(amax_s[mrow]) + 127) << 23);
        int sum = 0;
        uint32_t z[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int xi = __float2int_rn(v[j] * scale);
            sum += xi;
            z[j] = ((uint32_t)xi + 0x00808080u) ^ 0x00808080u;  // bytes 0..2: the signed digits
        }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        sum += __shfl_xor_sync(0xffffffffu, sum, 4);
        if (live) {
            const uint32_t chunk = b8 >> 4, grp = (b8 >> 3) & 1u, b = b8 & 7u;  // block b of the group: inputs 8 b .. 8 b + 7
            uint8_t *dst = xdig + (size_t)chunk * rows_chunk_bytes(MP) + (size_t)grp * 3u * MP * 64u + (size_t)mrow * 64u + 16u * (b >> 1) + 8u * (b & 1u);
#pragma unroll
            for (int d = 0; d < 3; ++d) {
                const uint32_t sel = (uint32_t)d | ((4u + (uint32_t)d) << 4);
                uint2 w;
                w.x = __byte_perm(__byte_perm(z[0], z[2], sel), __byte_perm(z[4], z[6], sel), 0x5410u);  // even inputs
                w.y = __byte_perm(__byte_perm(z[1], z[3], sel), __byte_perm(z[5], z[7], sel), 0x5410u);  // odd inputs
                *reinterpret_cast<uint2 *>(dst + (size_t)d * MP * 64u) = w;
            }
            if (b == 0) xsum[(chunk * 2u + grp) * MP + mrow] = (float)sum;
        }
    }
    __syncthreads();

    if (tr) tr[1] = rows_ns();
    if (item < items) prologue(kEarly, S - 1);

    // ---- tiles ----
    const uint32_t xdig_addr = (uint32_t)__cvta_generic_to_shared(xdig) + g * 64u + t * 16u;
    const uint32_t xsum_addr = (uint32_t)__cvta_generic_to_shared(xsum) + 2u * t * 4u;
    // this lane's 8 bytes of group G of row g in a stage: quarter 2 G + (t >> 1), swizzled as above, half t & 1
    const uint32_t rd_swz = 2u * ((g >> 1) & 1u);
    const uint32_t rd0 = 16u * (g * 4u + ((0u + (t >> 1)) ^ rd_swz)) + 8u * (t & 1u);
    const uint32_t rd1 = 16u * (g * 4u + ((2u + (t >> 1)) ^ rd_swz)) + 8u * (t & 1u);
    for (; item < items; item += blocks_per_part * kRowsWarps) {
        float acc[TW][NB][4];
#pragma unroll
        for (int w = 0; w < TW; ++w)
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) acc[w][nb][0] = acc[w][nb][1] = acc[w][nb][2] = acc[w][nb][3] = 0.f;
        for (uint32_t c = c_lo; c < c_hi; ++c) {
            issue_chunk(c + S - 1);
            cp_async_commit();
            cp_async_wait<S - 1>();
            __syncwarp();
            const uint32_t stage = ring + ((c - c_lo) % S) * kStage;
            const uint32_t pst = pring + (((c - c_lo) >> 2) % PS) * kParamStage + ((c - c_lo) & 3u) * 4u;
            const uint32_t xc = xdig_addr + (c - c_lo) * rows_chunk_bytes(MP);
            const uint32_t xs = xsum_addr + (c - c_lo) * (2u * MP * 4u);
#pragma unroll
            for (int grp = 0; grp < 2; ++grp) {
                // the activation's digits of this group: read once, used by every tile of the item
                uint4 xf[NB][3];
                uint2 xv[NB];
#pragma unroll
                for (int nb = 0; nb < NB; ++nb) {
#pragma unroll
                    for (int d = 0; d < 3; ++d) xf[nb][d] = lds_v4(xc + (uint32_t)((grp * 3 + d) * MP + nb * 8) * 64u);
                    xv[nb] = lds_v2(xs + (uint32_t)(grp * MP + nb * 8) * 4u);  // sums of x' of rows 2 t, 2 t + 1 of this block of 8
                }
#pragma unroll
                for (int w = 0; w < TW; ++w) {
                    const uint32_t wst = stage + w * kRowsStageBytes, pwst = pst + w * 512u;
                    const uint2 wA = lds_v2(wst + (grp ? rd1 : rd0)), wB = lds_v2(wst + 512u + (grp ? rd1 : rd0));
                    const uint32_t m4 = 0x0f0f0f0fu;
                    const uint32_t a_lo0 = wA.x & m4, a_hi0 = (wA.x >> 4) & m4, a_lo1 = wA.y & m4, a_hi1 = (wA.y >> 4) & m4;
                    const uint32_t b_lo0 = wB.x & m4, b_hi0 = (wB.x >> 4) & m4, b_lo1 = wB.y & m4, b_hi1 = (wB.y >> 4) & m4;
                    const uint32_t sa_c = lds_u32(pwst + g * 16u), sb_c = lds_u32(pwst + (g + 8u) * 16u);
                    const uint32_t ba_c = lds_u32(pwst + 256u + g * 16u), bb_c = lds_u32(pwst + 256u + (g + 8u) * 16u);
                    const float sa = bf16_bits_to_float(grp ? (sa_c >> 16) : (sa_c & 0xffffu));
                    const float sb = bf16_bits_to_float(grp ? (sb_c >> 16) : (sb_c & 0xffffu));
                    const float ba = bf16_bits_to_float(grp ? (ba_c >> 16) : (ba_c & 0xffffu));
                    const float bb = bf16_bits_to_float(grp ? (bb_c >> 16) : (bb_c & 0xffffu));
#pragma unroll
                    for (int nb = 0; nb < NB; ++nb) {
                        int q[3][4];
#pragma unroll
                        for (int d = 0; d < 3; ++d) {
                            q[d][0] = q[d][1] = q[d][2] = q[d][3] = 0;
                            mma_u8s8_16832(q[d], a_lo0, b_lo0, a_hi0, b_hi0, xf[nb][d].x, xf[nb][d].y);
                            mma_u8s8_16832(q[d], a_lo1, b_lo1, a_hi1, b_hi1, xf[nb][d].z, xf[nb][d].w);
                        }
                        // the group's integer dot product q0 + 256 q1 + 65536 q2 (exact; |q0 + 256 q1| < 2^25 is rounded to fp32 once)
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const float dot = fmaf(__int2float_rn(q[2][i]), 65536.f, __int2float_rn(q[0][i] + (q[1][i] << 8)));
                            acc[w][nb][i] = fmaf(dot, i < 2 ? sa : sb, acc[w][nb][i]);
                        }
                        const float x0 = __uint_as_float(xv[nb].x), x1 = __uint_as_float(xv[nb].y);
                        acc[w][nb][0] = fmaf(x0, ba, acc[w][nb][0]);
                        acc[w][nb][1] = fmaf(x1, ba, acc[w][nb][1]);
                        acc[w][nb][2] = fmaf(x0, bb, acc[w][nb][2]);
                        acc[w][nb][3] = fmaf(x1, bb, acc[w][nb][3]);
                    }
                }
            }
            __syncwarp();  // every lane is done with the stage before the next iteration refills the one before it
        }
        cp_async_wait<0>();
        __syncwarp();
        if (tr && first_tile) tr[2] = rows_ns();
        first_tile = false;
        // the next item's first weights travel while this one is finished
        const RowsJob *done_job[TW];
        uint32_t done_row0[TW];
        bool done_live[TW];
#pragma unroll
        for (int w = 0; w < TW; ++w) {
            done_job[w] = job[w];
            done_row0[w] = row0[w];
            done_live[w] = tile_live[w];
        }
        const uint32_t done_item = item;
        if (item + blocks_per_part * kRowsWarps < items) {
            open_item(item + blocks_per_part * kRowsWarps);
            prologue(0, S - 1);
        }

        // ---- the part's scaling undone; then the tile's parts ----
        const uint32_t rows_total = p.tiles * 16u;
#pragma unroll
        for (int w = 0; w < TW; ++w) {
            if (!done_live[w]) continue;  // (uniform)
            const uint32_t done_tile = done_item * TW + w;
            float val[NB][4];
#pragma unroll
            for (int nb = 0; nb < NB; ++nb)
#pragma unroll
                for (int i = 0; i < 4; ++i) val[nb][i] = acc[w][nb][i] * inv_s[nb * 8 + 2 * t + (i & 1)];
            bool last = true;
            if (p.parts > 1u) {
#pragma unroll
                for (int nb = 0; nb < NB; ++nb)
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const uint32_t mcol = nb * 8 + 2 * t + (i & 1), r = g + 8u * (i >> 1);
                        p.partials[((size_t)part * MP + mcol) * rows_total + (size_t)done_tile * 16u + r] = val[nb][i];
                    }
                __threadfence();
                __syncwarp();
                unsigned int before = 0;
                if (lane == 0) before = atomicAdd(p.counters + done_tile, 1u);
                before = __shfl_sync(0xffffffffu, before, 0);
                last = before + 1u == p.parts;
                if (last) {
                    __threadfence();
                    if (lane == 0) p.counters[done_tile] = 0;  // ready for the next launch
                }
            }
            if (last) {
#pragma unroll
                for (int nb = 0; nb < NB; ++nb)
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const uint32_t mcol = nb * 8 + 2 * t + (i & 1), r = g + 8u * (i >> 1);
                        if (mcol >= p.m || done_row0[w] + r >= done_job[w]->n) continue;
                        float sum = val[nb][i];
                        if (p.parts > 1u) {
                            sum = 0.f;
                            for (uint32_t q = 0; q < p.parts; ++q)  // part order, whoever came last
                                sum += __ldcg(p.partials + ((size_t)q * MP + mcol) * rows_total + (size_t)done_tile * 16u + r);
                        }
                        float *dst = done_job[w]->out + (size_t)mcol * done_job[w]->out_stride + done_row0[w] + r;
                        *dst = p.accumulate ? *dst + sum : sum;
                    }
            }
        }
    }
    cp_async_wait<0>();
    if (tr) tr[3] = rows_ns();
}

}  // namespace q4

// Largest part (in chunks) a block can hold for `mp` padded activation rows and `tw` tiles per warp, 0 if not even
// four chunks fit.
static uint32_t rows_part_capacity(uint32_t mp, uint32_t tw) {
    int dev = 0, optin = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    uint32_t chunks = 0;
    while (q4::rows_smem_bytes(mp, chunks + 1, tw) <= (size_t)optin && (chunks + 1) * mp <= 256u) ++chunks;
    return chunks >= 4 ? chunks : 0;
}

// How the K range of a launch is cut: the number of parts (0: the shape is not supported), the longest part, and how
// many tiles a warp walks at a time (two share the activation's fragments; up to 8 rows only).
extern "C" uint32_t q4k_rows_plan(uint32_t m, uint32_t k, uint32_t tiles, uint32_t sm_count, uint32_t *part_chunks, uint32_t *tiles_per_warp) {
    if (m < 1 || m > 16 || k == 0 || k % 512u != 0 || tiles == 0) return 0;
    const uint32_t mp = m <= 8 ? 8u : 16u;
    uint32_t best = 0;
    double best_cost = 0.0;
    for (uint32_t tw = 1; tw <= (mp == 8 ? 2u : 1u); ++tw) {
        const uint32_t cap = rows_part_capacity(mp, tw);
        if (cap == 0) continue;
        uint32_t chunks = 0;
        double cost = 0.0;
        const uint32_t parts = q4_rows_plan(k / 128u, tiles, sm_count, cap, tw, &chunks, &cost);
        if (parts && (best == 0 || cost < best_cost * 0.98)) {
            best = parts;
            best_cost = cost;
            *part_chunks = chunks;
            *tiles_per_warp = tw;
        }
    }
    return best;
}

template <int NB, int TW>
static cudaError_t rows_launch(const q4::RowsParams &p, uint32_t grid, size_t smem, cudaStream_t stream) {
    const cudaError_t e = cudaFuncSetAttribute(q4::q4_rows_kernel<NB, TW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    q4::q4_rows_kernel<NB, TW><<<grid, q4::kRowsWarps * 32, smem, stream>>>(p);
    return cudaGetLastError();
}

extern "C" cudaError_t q4k_rows(const q4::RowsParams *params, uint32_t sm_count, cudaStream_t stream) {
    const q4::RowsParams &p = *params;
    const uint32_t mp = p.m <= 8 ? 8u : 16u;
    if (p.tiles_per_warp != 1u && !(p.tiles_per_warp == 2u && mp == 8u)) return cudaErrorInvalidValue;
    const size_t smem = q4::rows_smem_bytes(mp, p.part_chunks, p.tiles_per_warp);
    const uint32_t grid = (sm_count / p.parts) * p.parts;
    if (grid == 0) return cudaErrorInvalidValue;
    if (mp == 16) return rows_launch<2, 1>(p, grid, smem, stream);
    return p.tiles_per_warp == 2u ? rows_launch<1, 2>(p, grid, smem, stream) : rows_launch<1, 1>(p, grid, smem, stream);
}
