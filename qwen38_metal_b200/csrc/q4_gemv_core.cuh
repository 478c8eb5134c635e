// Device code shared by the streaming projection kernels (single launches in q4_gemv.cu, the persistent decode
// kernel in q4_decode_stack.cu): the cp.async weight ring, chunk arithmetic on mma.sync, tile epilogue and the
// split-tile protocol.
#pragma once
#include <cuda_fp16.h>

#include "q4_decomp.h"
#include "q4_device.cuh"
#include "q4_kernels.h"

namespace q4 {

// ---------------------------------------------------------------------------------------------
// The projection kernel.
// ---------------------------------------------------------------------------------------------

// Weight bytes travel global -> shared with per-lane 16-byte async copies (cp.async), kStages chunks
// ahead of their use, so the number of bytes in flight does not depend on registers. Each warp owns a
// private ring; a lane reads back what it (or, in the byte-addressed variant, its quad) copied.
constexpr int kStages = 8;
// bytes per stage: aligned variant 2 row halves x 32 lanes x 16 B; byte-addressed variant
// 2 row halves x 8 quads x 5 windows x 16 B (the aligned windows enclosing 64 misaligned bytes)
constexpr int kStageBytesAligned = 2 * 32 * 16;
constexpr int kStageBytesWindowed = 2 * 8 * 5 * 16;

struct ParamRegs {
    uint32_t sa, ba;  // scale/bias bits for row g, this lane's group
    uint32_t sb, bb;  // same for row g+8
};

// `mis`: byte misalignment of the weights; `has_b`: the chunk's second affine group exists (byte-addressed variant)
template <bool ALIGNED>
__device__ __forceinline__ void issue_weights(uint32_t stage_addr, const uint8_t *wa, const uint8_t *wb, uint32_t lane,
                                              uint32_t t, bool pred, uint32_t mis = 0, bool has_b = true) {
    if (ALIGNED) {
        cp_async_16_pred(stage_addr + lane * 16u, wa, pred);
        cp_async_16_pred(stage_addr + 512u + lane * 16u, wb, pred);
    } else {
        // quad q = lane>>2 owns 80 bytes per row half: windows 0..3 from its four lanes, window 4 from lane 3.
        // Only windows that hold bytes of the row are requested (q4_decomp.h).
        const uint32_t a = stage_addr + (lane >> 2) * 80u + t * 16u, b = a + 640u;
        const bool own = pred && q4_window_wanted(t, mis, has_b);
        const bool fifth = pred && t == 3u && q4_fifth_window_wanted(mis, has_b);
        cp_async_16_pred(a, wa, own);
        cp_async_16_pred(b, wb, own);
        cp_async_16_pred(a + 16u, wa + 16, fifth);
        cp_async_16_pred(b + 16u, wb + 16, fifth);
    }
}

template <bool ALIGNED>
__device__ __forceinline__ void read_weights(uint32_t stage_addr, uint32_t lane, uint32_t t, uint32_t mis, uint4 &wa,
                                             uint4 &wb) {
    if (ALIGNED) {
        wa = lds_v4(stage_addr + lane * 16u);
        wb = lds_v4(stage_addr + 512u + lane * 16u);
    } else {
        const uint32_t a = stage_addr + (lane >> 2) * 80u + t * 16u;
        wa = realign_16(lds_v4(a), lds_v4(a + 16u), mis);
        wb = realign_16(lds_v4(a + 640u), lds_v4(a + 656u), mis);
    }
}

// parameters of one chunk for this lane's group; zeros (and no load) when `pred` is false
template <bool ALIGNED>
__device__ __forceinline__ void load_params(ParamRegs &c, const uint8_t *sa, const uint8_t *sb, const uint8_t *ba,
                                            const uint8_t *bb, bool pred = true) {
    c.sa = c.sb = c.ba = c.bb = 0;
    if (!pred) return;
    if (ALIGNED) {
        c.sa = (uint32_t)__ldg(reinterpret_cast<const unsigned short *>(sa));
        c.sb = (uint32_t)__ldg(reinterpret_cast<const unsigned short *>(sb));
        c.ba = (uint32_t)__ldg(reinterpret_cast<const unsigned short *>(ba));
        c.bb = (uint32_t)__ldg(reinterpret_cast<const unsigned short *>(bb));
    } else {
        c.sa = ldg_bf16_bits(sa);
        c.sb = ldg_bf16_bits(sb);
        c.ba = ldg_bf16_bits(ba);
        c.bb = ldg_bf16_bits(bb);
    }
}

// activation fragment of one chunk; lanes that supply zeros never load and keep their zeros
template <int NT>
__device__ __forceinline__ void load_x(uint4 (&xf)[NT][4], const uint16_t *xsrc, uint32_t x_mask, uint32_t x_col_stride) {
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        const uint4 *src = reinterpret_cast<const uint4 *>(xsrc + (size_t)(4 * j) * x_col_stride);
        const bool has_x = (x_mask >> j) & 1u;
#pragma unroll
        for (int w = 0; w < 4; ++w) ldg_v4_keep(xf[j][w], src + w, has_x);
    }
}

// The 8 MMAs of one chunk per column tile: d[j] = sum over the chunk of x*q for rows g, g+8 (raw group sums).
template <int NT>
__device__ __forceinline__ void chunk_mma(const uint4 &cwa, const uint4 &cwb, const uint4 (&xf)[NT][4], const Magic &mg,
                                          float (&d)[NT][4]) {
    const uint32_t wa[4] = {cwa.x, cwa.y, cwa.z, cwa.w};
    const uint32_t wb[4] = {cwb.x, cwb.y, cwb.z, cwb.w};
    // two independent accumulation chains (words 0,1 and words 2,3) halve the dependent MMA latency
    float e[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        d[j][0] = d[j][1] = d[j][2] = d[j][3] = 0.f;
        e[j][0] = e[j][1] = e[j][2] = e[j][3] = 0.f;
    }
#pragma unroll
    for (int w = 0; w < 4; ++w) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            // nibble pairs (2h, 2h+4) and (2h+1, 2h+5) of the word, rows g and g+8
            const uint32_t va = h ? (wa[w] >> 8) : wa[w], vb = h ? (wb[w] >> 8) : wb[w];
            const uint32_t a0 = nib_lo_to_f16x2(va, mg), a2 = nib_hi_to_f16x2(va, mg);
            const uint32_t a1 = nib_lo_to_f16x2(vb, mg), a3 = nib_hi_to_f16x2(vb, mg);
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const uint32_t xr[4] = {xf[j][w].x, xf[j][w].y, xf[j][w].z, xf[j][w].w};
                if (w < 2) mma_f16_16816(d[j], a0, a1, a2, a3, xr[2 * h], xr[2 * h + 1]);
                else mma_f16_16816(e[j], a0, a1, a2, a3, xr[2 * h], xr[2 * h + 1]);
            }
        }
    }
#pragma unroll
    for (int j = 0; j < NT; ++j) {
#pragma unroll
        for (int i = 0; i < 4; ++i) d[j][i] += e[j][i];
    }
}

// One chunk: 8 MMAs per column tile, then the affine step for the group this lane streamed.
//   xs  per-group column sums of the chunk for this lane's group and column pair
template <int NT>
__device__ __forceinline__ void consume_chunk(const uint4 &cwa, const uint4 &cwb, float sa, float sb, float ba, float bb,
                                              const uint4 (&xf)[NT][4], const float *xs, const Magic &mg,
                                              float (&acc)[NT][4]) {
    float d[NT][4];
    chunk_mma<NT>(cwa, cwb, xf, mg, d);
    // d[.][0],d[.][1]: row g, MMA columns 2t,2t+1; d[.][2],d[.][3]: row g+8. Those columns are activation
    // columns 4j + 2(t&1), +1 of the group this lane streamed.
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        const float2 s2 = __ldg(reinterpret_cast<const float2 *>(xs + 4 * j));
        acc[j][0] = fmaf(d[j][0], sa, fmaf(s2.x, ba, acc[j][0]));
        acc[j][1] = fmaf(d[j][1], sa, fmaf(s2.y, ba, acc[j][1]));
        acc[j][2] = fmaf(d[j][2], sb, fmaf(s2.x, bb, acc[j][2]));
        acc[j][3] = fmaf(d[j][3], sb, fmaf(s2.y, bb, acc[j][3]));
    }
}

// Final step for one tile: fold the two group halves (lanes t and t^2), gather the four
// columns of each tile into every lane, recombine fp32 splits, undo the row scaling, store.
template <int NT>
__device__ __forceinline__ void store_tile(const GemvParams &p, const float *row_inv, uint32_t tile, float (&acc)[NT][4],
                                           uint32_t g, uint32_t t, uint32_t job_index) {
    const GemvJob &job = p.jobs[job_index];
    float col[NT * 4][2];  // [activation column][row g / row g+8]
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        float mine[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) mine[i] = acc[j][i] + __shfl_xor_sync(0xffffffffu, acc[j][i], 2);
        float other[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) other[i] = __shfl_xor_sync(0xffffffffu, mine[i], 1);
        const bool odd = (t & 1u) != 0;
        // lane with even t holds columns 0,1 of the tile; odd t holds columns 2,3
        col[4 * j + 0][0] = odd ? other[0] : mine[0];
        col[4 * j + 1][0] = odd ? other[1] : mine[1];
        col[4 * j + 2][0] = odd ? mine[0] : other[0];
        col[4 * j + 3][0] = odd ? mine[1] : other[1];
        col[4 * j + 0][1] = odd ? other[2] : mine[2];
        col[4 * j + 1][1] = odd ? other[3] : mine[3];
        col[4 * j + 2][1] = odd ? mine[2] : other[2];
        col[4 * j + 3][1] = odd ? mine[3] : other[3];
    }
    if (t != 0) return;
    const uint32_t row0 = (tile - job.tile_begin) * 16u + g;
    const uint32_t parts = p.x_is_f32 ? 3u : 1u;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const uint32_t row = row0 + 8u * half;
        if (row >= job.n) continue;
#pragma unroll
        for (int m = 0; m < NT * 4; ++m) {
            if ((uint32_t)m >= p.m_rows) break;
            float y;
            if (parts == 1u) {
                y = col[m][half];
            } else {
                // (hi + mid) + lo of row m live in columns 3m, 3m+1, 3m+2
                y = 0.f;
#pragma unroll
                for (int c = 0; c < NT * 4; ++c) {
                    if (c == 3 * m) y = col[c][half];
                }
#pragma unroll
                for (int c = 0; c < NT * 4; ++c) {
                    if (c == 3 * m + 1 || c == 3 * m + 2) y += col[c][half];
                }
            }
            y *= row_inv[m];  // exact: a power of two
            float *dst = job.out + (uint64_t)m * job.out_stride + row;
            if (p.accumulate) y += *dst;  // residual form: dst += projection
            *dst = y;
            if (p.mirror) {  // the other ranks' copies of a row-sharded output (peer stores over NVLink)
                for (uint32_t r = 0; r < p.world; ++r) {
                    float *peer = p.mirror[job_index * kMaxPeers + r];
                    if (r != p.rank && peer) peer[(uint64_t)m * job.out_stride + row] = y;
                }
            }
        }
    }
}

// A whole tile is stored at once; a tile split between warps is parked in the warp's partial slot and
// summed, in worker order, by the last warp to arrive. The tile occupies the units [u0, u0 + span) of the launch.
template <int NT>
__device__ __forceinline__ void finish_tile(const GemvParams &p, const float *row_inv, const Q4Split &split, uint32_t worker,
                                            uint32_t tile, bool whole, float (&acc)[NT][4], uint32_t lane, uint32_t g,
                                            uint32_t t, uint32_t job_index, uint64_t u0, uint32_t span) {
    if (whole) {
        store_tile<NT>(p, row_inv, tile, acc, g, t, job_index);
        return;
    }
    uint32_t first, last;
    q4_split_span_contributors(split, u0, span, &first, &last);
    const uint64_t first_begin = q4_split_begin(split, first);
    // only the first contributor can have started in an earlier tile (slot 1); everyone else starts inside this one
    const uint32_t first_slot = 2u * first + (first_begin < u0 ? 1u : 0u);
    const uint32_t my_slot = worker == first ? first_slot : 2u * worker;
    float4 *slot = reinterpret_cast<float4 *>(p.partials) + ((uint64_t)my_slot * NT) * 32u;
#pragma unroll
    for (int j = 0; j < NT; ++j) slot[j * 32 + lane] = make_float4(acc[j][0], acc[j][1], acc[j][2], acc[j][3]);
    __threadfence();
    __syncwarp();
    uint32_t arrived = 0;
    if (lane == 0) arrived = atomicAdd(p.counters + first, 1u);
    arrived = __shfl_sync(0xffffffffu, arrived, 0);
    if (arrived == last - first) {
        __threadfence();
#pragma unroll
        for (int j = 0; j < NT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
        // partial slots are read four at a time (independent loads in flight) and added in worker order
        for (uint32_t w0 = first; w0 <= last; w0 += 4) {
            float4 pv[4][NT];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t w = w0 + i <= last ? w0 + i : last;
                const uint32_t ws = w == first ? first_slot : 2u * w;
                const float4 *src = reinterpret_cast<const float4 *>(p.partials) + ((uint64_t)ws * NT) * 32u;
#pragma unroll
                for (int j = 0; j < NT; ++j) pv[i][j] = __ldcg(src + j * 32 + lane);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                if (w0 + i <= last) {
#pragma unroll
                    for (int j = 0; j < NT; ++j) {
                        acc[j][0] += pv[i][j].x;
                        acc[j][1] += pv[i][j].y;
                        acc[j][2] += pv[i][j].z;
                        acc[j][3] += pv[i][j].w;
                    }
                }
            }
        }
        store_tile<NT>(p, row_inv, tile, acc, g, t, job_index);
        if (lane == 0) p.counters[first] = 0;  // ready for the next launch
    }
}

// General variant: any byte alignment of the three tensors, any group count. Weights come through
// aligned 16-byte windows, parameters through plain loads; when the group count is odd, lanes 2,3 of a
// quad have no group in the last chunk of a row and their parameters are zeroed.

// bf16 parameter of one chunk for this lane's group parity, as fp32: picks one half of the 32-bit word and moves
// it to the top (sel = 0x1044 for the low half, 0x3244 for the high half)
__device__ __forceinline__ float param_of(uint32_t word, uint32_t sel) {
    return __uint_as_float(__byte_perm(word, 0u, sel));
}

}  // namespace q4
