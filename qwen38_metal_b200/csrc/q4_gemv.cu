// Streaming affine-Q4 projection kernel for decode and short batches (1..8 activation rows).
//
// Replaces the reference's decode family -- qwen38_q4_affine_matvec_simd and its _unaligned
// twin (shaders/qwen38.metal:213-298), the batch2/batch3/batch_simd/short_compact kernels
// (shaders/qwen38.metal:1140-3640) and the pair kernels that share one activation between two
// matrices (shaders/qwen38.metal:1404-3757) -- with one kernel that takes a table of jobs:
// every projection of a launch reads the same prepared activation.
//
// Arithmetic is the reference's factored form (shaders/qwen38.metal:224-241):
//     y[n] = sum_g ( scale[n,g] * sum_{k in g} x[k]*q[n,k]  +  bias[n,g] * sum_{k in g} x[k] )
// The inner sums run on the warp-level tensor-core MMA (m16n8k16, bf16 x bf16 -> fp32): q is
// 0..15 and x is bf16, so every product is exact and only fp32 accumulation rounds. fp32
// activations are split into three bf16 terms (hi+mid+lo == x exactly) that ride in three MMA
// columns, so the fp32 entry points lose nothing.
//
// Data movement: each lane streams 16 bytes of two weight rows per K-chunk (128 inputs) with
// 128-bit no-allocate loads, several chunks in flight per lane; the four lanes of a quad cover 64
// contiguous bytes of a row. A quad's lanes 0,1 hold affine group A of the chunk and lanes 2,3
// group B; the activation fragment puts group A's x in MMA columns 0..3 and group B's in 4..7
// (zero elsewhere), so one MMA yields both groups' sums separately and each lane scales the
// sums of the group it loaded.
//
// Work is cut into near-equal contiguous unit ranges per warp (q4_decomp.h); tiles split
// between warps are combined, in worker order, by the last warp to arrive (no spinning).
#include "q4_kernels.h"

#include "q4_decomp.h"
#include "q4_device.cuh"

namespace q4 {

constexpr int kWarpsPerCta = 8;

// ---------------------------------------------------------------------------------------------
// Activation preparation: one pass over x that produces what every warp of the projection
// kernel needs -- bf16 columns in MMA fragment order and per-group sums.
//   xp  : [V][K] bf16; inside each block of 8 inputs the order is k0,k4,k1,k5,k2,k6,k3,k7
//         (lo/hi halves of the registers nib2_to_bf16x2 produces).
//   xsum: [K/64][vpad] fp32, sum of the column's values over the group; zero for v >= V.
// V = M for bf16 input; V = 3M for fp32 input (column 3m+p is part p of row m).
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) q4_prepare_x_kernel(const void *__restrict__ x, int x_is_f32, uint32_t m_rows,
                                                          uint32_t k, uint32_t vpad, uint16_t *__restrict__ xp,
                                                          float *__restrict__ xsum) {
    const uint32_t blocks_per_row = k / 8;
    const uint32_t groups = k / 64;
    const uint32_t parts = x_is_f32 ? 3u : 1u;
    // one thread per 8-input block; the 8 threads of a group are consecutive lanes
    uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    uint64_t total = (uint64_t)m_rows * blocks_per_row;
    bool active = idx < total;
    uint32_t row = active ? (uint32_t)(idx / blocks_per_row) : 0;
    uint32_t blk = active ? (uint32_t)(idx % blocks_per_row) : 0;
    float v[8];
    if (active) {
        if (x_is_f32) {
            const float4 *src = reinterpret_cast<const float4 *>(static_cast<const float *>(x) + (uint64_t)row * k + blk * 8);
            float4 a = src[0], b = src[1];
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        } else {
            uint4 raw = *reinterpret_cast<const uint4 *>(static_cast<const uint16_t *>(x) + (uint64_t)row * k + blk * 8);
            uint32_t r[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                v[2 * i] = bf16_bits_to_float(r[i] & 0xffffu);
                v[2 * i + 1] = bf16_bits_to_float(r[i] >> 16);
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = 0.f;
    }
    for (uint32_t p = 0; p < parts; ++p) {
        uint32_t bits[8];
        float part_sum = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            bits[i] = float_to_bf16_bits(v[i]);
            float taken = bf16_bits_to_float(bits[i]);
            part_sum += taken;
            v[i] -= taken;  // exact: the remainder has at most 16 significant bits
        }
        // sum over the 8 consecutive lanes that share a group
        part_sum += __shfl_xor_sync(0xffffffffu, part_sum, 1);
        part_sum += __shfl_xor_sync(0xffffffffu, part_sum, 2);
        part_sum += __shfl_xor_sync(0xffffffffu, part_sum, 4);
        if (active) {
            uint32_t col = row * parts + p;
            uint4 out;
            out.x = bits[0] | (bits[4] << 16);
            out.y = bits[1] | (bits[5] << 16);
            out.z = bits[2] | (bits[6] << 16);
            out.w = bits[3] | (bits[7] << 16);
            *reinterpret_cast<uint4 *>(xp + (uint64_t)col * k + blk * 8) = out;
            if ((threadIdx.x & 7u) == 0) xsum[(uint64_t)(blk / 8) * vpad + col] = part_sum;
        }
    }
    // zero the padding columns of xsum (columns V..vpad-1)
    uint32_t vcols = m_rows * parts;
    if (vcols < vpad) {
        uint64_t pad_total = (uint64_t)groups * (vpad - vcols);
        for (uint64_t i = idx; i < pad_total; i += (uint64_t)gridDim.x * blockDim.x) {
            uint32_t g = (uint32_t)(i / (vpad - vcols));
            uint32_t c = vcols + (uint32_t)(i % (vpad - vcols));
            xsum[(uint64_t)g * vpad + c] = 0.f;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// The projection kernel.
// ---------------------------------------------------------------------------------------------

// K-chunks in flight per lane (each: 2 x 16 B of weights + 4 bf16 parameters); two column tiles leave
// fewer registers for buffers
template <int NT>
struct Depth {
    static constexpr int value = NT == 1 ? 4 : 2;
};

struct ChunkRegs {
    uint4 wa, wb;       // 16 bytes of tile rows g and g+8
    uint32_t sa, ba;    // scale/bias bits for row g, this lane's group
    uint32_t sb, bb;    // same for row g+8
};

// Per-lane cursors of one tile segment. They point at the chunk the next refill will fetch for
// buffer 0; buffer i adds an immediate offset.
struct LaneView {
    const uint8_t *wa, *wb;  // this lane's 16 bytes in rows g and g+8
    const uint8_t *sa, *sb;  // scale of this lane's group (rows g, g+8)
    const uint8_t *ba, *bb;  // bias likewise
    uint32_t mis;            // weight address & 15 (byte-addressed path)
};

// Loads never need masking: a chunk past the lane's last group (odd group count) reads the start of
// the next row, or the padding behind the shard, and is cancelled by zeroed parameters when consumed.
template <bool ALIGNED>
__device__ __forceinline__ void load_chunk(ChunkRegs &c, const LaneView &v, int ahead) {
    const uint32_t woff = (uint32_t)ahead * 64u, poff = (uint32_t)ahead * 4u;
    if (ALIGNED) {
        c.wa = ldg_stream_v4(v.wa + woff);
        c.wb = ldg_stream_v4(v.wb + woff);
        c.sa = (uint32_t)__ldg(reinterpret_cast<const unsigned short *>(v.sa + poff));
        c.sb = (uint32_t)__ldg(reinterpret_cast<const unsigned short *>(v.sb + poff));
        c.ba = (uint32_t)__ldg(reinterpret_cast<const unsigned short *>(v.ba + poff));
        c.bb = (uint32_t)__ldg(reinterpret_cast<const unsigned short *>(v.bb + poff));
    } else {
        c.wa = ldg_stream_v4_unaligned(v.wa + woff, v.mis);
        c.wb = ldg_stream_v4_unaligned(v.wb + woff, v.mis);
        c.sa = ldg_bf16_bits(v.sa + poff);
        c.sb = ldg_bf16_bits(v.sb + poff);
        c.ba = ldg_bf16_bits(v.ba + poff);
        c.bb = ldg_bf16_bits(v.bb + poff);
    }
}

// One chunk: 8 MMAs per column tile, then the affine step for the group this lane streamed.
//   xf    activation fragment registers; lanes that supply zeros never load and keep their zeros
//   xsrc  this lane's fragment of the chunk for column tile 0 (column tiles are 4*x_col_stride apart)
//   xs    per-group column sums of the chunk for this lane's group and column pair
//   live  the lane's group exists in this chunk (false only in the last chunk of an odd group count)
template <int NT>
__device__ __forceinline__ void consume_chunk(const ChunkRegs &c, bool live, uint4 (&xf)[NT][4], const uint16_t *xsrc,
                                              uint32_t x_mask, uint32_t x_col_stride, const float *xs,
                                              const Magic &mg, float (&acc)[NT][4]) {
    const uint32_t wa[4] = {c.wa.x, c.wa.y, c.wa.z, c.wa.w};
    const uint32_t wb[4] = {c.wb.x, c.wb.y, c.wb.z, c.wb.w};
    const float sa = live ? bf16_bits_to_float(c.sa) : 0.f, sb = live ? bf16_bits_to_float(c.sb) : 0.f;
    const float ba = live ? bf16_bits_to_float(c.ba) : 0.f, bb = live ? bf16_bits_to_float(c.bb) : 0.f;
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        const uint4 *src = reinterpret_cast<const uint4 *>(xsrc + (size_t)(4 * j) * x_col_stride);
        const bool has_x = (x_mask >> j) & 1u;
#pragma unroll
        for (int w = 0; w < 4; ++w) ldg_v4_keep(xf[j][w], src + w, has_x);
    }
    float d[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) d[j][0] = d[j][1] = d[j][2] = d[j][3] = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t a0 = nib2_to_bf16x2(wa[w] >> (8 * h), mg);
            const uint32_t a2 = nib2_to_bf16x2(wa[w] >> (8 * h + 4), mg);
            const uint32_t a1 = nib2_to_bf16x2(wb[w] >> (8 * h), mg);
            const uint32_t a3 = nib2_to_bf16x2(wb[w] >> (8 * h + 4), mg);
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const uint32_t xr[4] = {xf[j][w].x, xf[j][w].y, xf[j][w].z, xf[j][w].w};
                mma_bf16_16816(d[j], a0, a1, a2, a3, xr[2 * h], xr[2 * h + 1]);
            }
        }
    }
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
// columns of each tile into every lane, recombine fp32 splits, store.
template <int NT>
__device__ __forceinline__ void store_tile(const GemvParams &p, uint32_t tile, float (&acc)[NT][4], uint32_t g,
                                           uint32_t t, uint32_t job_index) {
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
            float *dst = job.out + (uint64_t)m * job.out_stride + row;
            if (p.accumulate) y += *dst;  // residual form: dst += projection
            *dst = y;
        }
    }
}

template <int NT, bool ALIGNED>
__global__ void __launch_bounds__(kWarpsPerCta * 32, 2) q4_gemv_kernel(const __grid_constant__ GemvParams p) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t g = lane >> 2, t = lane & 3u;
    const uint32_t worker = blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
    if (worker >= p.workers) return;
    const Q4Split split{p.units, p.cpt, p.workers};
    uint64_t u = q4_split_begin(split, worker);
    const uint64_t u1 = q4_split_begin(split, worker + 1);
    const uint32_t cpt = p.cpt, groups = p.groups;
    // this lane supplies activation column (g & 3) of each column tile, for the group it streams:
    // MMA columns 0..3 carry group A (lanes t<2), columns 4..7 group B (lanes t>=2), zero elsewhere
    const bool x_lane = ((g < 4u) == (t < 2u));
    const uint32_t v_first = g & 3u;
    uint32_t x_mask = 0;  // bit j: this lane loads a fragment for column tile j
#pragma unroll
    for (int j = 0; j < NT; ++j) x_mask |= (x_lane && (v_first + 4u * j < p.v_cols)) ? (1u << j) : 0u;
    const uint16_t *xfrag0 = p.xp + (size_t)v_first * p.k + t * 32u;
    const float *xs0 = p.xsum + (size_t)(t >> 1) * p.vpad + 2u * (t & 1u);
    // chunks whose group exists for this lane: group = 2*chunk + (t>>1) < groups
    const uint32_t lane_chunks = (groups + 1u - (t >> 1)) >> 1;
    const Magic mg = make_magic();
    uint4 xf[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int w = 0; w < 4; ++w) xf[j][w] = make_uint4(0, 0, 0, 0);

    uint32_t tile = (uint32_t)(u / cpt);
    uint32_t c0 = (uint32_t)(u - (uint64_t)tile * cpt);
    uint32_t job_index = 0;
    while (u < u1) {
        const uint64_t left = u1 - u;
        const uint32_t c1 = (left < (uint64_t)(cpt - c0)) ? c0 + (uint32_t)left : cpt;
        while (job_index + 1 < p.n_jobs && tile >= p.jobs[job_index + 1].tile_begin) ++job_index;
        const GemvJob &job = p.jobs[job_index];
        LaneView v;
        {
            uint32_t row_a = (tile - job.tile_begin) * 16u + g;
            uint32_t row_b = row_a + 8u;
            row_a = row_a < job.n ? row_a : job.n - 1u;  // rows past N read a valid row and are never stored
            row_b = row_b < job.n ? row_b : job.n - 1u;
            const uint64_t row_bytes = (uint64_t)p.k >> 1;
            v.wa = job.w + (uint64_t)row_a * row_bytes + t * 16u + c0 * 64u;
            v.wb = job.w + (uint64_t)row_b * row_bytes + t * 16u + c0 * 64u;
            const uint64_t pa = ((uint64_t)row_a * groups + (t >> 1)) * 2u + c0 * 4u;
            const uint64_t pb = ((uint64_t)row_b * groups + (t >> 1)) * 2u + c0 * 4u;
            v.sa = job.s + pa;
            v.sb = job.s + pb;
            v.ba = job.b + pa;
            v.bb = job.b + pb;
            v.mis = job.w_misalign;
        }
        const uint16_t *xsrc = xfrag0 + c0 * 128u;
        const float *xs = xs0 + (size_t)c0 * 2u * p.vpad;
        const uint32_t xs_step = 2u * p.vpad;
        float acc[NT][4];
#pragma unroll
        for (int j = 0; j < NT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;

        // kDepth chunks in flight: a buffer is consumed, then refilled with the chunk kDepth ahead
        constexpr int kDepth = Depth<NT>::value;
        ChunkRegs buf[kDepth];
#pragma unroll
        for (int i = 0; i < kDepth; ++i)
            if (c0 + i < c1) load_chunk<ALIGNED>(buf[i], v, i);
        for (uint32_t c = c0; c < c1; c += kDepth) {
#pragma unroll
            for (int i = 0; i < kDepth; ++i) {
                if (c + i < c1) {
                    consume_chunk<NT>(buf[i], c + i < lane_chunks, xf, xsrc + i * 128, x_mask, p.k, xs + i * xs_step, mg, acc);
                    if (c + i + kDepth < c1) load_chunk<ALIGNED>(buf[i], v, i + kDepth);
                }
            }
            v.wa += kDepth * 64;
            v.wb += kDepth * 64;
            v.sa += kDepth * 4;
            v.sb += kDepth * 4;
            v.ba += kDepth * 4;
            v.bb += kDepth * 4;
            xsrc += kDepth * 128;
            xs += kDepth * xs_step;
        }

        if (c0 == 0 && c1 == cpt) {
            store_tile<NT>(p, tile, acc, g, t, job_index);
        } else {
            // split tile: park the lane accumulators, count in, last arrival sums in worker order
            uint32_t first, last;
            q4_split_contributors(split, tile, &first, &last);
            float4 *slot = reinterpret_cast<float4 *>(p.partials) + ((uint64_t)q4_split_slot(split, worker, tile) * NT) * 32u;
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
                for (uint32_t w = first; w <= last; ++w) {
                    const float4 *src = reinterpret_cast<const float4 *>(p.partials) + ((uint64_t)q4_split_slot(split, w, tile) * NT) * 32u;
#pragma unroll
                    for (int j = 0; j < NT; ++j) {
                        float4 pv = __ldcg(src + j * 32 + lane);
                        acc[j][0] += pv.x;
                        acc[j][1] += pv.y;
                        acc[j][2] += pv.z;
                        acc[j][3] += pv.w;
                    }
                }
                store_tile<NT>(p, tile, acc, g, t, job_index);
                if (lane == 0) p.counters[first] = 0;  // ready for the next launch
            }
        }
        u += c1 - c0;
        ++tile;
        c0 = 0;
    }
}

}  // namespace q4

// ---------------------------------------------------------------------------------------------
// Host launchers
// ---------------------------------------------------------------------------------------------

extern "C" cudaError_t q4k_prepare_x(const void *x, int x_is_f32, uint32_t m_rows, uint32_t k, uint32_t vpad,
                                     uint16_t *xp, float *xsum, cudaStream_t stream) {
    uint64_t total = (uint64_t)m_rows * (k / 8);
    uint32_t blocks = (uint32_t)((total + 255) / 256);
    q4::q4_prepare_x_kernel<<<blocks, 256, 0, stream>>>(x, x_is_f32, m_rows, k, vpad, xp, xsum);
    return cudaGetLastError();
}

extern "C" int q4k_gemv_warps_per_cta(void) { return q4::kWarpsPerCta; }

extern "C" uint32_t q4k_gemv_occupancy(int column_tiles, int aligned) {
    using namespace q4;
    int blocks = 0;
    cudaError_t e = cudaErrorInvalidValue;
    const int threads = kWarpsPerCta * 32;
    if (column_tiles == 1 && aligned) e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, q4_gemv_kernel<1, true>, threads, 0);
    if (column_tiles == 1 && !aligned) e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, q4_gemv_kernel<1, false>, threads, 0);
    if (column_tiles == 2 && aligned) e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, q4_gemv_kernel<2, true>, threads, 0);
    if (column_tiles == 2 && !aligned) e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, q4_gemv_kernel<2, false>, threads, 0);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return blocks > 0 ? (uint32_t)blocks : 0u;
}

extern "C" cudaError_t q4k_gemv(const q4::GemvParams *params, int column_tiles, int aligned, uint32_t ctas,
                                cudaStream_t stream) {
    using namespace q4;
    dim3 grid(ctas), block(kWarpsPerCta * 32);
    if (column_tiles == 1) {
        if (aligned) q4_gemv_kernel<1, true><<<grid, block, 0, stream>>>(*params);
        else q4_gemv_kernel<1, false><<<grid, block, 0, stream>>>(*params);
    } else if (column_tiles == 2) {
        if (aligned) q4_gemv_kernel<2, true><<<grid, block, 0, stream>>>(*params);
        else q4_gemv_kernel<2, false><<<grid, block, 0, stream>>>(*params);
    } else {
        return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}
