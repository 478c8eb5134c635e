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
// The inner sums run on the warp-level tensor-core MMA (m16n8k16, f16 x f16 -> fp32). q is 0..15 and
// the activation is held as fp16 after an exact power-of-two row scaling (undone in fp32 at the end),
// so every product is exact and only fp32 accumulation rounds: a bf16 activation fits fp16 exactly
// within 2^28 of the row maximum, and an fp32 activation is split into three fp16 terms
// (hi+mid+lo == x) that ride in three MMA columns.
//
// Data movement: each lane streams 16 bytes of two weight rows per K-chunk (128 inputs) with
// asynchronous global->shared copies issued eight chunks ahead; the four lanes of a quad cover 64
// contiguous bytes of a row. A quad's lanes 0,1 hold affine group A of the chunk and lanes 2,3
// group B; the activation fragment puts group A's x in MMA columns 0..3 and group B's in 4..7
// (zero elsewhere), so one MMA yields both groups' sums separately and each lane scales the
// sums of the group it loaded.
//
// Work is cut into near-equal contiguous unit ranges, one per warp (q4_decomp.h); a warp is a whole
// thread block, so all its bookkeeping is uniform. Tiles split between warps are combined, in worker
// order, by the last warp to arrive (no spinning).
#include "q4_kernels.h"

#include "q4_gemv_core.cuh"

namespace q4 {

// ---------------------------------------------------------------------------------------------
// Activation preparation: one block per activation row.
//   xp     : [V][kp] fp16, kp = K rounded up to 128 with zero fill; inside each block of 8 inputs the
//            order is k0,k4,k1,k5,k2,k6,k3,k7 (the pairing the nibble extraction produces)
//   xsum   : [kp/64][vpad] fp32, sum of the column's fp16 values over the group; zero where v >= V or
//            the group is padding
//   row_inv: [M] fp32, 2^-e of the row: x' = x * 2^e puts the row maximum in [2^14, 2^15)
// V = M for bf16 input; V = 3M for fp32 input (column 3m+p is part p of row m).
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) q4_prepare_x_kernel(const void *__restrict__ x, int x_is_f32, uint32_t k,
                                                          uint32_t kp, uint32_t vpad, uint16_t *__restrict__ xp,
                                                          float *__restrict__ xsum, float *__restrict__ row_inv) {
    __shared__ uint32_t warp_max[8];
    const uint32_t row = blockIdx.x;
    const uint32_t blocks = k / 8, blocks_p = kp / 8;
    const uint32_t parts = x_is_f32 ? 3u : 1u;
    const uint32_t v_cols = gridDim.x * parts;
    const float *xf = static_cast<const float *>(x) + (uint64_t)row * k;
    const uint16_t *xb = static_cast<const uint16_t *>(x) + (uint64_t)row * k;

    // pass 1: largest magnitude of the row (as fp32 bits; order-preserving for non-negative values)
    uint32_t amax = 0;
    for (uint32_t b = threadIdx.x; b < blocks; b += 256) {
        if (x_is_f32) {
            const float4 *src = reinterpret_cast<const float4 *>(xf + b * 8);
            float4 lo = src[0], hi = src[1];
            const float v[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
            for (int i = 0; i < 8; ++i) amax = max(amax, __float_as_uint(v[i]) & 0x7fffffffu);
        } else {
            uint4 raw = *reinterpret_cast<const uint4 *>(xb + b * 8);
            const uint32_t r[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                amax = max(amax, (r[i] << 16) & 0x7fffffffu);
                amax = max(amax, r[i] & 0x7fff0000u);
            }
        }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) amax = max(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    if ((threadIdx.x & 31u) == 0) warp_max[threadIdx.x >> 5] = amax;
    __syncthreads();
    amax = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = max(amax, warp_max[i]);
    int e = 14 - ((int)((amax >> 23) & 0xffu) - 127);  // floor(log2(max)) = exponent field - 127
    e = amax == 0 ? 0 : max(-100, min(100, e));
    const float scale = __uint_as_float((uint32_t)(e + 127) << 23);
    if (threadIdx.x == 0) row_inv[row] = __uint_as_float((uint32_t)(127 - e) << 23);

    // pass 2: scaled fp16 parts in fragment order, group sums
    for (uint32_t b = threadIdx.x; b < blocks_p; b += 256) {
        float v[8];
        if (b < blocks) {
            if (x_is_f32) {
                const float4 *src = reinterpret_cast<const float4 *>(xf + b * 8);
                float4 lo = src[0], hi = src[1];
                v[0] = lo.x; v[1] = lo.y; v[2] = lo.z; v[3] = lo.w; v[4] = hi.x; v[5] = hi.y; v[6] = hi.z; v[7] = hi.w;
            } else {
                uint4 raw = *reinterpret_cast<const uint4 *>(xb + b * 8);
                const uint32_t r[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    v[2 * i] = bf16_bits_to_float(r[i] & 0xffffu);
                    v[2 * i + 1] = bf16_bits_to_float(r[i] >> 16);
                }
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] *= scale;  // exact: a power of two
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = 0.f;
        }
        for (uint32_t p = 0; p < parts; ++p) {
            uint32_t bits[8];
            float part_sum = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const __half h = __float2half_rn(v[i]);
                bits[i] = (uint32_t)__half_as_ushort(h);
                const float taken = __half2float(h);
                part_sum += taken;
                v[i] -= taken;  // exact: the remainder has fewer significant bits than fp32 holds
            }
            // the 8 consecutive lanes of a group add up (a row has a whole number of groups)
            part_sum += __shfl_xor_sync(0xffffffffu, part_sum, 1);
            part_sum += __shfl_xor_sync(0xffffffffu, part_sum, 2);
            part_sum += __shfl_xor_sync(0xffffffffu, part_sum, 4);
            const uint32_t col = row * parts + p;
            uint4 out;
            out.x = bits[0] | (bits[4] << 16);
            out.y = bits[1] | (bits[5] << 16);
            out.z = bits[2] | (bits[6] << 16);
            out.w = bits[3] | (bits[7] << 16);
            *reinterpret_cast<uint4 *>(xp + (uint64_t)col * kp + b * 8) = out;
            if ((threadIdx.x & 7u) == 0) xsum[(uint64_t)(b / 8) * vpad + col] = part_sum;
        }
    }
    // zero the unused columns of xsum (columns V..vpad-1); block 0 does it for every group
    if (row == 0 && v_cols < vpad) {
        const uint32_t pad = vpad - v_cols, groups_p = kp / 64;
        for (uint32_t i = threadIdx.x; i < groups_p * pad; i += 256) xsum[(uint64_t)(i / pad) * vpad + v_cols + i % pad] = 0.f;
    }
}

template <int NT>
__global__ void __launch_bounds__(32, NT == 1 ? 20 : 16) q4_gemv_generic_kernel(const __grid_constant__ GemvParams p) {
    constexpr bool ALIGNED = false;
    extern __shared__ __align__(128) uint8_t ring_bytes[];
    const uint32_t lane = threadIdx.x;
    const uint32_t g = lane >> 2, t = lane & 3u;
    const uint32_t worker = blockIdx.x;
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
    const uint16_t *xfrag0 = p.xp + (size_t)v_first * p.kp + t * 32u;
    const float *xs0 = p.xsum + (size_t)(t >> 1) * p.vpad + 2u * (t & 1u);
    const uint32_t xs_step = 2u * p.vpad;
    // chunks whose group exists for this lane: group = 2*chunk + (t>>1) < groups
    const uint32_t lane_chunks = q4_lane_chunks(groups, t);
    const Magic mg = make_magic();
    constexpr uint32_t kStageBytes = ALIGNED ? kStageBytesAligned : kStageBytesWindowed;
    const uint32_t ring = (uint32_t)__cvta_generic_to_shared(ring_bytes);
    uint4 xf[2][NT][4];  // activation fragments of the chunk in use and the next one
#pragma unroll
    for (int b = 0; b < 2; ++b)
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int w = 0; w < 4; ++w) xf[b][j][w] = make_uint4(0, 0, 0, 0);

    uint32_t tile = (uint32_t)(u / cpt);
    uint32_t c0 = (uint32_t)(u - (uint64_t)tile * cpt);
    uint32_t job_index = 0;
    while (u < u1) {
        const uint64_t left = u1 - u;
        const uint32_t c1 = (left < (uint64_t)(cpt - c0)) ? c0 + (uint32_t)left : cpt;
        const uint32_t n = c1 - c0;  // chunks in this segment
        while (job_index + 1 < p.n_jobs && tile >= p.jobs[job_index + 1].tile_begin) ++job_index;
        const GemvJob &job = p.jobs[job_index];
        const uint32_t mis = ALIGNED ? 0u : job.w_misalign;
        // per-lane cursors at the segment's first chunk
        const uint8_t *wa, *wb, *sa, *sb, *ba, *bb;
        {
            uint32_t row_a = (tile - job.tile_begin) * 16u + g;
            uint32_t row_b = row_a + 8u;
            row_a = row_a < job.n ? row_a : job.n - 1u;  // rows past N read a valid row and are never stored
            row_b = row_b < job.n ? row_b : job.n - 1u;
            const uint64_t row_bytes = (uint64_t)p.k >> 1;
            wa = job.w + (uint64_t)row_a * row_bytes + t * 16u + c0 * 64u - mis;  // byte-addressed: the aligned window
            wb = job.w + (uint64_t)row_b * row_bytes + t * 16u + c0 * 64u - mis;
            const uint64_t pa = ((uint64_t)row_a * groups + (t >> 1)) * 2u + c0 * 4u;
            const uint64_t pb = ((uint64_t)row_b * groups + (t >> 1)) * 2u + c0 * 4u;
            sa = job.s + pa;
            sb = job.s + pb;
            ba = job.b + pa;
            bb = job.b + pb;
        }
        const uint16_t *xsrc = xfrag0 + c0 * 128u;
        const float *xs = xs0 + (size_t)c0 * xs_step;
        const uint32_t live_n = lane_chunks > c0 ? lane_chunks - c0 : 0u;  // segment chunks with a group for this lane
        float acc[NT][4];
#pragma unroll
        for (int j = 0; j < NT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;

        // prologue: weights of the first kStages chunks, parameters of the first two, activations of the first.
        // Parameters are only read for chunks of this segment in which the lane has a group: no byte outside the three
        // tensors' own 16-byte blocks is touched, so caller-supplied tensors need no padding.
        const uint32_t full_chunks = groups >> 1;  // chunks with both affine groups
        const uint32_t param_n = live_n < n ? live_n : n;
#pragma unroll
        for (int i = 0; i < kStages; ++i) {
            issue_weights<ALIGNED>(ring + i * kStageBytes, wa + i * 64, wb + i * 64, lane, t, (uint32_t)i < n, mis, c0 + i < full_chunks);
            if (i == 3 || i == 7) cp_async_commit();  // one group per half of the ring
        }
        ParamRegs prm[2];
        load_params<ALIGNED>(prm[0], sa, sb, ba, bb, 0 < param_n);
        load_params<ALIGNED>(prm[1], sa + 4, sb + 4, ba + 4, bb + 4, 1 < param_n);
        load_x<NT>(xf[0], xsrc, x_mask, p.kp);

        // Four chunks are consumed, then their four stages are refilled in one burst (chunks 8..11 ahead):
        // the burst asks for 256 contiguous bytes of each row at once, which keeps DRAM pages open.
        uint32_t half = 0;  // which half of the ring the next four chunks use
        for (uint32_t ci = 0; ci < n; ci += 4) {
            const uint32_t stage0 = ring + half * (4 * kStageBytes);
#pragma unroll
            for (int s = 0; s < 4; ++s) {
                if (ci + s < n) {
                    const int b = s & 1;
                    // each half of the ring is one copy group; only the other half's group may still be pending
                    if (s == 0) {
                        cp_async_wait<1>();
                        if (!ALIGNED) __syncwarp();  // a lane reads windows its quad neighbours copied
                    }
                    uint4 cwa, cwb;
                    read_weights<ALIGNED>(stage0 + s * kStageBytes, lane, t, mis, cwa, cwb);
                    load_x<NT>(xf[b ^ 1], xsrc + (s + 1) * 128, x_mask, p.kp);  // reads past the segment are harmless
                    consume_chunk<NT>(cwa, cwb, bf16_bits_to_float(prm[b].sa), bf16_bits_to_float(prm[b].sb),
                                      bf16_bits_to_float(prm[b].ba), bf16_bits_to_float(prm[b].bb), xf[b], xs + s * xs_step, mg, acc);
                    load_params<ALIGNED>(prm[b], sa + (s + 2) * 4, sb + (s + 2) * 4, ba + (s + 2) * 4, bb + (s + 2) * 4, ci + s + 2 < param_n);
                }
            }
            if (!ALIGNED) __syncwarp();  // everyone has read before the stages are refilled
#pragma unroll
            for (int s = 0; s < 4; ++s)
                issue_weights<ALIGNED>(stage0 + s * kStageBytes, wa + (s + kStages) * 64, wb + (s + kStages) * 64, lane, t,
                                       ci + s + kStages < n, mis, c0 + ci + s + kStages < full_chunks);
            cp_async_commit();
            wa += 4 * 64;
            wb += 4 * 64;
            sa += 16;
            sb += 16;
            ba += 16;
            bb += 16;
            xsrc += 4 * 128;
            xs += 4 * xs_step;
            half ^= 1u;
        }
        cp_async_wait<0>();

        finish_tile<NT>(p, p.row_inv, split, worker, tile, c0 == 0 && c1 == cpt, acc, lane, g, t, job_index, (uint64_t)tile * cpt, cpt);
        u += n;
        ++tile;
        c0 = 0;
    }
}

// Fast variant: weights, scales and biases start on 16-byte boundaries and the group count is a
// multiple of 8 (K % 512 == 0), so parameters ride the same async path as the weights: per four chunks
// one 16-byte copy per row and array (8 groups = 4 chunks), read back with one 128-bit shared load.
// Shared memory per warp: 8 weight stages of 1 KB and 2 parameter stages of 512 B.
constexpr int kFastRingBytes = kStages * kStageBytesAligned + 2 * 512;

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

template <int NT>
__global__ void __launch_bounds__(32, NT == 1 ? 20 : 16) q4_gemv_fast_kernel(const __grid_constant__ GemvParams p) {
    extern __shared__ __align__(128) uint8_t ring_bytes[];
    const uint32_t lane = threadIdx.x;
    if (p.trace && lane == 0) p.trace[blockIdx.x * 4 + 0] = global_ns();
    bool first_data = true;
    const uint32_t g = lane >> 2, t = lane & 3u;
    const uint32_t worker = blockIdx.x;
    const Q4Split split{p.units, p.cpt, p.workers};
    uint64_t u = q4_split_begin(split, worker);
    const uint64_t u1 = q4_split_begin(split, worker + 1);
    const uint32_t cpt = p.cpt, groups = p.groups;
    const bool x_lane = ((g < 4u) == (t < 2u));
    const uint32_t v_first = g & 3u;
    uint32_t x_mask = 0;
#pragma unroll
    for (int j = 0; j < NT; ++j) x_mask |= (x_lane && (v_first + 4u * j < p.v_cols)) ? (1u << j) : 0u;
    const uint16_t *xfrag0 = p.xp + (size_t)v_first * p.kp + t * 32u;
    const float *xs0 = p.xsum + (size_t)(t >> 1) * p.vpad + 2u * (t & 1u);
    const uint32_t xs_step = 2u * p.vpad;
    const uint32_t half_sel = (t >> 1) ? 0x3244u : 0x1044u;
    const Magic mg = make_magic();
    const uint32_t ring = (uint32_t)__cvta_generic_to_shared(ring_bytes);
    const uint32_t pring = ring + kStages * kStageBytesAligned;
    // parameter copies: lane l moves 16 bytes of row (l & 15) of array (l >> 4: scales, biases)
    const uint32_t prow = lane & 15u;
    uint4 xf[2][NT][4];
#pragma unroll
    for (int b = 0; b < 2; ++b)
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int w = 0; w < 4; ++w) xf[b][j][w] = make_uint4(0, 0, 0, 0);

    uint32_t tile = (uint32_t)(u / cpt);
    uint32_t c0 = (uint32_t)(u - (uint64_t)tile * cpt);
    uint32_t job_index = 0;
    while (u < u1) {
        const uint64_t left = u1 - u;
        const uint32_t c1 = (left < (uint64_t)(cpt - c0)) ? c0 + (uint32_t)left : cpt;
        while (job_index + 1 < p.n_jobs && tile >= p.jobs[job_index + 1].tile_begin) ++job_index;
        const GemvJob &job = p.jobs[job_index];
        const uint32_t cbase = c0 & ~3u;  // chunks are handled in aligned groups of four
        // per-lane cursors at chunk cbase
        const uint8_t *wa, *wb, *pp;
        {
            const uint32_t row0 = (tile - job.tile_begin) * 16u;
            uint32_t row_a = row0 + g, row_b = row0 + g + 8u, row_p = row0 + prow;
            row_a = row_a < job.n ? row_a : job.n - 1u;  // rows past N read a valid row and are never stored
            row_b = row_b < job.n ? row_b : job.n - 1u;
            row_p = row_p < job.n ? row_p : job.n - 1u;
            const uint64_t row_bytes = (uint64_t)p.k >> 1;
            wa = job.w + (uint64_t)row_a * row_bytes + t * 16u + cbase * 64u;
            wb = job.w + (uint64_t)row_b * row_bytes + t * 16u + cbase * 64u;
            pp = ((lane >> 4) ? job.b : job.s) + ((uint64_t)row_p * groups) * 2u + cbase * 4u;
        }
        const uint16_t *xsrc = xfrag0 + cbase * 128u;
        const float *xs = xs0 + (size_t)cbase * xs_step;
        float acc[NT][4];
#pragma unroll
        for (int j = 0; j < NT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;

        // prologue: the first two groups of four chunks (weights of chunks in [c0,c1) only), first activations
#pragma unroll
        for (int h = 0; h < 2; ++h) {
#pragma unroll
            for (int s = 0; s < 4; ++s) {
                const uint32_t c = cbase + 4 * h + s;
                const uint32_t stage = ring + (4 * h + s) * kStageBytesAligned;
                cp_async_16_pred(stage + lane * 16u, wa + (4 * h + s) * 64, c >= c0 && c < c1);
                cp_async_16_pred(stage + 512u + lane * 16u, wb + (4 * h + s) * 64, c >= c0 && c < c1);
            }
            cp_async_16_pred(pring + h * 512u + lane * 16u, pp + h * 16, cbase + 4 * h < c1);
            cp_async_commit();
        }
        if (c0 & 1u) load_x<NT>(xf[1], xsrc + (c0 - cbase) * 128u, x_mask, p.kp);
        else load_x<NT>(xf[0], xsrc + (c0 - cbase) * 128u, x_mask, p.kp);

        uint32_t half = 0;
        for (uint32_t cg = cbase; cg < c1; cg += 4) {
            const uint32_t stage0 = ring + half * (4 * kStageBytesAligned) + lane * 16u;
            const uint32_t pstage = pring + half * 512u;
            cp_async_wait<1>();  // this half's group has landed; the other half's may be pending
            __syncwarp();        // parameters were copied by other lanes
            if (p.trace && first_data) {
                if (lane == 0) p.trace[blockIdx.x * 4 + 1] = global_ns();
                first_data = false;
            }
            const uint4 psa = lds_v4(pstage + g * 16u), psb = lds_v4(pstage + (g + 8u) * 16u);
            const uint4 pba = lds_v4(pstage + 256u + g * 16u), pbb = lds_v4(pstage + 256u + (g + 8u) * 16u);
            const uint32_t wsa[4] = {psa.x, psa.y, psa.z, psa.w}, wsb[4] = {psb.x, psb.y, psb.z, psb.w};
            const uint32_t wba[4] = {pba.x, pba.y, pba.z, pba.w}, wbb[4] = {pbb.x, pbb.y, pbb.z, pbb.w};
            if (cg >= c0 && cg + 12 <= c1) {
                // steady state: all four chunks and all four refills lie inside the segment
                uint4 cwa = lds_v4(stage0), cwb = lds_v4(stage0 + 512u);
#pragma unroll
                for (int s = 0; s < 4; ++s) {
                    const int b = s & 1;
                    uint4 nwa = cwa, nwb = cwb;
                    if (s < 3) {  // next chunk's weights leave shared memory while this one is computed
                        nwa = lds_v4(stage0 + (s + 1) * kStageBytesAligned);
                        nwb = lds_v4(stage0 + (s + 1) * kStageBytesAligned + 512u);
                    }
                    load_x<NT>(xf[b ^ 1], xsrc + (s + 1) * 128, x_mask, p.kp);
                    consume_chunk<NT>(cwa, cwb, param_of(wsa[s], half_sel), param_of(wsb[s], half_sel),
                                      param_of(wba[s], half_sel), param_of(wbb[s], half_sel), xf[b], xs + s * xs_step, mg, acc);
                    cwa = nwa;
                    cwb = nwb;
                }
                __syncwarp();  // every lane is done with this half before it is refilled
#pragma unroll
                for (int s = 0; s < 4; ++s) {
                    cp_async_16(stage0 + s * kStageBytesAligned, wa + (8 + s) * 64);
                    cp_async_16(stage0 + s * kStageBytesAligned + 512u, wb + (8 + s) * 64);
                }
                cp_async_16(pstage + lane * 16u, pp + 32);
            } else {
#pragma unroll
                for (int s = 0; s < 4; ++s) {
                    const uint32_t c = cg + s;
                    if (c >= c0 && c < c1) {
                        const int b = s & 1;
                        const uint32_t stage = stage0 + s * kStageBytesAligned;
                        const uint4 cwa = lds_v4(stage), cwb = lds_v4(stage + 512u);
                        load_x<NT>(xf[b ^ 1], xsrc + (s + 1) * 128, x_mask, p.kp);  // reads past the segment are harmless
                        consume_chunk<NT>(cwa, cwb, param_of(wsa[s], half_sel), param_of(wsb[s], half_sel),
                                          param_of(wba[s], half_sel), param_of(wbb[s], half_sel), xf[b], xs + s * xs_step, mg, acc);
                    }
                }
                __syncwarp();
#pragma unroll
                for (int s = 0; s < 4; ++s) {
                    const bool more = cg + 8 + s < c1;
                    cp_async_16_pred(stage0 + s * kStageBytesAligned, wa + (8 + s) * 64, more);
                    cp_async_16_pred(stage0 + s * kStageBytesAligned + 512u, wb + (8 + s) * 64, more);
                }
                cp_async_16_pred(pstage + lane * 16u, pp + 32, cg + 8 < c1);
            }
            cp_async_commit();
            wa += 4 * 64;
            wb += 4 * 64;
            pp += 16;
            xsrc += 4 * 128;
            xs += 4 * xs_step;
            half ^= 1u;
        }
        cp_async_wait<0>();
        __syncwarp();
        if (p.trace && lane == 0) p.trace[blockIdx.x * 4 + 2] = global_ns();
        finish_tile<NT>(p, p.row_inv, split, worker, tile, c0 == 0 && c1 == cpt, acc, lane, g, t, job_index, (uint64_t)tile * cpt, cpt);
        u += c1 - c0;
        ++tile;
        c0 = 0;
    }
    if (p.trace && lane == 0) p.trace[blockIdx.x * 4 + 3] = global_ns();
}

}  // namespace q4

// ---------------------------------------------------------------------------------------------
// Host launchers
// ---------------------------------------------------------------------------------------------

extern "C" cudaError_t q4k_prepare_x(const void *x, int x_is_f32, uint32_t m_rows, uint32_t k, uint32_t kp, uint32_t vpad,
                                     uint16_t *xp, float *xsum, float *row_inv, cudaStream_t stream) {
    q4::q4_prepare_x_kernel<<<m_rows, 256, 0, stream>>>(x, x_is_f32, k, kp, vpad, xp, xsum, row_inv);
    return cudaGetLastError();
}

namespace {

constexpr size_t kGenericRingBytes = (size_t)q4::kStages * q4::kStageBytesWindowed;

template <int NT>
uint32_t occupancy_of(bool fast) {
    int blocks = 0;
    cudaError_t e = fast ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, q4::q4_gemv_fast_kernel<NT>, 32, q4::kFastRingBytes)
                         : cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, q4::q4_gemv_generic_kernel<NT>, 32, kGenericRingBytes);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return blocks > 0 ? (uint32_t)blocks : 0u;
}

}  // namespace

// resident warps (= blocks) per SM of a variant
extern "C" uint32_t q4k_gemv_occupancy(int column_tiles, int fast) {
    if (column_tiles == 1) return occupancy_of<1>(fast != 0);
    if (column_tiles == 2) return occupancy_of<2>(fast != 0);
    return 0;
}

// one warp per block: `workers` blocks. fast: every job of the launch meets the fast variant's
// alignment and shape conditions.
extern "C" cudaError_t q4k_gemv(const q4::GemvParams *params, int column_tiles, int fast, cudaStream_t stream) {
    const dim3 grid(params->workers), block(32);
    if (column_tiles == 1) {
        if (fast) q4::q4_gemv_fast_kernel<1><<<grid, block, q4::kFastRingBytes, stream>>>(*params);
        else q4::q4_gemv_generic_kernel<1><<<grid, block, kGenericRingBytes, stream>>>(*params);
    } else if (column_tiles == 2) {
        if (fast) q4::q4_gemv_fast_kernel<2><<<grid, block, q4::kFastRingBytes, stream>>>(*params);
        else q4::q4_gemv_generic_kernel<2><<<grid, block, kGenericRingBytes, stream>>>(*params);
    } else {
        return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}
