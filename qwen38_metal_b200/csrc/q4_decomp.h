// Work decomposition of the streaming (decode) projection kernel, shared by device and host
// code so the index arithmetic can be unit-tested on a CPU.
//
// A launch covers `tiles` row tiles (16 output rows each, over all jobs of the launch) times
// `cpt` K-chunks per tile (a chunk is 128 inputs = two affine groups = 64 packed bytes per
// row). The tiles*cpt units are numbered tile-major and cut into `workers` contiguous,
// near-equal ranges, one per warp. A tile whose units fall into more than one range is
// summed through per-warp partial slots by the last warp to arrive, in worker order.
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define Q4_HD __host__ __device__ __forceinline__
#else
#define Q4_HD inline
#endif

struct Q4Split {
    uint64_t units;    // tiles * cpt
    uint32_t cpt;      // chunks per tile
    uint32_t workers;  // warps in the grid
};

// first unit of worker w (w may equal workers: one past the last unit)
Q4_HD uint64_t q4_split_begin(const Q4Split &s, uint32_t w) {
    return (s.units * (uint64_t)w) / s.workers;
}

// the worker whose range holds unit u
Q4_HD uint32_t q4_split_owner(const Q4Split &s, uint64_t u) {
    return (uint32_t)((((u + 1) * (uint64_t)s.workers) - 1) / s.units);
}

// workers contributing to the units [u0, u0 + span): [first, last]
Q4_HD void q4_split_span_contributors(const Q4Split &s, uint64_t u0, uint32_t span, uint32_t *first, uint32_t *last) {
    *first = q4_split_owner(s, u0);
    *last = q4_split_owner(s, u0 + span - 1);
}

// workers contributing to tile t when every tile has s.cpt units: [first, last]
Q4_HD void q4_split_contributors(const Q4Split &s, uint32_t tile, uint32_t *first, uint32_t *last) {
    q4_split_span_contributors(s, (uint64_t)tile * s.cpt, s.cpt, first, last);
}

// partial slot worker w uses for tile t: slot 0 when t is the tile its range starts in, else 1
Q4_HD uint32_t q4_split_slot(const Q4Split &s, uint32_t w, uint32_t tile) {
    uint32_t head_tile = (uint32_t)(q4_split_begin(s, w) / s.cpt);
    return 2u * w + (tile == head_tile ? 0u : 1u);
}

// Byte-addressed variant of the streaming kernel: which aligned 16-byte windows it asks for. A chunk is 64 packed
// bytes of a row: lanes t = 0,1 of a quad hold affine group A (bytes 0..31), lanes 2,3 group B (bytes 32..63), and
// the lane's window is the aligned 16 bytes that start `mis` bytes before its share ([16t - mis, 16t - mis + 16)); a
// lane completes its 16 bytes from the window after its own, so the quad needs a fifth window when mis != 0. Every
// window the kernel asks for holds at least one byte of the row, so nothing outside the 16-byte blocks that the
// tensor itself touches is ever read. `has_b`: group B of this chunk exists (the last chunk of a row with an odd
// number of groups has only group A).
Q4_HD bool q4_window_wanted(uint32_t t, uint32_t mis, bool has_b) {
    if (t < 2u) return true;
    if (t == 2u) return has_b || mis != 0u;  // its first `mis` bytes complete lane 1's share
    return has_b;
}
Q4_HD bool q4_fifth_window_wanted(uint32_t mis, bool has_b) { return has_b && mis != 0u; }
// chunks of a row in which lane t (0..3) of a quad has an affine group: group 2*chunk + (t >> 1) < groups
Q4_HD uint32_t q4_lane_chunks(uint32_t groups, uint32_t t) { return (groups + 1u - (t >> 1)) >> 1; }

// Short-batch kernel: the K range (cpt chunks of 128 inputs, a multiple of four) is cut into `parts` runs that begin at
// multiples of four chunks (parameters travel in 16-byte pieces of eight groups). First chunk of `part`; part may
// equal parts (one past the last chunk).
Q4_HD uint32_t q4_rows_part_begin(uint32_t cpt, uint32_t parts, uint32_t part) { return ((cpt / 4u) * part / parts) * 4u; }

// How many parts to cut K into for `tiles` 16-row tiles on `sm_count` SMs of 16 warps, each warp walking `tw` tiles at
// a time, when a block can hold at most `cap` chunks of activation digits; 0 when no split fits. *part_chunks: chunks
// of the longest part; *cost_out: the estimate the choice was made by.
// Cost of a split in chunk times: every warp walks `rounds` items of the longest run, a chunk of two tiles costs 1.75
// (measured; the activation's fragments are read once for both), an item costs about ten more per tile pair or single
// tile (pipeline ramp, partial sums, the last part's addition), and SMs without a block count against it.
Q4_HD uint32_t q4_rows_plan(uint32_t cpt, uint32_t tiles, uint32_t sm_count, uint32_t cap, uint32_t tw, uint32_t *part_chunks, double *cost_out) {
    if (cpt == 0 || cpt % 4u != 0 || tiles == 0 || sm_count == 0 || tw == 0) return 0;
    const uint32_t quads = cpt / 4u, items = (tiles + tw - 1u) / tw;
    const double per_chunk = tw == 1u ? 1.0 : 1.75, per_item = tw == 1u ? 10.0 : 12.0;
    uint32_t best = 0;
    double best_cost = 0.0;
    for (uint32_t parts = 1; parts <= quads && parts <= sm_count && parts <= 32u; ++parts) {
        const uint32_t bpp = sm_count / parts, warps = bpp * 16u;
        const uint32_t run = ((quads + parts - 1) / parts) * 4u;
        if (run > cap) continue;
        const uint32_t rounds = (items + warps - 1) / warps;
        const double cost = (double)rounds * (per_item + run * per_chunk) * sm_count / (double)(bpp * parts);
        if (best == 0 || cost < best_cost * 0.98) {
            best_cost = cost;
            best = parts;
        }
    }
    if (best == 0) return 0;
    *part_chunks = ((quads + best - 1) / best) * 4u;
    if (cost_out) *cost_out = best_cost;
    return best;
}
