// Program format of the persistent decode kernel (q4_decode_stack.cu), shared with the host code that compiles a
// stage list into it (q4_runtime.cu). Plain structs, uploaded to device memory once per chain.
//
// A chain is a flat list of PHASES that every block walks in order. A phase is a set of projections over one
// activation held in shared memory, optionally preceded by a wait on the previous barrier plus the rebuild of that
// activation, and optionally followed by an arrival at the next barrier. Arrival and wait are separate steps: the
// phases between them are projections whose results nothing later in the chain reads (Q/K/V and the DeltaNet inputs
// of the reference's layer, src/metal_runtime.rs:3463-3517), so the weight stream keeps running while the barrier
// completes.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "q4_kernels.h"

namespace q4 {

constexpr uint32_t kPartialSets = 8;   // split-tile scratch sets, used round robin by consecutive phases
constexpr uint32_t kMaxPhases = 4096;  // phases per chain (the tag of a partial slot is launch * kMaxPhases + phase + 1)

// One projection of a phase. A tile is 16 accumulator rows: rows 0..7 ("side a") and rows 8..15 ("side b").
//   ordinary job: both sides come from one tensor, side b is 8 rows further down (rows_per_tile 16, b_row_offset 8);
//   gate/up pair: side a is a row of the gate tensor, side b the same row of the up tensor (rows_per_tile 8,
//                 b_row_offset 0); the epilogue forms bf16(silu(gate) * up) from the two sums of a lane.
// Rows may be strided views (w_stride, p_stride): a K-slice of a wider matrix is read in place.
struct StackJob {
    const uint8_t *w[2];   // packed weights at the first input of the slice, per side
    const uint8_t *s[2];   // scales
    const uint8_t *b[2];   // biases
    float *out[2];         // fp32 results per side, indexed by row; pair: either may be null
    float *peer_out[kMaxPeers];  // other ranks' copies of out[0] (ordinary jobs), null where not wanted
    // Tagged hand-off (ordinary jobs): every result is also stored as an 8-byte {value, tag} word into this GPU's copy
    // and every other rank's copy of a vector that the next stage's rebuild polls -- value and tag travel in one store,
    // so neither a fence nor a barrier stands between producer and consumer, on one GPU or across NVLink.
    unsigned long long *ll_out[kMaxPeers];  // indexed by row; null entries are skipped; all null: no hand-off
    unsigned long long *h_out;  // pair: {bf16(silu(a) * b) of rows 2i and 2i+1, tag} as one 8-byte word, indexed by i
    uint32_t n;            // rows per side
    uint32_t rows_per_tile, b_row_offset;
    uint32_t w_stride, p_stride;  // bytes between rows of the weight / parameter arrays (multiples of 16)
    uint32_t tile_begin;   // first tile of this job in the phase
    uint32_t unit_begin;   // first unit of this job in the phase
    uint32_t vcpt;         // units a tile counts for when the phase is cut into equal ranges (>= cpt; the extra ones are
                           // empty, so a job whose chunks cost more -- weights at a byte offset -- gets fewer per warp)
    uint32_t pair;
    uint32_t has_peers;
    uint32_t has_ll;
    uint32_t pad;
};

enum : uint32_t { kRebuildNone = 0, kRebuildBf16 = 1, kRebuildSwiglu = 2, kRebuildRms = 3, kRebuildH = 4, kRebuildF32 = 5 };
enum : uint32_t { kSyncNone = 0, kSyncLocal = 1, kSyncGlobal = 2 };

struct StackPhase {
    uint32_t job_begin, n_jobs;
    uint32_t k, kp, groups, cpt;  // inputs of this phase's activation (a K-slice counts its own inputs)
    uint32_t workers;             // warps that take part
    uint32_t tiles;               // 16-row tiles of all jobs
    // K-major mapping (0 or 1: off). Every tile is cut into `kparts` equal runs of chunks and a block works on ONE of
    // them -- part blockIdx % kparts of the 16 tiles (blockIdx / kparts) * 16 + warp -- so it rebuilds and holds only
    // that slice of the activation. Worker numbers stay tile * kparts + part.
    uint32_t kparts;
    uint32_t sliced;              // the activation buffer holds only the block's part (set on the phase that rebuilds it;
                                  // phases that reuse a buffer built whole leave it 0)
    uint32_t x_buf;               // which of the two shared-memory activation buffers the phase reads
    uint64_t units;
    uint32_t wait_kind;           // wait for the latest arrival (this GPU's blocks / all ranks) before the phase
    uint32_t x_kind;              // how the activation is rebuilt after the wait (kRebuild*)
    const void *src0, *src1;      // Bf16: bf16[k]; F32: fp32[k]; Swiglu: fp32 gate[k], up[k]; Rms: fp32 [src_parts][k]; H: tagged words [k/2]
    uint32_t src_parts, src_part_stride;  // Rms: the vector is the sum, in order, of src_parts vectors this many bytes apart
    uint32_t src_tagged;          // Rms: the source vectors are {value, tag} words written by phase src_tag_phase of this
    uint32_t src_tag_phase;       //      launch; the rebuild polls until every word carries that phase's tag (H: always)
    uint16_t *x_bf16_out;         // optional: block 0 stores the bf16 activation it built
    float *sum_out;               // optional (Rms): block 0 stores the summed fp32 vector
    float eps;
    uint32_t arrive_kind;         // arrival after the phase's units
    uint32_t slot_set;            // split-tile scratch set
    uint32_t pad;
};

// Cross-GPU part of a sharded chain: every rank runs the same program on its own slices.
struct StackPeers {
    uint32_t world, rank;
    unsigned long long *flag_local;            // arrivals of whole ranks at cross-GPU barriers, in this GPU's memory
    unsigned long long *flag_peer[kMaxPeers];  // the same word on every rank (this rank's included)
    unsigned long long *consumed;              // arrivals already accounted for by earlier launches (this GPU's memory)
    float2 *cand_local;                        // [kMaxPeers] (best logit, token id) per vocabulary slice
    float2 *cand_peer[kMaxPeers];
};

struct StackParams {
    const StackPhase *phases;
    const StackJob *jobs;
    uint32_t n_phases;
    uint32_t halfs[2];        // capacity of the two activation buffers in inputs (3 bytes each); the second may be 0
    unsigned int *local_bar;  // [0] arrivals of this GPU's blocks, [1] blocks that have finished; zero at launch, put back
                              // to zero by the last block of a launch
    int *error_flag;
    uint4 *partials;          // [kPartialSets][max_workers][32 lanes] of {sum a, tag, sum b, tag}
    unsigned int *launch_seq; // launches of this chain so far (read at the start, advanced at the end of the kernel)
    uint32_t max_workers;
    uint32_t spin_limit;      // polls before a wait gives up
    uint32_t flags;           // kFlag*
    const float *logits;      // output of the last phase to reduce to a token, or null
    uint32_t vocab, index_base;
    float *part_val;          // [gridDim.x]
    uint32_t *part_idx;       // [gridDim.x]
    uint32_t *token;
    float *best;
    const StackPeers *peers;  // null on one GPU
    uint32_t long_rebuild;    // some phase rebuilds a vector of more than two blocks of 8 per thread (picks the kernel instance)
    unsigned long long *trace;  // optional [blocks][n_phases][8] device-clock stamps
};

// A program of one phase inside the kernel parameters (q4_stack_inline_kernel).
struct InlineProgram {
    StackParams params;  // phases, jobs and n_phases are ignored
    StackPhase phase;
    StackJob jobs[kMaxJobs];
};

constexpr uint32_t kFlagRequestAfterRebuild = 2u;  // a phase that rebuilds its activation requests its first weights after the rebuild
constexpr uint32_t kFlagLateSkipsRequest = 4u;     // ... only for warps that finish a phase when all but (flags >> 8 & 255) blocks are through
constexpr uint32_t kProgressWord = 32;             // local_bar[kProgressWord]: blocks through with a phase, summed over the launch
constexpr uint32_t kFlagWarpFenceGpu = 1u;  // every warp fences at device scope before it arrives (default: block scope)

constexpr uint32_t kTraceStamps = 16;  // wait begin, wait end, rebuild end, warp 0 units end, block's arrival, SM id, last warp's units end,
                                      // thread 0 has read its source values (inside the rebuild)

}  // namespace q4

extern "C" {
uint32_t q4k_stack_warps(void);
uint32_t q4k_stack_max_k(void);       // longest activation the Bf16/Swiglu/Rms rebuilds handle
size_t q4k_stack_smem_bytes(uint32_t halfs0, uint32_t halfs1);
int q4k_stack_supported(uint32_t halfs0, uint32_t halfs1);
int q4k_stack_phase_is_long(const q4::StackPhase *phase);
cudaError_t q4k_stack_launch(const q4::StackParams *params, int sm_count, cudaStream_t stream);
int q4k_stack_inline_supported(uint32_t halfs);
cudaError_t q4k_stack_launch_inline(const q4::InlineProgram *program, int sm_count, cudaStream_t stream);
}
