// Host build of the device work-split arithmetic (qwen38_metal_b200/csrc/q4_decomp.h) for CPU tests.
#include "../qwen38_metal_b200/csrc/q4_decomp.h"
extern "C" {
uint64_t shim_begin(uint64_t units, uint32_t cpt, uint32_t workers, uint32_t w) { return q4_split_begin(Q4Split{units, cpt, workers}, w); }
uint32_t shim_owner(uint64_t units, uint32_t cpt, uint32_t workers, uint64_t u) { return q4_split_owner(Q4Split{units, cpt, workers}, u); }
void shim_contributors(uint64_t units, uint32_t cpt, uint32_t workers, uint32_t tile, uint32_t *first, uint32_t *last) {
    q4_split_contributors(Q4Split{units, cpt, workers}, tile, first, last);
}
int shim_window_wanted(uint32_t t, uint32_t mis, int has_b) { return q4_window_wanted(t, mis, has_b != 0) ? 1 : 0; }
int shim_fifth_window_wanted(uint32_t mis, int has_b) { return q4_fifth_window_wanted(mis, has_b != 0) ? 1 : 0; }
uint32_t shim_lane_chunks(uint32_t groups, uint32_t t) { return q4_lane_chunks(groups, t); }
uint32_t shim_rows_part_begin(uint32_t cpt, uint32_t parts, uint32_t part) { return q4_rows_part_begin(cpt, parts, part); }
uint32_t shim_rows_plan(uint32_t cpt, uint32_t tiles, uint32_t sm_count, uint32_t cap, uint32_t tw, uint32_t *part_chunks) { return q4_rows_plan(cpt, tiles, sm_count, cap, tw, part_chunks, nullptr); }
uint32_t shim_slot(uint64_t units, uint32_t cpt, uint32_t workers, uint32_t w, uint32_t tile) { return q4_split_slot(Q4Split{units, cpt, workers}, w, tile); }
}
