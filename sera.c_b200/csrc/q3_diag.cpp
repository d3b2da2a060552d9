/* q3_diag.cpp - pure-host inspection of the launch schedule through the C ABI
 * (no CUDA call): lets tests check on a machine without a GPU that every key
 * tile of every item is covered exactly once and that the pieces of cut items
 * have partial slots of their own. */
#include <string.h>

#include "q3_attn.h"
#include "q3_sched.h"

extern "C" bool q3_schedule_describe(uint32_t tokens, uint32_t n_kv_heads,
                                     uint32_t shared_len, const uint32_t *row_tag,
                                     const uint32_t *row_lp, uint32_t pages_per_branch,
                                     uint32_t n_branches, uint32_t num_ctas,
                                     uint32_t max_slots, bool lockstep,
                                     q3_sched_summary *summary,
                                     q3_sched_segment_info *segments,
                                     uint32_t max_segments, char *error,
                                     size_t error_len) {
    if (error && error_len) error[0] = '\0';
    if (!row_tag || !row_lp || !summary) {
        if (error && error_len) strncpy(error, "q3_schedule_describe: invalid argument", error_len - 1);
        return false;
    }
    std::vector<uint32_t> shared((shared_len + 15u) / 16u);
    for (size_t i = 0; i < shared.size(); i++) shared[i] = (uint32_t)i;
    std::vector<uint32_t> priv((size_t)pages_per_branch * n_branches);
    for (size_t i = 0; i < priv.size(); i++) priv[i] = (uint32_t)(shared.size() + i);
    q3_schedule s;
    if (!q3_build_schedule(s, tokens, n_kv_heads, shared_len, shared, row_tag, row_lp, priv,
                           pages_per_branch, num_ctas, max_slots, lockstep, error,
                           error_len))
        return false;
    summary->grid = s.grid;
    summary->n_segments = (uint32_t)s.segments.size();
    summary->n_cut_items = s.n_cut_items;
    summary->n_slots = s.n_slots;
    summary->total_key_tiles = s.total_key_tiles;
    if (segments) {
        uint32_t cta = 0;
        for (uint32_t i = 0; i < s.segments.size() && i < max_segments; i++) {
            while (cta + 1 <= s.grid && s.cta_seg_begin[cta + 1] <= i) cta++;
            const q3_segment &g = s.segments[i];
            segments[i].cta = cta;
            segments[i].tok0 = g.tok0;
            segments[i].kv_head = g.kv_head;
            segments[i].tile_begin = g.tile_begin;
            segments[i].tile_end = g.tile_end;
            segments[i].shared_tiles = g.shared_tiles;
            segments[i].partial_slot = g.partial_slot;
        }
    }
    return true;
}
