/* q3_sched.cpp - see q3_sched.h. Pure host code, no CUDA. */
#include "q3_sched.h"

#include <stdio.h>

#include <algorithm>

/* start-up cost of a segment, in quarter key tiles */
#ifndef Q3_SCHED_SEGMENT_COST
#define Q3_SCHED_SEGMENT_COST 10
#endif

static bool sched_fail(char *error, size_t error_len, const char *msg) {
    if (error && error_len) snprintf(error, error_len, "%s", msg);
    return false;
}

bool q3_build_schedule(q3_schedule &s, uint32_t tokens, uint32_t n_kv_heads,
                       uint32_t shared_len,
                       const std::vector<uint32_t> &shared_pages,
                       const uint32_t *row_tag, const uint32_t *row_lp,
                       const std::vector<uint32_t> &private_table,
                       uint32_t private_stride, uint32_t num_ctas,
                       uint32_t max_slots, bool lockstep, char *error,
                       size_t error_len) {
    s = q3_schedule();
    if (tokens == 0 || n_kv_heads == 0 || num_ctas == 0)
        return sched_fail(error, error_len, "schedule: empty launch");
    const uint32_t n_shared_pages = (shared_len + 15u) / 16u;
    if (shared_pages.size() < n_shared_pages)
        return sched_fail(error, error_len, "schedule: shared page table too short");
    s.tokens = tokens;
    s.n_kv_heads = n_kv_heads;
    s.shared_len = shared_len;
    s.n_shared_pages = n_shared_pages;
    s.page_ids.assign(shared_pages.begin(), shared_pages.begin() + n_shared_pages);
    s.page_ids.insert(s.page_ids.end(), private_table.begin(), private_table.end());
    s.row_tag.assign(row_tag, row_tag + tokens);
    s.row_lp.assign(row_lp, row_lp + tokens);

    /* Runs: distinct branches of each token tile, in order of first
     * appearance, each with the pages its rows can see. */
    const uint32_t n_tok_tiles = (tokens + Q3_TOK_TILE - 1) / Q3_TOK_TILE;
    std::vector<uint32_t> tile_run_begin(n_tok_tiles + 1);
    std::vector<uint32_t> tile_private_pages(n_tok_tiles);
    for (uint32_t tt = 0; tt < n_tok_tiles; tt++) {
        tile_run_begin[tt] = (uint32_t)s.runs.size();
        const uint32_t t0 = tt * Q3_TOK_TILE;
        const uint32_t t1 = std::min(tokens, t0 + Q3_TOK_TILE);
        const size_t first = s.runs.size();
        for (uint32_t t = t0; t < t1; t++) {
            const uint32_t need = row_lp[t] / 16u + 1u;
            size_t r = first;
            for (; r < s.runs.size(); r++)
                if (s.runs[r].tag == row_tag[t]) break;
            if (r == s.runs.size()) {
                if (need > private_stride ||
                    (uint64_t)row_tag[t] * private_stride + private_stride >
                        private_table.size())
                    return sched_fail(error, error_len,
                                      "schedule: private page table too short");
                q3_run run;
                run.table_off = n_shared_pages + row_tag[t] * private_stride;
                run.n_pages = need;
                run.tag = row_tag[t];
                run.pad = 0;
                s.runs.push_back(run);
            } else if (need > s.runs[r].n_pages) {
                if (need > private_stride)
                    return sched_fail(error, error_len,
                                      "schedule: private page table too short");
                s.runs[r].n_pages = need;
            }
        }
        uint32_t pages = 0;
        for (size_t r = first; r < s.runs.size(); r++) pages += s.runs[r].n_pages;
        tile_private_pages[tt] = pages;
    }
    tile_run_begin[n_tok_tiles] = (uint32_t)s.runs.size();

    /* Items in (kv_head, token tile) order and their key-tile counts. */
    const uint32_t shared_tiles =
        (n_shared_pages + Q3_KEY_TILE_PAGES - 1) / Q3_KEY_TILE_PAGES;
    uint64_t total = 0;
    std::vector<uint32_t> item_tiles(n_tok_tiles);
    for (uint32_t tt = 0; tt < n_tok_tiles; tt++) {
        item_tiles[tt] = shared_tiles + (tile_private_pages[tt] + Q3_KEY_TILE_PAGES - 1) /
                                            Q3_KEY_TILE_PAGES;
        total += item_tiles[tt];
    }
    total *= n_kv_heads;
    s.total_key_tiles = total;
    const uint32_t grid = (uint32_t)std::min<uint64_t>(num_ctas, total);
    s.grid = grid;
    s.cta_seg_begin.assign(grid + 1, 0);

    /* Assignment of key tiles to CTAs.
     *  - stream-K: CTA c owns global key tiles [c*total/grid, (c+1)*total/grid)
     *    of the item list; perfect balance, CTAs sit at staggered offsets of
     *    their items.
     *  - lockstep waves + stream-K tail (when `lockstep`): the first
     *    floor(items/grid)*grid items are handed out whole, wave by wave, so
     *    that all CTAs walk the same key tiles of neighbouring items at the
     *    same time and share them through L2; only the remaining items are
     *    cut stream-K style. Chosen by the caller when the shared KV of all
     *    heads would not stay in L2 under staggered access. */
    struct Item { uint32_t h, tt, n; };
    std::vector<Item> items;
    items.reserve((size_t)n_kv_heads * n_tok_tiles);
    for (uint32_t h = 0; h < n_kv_heads; h++)
        for (uint32_t tt = 0; tt < n_tok_tiles; tt++)
            items.push_back(Item{h, tt, item_tiles[tt]});
    struct Piece { uint32_t item, begin, end; };
    std::vector<std::vector<Piece>> per_cta(grid);
    size_t first_tail = 0;
    if (lockstep && items.size() >= grid) {
        const size_t waves = items.size() / grid;
        for (size_t w = 0; w < waves; w++)
            for (uint32_t c = 0; c < grid; c++) {
                const uint32_t i = (uint32_t)(w * grid + c);
                per_cta[c].push_back(Piece{i, 0, items[i].n});
            }
        first_tail = waves * grid;
    }
    {
        /* Cost-balanced stream-K over items [first_tail, end): a segment costs
         * its key tiles plus a fixed start-up (Q load, pipeline fill, epilogue),
         * so a CTA that receives many short items gets fewer tiles. Costs are
         * in quarter tiles. */
        const uint64_t F = Q3_SCHED_SEGMENT_COST;
        uint64_t rem = 0;   /* cost not yet handed out */
        for (size_t i = first_tail; i < items.size(); i++) rem += 4ull * items[i].n + F;
        rem += (uint64_t)(grid - 1) * F;   /* every CTA boundary cuts one item: its
                                              continuation pays the start-up again */
        uint32_t cta = 0;
        uint64_t budget = rem / grid, used = 0;
        for (size_t i = first_tail; i < items.size(); i++) {
            uint32_t done = 0;
            while (done < items[i].n) {
                if (cta + 1 < grid && used + F + 4 > budget) {
                    cta++;                        /* re-balance over what is left */
                    budget = rem / (grid - cta);
                    used = 0;
                }
                uint32_t take = items[i].n - done;
                if (cta + 1 < grid && budget > used + F)
                    take = (uint32_t)std::min<uint64_t>(take,
                                                        std::max<uint64_t>(1, (budget - used - F) / 4));
                per_cta[cta].push_back(Piece{(uint32_t)i, done, done + take});
                done += take;
                used += F + 4ull * take;
                rem -= std::min<uint64_t>(rem, F + 4ull * take);
            }
        }
    }
    /* Flatten; cut items get consecutive partial slots. */
    std::vector<uint32_t> item_pieces(items.size(), 0), item_slot(items.size(), 0);
    for (uint32_t c = 0; c < grid; c++)
        for (const Piece &pc : per_cta[c]) item_pieces[pc.item]++;
    for (size_t i = 0; i < items.size(); i++) {
        if (item_pieces[i] > 1) {
            if (s.n_slots + item_pieces[i] > max_slots)
                return sched_fail(error, error_len, "schedule: out of partial slots");
            item_slot[i] = s.n_slots;
            s.n_slots += item_pieces[i];
            s.n_cut_items++;
        }
    }
    std::vector<uint32_t> item_next(items.size(), 0), item_fix(items.size(), 0);
    {
        uint32_t n_fix = 0;
        for (size_t i = 0; i < items.size(); i++)
            if (item_pieces[i] > 1) item_fix[i] = n_fix++;
    }
    for (uint32_t c = 0; c < grid; c++) {
        /* pieces of cut items first: their last-arriver combination then
         * happens early instead of at the very end of the launch */
        std::stable_partition(per_cta[c].begin(), per_cta[c].end(),
                              [&](const Piece &pc) { return item_pieces[pc.item] > 1; });
        s.cta_seg_begin[c] = (uint32_t)s.segments.size();
        for (const Piece &pc : per_cta[c]) {
            const Item &it = items[pc.item];
            q3_segment seg;
            seg.tok0 = it.tt * Q3_TOK_TILE;
            seg.kv_head = it.h;
            seg.tile_begin = pc.begin;
            seg.tile_end = pc.end;
            seg.shared_tiles = shared_tiles;
            seg.partial_slot = item_pieces[pc.item] > 1
                                   ? (int32_t)(item_slot[pc.item] + item_next[pc.item]++)
                                   : -1;
            seg.run_begin = tile_run_begin[it.tt];
            seg.run_end = tile_run_begin[it.tt + 1];
            seg.slot_begin = item_slot[pc.item];
            seg.slot_count = item_pieces[pc.item] > 1 ? item_pieces[pc.item] : 0;
            seg.fix_index = item_fix[pc.item];
            seg.pad = 0;
            s.segments.push_back(seg);
        }
    }
    s.cta_seg_begin[grid] = (uint32_t)s.segments.size();
    return true;
}

void q3_build_decode_work(const uint32_t *ctx_lens, uint32_t num_seqs,
                          uint32_t extra_token, uint32_t chunk_pages,
                          std::vector<q3_decode_work> &work,
                          std::vector<uint32_t> &seq_work_begin) {
    work.clear();
    seq_work_begin.assign(num_seqs + 1, 0);
    for (uint32_t sidx = 0; sidx < num_seqs; sidx++) {
        seq_work_begin[sidx] = (uint32_t)work.size();
        const uint32_t keys = ctx_lens[sidx] + extra_token;
        const uint32_t pages = (keys + 15u) / 16u;
        /* equal-size chunks, none longer than chunk_pages */
        const uint32_t n_chunks = std::max(1u, (pages + chunk_pages - 1) / chunk_pages);
        for (uint32_t c = 0; c < n_chunks; c++) {
            q3_decode_work w;
            w.seq = sidx;
            w.page_begin = (uint32_t)((uint64_t)c * pages / n_chunks);
            w.page_end = (uint32_t)((uint64_t)(c + 1) * pages / n_chunks);
            w.slot = (uint32_t)work.size();
            work.push_back(w);
        }
    }
    seq_work_begin[num_seqs] = (uint32_t)work.size();
}
