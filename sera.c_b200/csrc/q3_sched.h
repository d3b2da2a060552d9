/* q3_sched.h - host-side launch schedule of the tensor-core attention kernel.
 * Pure C++ (no CUDA): built once per batch, reused by every layer.
 *
 * Vocabulary
 *   token tile  32 consecutive packed query tokens (two 16-token MMA tiles of
 *               16 tokens x 8 query heads = 128 rows each).
 *   item        one (token tile, KV head) pair: the unit that owns an output.
 *   key stream  of an item: first the shared-prefix pages in order, padded to
 *               a multiple of 8 pages, then the private pages of every
 *               distinct branch in the tile (branch by branch, pages 0..max
 *               local position / 16), padded likewise. 8 pages = 128 keys =
 *               one key tile.
 *   segment     a contiguous range of key tiles of one item given to one CTA.
 *               The whole launch is cut stream-K style: every CTA receives the
 *               same cost; every piece of a cut item writes un-normalised
 *               partials, and the piece that finishes last combines them
 *               with log-sum-exp inside the kernel (no waiting: an arrival
 *               counter per item). A CTA runs its pieces of cut items before
 *               its whole items, so those combinations happen early.
 */
#ifndef Q3_SCHED_H
#define Q3_SCHED_H

#include <stdint.h>

#include <vector>

#define Q3_TOK_TILE 32u     /* query tokens per CTA work item */
#define Q3_KEY_TILE_PAGES 8u

struct q3_run {            /* private pages of one branch inside a token tile */
    uint32_t table_off;    /* index into page_ids of the branch's page 0      */
    uint32_t n_pages;      /* pages 0..n_pages-1 are streamed                 */
    uint32_t tag;          /* branch handle (0 for a plain causal sequence)   */
    uint32_t pad;
};

struct q3_segment {
    uint32_t tok0;         /* first packed token of the token tile            */
    uint32_t kv_head;
    uint32_t tile_begin;   /* key tiles [tile_begin, tile_end) of the stream  */
    uint32_t tile_end;
    uint32_t shared_tiles; /* key tiles of the shared part of the stream      */
    int32_t partial_slot;  /* -1: this segment is the whole item              */
    uint32_t run_begin;    /* runs[run_begin, run_end) of the token tile      */
    uint32_t run_end;
    uint32_t slot_begin;   /* cut item: its partial slots [slot_begin, +count) */
    uint32_t slot_count;
    uint32_t fix_index;    /* cut item: index of its arrival counters          */
    uint32_t pad;
};

struct q3_decode_work {
    uint32_t seq;
    uint32_t page_begin;   /* pages [page_begin, page_end) of the sequence    */
    uint32_t page_end;
    uint32_t slot;         /* partial slot (per KV head: slot*Hkv + head)     */
};

struct q3_schedule {
    uint32_t tokens = 0, n_kv_heads = 0, shared_len = 0, n_shared_pages = 0;
    std::vector<uint32_t> page_ids;       /* [shared | private tables]        */
    std::vector<uint32_t> row_tag, row_lp; /* per packed token                */
    std::vector<q3_run> runs;
    std::vector<q3_segment> segments;
    std::vector<uint32_t> cta_seg_begin;  /* [grid + 1]                       */
    uint32_t n_cut_items = 0;             /* items split over several CTAs    */
    uint32_t grid = 0;
    uint32_t n_slots = 0;
    uint64_t total_key_tiles = 0;
};

/* Build runs, items and segments.
 *   row_tag/row_lp   per token: branch handle and local position (a plain
 *                    causal sequence uses tag 0 and lp = absolute position)
 *   shared_pages     page ids of the shared prefix (ceil(shared_len/16))
 *   private_table    all private page tables, concatenated; the table of tag
 *                    g starts at g * private_stride and holds private_stride
 *                    entries
 *   num_ctas         CTAs the launch may use (SM count)
 *   max_slots        partial slots available
 *   lockstep         hand out whole items in waves first (see q3_sched.cpp)
 * Returns false with a message on an inconsistent description. */
bool q3_build_schedule(q3_schedule &s, uint32_t tokens, uint32_t n_kv_heads,
                       uint32_t shared_len,
                       const std::vector<uint32_t> &shared_pages,
                       const uint32_t *row_tag, const uint32_t *row_lp,
                       const std::vector<uint32_t> &private_table,
                       uint32_t private_stride, uint32_t num_ctas,
                       uint32_t max_slots, bool lockstep, char *error,
                       size_t error_len);

/* Decode: cut every sequence into chunks of `chunk_pages` pages. */
void q3_build_decode_work(const uint32_t *ctx_lens, uint32_t num_seqs,
                          uint32_t extra_token, uint32_t chunk_pages,
                          std::vector<q3_decode_work> &work,
                          std::vector<uint32_t> &seq_work_begin);

#endif /* Q3_SCHED_H */
