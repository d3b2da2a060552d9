/* q3_prefix_cache.cpp - sealed prefixes kept across requests.
 *
 * The reference creates a prefix, prefills it, runs one decision batch and
 * destroys it, per request (ref: src/q3_systemone.cu:498-523, 740-741), so a
 * prompt shared by consecutive requests is prefilled again every time. With
 * the page pool a sealed prefix is just a page table: this cache keeps such
 * prefixes under a caller-chosen 64-bit key (a hash of the prompt's token ids),
 * hands them out by reference count, and evicts the least recently used
 * unreferenced ones when asked for room; their pages go back to the pool's
 * free list and are reused by the next prefix without any allocation.
 * Pure host code; single-threaded like the runtime it serves.
 */
#include <stdio.h>

#include <algorithm>
#include <new>
#include <vector>

#include "q3_internal.h"

struct q3_prefix_cache {
    struct Entry {
        uint64_t key;
        q3_prefix_kv *prefix;
        uint32_t refs;
        uint64_t tick;     /* last acquire / insert */
    };
    q3_attn_runtime *rt;
    uint32_t max_entries;
    uint64_t tick;
    std::vector<Entry> entries;
    q3_prefix_cache_stats stats;
};

static uint32_t entry_pages(const q3_prefix_cache::Entry &e) {
    return (uint32_t)e.prefix->pages.size();
}

/* Destroy the least recently used unreferenced entry; false if there is none. */
static bool evict_one(q3_prefix_cache *c) {
    size_t victim = c->entries.size();
    for (size_t i = 0; i < c->entries.size(); i++)
        if (c->entries[i].refs == 0 &&
            (victim == c->entries.size() || c->entries[i].tick < c->entries[victim].tick))
            victim = i;
    if (victim == c->entries.size()) return false;
    c->stats.pages_held -= entry_pages(c->entries[victim]);
    q3_prefix_destroy(c->entries[victim].prefix);
    c->entries.erase(c->entries.begin() + (long)victim);
    c->stats.evictions++;
    c->stats.entries = (uint32_t)c->entries.size();
    return true;
}

extern "C" q3_prefix_cache *q3_prefix_cache_create(q3_attn_runtime *rt, uint32_t max_entries,
                                                   char *error, size_t error_len) {
    q3_clear_error(error, error_len);
    if (!rt || max_entries == 0) {
        q3_fail(error, error_len, "q3_prefix_cache_create: invalid argument");
        return NULL;
    }
    q3_prefix_cache *c = new (std::nothrow) q3_prefix_cache();
    if (!c) {
        q3_fail(error, error_len, "q3_prefix_cache_create: allocation failed");
        return NULL;
    }
    c->rt = rt;
    c->max_entries = max_entries;
    c->tick = 0;
    c->stats = q3_prefix_cache_stats();
    return c;
}

extern "C" void q3_prefix_cache_destroy(q3_prefix_cache *c) {
    if (!c) return;
    for (auto &e : c->entries) q3_prefix_destroy(e.prefix);
    delete c;
}

extern "C" q3_prefix_kv *q3_prefix_cache_acquire(q3_prefix_cache *c, uint64_t key,
                                                 uint32_t token_count) {
    if (!c) return NULL;
    for (auto &e : c->entries)
        if (e.key == key && e.prefix->token_count == token_count) {
            e.refs++;
            e.tick = ++c->tick;
            c->stats.hits++;
            return e.prefix;
        }
    c->stats.misses++;
    return NULL;
}

extern "C" bool q3_prefix_cache_insert(q3_prefix_cache *c, uint64_t key, q3_prefix_kv *prefix,
                                       char *error, size_t error_len) {
    q3_clear_error(error, error_len);
    if (!c || !prefix) return q3_fail(error, error_len, "q3_prefix_cache_insert: null argument");
    if (prefix->rt != c->rt)
        return q3_fail(error, error_len, "q3_prefix_cache_insert: prefix of another runtime");
    if (!prefix->sealed)
        return q3_fail(error, error_len, "q3_prefix_cache_insert: prefix is not sealed");
    for (const auto &e : c->entries)
        if (e.prefix == prefix || (e.key == key && e.prefix->token_count == prefix->token_count))
            return q3_fail(error, error_len, "q3_prefix_cache_insert: already cached");
    while (c->entries.size() >= c->max_entries)
        if (!evict_one(c))
            return q3_fail(error, error_len,
                           "q3_prefix_cache_insert: cache full and every entry is referenced");
    q3_prefix_cache::Entry e;
    e.key = key;
    e.prefix = prefix;
    e.refs = 1;              /* the inserting request still uses it */
    e.tick = ++c->tick;
    c->entries.push_back(e);
    c->stats.inserts++;
    c->stats.entries = (uint32_t)c->entries.size();
    c->stats.pages_held += (uint32_t)prefix->pages.size();
    return true;
}

extern "C" bool q3_prefix_cache_release(q3_prefix_cache *c, q3_prefix_kv *prefix, char *error,
                                        size_t error_len) {
    q3_clear_error(error, error_len);
    if (!c || !prefix) return q3_fail(error, error_len, "q3_prefix_cache_release: null argument");
    for (auto &e : c->entries)
        if (e.prefix == prefix) {
            if (e.refs == 0)
                return q3_fail(error, error_len, "q3_prefix_cache_release: not referenced");
            e.refs--;
            return true;
        }
    return q3_fail(error, error_len, "q3_prefix_cache_release: not a cached prefix");
}

extern "C" uint32_t q3_prefix_cache_make_room(q3_prefix_cache *c, uint32_t pages_needed) {
    if (!c) return 0;
    uint32_t evicted = 0;
    while (c->rt->free_pages.size() < pages_needed && evict_one(c)) evicted++;
    return evicted;
}

extern "C" int q3_prefix_cache_holds(const q3_prefix_cache *c, const q3_prefix_kv *prefix) {
    if (!c || !prefix) return 0;
    for (const auto &e : c->entries)
        if (e.prefix == prefix) return 1;
    return 0;
}

extern "C" void q3_prefix_cache_get_stats(const q3_prefix_cache *c, q3_prefix_cache_stats *out) {
    if (c && out) *out = c->stats;
}
