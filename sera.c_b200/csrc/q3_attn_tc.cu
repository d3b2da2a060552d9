/* q3_attn_tc.cu - tensor-core attention over paged f16 KV for sm_100a.
 *
 * One kernel serves both tensor-bound cases of the path:
 *   causal GQA prefill      (ref: attention_kernel, src/q3_forward.cu:218-290)
 *   shared prefix + own suffix, packed branches
 *                           (ref: attention_segmented_kernel, :418-525)
 * The reference walks keys 0..P-1 of the prefix and then 0..lp of the row's own
 * branch with one running maximum; this kernel streams the same keys in tiles
 * of 128 (8 pages) with an online softmax, which is the same sum in a
 * different order. A plain causal sequence is the special case "no shared
 * prefix, one branch whose local position is the absolute position".
 *
 * Shape of the computation (per CTA, persistent over its schedule segments):
 *   M tile   128 rows = 16 query tokens x the 8 query heads of one KV head
 *            (GQA packing: the 8 heads share every K/V tile). Two M tiles per
 *            CTA (32 tokens) share every K/V tile in shared memory.
 *   S = Q K^T   tcgen05.mma kind::f16, A = Q (smem, K-major, 128B swizzle),
 *               B = K pages (smem, K-major), D = S in tensor memory (fp32).
 *               ONE S buffer serves both M tiles in turn: a softmax thread
 *               moves its S row into registers (tcgen05.ld) and hands the
 *               buffer back at once, so the other M tile's S - and this M
 *               tile's S of the next key tile - are computed while it
 *               exponentiates. (M = 128, N = 64 MMAs, which would allow two
 *               half-width S buffers per M tile, run at 55 instead of 32
 *               clocks on this part: shared-memory bound.)
 *   softmax     one thread per row: running max / sum in registers, P written
 *               as f16 into a P buffer of its own M tile (tcgen05.st), in two
 *               halves of 64 keys so that PV starts early.
 *   O += P V    tcgen05.mma, A = P from tensor memory, B = V pages (smem,
 *               MN-major), D = O in tensor memory (fp32).
 *   TMEM        S [0,128), P0 [128,192), P1 [192,256), O0 [256,384), O1 [384,512).
 *   K/V pages   4 KiB per page per head, fetched by TMA (128-byte swizzle)
 *               straight into the UMMA operand layouts: a K page as two
 *               64-column boxes - the eight pages of a key tile as two 128-row
 *               boxes when they follow one another in the pool -, a V page as
 *               one 3-D box holding both column halves. Every CTA issues its
 *               own loads, from this GPU's memory only.
 * Warp roles: 0 = TMA producer, 1 = issuer of the S MMAs (owns the TMEM
 * allocation), 2 / 3 = issuers of the PV MMAs of M tile 0 / 1 (three threads
 * issue, each waiting on its own events in order, so that no event waits
 * behind an unrelated one), 4-7 = softmax of M tile 0, 8-11 = softmax of M
 * tile 1.
 *
 * Work is cut stream-K style on the host (q3_sched.h): a CTA receives
 * segments (item, key-tile range). A segment that covers its whole item
 * writes the output rows; a piece of a cut item writes un-normalised fp32
 * partials plus (max, sum) and bumps an arrival counter per 32 rows; the warp
 * that arrives last combines all pieces of its rows with log-sum-exp (its own
 * partial straight from tensor memory) and writes them. No CTA waits for
 * another. A piece's O is stored lane-interleaved, so that the writer's and the
 * combining warp's accesses are 512 contiguous bytes per warp.
 *
 * Every mbarrier wait is bounded; on expiry the thread raises a flag in shared
 * memory, the status word is set and all roles leave; the producer first
 * waits (bounded) for the loads it still has in flight.
 *
 * Algorithmic cost: 4*128 FLOP per (query head row, visible key) pair; bytes
 * = Q in + O out + each distinct K/V page once.
 */
#include "q3_internal.h"
#include "q3_ptx.cuh"

using namespace q3ptx;

namespace {

constexpr uint32_t kThreads = 384;
constexpr uint32_t kNQ = 2;              /* M tiles per CTA */
constexpr uint32_t kStages = 2;          /* K and V ring depth */
constexpr uint32_t kMetaRing = 4;
constexpr uint32_t kTileBytes = 32768;   /* 128 x 128 f16 */
constexpr uint32_t kHalfBytes = 16384;   /* 128 rows x 64 f16 */
constexpr uint32_t kPageHalfBytes = 2048;

constexpr uint32_t kSmemQ = 0;
constexpr uint32_t kSmemK = kSmemQ + kNQ * kTileBytes;
constexpr uint32_t kSmemV = kSmemK + kStages * kTileBytes;
constexpr uint32_t kSmemMisc = kSmemV + kStages * kTileBytes;
constexpr uint32_t kSmemTotal = kSmemMisc + 2048 + 1024; /* + alignment slack */

constexpr uint32_t kSlotInvalid = 0, kSlotShared = 1, kSlotPrivate = 2;
constexpr uint32_t kNoTag = 0xFFFFFFFEu;

/* TMEM columns */
constexpr uint32_t kColS = 0;            /* the one S buffer (fp32, 128 columns)          */
constexpr uint32_t kColP = 128;          /* P_q (f16 pairs) at kColP + q*64               */
constexpr uint32_t kColO = 256;          /* O_q at kColO + q*128                          */

/* lazy rescale threshold in log2 units (P stays <= 2^8, exact enough in f16) */
constexpr float kTau = 8.0f;
/* polls granted to the drain of in-flight loads on the abort path */
constexpr uint32_t kDrainPolls = 1u << 16;

struct TileMeta {
    uint32_t nomask;
    uint32_t kind[8];
    uint32_t tag[8];
    uint32_t base[8];
    uint32_t nvis[8];
};

struct Barriers {
    uint64_t q_full, q_empty;
    uint64_t k_full[kStages], k_empty[kStages];
    uint64_t v_full[kStages], v_empty[kStages];
    uint64_t s_full[kNQ];        /* S of M tile q is complete (tcgen05.commit)            */
    uint64_t s_free;             /* 128 softmax threads moved their S row into registers  */
    uint64_t p_half[kNQ][2];     /* 128 threads stored P for keys [64h, 64h+64)           */
    uint64_t pv_done[kNQ][2];    /* the PV MMAs of that half are complete                 */
};

struct Misc {
    Barriers bar;
    uint32_t tmem_base;
    uint32_t abort_flag;
    TileMeta meta[kMetaRing];
};

struct GatherFlags {
    uint32_t *ptr[Q3_MAX_GATHER_RANKS];
    uint32_t n;
};

struct AttnParams {
    const uint32_t *page_ids;
    const q3_run *runs;
    const q3_segment *segments;
    const uint32_t *cta_seg_begin;
    const uint32_t *row_tag;
    const uint32_t *row_lp;
    uint32_t tokens;
    uint32_t n_heads;
    uint32_t n_shared_pages;
    uint32_t shared_len;
    uint32_t num_pages;
    uint32_t pool_row_base;     /* layer * n_kv_heads * num_pages * 16 */
    uint32_t pool_rows_total;   /* first out-of-range row: zero-filled by TMA */
    float scale_log2;           /* scale * log2(e) */
    uint32_t out_fp32;
    void *out;                  /* [tokens][n_heads][128] bf16, or fp32 */
    float *part_o;
    float2 *part_ml;
    uint32_t *fix_counters;     /* [cut items][2 M tiles][4 row quarters] arrivals */
    uint32_t *status;
};

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ float max3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}
/* packed fp32 pairs: one issue slot for two FMAs / adds */
__device__ __forceinline__ uint64_t pack2(float x, float y) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(x), "f"(y));
    return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float &x, float &y) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(x), "=f"(y) : "l"(v));
}
__device__ __forceinline__ uint64_t ffma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t fadd2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
/* 2^x for a pair without the special-function unit: round-to-nearest split
 * x = n + r, r in [-0.5, 0.5], cubic minimax for 2^r (relative error 7.5e-5,
 * below the f16 rounding of P), n added into the exponent field. The MUFU
 * executes 16 ex2 per clock per SM, exactly as many as the tensor core consumes
 * at full rate: with both pipes on the critical path, a share of the
 * exponentials on the FMA pipe gives the MUFU slack. Inputs must be finite and
 * >= -126. */
__device__ __forceinline__ void exp2_poly2(uint64_t x2, float &p0, float &p1) {
    const uint64_t magic = pack2(12582912.0f, 12582912.0f);       /* 1.5 * 2^23 */
    const uint64_t neg_magic = pack2(-12582912.0f, -12582912.0f);
    const uint64_t minus1 = pack2(-1.0f, -1.0f);
    const uint64_t xr = fadd2(x2, magic);                 /* n in the low mantissa bits */
    const uint64_t n = fadd2(xr, neg_magic);
    const uint64_t r = ffma2(n, minus1, x2);              /* r = x - n */
    uint64_t p = ffma2(r, pack2(0.055170901f, 0.055170901f), pack2(0.24260952f, 0.24260952f));
    p = ffma2(r, p, pack2(0.69326097f, 0.69326097f));
    p = ffma2(r, p, pack2(0.99992818f, 0.99992818f));
    float xr0, xr1, q0, q1;
    unpack2(xr, xr0, xr1);
    unpack2(p, q0, q1);
    p0 = __int_as_float(__float_as_int(q0) + (__float_as_int(xr0) << 23));
    p1 = __int_as_float(__float_as_int(q1) + (__float_as_int(xr1) << 23));
}
/* Pairs out of every 8 whose exponentials go through exp2_poly2. */
#ifndef Q3_POLY_PAIRS_OF_8
#define Q3_POLY_PAIRS_OF_8 0
#endif

/* Register budget: setmaxnreg must be executed identically by all four warps
 * of a warp group. Warps 0-3 (producer and the three MMA issuers) give
 * registers back; the two softmax groups (one S row of 128 fp32 per thread)
 * take them. 384 threads x 168 at launch = 128 x 40 + 256 x 232. */
__device__ __forceinline__ void regs_release() {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
}
__device__ __forceinline__ void regs_take() {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 232;");
}

/* Wait on a barrier unless the CTA is aborting; on expiry raise the abort flag. */
__device__ __forceinline__ bool wait_or_abort(uint64_t *bar, uint32_t parity,
                                              Misc *misc) {
    for (uint32_t i = 0; i < Q3_WAIT_POLLS; i++) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 255u) == 255u && *(volatile uint32_t *)&misc->abort_flag) return false;
    }
    atomicExch(&misc->abort_flag, 1u);
    return false;
}
/* For the waits of the softmax threads, which are normally satisfied long
 * before they are reached: a few non-blocking tests first. */
__device__ __forceinline__ bool quick_wait_or_abort(uint64_t *bar, uint32_t parity,
                                                    Misc *misc) {
#ifndef Q3_NO_QUICK_WAIT
    for (uint32_t i = 0; i < 8; i++)
        if (mbar_test_wait(bar, parity)) return true;
#endif
    return wait_or_abort(bar, parity, misc);
}
/* Abort path only: give a load that is still in flight time to land. */
__device__ __forceinline__ void drain_wait(uint64_t *bar, uint32_t parity) {
    for (uint32_t i = 0; i < kDrainPolls; i++)
        if (mbar_try_wait(bar, parity)) return;
}

/* Store 32 consecutive columns of one output row (already normalised). */
__device__ __forceinline__ void store_row_chunk(const AttnParams &p, size_t off,
                                                const float *v) {
    if (p.out_fp32) {
#pragma unroll
        for (uint32_t i = 0; i < 8; i++)
            *reinterpret_cast<float4 *>(reinterpret_cast<float *>(p.out) + off + i * 4) =
                make_float4(v[i * 4], v[i * 4 + 1], v[i * 4 + 2], v[i * 4 + 3]);
    } else {
#pragma unroll
        for (uint32_t i = 0; i < 4; i++) {
            uint4 u;
            __nv_bfloat162 *h = reinterpret_cast<__nv_bfloat162 *>(&u);
#pragma unroll
            for (uint32_t e = 0; e < 4; e++)
                h[e] = __floats2bfloat162_rn(v[i * 8 + 2 * e], v[i * 8 + 2 * e + 1]);
            *reinterpret_cast<uint4 *>(reinterpret_cast<__nv_bfloat16 *>(p.out) + off + i * 8) = u;
        }
    }
}

__global__ void __launch_bounds__(kThreads, 1)
attention_tc_kernel(const __grid_constant__ CUtensorMap q_map,
                    const __grid_constant__ CUtensorMap k_map,
                    const __grid_constant__ CUtensorMap v_map_page,
                    const __grid_constant__ CUtensorMap k_map_tile, const AttnParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    Misc *misc = reinterpret_cast<Misc *>(smem + kSmemMisc);
    Barriers &bar = misc->bar;
    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31u;

    if (threadIdx.x == 0) {
        mbar_init(&bar.q_full, 1);
        mbar_init(&bar.q_empty, 1);
        for (uint32_t s = 0; s < kStages; s++) {
            mbar_init(&bar.k_full[s], 1);
            mbar_init(&bar.k_empty[s], 1);
            mbar_init(&bar.v_full[s], 1);
            mbar_init(&bar.v_empty[s], kNQ);     /* one commit per PV issuer */
        }
        mbar_init(&bar.s_free, 128);
        for (uint32_t q = 0; q < kNQ; q++) {
            mbar_init(&bar.s_full[q], 1);
            for (uint32_t h = 0; h < 2; h++) {
                mbar_init(&bar.p_half[q][h], 128);
                mbar_init(&bar.pv_done[q][h], 1);
            }
        }
        misc->abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc(&misc->tmem_base, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = misc->tmem_base;

    const uint32_t seg_begin = p.cta_seg_begin[blockIdx.x];
    const uint32_t seg_end = p.cta_seg_begin[blockIdx.x + 1];

    if (warp < 4) regs_release();
    if (warp == 0) {
        /* ===================== TMA producer ===================== */
        if (lane == 0) {
            prefetch_tmap(&q_map);
            prefetch_tmap(&k_map);
            prefetch_tmap(&v_map_page);
            prefetch_tmap(&k_map_tile);
        }
        uint32_t it = 0;          /* K tiles armed so far */
        uint32_t v_armed = 0;     /* V tiles armed so far */
        uint32_t q_armed = 0;     /* Q loads armed so far */
        bool alive = true;
        for (uint32_t si = seg_begin; si < seg_end && alive; si++) {
            const q3_segment seg = p.segments[si];
            /* CTA-wide row summary, for the "whole tile visible" shortcut */
            const uint32_t tok = seg.tok0 + lane;
            const bool tvalid = tok < p.tokens;
            const uint32_t my_tag = tvalid ? p.row_tag[tok] : 0u;
            const uint32_t my_lp = tvalid ? p.row_lp[tok] : 0xFFFFFFFFu;
            const uint32_t first_tag = __shfl_sync(0xffffffffu, my_tag, 0);
            const bool uniform =
                __all_sync(0xffffffffu, !tvalid || my_tag == first_tag);
            uint32_t min_lp = my_lp;
            for (uint32_t o = 16; o; o >>= 1)
                min_lp = min(min_lp, __shfl_xor_sync(0xffffffffu, min_lp, o));

            if (si != seg_begin)
                alive = wait_or_abort(&bar.q_empty, (si - seg_begin - 1) & 1u, misc);
            alive = __all_sync(0xffffffffu, alive);
            if (!alive) break;
            if (lane == 0) {
                mbar_arrive_expect_tx(&bar.q_full, kNQ * kTileBytes);
                for (uint32_t q = 0; q < kNQ; q++)
                    for (uint32_t half = 0; half < 2; half++)
                        tma_load_3d(smem + kSmemQ + q * kTileBytes + half * kHalfBytes,
                                    &q_map, (int32_t)(half * 64),
                                    (int32_t)(seg.kv_head * Q3_G),
                                    (int32_t)(seg.tok0 + q * 16), &bar.q_full);
            }
            q_armed++;
            /* Arm the K and V loads of one key tile: lanes 0..7 fetch one page
             * each from pool row `row` (K: two 64-column boxes; V: one box with
             * both halves); when the eight pages follow one another in the pool
             * (`run`), lane 0 fetches K as two boxes of 128 rows. A copy costs
             * the issuing warp about 60 clocks whatever its size, one lane after
             * the other: 32 page copies per key tile were 2 k clocks of this
             * warp, more than the tensor work of the tile; now 24, or 10 in a run. */
            auto arm_tile = [&](int32_t row, bool run) {
                const uint32_t stage = it % kStages;
                const uint32_t ph = (it / kStages) & 1u;
                if (lane == 0) mbar_arrive_expect_tx(&bar.k_full[stage], kTileBytes);
                __syncwarp();
                if (run) {
                    if (lane == 0) {
                        uint8_t *dst = smem + kSmemK + stage * kTileBytes;
                        tma_load_2d(dst, &k_map_tile, 0, row, &bar.k_full[stage]);
                        tma_load_2d(dst + kHalfBytes, &k_map_tile, 64, row, &bar.k_full[stage]);
                    }
                } else if (lane < 8) {
                    uint8_t *dst = smem + kSmemK + stage * kTileBytes + lane * kPageHalfBytes;
                    tma_load_2d(dst, &k_map, 0, row, &bar.k_full[stage]);
                    tma_load_2d(dst + kHalfBytes, &k_map, 64, row, &bar.k_full[stage]);
                }
                it++;
                alive = wait_or_abort(&bar.v_empty[stage], ph ^ 1u, misc);
                alive = __all_sync(0xffffffffu, alive);
                if (!alive) return;
                if (lane == 0) mbar_arrive_expect_tx(&bar.v_full[stage], kTileBytes);
                __syncwarp();
                /* V: one copy per page, both column halves ([half][16 keys][128 B],
                 * 4 KiB per page). A PV MMA step consumes one page, so its operand
                 * descriptor can point at any page; K, whose MMA walks all 128
                 * keys of a column half at one stride, cannot be laid out so. */
                if (lane < 8)
                    tma_load_3d(smem + kSmemV + stage * kTileBytes + lane * 2u * kPageHalfBytes,
                                &v_map_page, 0, row, 0, &bar.v_full[stage]);
                v_armed++;
            };
            const uint32_t row_base = p.pool_row_base + seg.kv_head * p.num_pages * Q3_PAGE;
            uint32_t tile = seg.tile_begin;

            /* Key tiles whose 128 keys every row of the item sees: no mask data,
             * and the page ids of the next tile are fetched while this tile's
             * loads are armed. This loop sets the pace of the whole CTA when it
             * is slow: with the general code below for every tile the producer
             * needed 3.5 k clocks per key tile (page-id load, run lookup and
             * mask summary between two tiles' loads), more than the softmax
             * threads. Tiles [tile, fend) take their pages from
             * page_ids[table + (tile - t_off) * 8 ...]. */
            auto fast_tiles = [&](uint32_t fend, uint32_t table, uint32_t t_off) {
                uint32_t pg = 0;
                if (tile < fend && lane < 8) pg = p.page_ids[table + (tile - t_off) * 8 + lane];
                for (; tile < fend; tile++) {
                    const int32_t row = (int32_t)(row_base + pg * Q3_PAGE);
                    const uint32_t pg0 = __shfl_sync(0xffffffffu, pg, 0);
                    const bool run = __all_sync(0xffffffffu, lane >= 8 || pg == pg0 + lane);
                    if (tile + 1 < fend && lane < 8)
                        pg = p.page_ids[table + (tile + 1 - t_off) * 8 + lane];
                    alive = wait_or_abort(&bar.k_empty[it % kStages], ((it / kStages) & 1u) ^ 1u,
                                          misc);
                    alive = __all_sync(0xffffffffu, alive);
                    if (!alive) return;
                    if (lane == 0) misc->meta[it % kMetaRing].nomask = 1u;
                    arm_tile(row, run);
                    if (!alive) return;
                }
            };
            /* the shared prefix, up to its last full tile */
            fast_tiles(min(seg.tile_end, min(seg.shared_tiles, p.shared_len >> 7)), 0u, 0u);
            if (!alive) break;
            /* an item of one branch (a causal prefill chunk, a long suffix): its own
             * keys below the first row's position */
            if (tile >= seg.shared_tiles && seg.run_end == seg.run_begin + 1 && uniform) {
                const q3_run run = p.runs[seg.run_begin];
                if (run.tag == first_tag && min_lp != 0xFFFFFFFFu)
                    fast_tiles(min(seg.tile_end,
                                   seg.shared_tiles + min((min_lp + 1u) >> 7, run.n_pages >> 3)),
                               run.table_off, seg.shared_tiles);
                if (!alive) break;
            }

            /* The remaining tiles: a partly filled shared page, the branches'
             * own pages. Lanes 0..7 resolve one page slot each. */
            for (; tile < seg.tile_end; tile++) {
                uint32_t kind = kSlotInvalid, tag = 0, base = 0, nvis = 0;
                uint32_t page = 0;
                if (lane < 8) {
                    if (tile < seg.shared_tiles) {
                        const uint32_t pidx = tile * 8 + lane;
                        if (pidx < p.n_shared_pages) {
                            page = p.page_ids[pidx];
                            kind = kSlotShared;
                            nvis = min(16u, p.shared_len - pidx * 16u);
                        }
                    } else {
                        uint32_t f = (tile - seg.shared_tiles) * 8 + lane;
                        for (uint32_t r = seg.run_begin; r < seg.run_end; r++) {
                            const q3_run run = p.runs[r];
                            if (f < run.n_pages) {
                                page = p.page_ids[run.table_off + f];
                                kind = kSlotPrivate;
                                tag = run.tag;
                                base = f * 16u;
                                break;
                            }
                            f -= run.n_pages;
                        }
                    }
                }
                const bool whole =
                    (kind == kSlotShared && nvis == 16u) ||
                    (kind == kSlotPrivate && uniform && tag == first_tag &&
                     base + 15u <= min_lp);
                const uint32_t whole_mask = __ballot_sync(0xffffffffu, whole) & 0xFFu;
                const int32_t row = kind == kSlotInvalid ? (int32_t)p.pool_rows_total
                                                         : (int32_t)(row_base + page * Q3_PAGE);
                alive = wait_or_abort(&bar.k_empty[it % kStages], ((it / kStages) & 1u) ^ 1u, misc);
                alive = __all_sync(0xffffffffu, alive);
                if (!alive) break;
                TileMeta &m = misc->meta[it % kMetaRing];
                if (lane < 8) {
                    m.kind[lane] = kind;
                    m.tag[lane] = tag;
                    m.base[lane] = base;
                    m.nvis[lane] = nvis;
                }
                if (lane == 0) m.nomask = whole_mask == 0xFFu;
                arm_tile(row, false);
                if (!alive) break;
            }
        }
        if (!alive && lane == 0) {
            /* leaving early: the loads armed last may still be writing shared
             * memory; wait for them (bounded) before the CTA can exit */
            if (q_armed) drain_wait(&bar.q_full, (q_armed - 1) & 1u);
            for (uint32_t b = 0; b < kStages; b++) {
                if (it > b) {
                    const uint32_t i = it - 1 - b;
                    drain_wait(&bar.k_full[i % kStages], (i / kStages) & 1u);
                }
                if (v_armed > b) {
                    const uint32_t i = v_armed - 1 - b;
                    drain_wait(&bar.v_full[i % kStages], (i / kStages) & 1u);
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        /* ===================== issuer of S = Q K^T =====================
         * One S buffer, used by the two M tiles in turn: S number g = 2*it + q
         * may be issued once the softmax threads of S number g-1 have moved
         * their rows into registers. */
        if (elect_one()) {
            constexpr uint32_t idesc_qk = umma_idesc_f16(128, 128, false);
            const uint32_t q_addr = smem_u32(smem + kSmemQ);
            const uint32_t k_addr = smem_u32(smem + kSmemK);
            uint32_t it = 0;
            bool alive = true;
            for (uint32_t si = seg_begin; si < seg_end && alive; si++) {
                const q3_segment seg = p.segments[si];
                const uint32_t n = seg.tile_end - seg.tile_begin;
                alive = wait_or_abort(&bar.q_full, (si - seg_begin) & 1u, misc);
                for (uint32_t j = 0; j < n && alive; j++, it++) {
                    const uint32_t stage = it % kStages;
                    for (uint32_t q = 0; q < kNQ && alive; q++) {
                        const uint32_t g = 2u * it + q;
                        if (g > 0) alive = wait_or_abort(&bar.s_free, (g - 1u) & 1u, misc);
                        if (alive && q == 0)
                            alive = wait_or_abort(&bar.k_full[stage], (it / kStages) & 1u, misc);
                        if (!alive) break;
                        tc_fence_after();
                        /* 8 steps of K = 16 over head_dim = 128 */
#pragma unroll
                        for (uint32_t ks = 0; ks < 8; ks++) {
                            const uint32_t off = (ks >> 2) * kHalfBytes + (ks & 3u) * 32u;
                            umma_ss(tmem + kColS,
                                    umma_desc(q_addr + q * kTileBytes + off, 16, 1024),
                                    umma_desc(k_addr + stage * kTileBytes + off, 16, 1024),
                                    idesc_qk, ks > 0);
                        }
                        umma_commit(&bar.s_full[q]);
                    }
                    if (!alive) break;
                    umma_commit(&bar.k_empty[stage]);
                    if (j + 1 == n) umma_commit(&bar.q_empty);
                }
            }
        }
        __syncwarp();
    } else if (warp < 4) {
        /* ===================== issuers of O_q += P_q V =================== */
        if (elect_one()) {
            const uint32_t q = warp - 2u;
            constexpr uint32_t idesc_pv = umma_idesc_f16(128, 128, true);
            const uint32_t v_addr = smem_u32(smem + kSmemV);
            uint32_t it = 0;
            bool alive = true;
            for (uint32_t si = seg_begin; si < seg_end && alive; si++) {
                const q3_segment seg = p.segments[si];
                const uint32_t n = seg.tile_end - seg.tile_begin;
                for (uint32_t j = 0; j < n && alive; j++, it++) {
                    const uint32_t stage = it % kStages;
                    for (uint32_t half = 0; half < 2 && alive; half++) {
                        alive = wait_or_abort(&bar.p_half[q][half], it & 1u, misc);
                        if (alive && half == 0)
                            alive = wait_or_abort(&bar.v_full[stage], (it / kStages) & 1u, misc);
                        if (!alive) break;
                        tc_fence_after();
                        /* keys [64*half, 64*half+64): 4 steps of K = 16 keys = one
                         * page each; V is MN-major (a page is 4 KiB: its two
                         * 64-column blocks 2 KiB apart, 8-key groups 1 KiB apart) */
#pragma unroll
                        for (uint32_t ks = half * 4; ks < half * 4 + 4; ks++)
                            umma_ts(tmem + kColO + q * 128u, tmem + kColP + q * 64u + ks * 8u,
                                    umma_desc(v_addr + stage * kTileBytes + ks * 4096u,
                                              2u * 1024u, 1024),
                                    idesc_pv, (j > 0 || ks > 0) ? 1u : 0u);
                        umma_commit(&bar.pv_done[q][half]);
                    }
                    if (!alive) break;
                    umma_commit(&bar.v_empty[stage]);
                }
            }
        }
        __syncwarp();
    } else {
        /* ===================== softmax groups ==================== */
        regs_take();
        const uint32_t q = (warp - 4) >> 2;                 /* M tile of this group */
        const uint32_t row = (warp & 3u) * 32u + lane;       /* TMEM lane == tile row */
        const uint32_t lane_addr = ((warp & 3u) * 32u) << 16;
        const uint32_t s_addr = tmem + lane_addr + kColS;
        const uint32_t p_addr = tmem + lane_addr + kColP + q * 64u;
        const uint32_t o_addr = tmem + lane_addr + kColO + q * 128u;
        const float c = p.scale_log2;
        const float tau_raw = kTau / c;
        uint32_t it = 0;
        bool alive = true;

        for (uint32_t si = seg_begin; si < seg_end && alive; si++) {
            const q3_segment seg = p.segments[si];
            const uint32_t n = seg.tile_end - seg.tile_begin;
            const uint32_t token = seg.tok0 + q * 16u + (row >> 3);
            const uint32_t head = seg.kv_head * Q3_G + (row & 7u);
            const bool valid = token < p.tokens;
            const uint32_t tag_r = valid ? p.row_tag[token] : kNoTag;
            const uint32_t lp_r = valid ? p.row_lp[token] : 0u;
            float m_ref = -INFINITY, l = 0.f;

            for (uint32_t j = 0; j < n && alive; j++, it++) {
                alive = quick_wait_or_abort(&bar.s_full[q], it & 1u, misc);
                alive = __all_sync(0xffffffffu, alive);
                if (!alive) break;
                tc_fence_after();
                float s[128];
#pragma unroll
                for (uint32_t ch = 0; ch < 4; ch++)
                    tmem_ld32(s_addr + ch * 32u, reinterpret_cast<uint32_t *>(s) + ch * 32u);
                tmem_wait_ld();
                /* the row is in registers: the S buffer may be overwritten */
                tc_fence_before();
                mbar_arrive(&bar.s_free);
                const TileMeta &m = misc->meta[it % kMetaRing];
                if (!m.nomask) {
#pragma unroll
                    for (uint32_t i = 0; i < 8; i++) {
                        const uint32_t kind = m.kind[i];
                        uint32_t nvis = 0;
                        if (kind == kSlotShared) {
                            nvis = m.nvis[i];
                        } else if (kind == kSlotPrivate && m.tag[i] == tag_r) {
                            const uint32_t b = m.base[i];
                            nvis = lp_r >= b ? min(16u, lp_r - b + 1u) : 0u;
                        }
#pragma unroll
                        for (uint32_t k2 = 0; k2 < 16; k2++)
                            if (k2 >= nvis) s[i * 16 + k2] = -INFINITY;
                    }
                }
                /* row max: 8 independent chains of 3-input max */
                float mx;
                {
                    float mc[8];
#pragma unroll
                    for (uint32_t ch = 0; ch < 8; ch++) {
                        const float *v = s + ch * 16;
                        float t = max3(v[0], v[1], v[2]);
#pragma unroll
                        for (uint32_t i = 3; i < 15; i += 2) t = max3(t, v[i], v[i + 1]);
                        mc[ch] = fmaxf(t, v[15]);
                    }
                    mx = fmaxf(max3(mc[0], mc[1], mc[2]),
                               max3(mc[3], mc[4], fmaxf(mc[5], fmaxf(mc[6], mc[7]))));
                }

                if (j == 0) {
                    m_ref = mx;
                } else {
                    const bool need = mx > m_ref + tau_raw;
                    if (__any_sync(0xffffffffu, need)) {
                        /* O_q must be at rest: the PV of the previous key tile done */
                        alive = wait_or_abort(&bar.pv_done[q][1], (it - 1u) & 1u, misc);
                        alive = __all_sync(0xffffffffu, alive);
                        if (!alive) break;
                        tc_fence_after();
                        const float f = need ? fast_exp2((m_ref - mx) * c) : 1.0f;
                        if (need) m_ref = mx;
                        l *= f;
#pragma unroll
                        for (uint32_t ch = 0; ch < 4; ch++) {
                            uint32_t o[32];
                            tmem_ld32(o_addr + ch * 32u, o);
                            tmem_wait_ld();
#pragma unroll
                            for (uint32_t i = 0; i < 32; i++)
                                o[i] = __float_as_uint(__uint_as_float(o[i]) * f);
                            tmem_st32(o_addr + ch * 32u, o);
                        }
                        tmem_wait_st();
                    }
                }
                const float neg = (m_ref == -INFINITY) ? 0.f : -m_ref * c;
                uint32_t pk[64];
                {
                    const uint64_t c2 = pack2(c, c), neg2 = pack2(neg, neg);
                    uint64_t acc[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll
                    for (uint32_t i = 0; i < 64; i++) {
                        if (i == 32) {
                            /* keys 0..63 are ready. The P buffer still feeds the
                             * previous key tile's PV until pv_done says otherwise
                             * (the second half's completion implies the first's:
                             * one thread issues both, in order). */
                            if (it > 0) {
                                alive = quick_wait_or_abort(&bar.pv_done[q][1], (it - 1u) & 1u, misc);
                                alive = __all_sync(0xffffffffu, alive);
                            }
                            if (alive) {
                                tc_fence_after();
                                tmem_st32(p_addr, pk);
                                tmem_wait_st();
                                tc_fence_before();
                                mbar_arrive(&bar.p_half[q][0]);
                            }
                        }
                        float x0, x1, p0, p1;
                        const uint64_t x2 = ffma2(pack2(s[2 * i], s[2 * i + 1]), c2, neg2);
                        unpack2(x2, x0, x1);
                        if ((int)(i & 7u) < (int)Q3_POLY_PAIRS_OF_8) {
                            exp2_poly2(pack2(fmaxf(x0, -126.f), fmaxf(x1, -126.f)), p0, p1);
                        } else {
                            p0 = fast_exp2(x0);
                            p1 = fast_exp2(x1);
                        }
                        acc[i & 3u] = fadd2(acc[i & 3u], pack2(p0, p1));
                        const __half2 h = __floats2half2_rn(p0, p1);
                        pk[i] = *reinterpret_cast<const uint32_t *>(&h);
                    }
                    float a0, a1;
                    unpack2(fadd2(fadd2(acc[0], acc[1]), fadd2(acc[2], acc[3])), a0, a1);
                    l += a0 + a1;
                }
                if (!alive) break;
                tmem_st32(p_addr + 32u, pk + 32);
                tmem_wait_st();
                tc_fence_before();
                mbar_arrive(&bar.p_half[q][1]);
            }
            if (!alive) break;
            /* ---- segment epilogue: O_q after the last key tile ---- */
            alive = wait_or_abort(&bar.pv_done[q][1], (it - 1u) & 1u, misc);
            alive = __all_sync(0xffffffffu, alive);
            if (!alive) break;
            tc_fence_after();
            const size_t orow = ((size_t)token * p.n_heads + head) * Q3_D;
            if (seg.partial_slot < 0) {
                const float inv = 1.0f / l;
#pragma unroll
                for (uint32_t ch = 0; ch < 4; ch++) {
                    uint32_t o[32];
                    tmem_ld32(o_addr + ch * 32u, o);
                    tmem_wait_ld();
                    float v[32];
#pragma unroll
                    for (uint32_t i = 0; i < 32; i++) v[i] = __uint_as_float(o[i]) * inv;
                    if (valid) store_row_chunk(p, orow + ch * 32, v);
                }
            } else {
                /* piece of a cut item: publish the un-normalised partial ...
                 * Layout of a piece's O: [M tile][row quarter][32 chunks of 4
                 * columns][32 lanes] x 16 bytes, so that a warp's store (and the
                 * combining warp's load) of one chunk is 512 contiguous bytes. */
                const size_t prow = (size_t)seg.partial_slot * 256 + q * 128 + row;
                uint4 *dst = reinterpret_cast<uint4 *>(p.part_o) +
                             ((((size_t)seg.partial_slot * 2 + q) * 4 + (warp & 3u)) << 10) + lane;
#pragma unroll
                for (uint32_t ch = 0; ch < 4; ch++) {
                    uint32_t o[32];
                    tmem_ld32(o_addr + ch * 32u, o);
                    tmem_wait_ld();
#pragma unroll
                    for (uint32_t i = 0; i < 8; i++)
                        dst[(ch * 8 + i) * 32] =
                            make_uint4(o[i * 4], o[i * 4 + 1], o[i * 4 + 2], o[i * 4 + 3]);
                }
                p.part_ml[prow] =
                    make_float2(m_ref == -INFINITY ? -INFINITY : m_ref * c, l);
                __threadfence();
                /* ... and count the arrival of this warp's 32 rows. The warp
                 * that arrives last at (item, M tile, row quarter) combines all
                 * pieces of those rows; nobody waits for anybody:
                 *   M = max_i m_i;  out = sum_i 2^(m_i-M) O_i / sum_i 2^(m_i-M) l_i
                 * equal to one running max over all keys
                 * (ref: src/q3_forward.cu:452-518) up to rounding. */
                __syncwarp();
                uint32_t last = 0;
                if (lane == 0) {
                    uint32_t *cnt = p.fix_counters + (seg.fix_index * 2 + q) * 4 + (warp & 3u);
                    last = atomicAdd(cnt, 1u) + 1 == seg.slot_count;
                    if (last) *cnt = 0;            /* ready for the next launch */
                }
                last = __shfl_sync(0xffffffffu, last, 0);
                if (last) {
                    __threadfence();
                    /* this thread's own partial is still in tensor memory; only
                     * the other pieces' rows are read back (from L2) */
                    const uint32_t own = (uint32_t)seg.partial_slot - seg.slot_begin;
                    const size_t base = (size_t)seg.slot_begin * 256 + q * 128 + row;
                    const float m_own = m_ref == -INFINITY ? -INFINITY : m_ref * c;
                    float M = m_own;
                    for (uint32_t i = 0; i < seg.slot_count; i++)
                        if (i != own)
                            M = fmaxf(M, __ldcg(&p.part_ml[base + (size_t)i * 256]).x);
                    /* sums run in slot order whichever piece came last, so the
                     * result is bit-identical from run to run */
                    const float w_own = m_own == -INFINITY ? 0.f : exp2f(m_own - M);
                    float den = 0.f;
                    for (uint32_t i = 0; i < seg.slot_count; i++) {
                        if (i == own) {
                            den += w_own * l;
                        } else {
                            const float2 ml = __ldcg(&p.part_ml[base + (size_t)i * 256]);
                            den += ml.x == -INFINITY ? 0.f : exp2f(ml.x - M) * ml.y;
                        }
                    }
                    const float inv = 1.0f / den;
                    const float w_self = w_own * inv;
                    const float4 *piece0 =
                        reinterpret_cast<const float4 *>(p.part_o) +
                        ((((size_t)seg.slot_begin * 2 + q) * 4 + (warp & 3u)) << 10) + lane;
                    /* 64 columns per pass: a pass costs one L2 round trip per other
                     * piece (16 loads of 16 bytes in flight per thread), so the
                     * whole combination is 2 x (pieces - 1) round trips. Pieces
                     * are summed in slot order whichever came last: the result is
                     * bit-identical from run to run. */
#pragma unroll 1
                    for (uint32_t hf = 0; hf < 2; hf++) {
                        float v[64];
#pragma unroll
                        for (uint32_t i = 0; i < 64; i++) v[i] = 0.f;
#pragma unroll 1
                        for (uint32_t sidx = 0; sidx < seg.slot_count; sidx++) {
                            if (sidx == own) {
#pragma unroll
                                for (uint32_t c2 = 0; c2 < 2; c2++) {
                                    uint32_t o[32];
                                    tmem_ld32(o_addr + hf * 64u + c2 * 32u, o);
                                    tmem_wait_ld();
#pragma unroll
                                    for (uint32_t i = 0; i < 32; i++)
                                        v[c2 * 32 + i] += w_self * __uint_as_float(o[i]);
                                }
                                continue;
                            }
                            const float4 *src = piece0 + ((size_t)sidx << 13) + hf * 512;
                            float4 f[16];
#pragma unroll
                            for (uint32_t i = 0; i < 16; i++) f[i] = __ldcg(src + i * 32);
                            const float mx2 = __ldcg(&p.part_ml[base + (size_t)sidx * 256]).x;
                            const float wgt = mx2 == -INFINITY ? 0.f : exp2f(mx2 - M) * inv;
#pragma unroll
                            for (uint32_t i = 0; i < 16; i++) {
                                v[i * 4] += wgt * f[i].x;
                                v[i * 4 + 1] += wgt * f[i].y;
                                v[i * 4 + 2] += wgt * f[i].z;
                                v[i * 4 + 3] += wgt * f[i].w;
                            }
                        }
                        if (valid) {
                            store_row_chunk(p, orow + hf * 64, v);
                            store_row_chunk(p, orow + hf * 64 + 32, v + 32);
                        }
                    }
                }
            }
            /* the next segment's first PV overwrites O_q only after p_half of
             * its first tile, which this thread raises after these loads */
            tc_fence_before();
        }
    }

    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && misc->abort_flag) atomicOr(p.status, Q3_STATUS_WAIT_TIMEOUT);
    if (warp == 1) tmem_dealloc(tmem, 512);
}

/* After a layer's rows are stored: publish `seq` in every rank's flag array
 * (slot = this rank). One thread; the fence orders the flag after the rows of
 * the preceding kernels of this stream. */
__global__ void gather_signal_kernel(const GatherFlags flags, uint32_t rank, uint32_t seq,
                                     const uint32_t *epoch) {
    if (threadIdx.x == 0) {
        seq += *epoch;
        __threadfence_system();
        for (uint32_t d = 0; d < flags.n; d++)
            asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flags.ptr[d] + rank),
                         "r"(seq)
                         : "memory");
    }
}

/* Wait (bounded) until every rank has published at least `seq` in this rank's
 * flag array, i.e. the gathered buffer holds that layer from every rank. */
__global__ void gather_wait_kernel(const uint32_t *flags, uint32_t n_ranks, uint32_t seq,
                                   const uint32_t *epoch, uint32_t *status) {
    const uint32_t r = threadIdx.x;
    if (r >= n_ranks) return;
    seq += *epoch;
    for (uint32_t i = 0; i < (1u << 20); i++) {   /* about a second */
        uint32_t v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flags + r) : "memory");
        if ((int32_t)(v - seq) >= 0) return;
        __nanosleep(64);
    }
    atomicOr(status, Q3_STATUS_GATHER_TIMEOUT);
}

/* Sequence numbers of later calls start `count` higher: a recorded step passes
 * step-relative numbers and ends with this. */
__global__ void gather_advance_kernel(uint32_t *epoch, uint32_t count) {
    if (threadIdx.x == 0) *epoch += count;
}

}  // namespace

bool q3_launch_gather_advance(q3_attn_runtime *rt, uint32_t count, char *error,
                              size_t error_len) {
    gather_advance_kernel<<<1, 32, 0, rt->stream>>>(rt->gather_epoch_dev, count);
    Q3_LAUNCH_CHECK("gather_advance launch failed");
    rt->n_launch++;
    return true;
}

bool q3_launch_gather_signal(q3_attn_runtime *rt, const q3_gather_peers *g, uint32_t seq,
                             cudaStream_t stream, char *error, size_t error_len) {
    GatherFlags f;
    f.n = g->n_ranks;
    for (uint32_t d = 0; d < g->n_ranks; d++) f.ptr[d] = g->flags[d];
    gather_signal_kernel<<<1, 32, 0, stream>>>(f, g->rank, seq, rt->gather_epoch_dev);
    Q3_LAUNCH_CHECK("gather_signal launch failed");
    rt->n_launch++;
    return true;
}

bool q3_launch_gather_wait(q3_attn_runtime *rt, const q3_gather_peers *g, uint32_t seq,
                           char *error, size_t error_len) {
    q3_phase_begin(rt, Q3_PHASE_GATHER_WAIT);
    gather_wait_kernel<<<1, 32, 0, rt->stream>>>(g->flags[g->rank], g->n_ranks, seq,
                                                 rt->gather_epoch_dev, rt->status_dev);
    q3_phase_end(rt);
    Q3_LAUNCH_CHECK("gather_wait launch failed");
    rt->n_launch++;
    return true;
}

/* Per device, at runtime creation: opt in to the large dynamic shared memory. */
bool q3_prepare_attention_kernel(char *error, size_t error_len) {
    cudaError_t e = cudaFuncSetAttribute(attention_tc_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)kSmemTotal);
    if (e != cudaSuccess)
        return q3_fail_cuda(error, error_len, "attention_tc: shared memory opt-in", e);
    return true;
}

bool q3_launch_attention(q3_attn_runtime *rt, uint32_t layer, const q3_stage *st,
                         void *out_bf16, char *error, size_t error_len) {
    const q3_attn_config &c = rt->cfg;
    CUtensorMap q_map;
    if (!q3_encode_tmap_q(&q_map, rt->q2, c.n_heads, st->tokens, error, error_len))
        return false;
    AttnParams p;
    p.page_ids = st->page_ids;
    p.runs = st->runs;
    p.segments = st->segments;
    p.cta_seg_begin = st->cta_seg_begin;
    p.row_tag = st->row_tag;
    p.row_lp = st->row_lp;
    p.tokens = st->tokens;
    p.n_heads = c.n_heads;
    p.n_shared_pages = st->n_shared_pages;
    p.shared_len = st->shared_len;
    p.num_pages = c.num_pages;
    p.pool_row_base = layer * c.n_kv_heads * c.num_pages * Q3_PAGE;
    p.pool_rows_total = c.num_layers * c.n_kv_heads * c.num_pages * Q3_PAGE;
    p.scale_log2 = (1.0f / sqrtf((float)Q3_D)) * 1.4426950408889634f;
    p.out_fp32 = c.out_fp32;
    p.out = out_bf16;
    p.part_o = rt->part_o;
    p.part_ml = rt->part_ml;
    p.fix_counters = rt->fix_counters;
    p.status = rt->status_dev;
    q3_phase_begin(rt, Q3_PHASE_ATTENTION);
    attention_tc_kernel<<<st->grid, kThreads, kSmemTotal, rt->stream>>>(
        q_map, rt->k_map, rt->v_map_page, rt->k_map_tile, p);
    q3_phase_end(rt);
    Q3_LAUNCH_CHECK("attention_tc launch failed");
    rt->n_launch++;
    return true;
}
