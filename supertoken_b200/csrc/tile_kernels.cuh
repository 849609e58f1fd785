// K2 (pair histogram) and K3 (merge) as warp-specialised TMA pipelines over the tiled stream.
//
// One persistent CTA = STBPE_NCW consumer warps + 1 producer warp around a ring of STBPE_NS
// shared-memory stages of one tile (STBPE_TILE tokens, 4 KB) each.
//   producer warp : looks up tile records 32 tiles at a time (one tile per lane), gathers each
//                   tile's halo (two live tokens before it, three after it) and issues one
//                   bulk-async (TMA) copy per tile into the ring; an mbarrier per stage carries the
//                   byte count.  Lanes issue in parallel (half a warp at a time).
//   consumer warp : owns every STBPE_NCW-th tile of the CTA's sequence.  It waits on the stage's
//                   "full" barrier and processes the whole tile by itself with ballots and
//                   shuffles, so the main loop has no CTA-wide barrier.  A rewritten tile is
//                   compacted in place in the stage and goes back to HBM with a bulk-async store
//                   straight from shared memory; the stage is handed back ("empty" barrier) once
//                   the store has read it.
// No multicast, no tensor map: plain 1-D bulk copies (16-byte aligned addresses and sizes).
//
// Every wait is bounded: a wait that runs out sets STBPE_DERR_TIMEOUT and the role leaves its loop.
#pragma once
#include "common.cuh"

#define STBPE_DERR_TIMEOUT 32u
#define STBPE_SPIN_LIMIT (1u << 20)
#ifndef STBPE_NCW
#define STBPE_NCW 8                              // consumer warps per CTA
#endif
#ifndef STBPE_NS
#define STBPE_NS 8                               // ring stages per CTA
#endif
#ifndef STBPE_MIN_CTAS
#define STBPE_MIN_CTAS 3                         // resident CTAs per SM the kernels are compiled for
#endif
// Measured on the first 20 merges of a 1 GiB corpus (every tile visited and rewritten): 8 warps x 16
// stages x 2 CTAs per SM 1.93 TB/s, 8 x 8 x 3 CTAs (24 consumer warps per SM, one stage each)
// 2.06 TB/s, 16 x 16 x 2 and 12 x 12 x 2 slower (registers spill or fewer CTAs fit), 8 x 24 x 2 far
// slower (one CTA per SM).
// STBPE_NS must be a multiple of STBPE_NCW: then a stage is always consumed by the same warp, and
// a parity wait can never be more than one phase ahead of its barrier (a waiter that is two
// phases early would see the older phase of equal parity as "complete" and run onto stale data)
static_assert(STBPE_NS % STBPE_NCW == 0 && STBPE_NS >= 8 && STBPE_NCW <= 32, "ring size must be a multiple of the consumer warps");
#define STBPE_ISSUE_GROUP (STBPE_NS >= 32 ? 32 : (STBPE_NS >= 16 ? 16 : 8))  // producer lanes that issue together
#define STBPE_CTA_THREADS ((STBPE_NCW + 1) * 32)  // + producer warp
#define STBPE_CHUNK 128                          // tokens per warp step (4 per lane)
#define STBPE_QCAP 64                            // per-warp queue of match windows awaiting their delta terms
#define STBPE_QWORDS 8                           // words per queued window: 6 tokens, tile of the token before the head, own tile
// A stage holds one tile between two pads of four words: the two live tokens before the tile end
// the front pad, the three after it follow the tile's last token, so a window around any token of
// the tile is a run of consecutive shared-memory words.  The tile itself starts 16 bytes into the
// stage (bulk copies need 16-byte aligned shared-memory addresses).
#define STBPE_STAGE_WORDS (STBPE_TILE + 8)

struct StageMeta {
    int tile;  // -1 = end of the sequence for the consumer warp that receives it
    int len;
    int slot;  // record slot that is current before this merge
    uint32_t prev;
    uint32_t nxt[3];
    uint32_t prev2;
    int next_tile;  // tile that holds nxt[0] (-1: none)
    int prev_tile;  // tile that holds prev (-1: none)
    int pad[2];
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(2000u)  // let the hardware park the thread for up to ~2 us
        : "memory");
    return ok != 0;
}
// bounded wait; false = gave up (device error bit set)
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, unsigned int *derr) {
    for (uint32_t i = 0; i < STBPE_SPIN_LIMIT; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    atomicOr(derr, STBPE_DERR_TIMEOUT);
    return false;
}
__device__ __forceinline__ void tma_load_1d(void *smem_dst, const void *gsrc, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(smem_dst)),
                 "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tma_store_1d(void *gdst, const void *smem_src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst),
                 "r"(smem_u32(smem_src)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void tma_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void tma_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void tma_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Shared-memory carve-up of one CTA: stages, aggregation table, barriers, metadata.
struct TilePipe {
    uint32_t *tok0;
    StageMeta *meta;
    uint64_t *full;
    uint64_t *empty;
    uint32_t *queue;  // STBPE_NCW queues of STBPE_QCAP windows of STBPE_QWORDS words (merge kernel)
    SmemTable tab;

    __device__ __forceinline__ void carve(unsigned char *base, unsigned int table_slots) {
        tok0 = reinterpret_cast<uint32_t *>(base);
        unsigned char *p = base + (size_t)STBPE_NS * STBPE_STAGE_WORDS * sizeof(uint32_t);
        tab.keys = reinterpret_cast<u64 *>(p);
        p += (size_t)table_slots * sizeof(u64);
        tab.vals = reinterpret_cast<int *>(p);
        p += (size_t)table_slots * sizeof(int);
        tab.mask = table_slots - 1;
        full = reinterpret_cast<uint64_t *>(p);
        empty = full + STBPE_NS;
        p += 2 * STBPE_NS * sizeof(uint64_t);
        meta = reinterpret_cast<StageMeta *>(p);
        p += STBPE_NS * sizeof(StageMeta);
        queue = reinterpret_cast<uint32_t *>(p);
    }
    __device__ __forceinline__ uint32_t *tok(int stage) const { return tok0 + (size_t)stage * STBPE_STAGE_WORDS + 4; }
    static size_t bytes(unsigned int table_slots) {
        return (size_t)STBPE_NS * STBPE_STAGE_WORDS * sizeof(uint32_t) + (size_t)table_slots * 12 +
               2 * STBPE_NS * sizeof(uint64_t) + STBPE_NS * sizeof(StageMeta) +
               (size_t)STBPE_NCW * STBPE_QCAP * STBPE_QWORDS * sizeof(uint32_t) + 16;
    }
};

__device__ __forceinline__ void pipe_setup(TilePipe &pipe) {
    if (threadIdx.x == 0) {
        for (int s = 0; s < STBPE_NS; ++s) {
            mbar_init(&pipe.full[s], 1);
            mbar_init(&pipe.empty[s], 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    smem_table_clear(pipe.tab);
    __syncthreads();
}

// Producer warp: feeds this CTA's tiles through the ring, then one end marker per consumer warp.
// n_work < 0: tiles blockIdx.x, +gridDim.x, ...; otherwise the tiles listed in worklist items
// blockIdx.x, +gridDim.x, ...
// `first_item`: worklist item blockIdx.x + lane * gridDim.x, read by the caller ahead of n_work.
__device__ __forceinline__ void produce_tiles(const EngineDev &e, TilePipe &pipe, int m, int lane, int n_work,
                                              unsigned int first_item) {
    unsigned int *derr = &e.st->error;
    const unsigned int lt = (1u << lane) - 1u;
    int it_base = 0;
    bool alive = true;
    for (long long j0 = 0; alive; j0 += 32) {
        int tile = -1;
        bool more;  // does the sequence continue past this batch?
        const long long first = blockIdx.x + j0 * gridDim.x;
        const long long limit = n_work < 0 ? (long long)e.n_tiles : (long long)n_work;
        if (first >= limit) break;
        const long long mine = first + (long long)lane * gridDim.x;
        if (mine < limit) tile = n_work < 0 ? (int)mine : (j0 == 0 ? (int)first_item : (int)e.worklist[mine]);
        more = first + 32ll * gridDim.x < limit;
        TileRec rec;
        int slot = 0, len = 0, next_tile = -1, prev_tile = -1;
        uint32_t prev = STBPE_NONE, prev2 = STBPE_NONE, nxt[3] = {STBPE_NONE, STBPE_NONE, STBPE_NONE};
        if (tile >= 0) {
            // the tile's records and its neighbours' are adjacent: one round trip for the three
            TileRec before, after;
            const bool has_before = tile > 0, has_after = tile + 1 < e.n_tiles;
            slot = current_rec(e, tile, m, rec);
            if (has_before) current_rec(e, tile - 1, m, before);
            if (has_after) current_rec(e, tile + 1, m, after);
            len = rec.len;
            if (len > 0)
                gather_halo(e, tile, m, prev, prev2, nxt, next_tile, prev_tile, has_before ? &before : nullptr,
                            has_after ? &after : nullptr);
        }
        const unsigned int has = __ballot_sync(0xFFFFFFFFu, len > 0);
        const int my_it = it_base + __popc(has & lt);
        // a group of lanes issues at a time: the group is no larger than the ring, so its lanes own
        // distinct stages
        for (int g = 0; g < 32; g += STBPE_ISSUE_GROUP) {
            bool ok = true;
            if (len > 0 && (lane & ~(STBPE_ISSUE_GROUP - 1)) == g) {
                const int stage = my_it % STBPE_NS;
                const uint32_t par = (((uint32_t)(my_it / STBPE_NS)) & 1u) ^ 1u;
                ok = mbar_wait(&pipe.empty[stage], par, derr);
                if (ok) {
                    StageMeta *mt = &pipe.meta[stage];
                    mt->tile = tile;
                    mt->len = len;
                    mt->slot = slot;
                    mt->prev = prev;
                    mt->prev2 = prev2;
                    mt->nxt[0] = nxt[0];
                    mt->nxt[1] = nxt[1];
                    mt->nxt[2] = nxt[2];
                    mt->next_tile = next_tile;
                    mt->prev_tile = prev_tile;
                    const uint32_t bytes = ((uint32_t)len * 4u + 15u) & ~15u;
                    mbar_arrive_expect_tx(&pipe.full[stage], bytes);
                    tma_load_1d(pipe.tok(stage), e.tiles + (i64)tile * STBPE_TILE, bytes, &pipe.full[stage]);
                }
            }
            alive = __all_sync(0xFFFFFFFFu, ok) && alive;
        }
        it_base += __popc(has);
        if (!more) break;
    }
    if (alive && lane < STBPE_NCW) {  // end markers: the next NCW iterations, one per consumer warp
        const int my_it = it_base + lane;
        const int stage = my_it % STBPE_NS;
        const uint32_t par = (((uint32_t)(my_it / STBPE_NS)) & 1u) ^ 1u;
        if (mbar_wait(&pipe.empty[stage], par, derr)) {
            pipe.meta[stage].tile = -1;
            mbar_arrive(&pipe.full[stage]);
        }
    }
}

// token at tile position q in [len, len+2] comes from the halo; beyond that nothing
__device__ __forceinline__ uint32_t tok_or_halo(const uint32_t *s_tok, const StageMeta *mp, int len, int q) {
    if (q < len) return s_tok[q];
    const int h = q - len;
    return h < 3 ? mp->nxt[h] : STBPE_NONE;
}

// ---------------------------------------------------------------------------------------
// K2  full adjacent-pair histogram (gpu_tokenizer/utils.py:558-635 without the sort):
// every countable pair adds +1 into the CTA's shared-memory table, flushed at the end into
// the pair table (or, multi-GPU, into the rank-local delta table).
// ---------------------------------------------------------------------------------------
template <bool MG>
__global__ void __launch_bounds__(STBPE_CTA_THREADS, STBPE_MIN_CTAS) count_kernel(EngineDev e, unsigned int smem_slots) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    TilePipe pipe;
    pipe.carve(smem_raw, smem_slots);
    pipe_setup(pipe);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int m = 0x7FFFFFFF;  // every record version counts as "before"
    if (warp == STBPE_NCW) {
        produce_tiles(e, pipe, m, lane, -1, 0u);
    } else {
        unsigned int *derr = &e.st->error;
        for (int it = warp;; it += STBPE_NCW) {
            const int stage = it % STBPE_NS;
            if (!mbar_wait(&pipe.full[stage], ((uint32_t)(it / STBPE_NS)) & 1u, derr)) break;
            const StageMeta *mp = &pipe.meta[stage];
            if (mp->tile < 0) break;
            const uint32_t *s_tok = pipe.tok(stage);
            const int len = mp->len;
            for (int cq = 0; cq < len; cq += STBPE_CHUNK) {
                const int q0 = cq + lane * 4;
                const uint4 raw = *reinterpret_cast<const uint4 *>(s_tok + q0);
                uint32_t v[5] = {raw.x, raw.y, raw.z, raw.w, 0};
                uint32_t n0 = __shfl_down_sync(0xFFFFFFFFu, v[0], 1);
                if (lane == 31) n0 = tok_or_halo(s_tok, mp, len, cq + STBPE_CHUNK);
                v[4] = n0;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    if (q0 + k < len) {
                        const uint32_t t1 = (q0 + k + 1 < len) ? v[k + 1] : mp->nxt[0];
                        if (!(t1 & STBPE_FLAG))
                            smem_table_add<MG>(pipe.tab, e, ((u64)(v[k] & STBPE_IDMASK) << 32) | (u64)t1, 1);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&pipe.empty[stage]);
        }
    }
    __syncthreads();
    smem_table_flush<MG>(pipe.tab, e);
}

// ---------------------------------------------------------------------------------------
// K3  one merge: find + rewrite + in-tile compaction + delta counts
//
// With M[i] = (id[i]==a && id[i+1]==b && token i+1 does not start a row) evaluated on
// the pre-merge stream (gpu_tokenizer/utils.py:520-527), token i is dropped when M[i-1]
// and becomes `new` when M[i] (utils.py:529-531).  The histogram of the result equals a
// full recount of the rewritten rows when these terms are added (the entry of (a,b) itself
// is zeroed when the merge is selected):
//   a != b, per match head i (x = token i-1, y = token i+2, both only if in the same row):
//       x exists : if x is the dropped b of a preceding match  +1 (new,new)
//                  else                                         -1 (x,a)  +1 (x,new)
//       y exists : -1 (b,y);  +1 (new,y) unless y starts the next match (whose head then adds
//                  the (new,new) term)
//   a == b, per run of k >= 2 equal tokens (it collapses into ONE new token):
//       head (first token), x exists : -1 (x,a)  +1 (x,new)
//       tail (last token),  y exists : -1 (a,y)  +1 (new,y)
// ---------------------------------------------------------------------------------------
template <bool MG>
__device__ __forceinline__ void merge_delta_terms(const SmemTable &tab, const EngineDev &e, uint32_t a, uint32_t b,
                                                  uint32_t nw, uint32_t tm2, uint32_t tm1, uint32_t t0, uint32_t t1,
                                                  uint32_t t2, uint32_t t3, int tile_x, int tile_own) {
    // Every window yields at most two -1 terms, two +1 terms and two filter entries (every pair that
    // comes into being is entered into the pair filter of the tile that holds its left token: tile_x
    // for the token before the head, tile_own for the head).  The terms are worked out first and
    // added afterwards, so that the lanes of a warp, whose windows fall into different cases, run
    // through one sequence of adds together instead of one sequence per case.
    u64 km0 = 0, kp0 = 0, km1 = 0, kp1 = 0;  // keys of the -1 / +1 terms on the left and on the right
    bool m0 = false, p0 = false, m1 = false, p1 = false, f1 = false;
    u64 kf1 = 0;
    if (a != b) {
        if (!(t0 & STBPE_FLAG)) {  // x exists
            const bool x_dropped = (tm1 == b) && ((tm2 & STBPE_IDMASK) == a);
            const u64 x = (u64)(tm1 & STBPE_IDMASK) << 32;
            km0 = x | (u64)a;
            m0 = !x_dropped;
            // the preceding head became `new` where x's left neighbour was
            kp0 = x_dropped ? (((u64)nw << 32) | (u64)nw) : (x | (u64)nw);
            p0 = true;
        }
        if (!(t2 & STBPE_FLAG)) {  // y exists
            const bool M2 = (t2 == a) && (t3 == b);  // y heads the next match, which adds (new,new) itself
            km1 = ((u64)b << 32) | (u64)t2;
            m1 = true;
            kp1 = ((u64)nw << 32) | (u64)t2;
            p1 = !M2;
            kf1 = M2 ? (((u64)nw << 32) | (u64)nw) : kp1;
            f1 = true;
        }
    } else {
        const bool head = ((t0 & STBPE_IDMASK) == a) && (t1 == b);
        if (head) {
            if (!(t0 & STBPE_FLAG)) {
                const u64 x = (u64)(tm1 & STBPE_IDMASK) << 32;
                km0 = x | (u64)a;
                kp0 = x | (u64)nw;
                m0 = p0 = true;
            }
        } else if (!(t1 & STBPE_FLAG)) {  // tail of the run, y = t1
            km1 = ((u64)a << 32) | (u64)t1;
            kp1 = ((u64)nw << 32) | (u64)t1;
            m1 = p1 = true;
            kf1 = kp1;  // right when the run started in this tile; the tile where a run that crosses
            f1 = true;  // tiles started is a wildcard instead
        }
    }
    if (m0) smem_table_add<MG>(tab, e, km0, -1);
    if (p0) smem_table_add<MG>(tab, e, kp0, 1);
    if (m1) smem_table_add<MG>(tab, e, km1, -1);
    if (p1) smem_table_add<MG>(tab, e, kp1, 1);
    if (p0) filter_set(e, tile_x, kp0);
    if (f1) filter_set(e, tile_own, kf1);
}

// Remove the first live token of a tile that this merge does not otherwise visit: it is the b of
// a match whose head is the last token of the preceding tile.  One warp shifts the tile left by one
// token in global memory (chunk by chunk: all reads of a chunk, then its writes) and writes the
// tile's next record.  Nobody else touches this tile during the merge.
__device__ __noinline__ void drop_first_token(const EngineDev &e, int tile, int m, int lane) {
    TileRec r;
    const int slot = current_rec(e, tile, m, r);
    uint32_t *g = e.tiles + (i64)tile * STBPE_TILE;
    const int newlen = r.len - 1;
    for (int c = 0; c < newlen; c += 128) {
        uint32_t v[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int q = c + lane * 4 + k;
            v[k] = q < newlen ? g[q + 1] : 0u;
        }
        __syncwarp();
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int q = c + lane * 4 + k;
            if (q < newlen) g[q] = v[k];
        }
        __syncwarp();
    }
    if (lane == 0) {
        TileRec *dst = &e.recs[2 * tile + (slot ^ 1)];
        dst->len = newlen;
        dst->head[0] = newlen > 0 ? r.head[1] : STBPE_NONE;
        dst->head[1] = newlen > 1 ? r.head[2] : STBPE_NONE;
        dst->head[2] = newlen > 2 ? g[2] : STBPE_NONE;
        dst->tail = newlen > 0 ? r.tail : STBPE_NONE;
        dst->tail2 = newlen > 1 ? r.tail2 : STBPE_NONE;
        dst->ver = m;
        atomicAdd(&e.st->n_fixups, 1u);
    }
    __syncwarp();
}

// Match windows are queued per warp and their delta terms are added 32 at a time, one window
// per lane: a table add is a dependent chain of a few hundred cycles, which a single lane
// walking its own matches one after the other would pay in full for every term.
template <bool MG>
__device__ __forceinline__ void drain_queue(const SmemTable &tab, const EngineDev &e, uint32_t a, uint32_t b,
                                            uint32_t nw, const uint32_t *q, int n, int lane) {
    __syncwarp();
    for (int i = lane; i < n; i += 32) {
        const uint4 lo = *reinterpret_cast<const uint4 *>(q + i * STBPE_QWORDS);
        const uint4 hi = *reinterpret_cast<const uint4 *>(q + i * STBPE_QWORDS + 4);
        merge_delta_terms<MG>(tab, e, a, b, nw, lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, (int)hi.z, (int)hi.w);
    }
    __syncwarp();
}

// One warp, one tile.  The tile sits in shared memory with its halo around it (s[-2], s[-1] = the two
// live tokens before it, s[len .. len+2] = the three after it).  The warp works in passes over the
// whole tile instead of chunk by chunk, so that the cross-lane steps are paid once per tile:
//   1. match heads of all 1024 positions into one 32-bit mask per lane (bit 4c+k = position
//      128c + 4*lane + k); the dropped positions follow from the masks of the neighbouring lane;
//   2. per-chunk drop counts packed into bytes and scanned across the lanes once;
//   3. windows of the positions that own delta terms go to the warp's queue (read from the intact
//      pre-merge tile), then the surviving heads are rewritten in place;
//   4. chunks at or behind the first drop are re-read and written back compacted.
template <bool MG>
__global__ void __launch_bounds__(STBPE_CTA_THREADS, STBPE_MIN_CTAS) merge_kernel(EngineDev e, unsigned int smem_slots) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    // the shared-memory set-up needs nothing from the kernels before this one: inside the captured
    // loop it runs while they finish
    dep_release();
    TilePipe pipe;
    pipe.carve(smem_raw, smem_slots);
    pipe_setup(pipe);
    dep_wait();
    DevState *st = e.st;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // everything the kernel needs from the loop state in one round trip, and with it the producer
    // warp's first worklist items (the list is as long as the stream has tiles; items past n_work
    // are stale and not used)
    const int stopped = st->stopped, exchange_only = st->exchange_only;
    const uint32_t a = (uint32_t)st->cur_a, b = (uint32_t)st->cur_b, nw = (uint32_t)st->cur_new;
    const int m = st->merges_done;  // number of this merge (>= 1)
    const int n_work = st->n_work;  // < 0: every tile
    const bool fv = st->filter_valid != 0;  // the pair filter is being maintained
    unsigned int first_item = 0;
    if (warp == STBPE_NCW) {
        const long long mine = blockIdx.x + (long long)lane * gridDim.x;
        if (mine < (long long)e.n_tiles) first_item = e.worklist[mine];
    }
    if (stopped || exchange_only) return;
    if (m < 1) return;  // nothing has been selected yet
    const bool same = (a == b);
    if (warp == STBPE_NCW) {
        produce_tiles(e, pipe, m, lane, n_work, first_item);
    } else {
        unsigned int *derr = &st->error;
        i64 removed = 0;
        int matches = 0;
        i64 bytes_in = 0, bytes_out = 0;  // lane 0: bulk-copy bytes of this warp's tiles (statistics)
        int pending = -1;  // lane 0: stage whose bulk store may still be reading shared memory
        uint32_t *queue = pipe.queue + (size_t)warp * STBPE_QCAP * STBPE_QWORDS;
        int qn = 0;  // warp-uniform
        const unsigned int lt = (1u << lane) - 1u;
        for (int it = warp;; it += STBPE_NCW) {
            const int stage = it % STBPE_NS;
            if (lane == 0 && pending >= 0) {  // the previous tile's store has had a whole tile time
                tma_wait_read_all();
                mbar_arrive(&pipe.empty[pending]);
                pending = -1;
            }
            if (!mbar_wait(&pipe.full[stage], ((uint32_t)(it / STBPE_NS)) & 1u, derr)) break;
            const StageMeta *mp = &pipe.meta[stage];
            const int tile = mp->tile;
            if (tile < 0) break;
            uint32_t *s = pipe.tok(stage);
            const int len = mp->len;
            bytes_in += ((len * 4 + 15) & ~15) + 2 * (int)sizeof(TileRec);
            // halo around the tile (the bulk copy may have written up to three words past len)
            if (lane == 0) {
                s[-2] = mp->prev2;
                s[-1] = mp->prev;
            } else if (lane <= 3) {
                s[len + lane - 1] = mp->nxt[lane - 1];
            }
            __syncwarp();
            const int nch = (len + STBPE_CHUNK - 1) / STBPE_CHUNK;
            // ---- pass 1: match heads.  Comparing the whole word of the right-hand token with b also
            // checks that it does not start a row.
            uint32_t hmask = 0;
#pragma unroll
            for (int c = 0; c < STBPE_TILE / STBPE_CHUNK; ++c) {
                if (c < nch) {
                    const uint4 v = *reinterpret_cast<const uint4 *>(s + c * STBPE_CHUNK + lane * 4);
                    uint32_t nx = __shfl_down_sync(0xFFFFFFFFu, v.x, 1);
                    if (lane == 31) nx = s[(c + 1) * STBPE_CHUNK];
                    unsigned int h = 0;
                    if (((v.x & STBPE_IDMASK) == a) && (v.y == b)) h |= 1u;
                    if (((v.y & STBPE_IDMASK) == a) && (v.z == b)) h |= 2u;
                    if (((v.z & STBPE_IDMASK) == a) && (v.w == b)) h |= 4u;
                    if (((v.w & STBPE_IDMASK) == a) && (nx == b)) h |= 8u;
                    hmask |= h << (4 * c);
                }
            }
            // positions of this lane that lie inside the tile
            const int cf = len / STBPE_CHUNK;  // full chunks
            uint32_t vmask = 0xFFFFFFFFu;
            if (cf < STBPE_TILE / STBPE_CHUNK) {
                const int rem = min(4, max(0, len - cf * STBPE_CHUNK - lane * 4));
                vmask = ((1u << (4 * cf)) - 1u) | (((1u << rem) - 1u) << (4 * cf));
            }
            hmask &= vmask;
            // a position is dropped when the position before it heads a match: inside the lane a shift
            // of the mask, at the lane's first token the last token of the lane before it, and for
            // lane 0 the last token of lane 31 in the chunk before (the tile's first token: the halo)
            const uint32_t up = __shfl_up_sync(0xFFFFFFFFu, hmask, 1);
            const uint32_t h31 = __shfl_sync(0xFFFFFFFFu, hmask, 31);
            uint32_t top = (up >> 3) & 0x11111111u;
            if (lane == 0) {
                const bool carry_in = ((mp->prev & STBPE_IDMASK) == a) && (s[0] == b);
                top = (((h31 >> 3) & 0x01111111u) << 4) | (carry_in ? 1u : 0u);
            }
            const uint32_t drops = (((hmask << 1) & 0xEEEEEEEEu) | top) & vmask;
            const uint32_t touched = hmask | drops;
            if (__ballot_sync(0xFFFFFFFFu, touched != 0u) == 0u) {  // the filter let a tile through in vain
                __syncwarp();
                if (lane == 0) mbar_arrive(&pipe.empty[stage]);
                continue;
            }
            matches += __popc(hmask);
            const int lastq = len - 1;
            const bool last_head =
                (__shfl_sync(0xFFFFFFFFu, hmask, (lastq & (STBPE_CHUNK - 1)) >> 2) >> (4 * (lastq / STBPE_CHUNK) + (lastq & 3))) & 1u;
            // first position whose word changes (bit order inside a lane is position order)
            int firstq = 0x7FFFFFFF;
            if (touched) {
                const int bit = __ffs(touched) - 1;
                firstq = (bit >> 2) * STBPE_CHUNK + lane * 4 + (bit & 3);
            }
            firstq = __reduce_min_sync(0xFFFFFFFFu, firstq);

            // ---- pass 2: drops before every position.  Per-chunk drop counts of this lane as bytes
            // (even chunks in `lo`, odd chunks in `hi`; a chunk holds at most 128 drops), one
            // inclusive scan over the lanes for all eight chunks.
            uint32_t own_lo, own_hi, inc_lo, inc_hi;
            {
                uint32_t x = drops - ((drops >> 1) & 0x55555555u);
                x = (x & 0x33333333u) + ((x >> 2) & 0x33333333u);  // drops per nibble
                own_lo = x & 0x0F0F0F0Fu;
                own_hi = (x >> 4) & 0x0F0F0F0Fu;
                inc_lo = own_lo, inc_hi = own_hi;
#pragma unroll
                for (int d = 1; d < 32; d <<= 1) {
                    const uint32_t nl = __shfl_up_sync(0xFFFFFFFFu, inc_lo, d);
                    const uint32_t nh = __shfl_up_sync(0xFFFFFFFFu, inc_hi, d);
                    if (lane >= d) {
                        inc_lo += nl;
                        inc_hi += nh;
                    }
                }
            }
            const uint32_t tot_lo = __shfl_sync(0xFFFFFFFFu, inc_lo, 31), tot_hi = __shfl_sync(0xFFFFFFFFu, inc_hi, 31);
            const uint32_t exc_lo = inc_lo - own_lo, exc_hi = inc_hi - own_hi;  // drops in lanes before this one
            int cb[STBPE_TILE / STBPE_CHUNK + 1];  // drops before chunk c (warp-uniform)
            cb[0] = 0;
#pragma unroll
            for (int c = 0; c < STBPE_TILE / STBPE_CHUNK; ++c)
                cb[c + 1] = cb[c] + (int)((((c & 1) ? tot_hi : tot_lo) >> (8 * (c >> 1))) & 0xFFu);
            const int newlen = len - cb[STBPE_TILE / STBPE_CHUNK];

            // ---- pass 3: windows of the positions that own delta terms (match heads when a != b; the
            // first and the last token of a run of equal tokens when a == b), one per lane and round
            {
                uint32_t owners = same ? (hmask ^ drops) : hmask;
                for (;;) {
                    const unsigned int om = __ballot_sync(0xFFFFFFFFu, owners != 0u);
                    if (om == 0u) break;
                    if (owners) {
                        const int bit = __ffs(owners) - 1;
                        owners &= owners - 1u;
                        const int q = (bit >> 2) * STBPE_CHUNK + lane * 4 + (bit & 3);
                        const uint32_t *w = s + q - 2;
                        uint4 lo, hi;
                        lo.x = w[0], lo.y = w[1], lo.z = w[2], lo.w = w[3];
                        hi.x = w[4], hi.y = w[5];
                        // tiles whose filter bits the new pairs go into; -1 (no tile) while the filter is stale
                        hi.z = (uint32_t)(fv ? (q > 0 ? tile : mp->prev_tile) : -1);
                        hi.w = (uint32_t)(fv ? tile : -1);
                        uint32_t *d = queue + (qn + __popc(om & lt)) * STBPE_QWORDS;
                        *reinterpret_cast<uint4 *>(d) = lo;
                        *reinterpret_cast<uint4 *>(d + 4) = hi;
                    }
                    qn += __popc(om);
                    if (qn >= 32) {
                        drain_queue<MG>(pipe.tab, e, a, b, nw, queue, qn, lane);
                        qn = 0;
                    }
                }
            }
            __syncwarp();  // every window has been read: the tile may change now
            {   // surviving heads become the new token (the row-start flag stays)
                uint32_t pm = hmask & ~drops;
                while (pm) {
                    const int bit = __ffs(pm) - 1;
                    pm &= pm - 1u;
                    const int q = (bit >> 2) * STBPE_CHUNK + lane * 4 + (bit & 3);
                    s[q] = nw | (s[q] & STBPE_FLAG);
                }
            }
            __syncwarp();
            // ---- pass 4: compaction.  Chunks in front of the first drop stay where they are.
            // (The per-chunk loops of passes 1 and 4 stay unrolled: rolled up, with the drops before a
            // chunk kept as a running sum, the kernel was 8 KB shorter and 2-5 % slower.)
            const uint32_t keepm = vmask & ~drops;
#pragma unroll
            for (int c = 0; c < STBPE_TILE / STBPE_CHUNK; ++c) {
                if (c < nch && cb[c + 1] != 0) {
                    const uint4 v = *reinterpret_cast<const uint4 *>(s + c * STBPE_CHUNK + lane * 4);
                    __syncwarp();  // all lanes hold their tokens before anyone overwrites the chunk
                    const unsigned int keep = (keepm >> (4 * c)) & 15u;
                    const int before = cb[c] + (int)((((c & 1) ? exc_hi : exc_lo) >> (8 * (c >> 1))) & 0xFFu);
                    uint32_t *o = s + c * STBPE_CHUNK + lane * 4 - before;
                    if (keep & 1u) *o++ = v.x;
                    if (keep & 2u) *o++ = v.y;
                    if (keep & 4u) *o++ = v.z;
                    if (keep & 8u) *o++ = v.w;
                }
            }
            fence_async_smem();  // the bulk store reads these writes through the async proxy
            __syncwarp();
            if (fv && same && last_head && lane == 0) {
                // the run of a's goes on in the next tile: the pair that will start at the collapsed
                // token is decided by whoever finds the run's tail, so visit this tile from now on
                unsigned int *p = e.presence + (size_t)STBPE_PROWS * e.presence_words + ((unsigned int)tile >> 5);
                atomicOr(p, 1u << (tile & 31));
            }
            if (last_head && n_work >= 0 && mp->next_tile >= 0) {
                // the dropped partner opens the next non-empty tile; if this merge does not visit
                // that tile, drop it here
                const unsigned int su = (unsigned int)mp->next_tile;
                if (!((e.cand_bits[su >> 5] >> (su & 31)) & 1u)) {
                    drop_first_token(e, mp->next_tile, m, lane);
                    if (lane == 0) {
                        removed += 1;
                        // a == b: the dropped token is the tail of the run and would have owned the
                        // terms of the pair behind the run; its tile is not visited, so add them here
                        const uint32_t y = mp->nxt[1];
                        if (same && !(y & STBPE_FLAG)) {
                            smem_table_add<MG>(pipe.tab, e, ((u64)a << 32) | (u64)y, -1);
                            smem_table_add<MG>(pipe.tab, e, ((u64)nw << 32) | (u64)y, 1);
                            if (fv) filter_set(e, tile, ((u64)nw << 32) | (u64)y);
                        }
                    }
                }
            }
            if (lane == 0) {
                // only the part of the tile from the first changed word on goes back to HBM
                const int start = firstq & ~3;
                if (newlen > start) {
                    tma_store_1d(e.tiles + (i64)tile * STBPE_TILE + start, s + start,
                                 ((uint32_t)(newlen - start) * 4u + 15u) & ~15u);
                    tma_commit();
                    pending = stage;
                    bytes_out += ((newlen - start) * 4 + 15) & ~15;
                }
                bytes_out += (int)sizeof(TileRec);
                // the record that is not current before this merge; readers of this merge never pick a
                // record stamped m, so payload and stamp need no ordering between them
                TileRec *dst = &e.recs[2 * tile + (mp->slot ^ 1)];
                dst->len = newlen;
                for (int i = 0; i < 3; ++i) dst->head[i] = i < newlen ? s[i] : STBPE_NONE;
                dst->tail = newlen > 0 ? s[newlen - 1] : STBPE_NONE;
                dst->tail2 = newlen > 1 ? s[newlen - 2] : STBPE_NONE;
                dst->ver = m;
                removed += len - newlen;
                if (pending != stage) mbar_arrive(&pipe.empty[stage]);
            }
        }
        drain_queue<MG>(pipe.tab, e, a, b, nw, queue, qn, lane);
        if (lane == 0) {
            tma_wait_all();  // bulk stores must have landed before the grid ends
            if (removed) atomicAdd((u64 *)&st->n_live, (u64)(-removed));
            if (bytes_in) atomicAdd(&st->tile_bytes_in, (u64)bytes_in);
            if (bytes_out) atomicAdd(&st->tile_bytes_out, (u64)bytes_out);
        }
        matches = __reduce_add_sync(0xFFFFFFFFu, matches);
        if (lane == 0 && matches) atomicAdd((u64 *)&st->n_matches, (u64)(i64)matches);
    }
    __syncthreads();
    smem_table_flush<MG>(pipe.tab, e);
}
