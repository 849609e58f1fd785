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
#define STBPE_NCW 8                              // consumer warps per CTA
#define STBPE_NS 16                              // ring stages per CTA
// STBPE_NS must be a multiple of STBPE_NCW: then a stage is always consumed by the same warp, and
// a parity wait can never be more than one phase ahead of its barrier (a waiter that is two
// phases early would see the older phase of equal parity as "complete" and run onto stale data)
static_assert(STBPE_NS % STBPE_NCW == 0 && STBPE_NS >= 16, "ring size must be a multiple of the consumer warps");
#define STBPE_CTA_THREADS ((STBPE_NCW + 1) * 32)  // + producer warp
#define STBPE_CHUNK 128                          // tokens per warp step (4 per lane)
#define STBPE_QCAP 64                            // per-warp queue of match windows awaiting their delta terms
#define STBPE_QWORDS 8                           // words per queued window: 6 tokens, tile of the token before the head, own tile

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
        unsigned char *p = base + (size_t)STBPE_NS * STBPE_TILE * sizeof(uint32_t);
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
    __device__ __forceinline__ uint32_t *tok(int stage) const { return tok0 + (size_t)stage * STBPE_TILE; }
    static size_t bytes(unsigned int table_slots) {
        return (size_t)STBPE_NS * STBPE_TILE * sizeof(uint32_t) + (size_t)table_slots * 12 +
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
__device__ __forceinline__ void produce_tiles(const EngineDev &e, TilePipe &pipe, int m, int lane, int n_work) {
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
        if (mine < limit) tile = n_work < 0 ? (int)mine : (int)e.worklist[mine];
        more = first + 32ll * gridDim.x < limit;
        TileRec rec;
        int slot = 0, len = 0, next_tile = -1, prev_tile = -1;
        uint32_t prev = STBPE_NONE, prev2 = STBPE_NONE, nxt[3] = {STBPE_NONE, STBPE_NONE, STBPE_NONE};
        if (tile >= 0) {
            slot = current_rec(e, tile, m, rec);
            len = rec.len;
            if (len > 0) gather_halo(e, tile, m, prev, prev2, nxt, next_tile, prev_tile);
        }
        const unsigned int has = __ballot_sync(0xFFFFFFFFu, len > 0);
        const int my_it = it_base + __popc(has & lt);
        // half a warp issues at a time: 16 <= STBPE_NS, so the lanes of a group own distinct stages
        for (int g = 0; g < 32; g += 16) {
            bool ok = true;
            if (len > 0 && (lane & 16) == g) {
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
__global__ void __launch_bounds__(STBPE_CTA_THREADS, 2) count_kernel(EngineDev e, unsigned int smem_slots) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    TilePipe pipe;
    pipe.carve(smem_raw, smem_slots);
    pipe_setup(pipe);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int m = 0x7FFFFFFF;  // every record version counts as "before"
    if (warp == STBPE_NCW) {
        produce_tiles(e, pipe, m, lane, -1);
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
    // every pair that comes into being (+1 term) is also entered into the pair filter of the tile
    // that holds its left token: tile_x for the token before the head, tile_own for the head
    if (a != b) {
        if (!(t0 & STBPE_FLAG)) {
            const bool x_dropped = (tm1 == b) && ((tm2 & STBPE_IDMASK) == a);
            if (x_dropped) {
                const u64 k = ((u64)nw << 32) | (u64)nw;
                smem_table_add<MG>(tab, e, k, 1);
                filter_set(e, tile_x, k);  // the preceding head became `new` where x's left neighbour was
            } else {
                const u64 x = (u64)(tm1 & STBPE_IDMASK) << 32;
                smem_table_add<MG>(tab, e, x | (u64)a, -1);
                smem_table_add<MG>(tab, e, x | (u64)nw, 1);
                filter_set(e, tile_x, x | (u64)nw);
            }
        }
        if (!(t2 & STBPE_FLAG)) {
            smem_table_add<MG>(tab, e, ((u64)b << 32) | (u64)t2, -1);
            const bool M2 = (t2 == a) && (t3 == b);
            const u64 k = ((u64)nw << 32) | (u64)(M2 ? nw : t2);
            if (!M2) smem_table_add<MG>(tab, e, k, 1);
            filter_set(e, tile_own, k);
        }
    } else {
        const bool head = ((t0 & STBPE_IDMASK) == a) && (t1 == b);
        if (head) {
            if (!(t0 & STBPE_FLAG)) {
                const u64 x = (u64)(tm1 & STBPE_IDMASK) << 32;
                smem_table_add<MG>(tab, e, x | (u64)a, -1);
                smem_table_add<MG>(tab, e, x | (u64)nw, 1);
                filter_set(e, tile_x, x | (u64)nw);
            }
        } else if (!(t1 & STBPE_FLAG)) {
            smem_table_add<MG>(tab, e, ((u64)a << 32) | (u64)t1, -1);
            const u64 k = ((u64)nw << 32) | (u64)t1;
            smem_table_add<MG>(tab, e, k, 1);
            filter_set(e, tile_own, k);  // right when the run started in this tile; the tile where a
                                          // run that crosses tiles started is a wildcard instead
        }
    }
}

// Remove the first live token of a tile that this merge does not otherwise visit: it is the b of
// a match whose head is the last token of the preceding tile.  One warp shifts the tile left by one
// token in global memory (chunk by chunk: all reads of a chunk, then its writes) and writes the
// tile's next record.  Nobody else touches this tile during the merge.
__device__ __forceinline__ void drop_first_token(const EngineDev &e, int tile, int m, int lane) {
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
        const uint32_t *d = q + i * STBPE_QWORDS;
        merge_delta_terms<MG>(tab, e, a, b, nw, d[0], d[1], d[2], d[3], d[4], d[5], (int)d[6], (int)d[7]);
    }
    __syncwarp();
}

template <bool MG>
__global__ void __launch_bounds__(STBPE_CTA_THREADS, 2) merge_kernel(EngineDev e, unsigned int smem_slots) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    DevState *st = e.st;
    if (st->stopped || st->exchange_only) return;
    const uint32_t a = (uint32_t)st->cur_a, b = (uint32_t)st->cur_b, nw = (uint32_t)st->cur_new;
    const int m = st->merges_done;  // number of this merge (>= 1)
    if (m < 1) return;              // nothing has been selected yet
    const bool same = (a == b);

    TilePipe pipe;
    pipe.carve(smem_raw, smem_slots);
    pipe_setup(pipe);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n_work = st->n_work;  // < 0: every tile
    if (warp == STBPE_NCW) {
        produce_tiles(e, pipe, m, lane, n_work);
    } else {
        unsigned int *derr = &st->error;
        i64 removed = 0, matches = 0;
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
            uint32_t *s_tok = pipe.tok(stage);
            const int len = mp->len;
            int base = 0;          // tokens written so far (compacted in place)
            bool changed = false;  // warp-uniform
            bool any_head = false, last_head = false;  // warp-uniform
            // does the first token of the next chunk vanish (its left neighbour heads a match)?
            bool carry_drop = ((mp->prev & STBPE_IDMASK) == a) && (s_tok[0] == b);
            uint32_t pw4 = mp->prev2, pw5 = mp->prev;  // this lane's tokens 2,3 of the previous chunk (pre-merge)
            for (int cq = 0; cq < len; cq += STBPE_CHUNK) {
                const int q0 = cq + lane * 4;
                const uint4 raw = *reinterpret_cast<const uint4 *>(s_tok + q0);
                uint32_t w[9];  // pre-merge window: positions q0-2 .. q0+6
                w[2] = raw.x, w[3] = raw.y, w[4] = raw.z, w[5] = raw.w;
                const bool whole = (cq + STBPE_CHUNK <= len);  // warp-uniform
                unsigned int valid = 0xFu;                      // which of my 4 positions are in the tile
                if (!whole) {
                    valid = 0;
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        if (q0 + k < len) valid |= 1u << k;
                        else w[2 + k] = tok_or_halo(s_tok, mp, len, q0 + k);
                    }
                }
                // cheap test first: does any match start in this chunk?  Comparing the whole word of
                // a right-hand token with b also checks that it does not start a row.
                w[6] = __shfl_down_sync(0xFFFFFFFFu, w[2], 1);
                if (lane == 31) w[6] = tok_or_halo(s_tok, mp, len, cq + STBPE_CHUNK);
                unsigned int heads = 0;
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    if (((w[2 + k] & STBPE_IDMASK) == a) && (w[3 + k] == b)) heads |= 1u << k;
                heads &= valid;
                const int nvalid = min(STBPE_CHUNK, len - cq);
                if (__ballot_sync(0xFFFFFFFFu, heads != 0u) == 0u && !carry_drop) {
                    // nothing here matches or vanishes: keep, or slide left behind earlier drops
                    if (base != cq) {
                        __syncwarp();
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            if ((valid >> k) & 1u) s_tok[base + lane * 4 + k] = w[2 + k];
                    }
                    base += nvalid;
                    pw4 = w[4], pw5 = w[5];
                    continue;
                }
                // full window: neighbours across lanes
                w[0] = __shfl_up_sync(0xFFFFFFFFu, w[4], 1);
                w[1] = __shfl_up_sync(0xFFFFFFFFu, w[5], 1);
                w[7] = __shfl_down_sync(0xFFFFFFFFu, w[3], 1);
                w[8] = __shfl_down_sync(0xFFFFFFFFu, w[4], 1);
                {
                    const uint32_t c2 = __shfl_sync(0xFFFFFFFFu, pw4, 31), c1 = __shfl_sync(0xFFFFFFFFu, pw5, 31);
                    if (lane == 0) {
                        w[0] = cq ? c2 : mp->prev2;
                        w[1] = cq ? c1 : mp->prev;
                    }
                }
                if (lane == 31) {
                    w[7] = tok_or_halo(s_tok, mp, len, cq + STBPE_CHUNK + 1);
                    w[8] = tok_or_halo(s_tok, mp, len, cq + STBPE_CHUNK + 2);
                }
                uint32_t out[4];
                unsigned int keep = 0;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    out[k] = w[2 + k];
                    bool owns = false;
                    if ((valid >> k) & 1u) {
                        const uint32_t t0 = w[2 + k];
                        const bool M0 = (heads >> k) & 1u;
                        const bool D0 = (t0 == b) && ((w[1 + k] & STBPE_IDMASK) == a);
                        if (M0) out[k] = nw | (t0 & STBPE_FLAG);
                        if (!D0) keep |= 1u << k;
                        matches += (int)M0;
                        owns = same ? (M0 != D0) : M0;  // match head (a != b) or run head / tail (a == b)
                    }
                    const unsigned int om = __ballot_sync(0xFFFFFFFFu, owns);
                    if (om) {
                        if (owns) {
                            uint32_t *d = queue + (qn + __popc(om & lt)) * STBPE_QWORDS;
                            d[0] = w[k], d[1] = w[1 + k], d[2] = w[2 + k], d[3] = w[3 + k], d[4] = w[4 + k], d[5] = w[5 + k];
                            d[6] = (uint32_t)((q0 + k) > 0 ? tile : mp->prev_tile);
                            d[7] = (uint32_t)tile;
                        }
                        qn += __popc(om);
                        if (qn >= 32) {
                            drain_queue<MG>(pipe.tab, e, a, b, nw, queue, qn, lane);
                            qn = 0;
                        }
                    }
                }
                changed = true;  // a head or a carried drop: the tile is rewritten
                {
                    const unsigned int hb = __ballot_sync(0xFFFFFFFFu, heads != 0u);
                    any_head |= hb != 0u;
                    const int lastq = len - 1 - cq;  // position of the tile's last token in this chunk
                    if (lastq >= 0 && lastq < STBPE_CHUNK)
                        last_head = (__shfl_sync(0xFFFFFFFFu, heads, lastq >> 2) >> (lastq & 3)) & 1u;
                }
                // the last position of the chunk heads a match: its partner opens the next chunk
                carry_drop = ((__ballot_sync(0xFFFFFFFFu, (heads >> 3) & 1u) >> 31) & 1u) && whole;
                const int cnt = __popc(keep);
                int incl = cnt;
#pragma unroll
                for (int d = 1; d < 32; d <<= 1) {
                    const int n = __shfl_up_sync(0xFFFFFFFFu, incl, d);
                    if (lane >= d) incl += n;
                }
                int pos = base + incl - cnt;
                __syncwarp();  // all lanes hold their window before anyone overwrites the stage
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    if ((keep >> k) & 1u) s_tok[pos++] = out[k];
                base += __shfl_sync(0xFFFFFFFFu, incl, 31);
                pw4 = w[4], pw5 = w[5];
            }
            if (!changed) {
                __syncwarp();
                if (lane == 0) mbar_arrive(&pipe.empty[stage]);
                continue;
            }
            const int newlen = base;
            fence_async_smem();  // the bulk store reads these writes through the async proxy
            __syncwarp();
            if (same && last_head && lane == 0) {
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
                            filter_set(e, tile, ((u64)nw << 32) | (u64)y);
                        }
                    }
                }
            }
            if (lane == 0) {
                if (newlen > 0) {
                    tma_store_1d(e.tiles + (i64)tile * STBPE_TILE, s_tok, ((uint32_t)newlen * 4u + 15u) & ~15u);
                    tma_commit();
                    pending = stage;
                }
                // the record that is not current before this merge; readers of this merge never pick a
                // record stamped m, so payload and stamp need no ordering between them
                TileRec *dst = &e.recs[2 * tile + (mp->slot ^ 1)];
                dst->len = newlen;
                for (int i = 0; i < 3; ++i) dst->head[i] = i < newlen ? s_tok[i] : STBPE_NONE;
                dst->tail = newlen > 0 ? s_tok[newlen - 1] : STBPE_NONE;
                dst->tail2 = newlen > 1 ? s_tok[newlen - 2] : STBPE_NONE;
                dst->ver = m;
                removed += len - newlen;
                if (newlen == 0) mbar_arrive(&pipe.empty[stage]);
            }
        }
        drain_queue<MG>(pipe.tab, e, a, b, nw, queue, qn, lane);
        if (lane == 0) {
            tma_wait_all();  // bulk stores must have landed before the grid ends
            if (removed) atomicAdd((u64 *)&st->n_live, (u64)(-removed));
        }
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) matches += __shfl_down_sync(0xFFFFFFFFu, matches, d);
        if (lane == 0 && matches) atomicAdd((u64 *)&st->n_matches, (u64)matches);
    }
    __syncthreads();
    smem_table_flush<MG>(pipe.tab, e);
}
