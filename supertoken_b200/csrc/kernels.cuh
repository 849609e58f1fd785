// Kernels of the BPE merge-loop engine (sm_100a).  See common.cuh for the data layout.
#pragma once
#include "common.cuh"

// ---------------------------------------------------------------------------------------
// K1  pack: bytes / ids -> uint32 stream words, row-start flags, tile records
// ---------------------------------------------------------------------------------------
// identity byte -> id map of the reference's packer (gpu_tokenizer/cpu_packer.py:17-26)
__global__ void pack_bytes_kernel(const uint8_t *__restrict__ src, i64 n, uint32_t *__restrict__ dst) {
    i64 i = ((i64)blockIdx.x * blockDim.x + threadIdx.x) * 16;
    i64 stride = (i64)gridDim.x * blockDim.x * 16;
    bool aligned = ((((uintptr_t)src) | ((uintptr_t)dst)) & 15) == 0;
    for (; i < n; i += stride) {
        if (aligned && i + 16 <= n) {
            uint4 v = *reinterpret_cast<const uint4 *>(src + i);
            uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                uint4 o;
                o.x = w[q] & 0xFF;
                o.y = (w[q] >> 8) & 0xFF;
                o.z = (w[q] >> 16) & 0xFF;
                o.w = w[q] >> 24;
                *reinterpret_cast<uint4 *>(dst + i + 4 * q) = o;
            }
        } else {
            for (i64 k = i; k < n && k < i + 16; ++k) dst[k] = src[k];
        }
    }
}

__global__ void pack_ids_kernel(const int32_t *__restrict__ src, i64 n, uint32_t *__restrict__ dst,
                                unsigned int *bad) {
    i64 i = (i64)blockIdx.x * blockDim.x + threadIdx.x;
    i64 stride = (i64)gridDim.x * blockDim.x;
    for (; i < n; i += stride) {
        int32_t v = src[i];
        if (v < 0 || v == 0x7FFFFFFF) atomicOr(bad, STBPE_DERR_BAD_ID);  // ids must leave bit 31 and NONE free
        dst[i] = (uint32_t)v & STBPE_IDMASK;
    }
}

__global__ void mark_row_starts_kernel(const i64 *__restrict__ off, i64 n_rows, uint32_t *stream) {
    i64 r = (i64)blockIdx.x * blockDim.x + threadIdx.x;
    if (r < n_rows && off[r] < off[r + 1]) stream[off[r]] |= STBPE_FLAG;
}

__global__ void init_recs_kernel(EngineDev e, i64 n_tokens) {
    int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= e.n_tiles) return;
    i64 base = (i64)t * STBPE_TILE;
    i64 rem = n_tokens - base;
    int len = rem >= STBPE_TILE ? STBPE_TILE : (int)rem;
    TileRec r;
    r.ver = 0;
    r.len = len;
    for (int i = 0; i < 3; ++i) r.head[i] = i < len ? e.tiles[base + i] : STBPE_NONE;
    r.tail = len > 0 ? e.tiles[base + len - 1] : STBPE_NONE;
    r.tail2 = len > 1 ? e.tiles[base + len - 2] : STBPE_NONE;
    r.pad = 0;
    e.recs[2 * t] = r;
    r.ver = -1;
    r.len = 0;
    e.recs[2 * t + 1] = r;
}

__global__ void clear_table_kernel(EngineDev e) {
    u64 i = (u64)blockIdx.x * blockDim.x + threadIdx.x;
    u64 stride = (u64)gridDim.x * blockDim.x;
    for (; i <= e.mask; i += stride) {
        Slot s;
        s.key = STBPE_EMPTY;
        s.count = 0;
        e.table[i] = s;
    }
}

#include "tile_kernels.cuh"

// ---------------------------------------------------------------------------------------
// K2, byte-level fast path.  Right after a load of bytes the stream is dense (every tile full)
// and every id is below 256, so a pair key fits 16 bits and the whole histogram fits a CTA's
// shared memory as 65 536 16-bit counters (two per 32-bit word, 128 KB).  Each token costs one
// shared-memory atomic on a direct index: no hashing, no key compare.
// A 16-bit counter is kept below 2^15: the thread whose add takes it to 0x8000 moves 0x8000 of it
// to the global 64-bit counter.  Should a counter ever be seen above 0xC000 (16 384 further
// adds would have to slip in before that subtraction lands) the kernel raises
// STBPE_DERR_DENSE_OVERFLOW and the host recounts with the general kernel, so the result is exact
// or the failure is reported, never silently wrong.
// ---------------------------------------------------------------------------------------
// Word of the shared-memory table that holds the counter of a 16-bit key (two counters per word).
// The bank would be bits 1-5 of the right byte alone, and text concentrates those on a dozen values
// (lower-case letters, the space), so the low five bits are XOR-ed with the low bits of the left
// byte: a bijection inside each left-byte row that spreads hot right bytes over the banks.
__device__ __forceinline__ unsigned int dense_word(unsigned int key) { return (key >> 1) ^ ((key >> 8) & 31u); }

// rare path of dense_add: the add took one of the two 16-bit halves of the word to 0x8000 or beyond
__device__ __noinline__ void dense_hand_over(unsigned int *s_tab, u64 *g_dense, unsigned int *derr,
                                             unsigned int key, unsigned int now) {
    const unsigned int sh = (key & 1u) * 16u;
    const unsigned int h = (now >> sh) & 0xFFFFu;  // this key's counter after the add
    if (h == 0x8000u) {
        atomicSub(&s_tab[dense_word(key)], 0x8000u << sh);
        atomicAdd(&g_dense[key], 0x8000ull);
    } else if (h > 0xC000u) {
        atomicOr(derr, STBPE_DERR_DENSE_OVERFLOW);
    }
    // 0x8000 < h <= 0xC000: another thread is handing this counter over; h < 0x8000: it was the other half
}

__device__ __forceinline__ void dense_add(unsigned int *s_tab, u64 *g_dense, unsigned int *derr, uint32_t t0,
                                          uint32_t t1) {
    if ((int)t1 < 0) return;  // the right token starts a row (or lies past the end): bit 31 set
    // key = (low byte of t0) << 8 | t1; bytes 1 and 2 of t1 are zero for ids below 256
    const unsigned int key = __byte_perm(t1, t0, 0x2140);
    const unsigned int inc = (key & 1u) ? 0x10000u : 1u;
    const unsigned int now = atomicAdd(&s_tab[dense_word(key)], inc) + inc;
    if (now & 0x80008000u) dense_hand_over(s_tab, g_dense, derr, key, now);
}

#define STBPE_DENSE_THREADS 1024
#define STBPE_DENSE_UNROLL 4
__global__ void __launch_bounds__(STBPE_DENSE_THREADS, 1)
    count_dense_kernel(EngineDev e, i64 n_tokens, u64 *g_dense) {
    extern __shared__ __align__(16) unsigned int s_tab[];  // 32 768 words
    for (int i = threadIdx.x; i < 32768; i += STBPE_DENSE_THREADS) s_tab[i] = 0u;
    __syncthreads();
    const uint32_t *tok = e.tiles;
    unsigned int *derr = &e.st->error;
    const int lane = threadIdx.x & 31;
    const i64 span = (i64)STBPE_DENSE_THREADS * 4;  // tokens per CTA step
    for (i64 base = (i64)blockIdx.x * span * STBPE_DENSE_UNROLL; base < n_tokens;
         base += (i64)gridDim.x * span * STBPE_DENSE_UNROLL) {
        uint4 v[STBPE_DENSE_UNROLL];
        uint32_t nx[STBPE_DENSE_UNROLL];
#pragma unroll
        for (int u = 0; u < STBPE_DENSE_UNROLL; ++u) {  // all loads first: several in flight per thread
            const i64 i = base + u * span + (i64)threadIdx.x * 4;
            if (i + 4 <= n_tokens) {
                v[u] = *reinterpret_cast<const uint4 *>(tok + i);
            } else {
                v[u].x = i < n_tokens ? tok[i] : STBPE_NONE;
                v[u].y = i + 1 < n_tokens ? tok[i + 1] : STBPE_NONE;
                v[u].z = i + 2 < n_tokens ? tok[i + 2] : STBPE_NONE;
                v[u].w = i + 3 < n_tokens ? tok[i + 3] : STBPE_NONE;
            }
            nx[u] = (lane == 31) ? (i + 4 < n_tokens ? tok[i + 4] : STBPE_NONE) : 0u;
        }
        // tokens past the end were loaded as STBPE_NONE: as a right-hand token NONE carries the
        // row-start flag (no pair), and a left-hand NONE is always followed by another NONE
#pragma unroll
        for (int u = 0; u < STBPE_DENSE_UNROLL; ++u) {
            uint32_t n0 = __shfl_down_sync(0xFFFFFFFFu, v[u].x, 1);
            if (lane == 31) n0 = nx[u];
            dense_add(s_tab, g_dense, derr, v[u].x, v[u].y);
            dense_add(s_tab, g_dense, derr, v[u].y, v[u].z);
            dense_add(s_tab, g_dense, derr, v[u].z, v[u].w);
            dense_add(s_tab, g_dense, derr, v[u].w, n0);
        }
    }
    __syncthreads();
    for (int p = threadIdx.x; p < 32768; p += STBPE_DENSE_THREADS) {
        const unsigned int x = s_tab[p];
        const unsigned int w = (unsigned int)p ^ (((unsigned int)p >> 7) & 31u);  // inverse of dense_word
        if (x & 0xFFFFu) atomicAdd(&g_dense[2 * w], (u64)(x & 0xFFFFu));
        if (x >> 16) atomicAdd(&g_dense[2 * w + 1], (u64)(x >> 16));
    }
}

// Insert a key that is known to be absent (every directly indexed counter is its own key, and the
// table was cleared before the count): one compare-and-swap claims the slot, the count is a plain
// store, and nothing is marked dirty because a full refresh follows the initial count.
__device__ __forceinline__ bool table_insert_unique(const EngineDev &e, u64 key, i64 count) {
    u64 h = slot_of(e, key);
    for (unsigned int probe = 0; probe < STBPE_MAX_PROBE; ++probe) {
        Slot *s = &e.table[h];
        if (atomicCAS(&s->key, STBPE_EMPTY, key) == STBPE_EMPTY) {
            s->count = count;
            return true;
        }
        h = (h + 1) & e.mask;
    }
    atomicOr(&e.st->error, STBPE_DERR_TABLE_FULL);
    return false;
}

#include "wide_count.cuh"

// dense 16-bit keys -> entries of the pair table (or of the rank-local delta table)
template <bool MG>
__global__ void dense_to_table_kernel(EngineDev e, const u64 *g_dense) {
    const int k = blockIdx.x * blockDim.x + threadIdx.x;
    if (k >= 65536) return;
    const u64 c = g_dense[k];
    if (c) sink_add<MG>(e, ((u64)(k >> 8) << 32) | (u64)(k & 0xFF), (i64)c);
}

// ---------------------------------------------------------------------------------------
// K4  arg-max: block maxima refresh + reduction with the reference's tie-break
// ---------------------------------------------------------------------------------------
// recompute the maximum of blocks [w0, n) of the dirty list (or of all blocks), one warp per block
__device__ __forceinline__ void refresh_blocks(const EngineDev &e, int all, unsigned int n, unsigned int w,
                                               unsigned int nwarps) {
    const unsigned int lane = threadIdx.x & 31;
    for (; w < n; w += nwarps) {
        const unsigned int blk = all ? w : e.dirty_list[w];
        const Slot *base = e.table + (u64)blk * STBPE_BLK;
        u64 bk = STBPE_EMPTY;
        i64 bc = 0;
#pragma unroll
        for (int j = 0; j < STBPE_BLK / 32; ++j) {
            const uint4 raw = *reinterpret_cast<const uint4 *>(base + j * 32 + lane);
            const u64 k = ((u64)raw.y << 32) | raw.x;
            const i64 c = (i64)(((u64)raw.w << 32) | raw.z);
            if (k != STBPE_EMPTY && c > 0 && better(k, c, bk, bc)) {
                bk = k;
                bc = c;
            }
        }
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) {
            const u64 ok = __shfl_down_sync(0xFFFFFFFFu, bk, d);
            const i64 oc = __shfl_down_sync(0xFFFFFFFFu, bc, d);
            if (better(ok, oc, bk, bc)) {
                bk = ok;
                bc = oc;
            }
        }
        if (lane == 0) {
            Slot s;
            s.key = bk;
            s.count = bc;
            const Slot was = e.blockmax[blk];
            e.blockmax[blk] = s;
            e.dirty_flag[blk] = 0u;
            const unsigned int sb = blk >> 8;
            // the super-block is recomputed only if this block's maximum really changed
            if (!all && (was.key != s.key || was.count != s.count) && atomicExch(&e.dirty2_flag[sb], 1u) == 0u)
                e.dirty2_list[atomicAdd(&e.st->n_dirty2, 1u)] = sb;
        }
    }
}

__global__ void refresh_kernel(EngineDev e, int all) {
    dep_release();
    dep_wait();
    const unsigned int n = all ? e.n_blocks : min(e.st->n_dirty, e.n_blocks);
    refresh_blocks(e, all, n, (blockIdx.x * blockDim.x + threadIdx.x) >> 5, (gridDim.x * blockDim.x) >> 5);
}

__device__ __forceinline__ i64 find_slot(const EngineDev &e, u64 key) {
    u64 h = slot_of(e, key);
    for (unsigned int probe = 0; probe < STBPE_MAX_PROBE; ++probe) {
        const u64 k = *(volatile u64 *)&e.table[h].key;
        if (k == key) return (i64)h;
        if (k == STBPE_EMPTY) return -1;
        h = (h + 1) & e.mask;
    }
    return -1;
}

// Bookkeeping of one selected merge (gpu_tokenizer/bpe_trainer.py:4358-4373): log it, make it
// current, zero its table entry (no (a,b) pair survives its own merge).
__device__ __forceinline__ void begin_merge(const EngineDev &e, u64 key, i64 count, int new_id,
                                            bool may_be_absent) {
    DevState *st = e.st;
    const int mnum = st->merges_done;
    e.merges[2 * mnum] = (int32_t)(key >> 32);
    e.merges[2 * mnum + 1] = (int32_t)(key & 0xFFFFFFFFull);
    e.merge_counts[mnum] = count;
    e.live_before[mnum] = st->n_live;
    st->cur_a = (int)(key >> 32);
    st->cur_b = (int)(key & 0xFFFFFFFFull);
    st->cur_new = new_id;
    st->cur_count = count;
    st->merges_done = mnum + 1;
    st->n_work = 0;  // the worklist of this merge starts empty (worklist_kernel appends)
    const i64 h = find_slot(e, key);
    if (h >= 0) {
        e.table[h].count = 0;
        mark_dirty(e, (u64)h);
    } else if (!may_be_absent) {
        atomicOr(&st->error, STBPE_DERR_KEY_MISSING);
    }
}

// stop rules of the loop: bpe_trainer.py:4304-4308 (no pairs), :2491-2494 / :4361-4364 (count < 2)
__device__ __forceinline__ void advance_or_stop(const EngineDev &e, u64 key, i64 count) {
    DevState *st = e.st;
    st->n_dirty = 0;
    if (st->error) {
        st->stopped = 1;
        st->stop_reason = 4;
    } else if (st->merges_done >= st->target) {
        st->stopped = 1;
        st->stop_reason = 1;
    } else if (count <= 0) {
        st->stopped = 1;
        st->stop_reason = 2;
    } else if (count < 2) {
        st->stopped = 1;
        st->stop_reason = 3;
    } else {
        begin_merge(e, key, count, st->base_vocab + st->merges_done, e.world > 1);
    }
}

// mode 0: peek (result into st->peek_*), 1: advance the loop, 2: write candidate to cand[0..3].
// all2 != 0: recompute every super-block maximum (after a full rebuild of the block maxima),
// otherwise only the super-blocks the last refresh marked.  The last CTA to finish reduces the
// super-block maxima and finalises.
#define STBPE_SELECT_THREADS 256
__device__ __forceinline__ void block_best(u64 &bk, i64 &bc, u64 *s_k, i64 *s_c) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
        const u64 ok = __shfl_down_sync(0xFFFFFFFFu, bk, d);
        const i64 oc = __shfl_down_sync(0xFFFFFFFFu, bc, d);
        if (better(ok, oc, bk, bc)) {
            bk = ok;
            bc = oc;
        }
    }
    if (lane == 0) {
        s_k[warp] = bk;
        s_c[warp] = bc;
    }
    __syncthreads();
    if (threadIdx.x == 0)
        for (int w = 1; w < STBPE_SELECT_THREADS / 32; ++w)
            if (better(s_k[w], s_c[w], bk, bc)) {
                bk = s_k[w];
                bc = s_c[w];
            }
    __syncthreads();
}

#include "peer_kernels.cuh"

// recompute the maximum of super-blocks [w, n) of the second dirty list (or of all): one warp per
// super-block, 256 block maxima, 8 per lane
__device__ __forceinline__ void refresh_super_blocks(const EngineDev &e, int all2, unsigned int n2, unsigned int w,
                                                     unsigned int nwarps) {
    const unsigned int lane = threadIdx.x & 31;
    for (unsigned int i = w; i < n2; i += nwarps) {
        const unsigned int sb = all2 ? i : e.dirty2_list[i];
        u64 bk = STBPE_EMPTY;
        i64 bc = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const unsigned int blk = sb * 256u + j * 32u + lane;
            if (blk < e.n_blocks) {
                const uint4 raw = __ldcg(reinterpret_cast<const uint4 *>(e.blockmax + blk));
                const u64 k = ((u64)raw.y << 32) | raw.x;
                const i64 c = (i64)(((u64)raw.w << 32) | raw.z);
                if (c > 0 && better(k, c, bk, bc)) {
                    bk = k;
                    bc = c;
                }
            }
        }
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) {
            const u64 ok = __shfl_down_sync(0xFFFFFFFFu, bk, d);
            const i64 oc = __shfl_down_sync(0xFFFFFFFFu, bc, d);
            if (better(ok, oc, bk, bc)) {
                bk = ok;
                bc = oc;
            }
        }
        if (lane == 0) {
            Slot s;
            s.key = bk;
            s.count = bc;
            e.supermax[sb] = s;
            e.dirty2_flag[sb] = 0u;
        }
    }
}

// mode 0: peek (result into the state); 1: single rank, advance or stop; 2: candidate of this rank
// into cand; 3: candidate of this rank into every peer mailbox, then wait for the peers' candidates
// and commit (target = the merge target of the engine)
__global__ void __launch_bounds__(STBPE_SELECT_THREADS)
    select_kernel(EngineDev e, int mode, int all2, i64 *cand, int target = 0) {
    dep_release();
    dep_wait();
    DevState *st = e.st;
    const int stopped = st->stopped;            // both in one round trip
    const unsigned int n_dirty2 = st->n_dirty2;
    if (mode == 1 && stopped) return;
    __shared__ u64 s_k[STBPE_SELECT_THREADS / 32];
    __shared__ i64 s_c[STBPE_SELECT_THREADS / 32];
    __shared__ int s_last;
    const unsigned int n2 = all2 ? e.n_super2 : min(n_dirty2, e.n_super2);
    refresh_super_blocks(e, all2, n2, blockIdx.x * (STBPE_SELECT_THREADS / 32) + (threadIdx.x >> 5),
                         gridDim.x * (STBPE_SELECT_THREADS / 32));
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        s_last = (atomicAdd(&st->ticket, 1u) == gridDim.x - 1);
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    u64 bk = STBPE_EMPTY;
    i64 bc = 0;
    for (unsigned int i = threadIdx.x; i < e.n_super2; i += STBPE_SELECT_THREADS) {
        const volatile Slot *p = e.supermax + i;
        const u64 k = p->key;
        const i64 c = p->count;
        if (c > 0 && better(k, c, bk, bc)) {
            bk = k;
            bc = c;
        }
    }
    block_best(bk, bc, s_k, s_c);
    if (threadIdx.x != 0) return;
    st->ticket = 0;
    st->n_dirty2 = 0;
    if (mode == 0) {
        st->peek_key = bk;
        st->peek_count = bc;
    } else if (mode == 1) {
        advance_or_stop(e, bk, bc);
    } else if (mode == 2) {
        cand[0] = (i64)bk;
        cand[1] = bc;
        cand[2] = st->round_incomplete;
        cand[3] = 0;
    } else {
        publish_candidate(e, bk, bc, st->round_incomplete);
        commit_from_mailbox(e, target);
    }
}

// ---------------------------------------------------------------------------------------
// Tile skipping.  A merge (a,b) changes a tile only if a match head sits in it (the pair (a,b)
// starts there) or if its first token is the partner of a head that ends the tile before it.  The
// pair filter records, per tile, which pairs start in it (including the pair formed by its last
// token and the first token of the next non-empty tile), so
//     visit tile t  iff  all three filter rows of (a,b) have bit t set.
// A partner in a tile that is not visited is dropped by the warp that owns the head (fix-up in the
// merge kernel).  This kernel builds the bitmap of visited tiles and the compact worklist.
// ---------------------------------------------------------------------------------------
// the tiles merge (cur_a, cur_b) must visit: bitmap and compact list; `block` of `n_blocks` thread
// blocks of blockDim.x threads share the words of the bitmap
__device__ __forceinline__ void build_worklist(const EngineDev &e, int block, int n_blocks, int cur_a, int cur_b) {
    DevState *st = e.st;
    unsigned int r1, r2, r3;
    filter_rows(((u64)(uint32_t)cur_a << 32) | (u64)(uint32_t)cur_b, r1, r2, r3);
    const unsigned int *row1 = e.presence + (size_t)r1 * e.presence_words;
    const unsigned int *row2 = e.presence + (size_t)r2 * e.presence_words;
    const unsigned int *row3 = e.presence + (size_t)r3 * e.presence_words;
    const unsigned int *wild = e.presence + (size_t)STBPE_PROWS * e.presence_words;
    const int n_words = (e.n_tiles + 31) / 32;
    const int lane = threadIdx.x & 31;
    for (int w0 = block * blockDim.x; w0 < n_words; w0 += n_blocks * blockDim.x) {
        const int w = w0 + threadIdx.x;
        unsigned int c = 0;
        if (w < n_words) {
            c = (__ldcg(row1 + w) & __ldcg(row2 + w) & __ldcg(row3 + w)) | __ldcg(wild + w);
            const int rem = e.n_tiles - w * 32;
            if (rem < 32) c &= (1u << rem) - 1u;
            e.cand_bits[w] = c;
        }
        // warp-aggregated append of the set bits
        const int cnt = __popc(c);
        int incl = cnt;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int n = __shfl_up_sync(0xFFFFFFFFu, incl, d);
            if (lane >= d) incl += n;
        }
        const int total = __shfl_sync(0xFFFFFFFFu, incl, 31);
        int base = 0;
        if (lane == 31 && total) base = atomicAdd(&st->n_work, total);
        base = __shfl_sync(0xFFFFFFFFu, base, 31) + incl - cnt;
        while (c) {
            const int bit = __ffs(c) - 1;
            c &= c - 1;
            e.worklist[base++] = (unsigned int)(w * 32 + bit);
        }
    }
}

__global__ void __launch_bounds__(1024) worklist_kernel(EngineDev e) {
    dep_release();
    dep_wait();
    DevState *st = e.st;
    const int stopped = st->stopped, exchange_only = st->exchange_only, filter_valid = st->filter_valid;
    const int cur_a = st->cur_a, cur_b = st->cur_b;  // all in one round trip
    if (stopped || exchange_only) return;
    if (!filter_valid) {  // stale filter: the merge visits every tile
        if (blockIdx.x == 0 && threadIdx.x == 0) st->n_work = -1;
        return;
    }
    build_worklist(e, blockIdx.x, gridDim.x, cur_a, cur_b);
}

// (Re)build the pair filter from the stream: after a load and after every re-pack.  One CTA handles
// 32 consecutive tiles, i.e. one word of every row: it collects the bits in shared memory and then
// writes the STBPE_PROWS words with plain stores.
__global__ void __launch_bounds__(1024) presence_rebuild_kernel(EngineDev e) {
    extern __shared__ unsigned int s_rows[];  // STBPE_PROWS words
    const int n_groups = (e.n_tiles + 31) / 32;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int grp = blockIdx.x; grp < n_groups; grp += gridDim.x) {
        for (int i = threadIdx.x; i < STBPE_PROWS; i += blockDim.x) s_rows[i] = 0u;
        __syncthreads();
        const int tile = grp * 32 + warp;  // blockDim.x == 1024: one warp per tile of the group
        if (tile < e.n_tiles) {
            TileRec r;
            current_rec(e, tile, 0x7FFFFFFF, r);
            if (r.len > 0) {
                const uint32_t *g = e.tiles + (i64)tile * STBPE_TILE;
                uint32_t nxt0 = STBPE_NONE;  // first live token after the tile
                for (int t = tile + 1; t < e.n_tiles; ++t) {
                    TileRec rn;
                    current_rec(e, t, 0x7FFFFFFF, rn);
                    if (rn.len > 0) {
                        nxt0 = rn.head[0];
                        break;
                    }
                }
                for (int i = lane; i < r.len; i += 32) {
                    const uint32_t t1 = (i + 1 < r.len) ? g[i + 1] : nxt0;
                    if (t1 & STBPE_FLAG) continue;  // not a countable pair
                    unsigned int r1, r2, r3;
                    filter_rows(((u64)(g[i] & STBPE_IDMASK) << 32) | (u64)t1, r1, r2, r3);
                    atomicOr(&s_rows[r1], 1u << warp);
                    atomicOr(&s_rows[r2], 1u << warp);
                    atomicOr(&s_rows[r3], 1u << warp);
                }
            }
        }
        __syncthreads();
        for (int i = threadIdx.x; i < STBPE_PROWS; i += blockDim.x)
            e.presence[(size_t)i * e.presence_words + grp] = s_rows[i];
        if (threadIdx.x == 0) e.presence[(size_t)STBPE_PROWS * e.presence_words + grp] = 0u;  // no wildcards
        __syncthreads();
    }
}

// number of keys that hold exactly `count` (tie statistics; full table scan, on demand only)
__global__ void count_ties_kernel(EngineDev e) {
    const i64 target = e.st->peek_count;
    i64 n = 0;
    for (u64 i = (u64)blockIdx.x * blockDim.x + threadIdx.x; i <= e.mask; i += (u64)gridDim.x * blockDim.x) {
        const Slot s = e.table[i];
        if (s.key != STBPE_EMPTY && s.count == target) ++n;
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) n += __shfl_down_sync(0xFFFFFFFFu, n, d);
    if ((threadIdx.x & 31) == 0 && n) atomicAdd((u64 *)&e.st->peek_ties, (u64)n);
}

// host-requested merge (stbpe_apply_merge): same bookkeeping as a selected one
__global__ void force_merge_kernel(EngineDev e, int a, int b, int new_id) {
    DevState *st = e.st;
    st->n_dirty = 0;
    st->stopped = 0;
    st->stop_reason = 0;
    st->n_matches = 0;
    const u64 key = ((u64)(uint32_t)a << 32) | (u64)(uint32_t)b;
    const i64 h = find_slot(e, key);
    const i64 count = h >= 0 ? e.table[h].count : 0;
    begin_merge(e, key, count, new_id, true);  // merging a pair that never occurs is legal
}

// ---------------------------------------------------------------------------------------
// exports
// ---------------------------------------------------------------------------------------
__global__ void export_table_kernel(EngineDev e, u64 *keys, i64 *counts, i64 cap) {
    for (u64 i = (u64)blockIdx.x * blockDim.x + threadIdx.x; i <= e.mask; i += (u64)gridDim.x * blockDim.x) {
        const Slot s = e.table[i];
        if (s.key != STBPE_EMPTY && s.count != 0) {
            const i64 j = (i64)atomicAdd((u64 *)&e.st->export_n, 1ull);
            if (j < cap) {
                keys[j] = s.key;
                counts[j] = s.count;
            }
        }
    }
}

// keys whose count equals `count` (unordered; the host sorts the few there are)
__global__ void export_ties_kernel(EngineDev e, i64 count, u64 *keys, i64 cap) {
    for (u64 i = (u64)blockIdx.x * blockDim.x + threadIdx.x; i <= e.mask; i += (u64)gridDim.x * blockDim.x) {
        const Slot s = e.table[i];
        if (s.key != STBPE_EMPTY && s.count == count) {
            const i64 j = (i64)atomicAdd((u64 *)&e.st->export_n, 1ull);
            if (j < cap) keys[j] = s.key;
        }
    }
}

// tile_off[t] = exclusive prefix of the current tile lengths (computed by the host)
__global__ void export_stream_kernel(EngineDev e, const i64 *__restrict__ tile_off, int32_t *out) {
    for (int tile = blockIdx.x; tile < e.n_tiles; tile += gridDim.x) {
        const int len = (int)(tile_off[tile + 1] - tile_off[tile]);
        const uint32_t *g = e.tiles + (i64)tile * STBPE_TILE;
        for (int i = threadIdx.x; i < len; i += blockDim.x) out[tile_off[tile] + i] = (int32_t)g[i];
    }
}

// Re-pack: tiles only ever shrink, so after many merges they are sparsely filled and the per-tile
// cost of the pipeline is spread over few tokens.  The live tokens of all tiles are copied, in
// order, into a dense stream (tile_off = exclusive prefix of the tile lengths).
__global__ void repack_copy_kernel(EngineDev e, const i64 *__restrict__ tile_off, uint32_t *__restrict__ dst) {
    const int warps_per_block = blockDim.x >> 5, lane = threadIdx.x & 31;
    for (long long tile = (long long)blockIdx.x * warps_per_block + (threadIdx.x >> 5); tile < e.n_tiles;
         tile += (long long)gridDim.x * warps_per_block) {
        const i64 o = tile_off[tile];
        const int len = (int)(tile_off[tile + 1] - o);
        const uint32_t *g = e.tiles + (i64)tile * STBPE_TILE;
        for (int i = lane; i < len; i += 32) dst[o + i] = g[i];
    }
}

__global__ void tile_lens_kernel(EngineDev e, i64 *lens) {
    int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= e.n_tiles) return;
    TileRec r;
    current_rec(e, t, 0x7FFFFFFF, r);
    lens[t] = r.len;
}

// ---------------------------------------------------------------------------------------
// multi-GPU: drain the rank-local delta table into per-owner outbox chunks; apply an inbox
// ---------------------------------------------------------------------------------------
// chunk headers start a round at zero: done once when the buffers are set and after every exchange
// (apply_inbox_kernel), so a round needs no separate reset launch
__global__ void outbox_reset_kernel(EngineDev e) {
    int p = blockIdx.x * blockDim.x + threadIdx.x;
    if (p < e.world) {
        Slot h;
        h.key = 0;
        h.count = 0;
        e.outbox[(i64)p * (e.cap_per_peer + 1)] = h;
    }
    if (p == 0) {
        e.st->n_lkept = 0;
        e.st->round_incomplete = 0;
    }
}

// Move the rank-local deltas into the per-owner outbox chunks.  A chunk holds cap_per_peer
// entries; what does not fit stays in the local table and is listed again for the next round
// (the header count of a chunk keeps counting past the capacity, which tells the receiver that
// more is to come).
__global__ void drain_ltable_kernel(EngineDev e) {
    __shared__ int s_last;
    const unsigned int n = e.st->n_ltouched;
    unsigned int *kept = e.ltouched + (e.lmask + 1);
    for (unsigned int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const unsigned int idx = e.ltouched[i];
        Slot *s = &e.ltable[idx];
        const Slot v = *s;
        if (v.count != 0) {
            const int owner = owner_of(v.key, e.world);
            Slot *chunk = e.outbox + (i64)owner * (e.cap_per_peer + 1);
            const i64 j = (i64)atomicAdd(&chunk[0].key, 1ull);
            if (j >= e.cap_per_peer) {
                kept[atomicAdd(&e.st->n_lkept, 1u)] = idx;
                e.st->round_incomplete = 1;
                continue;
            }
            chunk[1 + j] = v;
        }
        s->key = STBPE_EMPTY;
        s->count = 0;
    }
    // the last CTA to finish turns the kept entries into the list the next inserts append to
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        s_last = (atomicAdd(&e.st->ticket, 1u) == gridDim.x - 1);
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    const unsigned int nk = *(volatile unsigned int *)&e.st->n_lkept;
    for (unsigned int i = threadIdx.x; i < nk; i += blockDim.x) e.ltouched[i] = ((volatile unsigned int *)kept)[i];
    __syncthreads();
    if (threadIdx.x == 0) {
        e.st->n_ltouched = nk;
        e.st->n_lkept = 0;
        e.st->ticket = 0;
    }
}

__global__ void apply_inbox_kernel(EngineDev e) {
    if (blockIdx.x == 0 && threadIdx.x < e.world) {  // the exchange is over: headers for the next round
        Slot h;
        h.key = 0;
        h.count = 0;
        e.outbox[(i64)threadIdx.x * (e.cap_per_peer + 1)] = h;
    }
    for (int p = 0; p < e.world; ++p) {
        const Slot *chunk = e.inbox + (i64)p * (e.cap_per_peer + 1);
        i64 n = (i64)chunk[0].key;
        if (n > e.cap_per_peer) {
            n = e.cap_per_peer;
            if (blockIdx.x == 0 && threadIdx.x == 0) e.st->round_incomplete = 1;
        }
        for (i64 i = (i64)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (i64)gridDim.x * blockDim.x) {
            const Slot v = chunk[1 + i];
            table_add(e, v.key, v.count);
        }
    }
}

// Every rank evaluates the same gathered candidates {key, count, incomplete, -} and reaches the
// same decision: if any rank still has deltas in flight the next round only exchanges, otherwise
// the best candidate (highest count, smallest key) is committed or a stop rule fires.
__global__ void commit_kernel(EngineDev e, const i64 *all_cands, int target) {
    DevState *st = e.st;
    st->target = target;
    st->round_incomplete = 0;  // the candidates carried this round's flag; the next round starts clean
    if (st->stopped) return;
    u64 bk = STBPE_EMPTY;
    i64 bc = 0;
    bool incomplete = false;
    for (int r = 0; r < e.world; ++r) {
        const u64 k = (u64)all_cands[4 * r];
        const i64 c = all_cands[4 * r + 1];
        incomplete |= all_cands[4 * r + 2] != 0;
        if (c > 0 && better(k, c, bk, bc)) {
            bk = k;
            bc = c;
        }
    }
    if (incomplete) {
        st->n_dirty = 0;
        st->exchange_only = 1;
        return;
    }
    st->exchange_only = 0;
    advance_or_stop(e, bk, bc);
}
