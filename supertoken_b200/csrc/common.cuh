// Shared device-side definitions of the BPE merge-loop engine (sm_100a).
//
// Data layout in HBM
//   token stream : tiles of STBPE_TILE uint32 words; a tile keeps its live tokens compacted
//                  at the front, its length lives in the tile record.  Bit 31 of a word
//                  marks the first token of a row; a pair (i, i+1) is countable iff token
//                  i+1 does not carry that bit (rows are the only pair-breaking boundary,
//                  gpu_tokenizer/utils.py:586).
//   tile records : two versioned 32-byte records per tile {ver, len, first three live
//                  tokens, last live token}.  During merge number m a tile is rewritten in
//                  place by exactly one CTA, while neighbouring CTAs need its PRE-merge
//                  head and tail.  A writer therefore fills the record with the older
//                  version and stamps it m; readers use the record with the largest
//                  version below m, which nobody writes during merge m.
//   pair table   : open addressing, linear probing, 16-byte slots {key = (a<<32)|b,
//                  int64 count}.  Keys are never removed; a count may return to zero.
//   block maxima : best (count, smallest key) of every block of 256 slots, and of every
//                  256 blocks above that; only blocks touched by a merge are recomputed, the
//                  arg-max reduces the few top-level maxima.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#define STBPE_TILE 1024  // tokens per tile: one consumer warp owns a whole tile
#define STBPE_NONE 0xFFFFFFFFu
#define STBPE_FLAG 0x80000000u
#define STBPE_IDMASK 0x7FFFFFFFu
#define STBPE_EMPTY 0xFFFFFFFFFFFFFFFFull
#define STBPE_BLK 256
#define STBPE_PROWS 16384  // rows of the pair filter: pair keys are hashed onto them (three hashes)
#define STBPE_MAX_PROBE (1u << 20)

// device error bits
#define STBPE_DERR_TABLE_FULL 1u
#define STBPE_DERR_OUTBOX_FULL 2u
#define STBPE_DERR_LTABLE_FULL 4u
#define STBPE_DERR_KEY_MISSING 8u
#define STBPE_DERR_BAD_ID 16u
#define STBPE_DERR_DENSE_OVERFLOW 64u

typedef unsigned long long u64;
typedef long long i64;

struct __align__(16) Slot {
    u64 key;
    i64 count;
};

struct __align__(16) TileRec {
    int ver;  // merge number that wrote this record; 0 = written at load; <0 = never written
    int len;
    uint32_t head[3];
    uint32_t tail;   // last live token
    uint32_t tail2;  // second to last live token (STBPE_NONE when len < 2)
    uint32_t pad;
};

struct DevState {
    int cur_a, cur_b, cur_new;
    int filter_valid;          // the pair filter describes the stream: merges maintain it and skip tiles by it;
                               // 0 = stale (every merge visits every tile and leaves the filter alone)
    i64 cur_count;
    int merges_done, target, base_vocab, stopped;
    int stop_reason;
    unsigned int n_dirty;
    unsigned int error;
    unsigned int ticket;
    u64 n_keys;
    i64 n_live;
    i64 n_matches;
    u64 peek_key;
    i64 peek_count;
    i64 peek_ties;
    unsigned int n_ltouched;   // entries of the rank-local delta table awaiting the drain
    unsigned int n_lkept;      // entries the last drain had to keep (outbox chunk full)
    i64 export_n;
    unsigned int n_dirty2;     // super-blocks whose maximum must be recomputed
    unsigned int pad1;
    int n_work;                // tiles on this merge's worklist; < 0 = every tile
    int pad3;
    unsigned int n_fixups;     // partners dropped in a tile the merge did not visit (statistics)
    int pad2;
    int exchange_only;         // multi-GPU: deltas still in flight, the next round only exchanges
    int round_incomplete;      // multi-GPU: this rank saw a full chunk or kept entries this round
    u64 tile_bytes_in;         // merge kernel: bytes its bulk copies and record look-ups brought in ...
    u64 tile_bytes_out;        // ... and bytes it stored (rewritten tile parts and records), since the load
};

// Peer mailboxes (multi-GPU exchange over NVLink peer memory, no library collective).  Every rank owns
// one mailbox in its own HBM that its peers map: a header of flags and candidates followed by one
// inbox chunk per sender.  Flags carry the round number and only grow, so nothing is ever reset.
#define STBPE_MAX_PEERS 16
#define STBPE_MAIL_HEADER_BYTES 2048
struct MailHeader {
    u64 inbox_flag[STBPE_MAX_PEERS];     // [src] = last round whose chunk from src is complete here
    u64 cand_flag[STBPE_MAX_PEERS];      // [src] = last round whose candidate from src is here
    i64 cands[STBPE_MAX_PEERS][4];       // [src] = {key, count, incomplete, -}
    u64 round;                           // rounds this rank has committed (own use only)
    unsigned int out_count[STBPE_MAX_PEERS];  // entries sent to each owner this round (own use only)
};
static_assert(sizeof(MailHeader) <= STBPE_MAIL_HEADER_BYTES, "mailbox header does not fit");

struct EngineDev {
    unsigned char *mail[STBPE_MAX_PEERS];  // mailbox of every rank ([rank] = own), or null
    uint32_t *tiles;
    TileRec *recs;  // 2 per tile
    int n_tiles;
    Slot *table;
    u64 mask;
    int slot_bits;  // slot index bits below the table slice of a partition (slots = slices << slot_bits)
    Slot *blockmax;
    unsigned int *dirty_flag;
    unsigned int *dirty_list;
    unsigned int n_blocks;
    // presence[r][w]: bit t of word w of row r says "a pair whose key hashes to r may start in tile
    // 32*w + t" (the tile of the pair's left token; set when such a pair comes into being, never
    // cleared until the next re-pack).  A Bloom filter with three hashes per pair: false positives
    // cost a wasted visit, never a missed one.  Row STBPE_PROWS is a wildcard: tiles that every
    // merge visits because the pair that starts at their last token is not known exactly (their
    // last token is the result of a run of equal tokens that ran on into the next tile).
    unsigned int *presence;
    unsigned int presence_words;  // words per row
    unsigned int *cand_bits;      // tiles the current merge must visit
    unsigned int *worklist;
    Slot *supermax;             // best entry of every 256 blocks (second level of the arg-max)
    unsigned int *dirty2_flag;
    unsigned int *dirty2_list;
    unsigned int n_super2;
    DevState *st;
    int32_t *merges;
    i64 *merge_counts;
    i64 *live_before;
    // multi-GPU: rank-local delta table, emptied into the per-owner outbox
    int world, rank;
    Slot *ltable;
    u64 lmask;
    unsigned int *ltouched;  // 2 lists of lslots entries: [0] filled by inserts, [1] by the drain
    Slot *outbox;  // [world][1 + cap] entries; entry 0 of a chunk = {count, 0}
    Slot *inbox;
    i64 cap_per_peer;
};

__device__ __forceinline__ MailHeader *mail_header(const EngineDev &e, int r) {
    return reinterpret_cast<MailHeader *>(e.mail[r]);
}
// chunk that rank `src` fills in the mailbox of rank `dst`
__device__ __forceinline__ Slot *mail_chunk(const EngineDev &e, int dst, int src) {
    return reinterpret_cast<Slot *>(e.mail[dst] + STBPE_MAIL_HEADER_BYTES) + (i64)src * (e.cap_per_peer + 1);
}

__device__ __forceinline__ u64 mix64(u64 x) {
    x ^= x >> 33;
    x *= 0xff51afd7ed558ccdULL;
    x ^= x >> 33;
    x *= 0xc4ceb9fe1a85ec53ULL;
    x ^= x >> 33;
    return x;
}


// Partition of a pair key: the top STBPE_PART_BITS bits of an invertible 32-bit mix of the key folded
// to 32 bits (for ids below 65 536 the fold is (a << 16) | b itself, so the mixed word identifies the
// pair).  One function places a key three ways: the partition is the top bits of its slot in the
// pair table (so the keys of a partition fill one contiguous slice of the table, which the
// partitioned first count keeps in L2 while it fills it), it is the partition of that count, and
// its residue modulo the number of ranks is the rank that owns the key.
#define STBPE_PART_BITS 8
#define STBPE_PARTS (1 << STBPE_PART_BITS)
__host__ __device__ __forceinline__ uint32_t mix32(uint32_t x) {
    x ^= x >> 16;
    x *= 0x7feb352du;
    x ^= x >> 15;
    x *= 0x846ca68bu;
    x ^= x >> 16;
    return x;
}
__host__ __device__ __forceinline__ uint32_t unmix32(uint32_t x) {  // inverse of mix32
    x ^= x >> 16;
    x *= 0x43021123u;
    x ^= (x >> 15) ^ (x >> 30);
    x *= 0x1d69e2a5u;
    x ^= x >> 16;
    return x;
}
__host__ __device__ __forceinline__ uint32_t fold_key(u64 key) {
    const uint32_t a = (uint32_t)(key >> 32), b = (uint32_t)key;
    return (a << 16) ^ b ^ ((a >> 16) * 0x9E3779B1u) ^ ((b >> 16) * 0x85EBCA77u);
}
__host__ __device__ __forceinline__ unsigned int part_of(u64 key) {
    return mix32(fold_key(key)) >> (32 - STBPE_PART_BITS);
}

__device__ __forceinline__ int owner_of(u64 key, int world) {
    return (int)(part_of(key) % (unsigned int)world);
}

// Table slice of a partition.  A rank holds only the keys it owns, i.e. the partitions with its
// residue modulo the number of ranks: their slices are numbered densely (partition / ranks), so the
// whole table is in use whatever the number of ranks.
__device__ __forceinline__ unsigned int slice_of(const EngineDev &e, unsigned int part) {
    return part / (unsigned int)e.world;
}
// first slot probed for a key: its partition's slice in the top bits, then the top bits of the 64-bit mix
__device__ __forceinline__ u64 slot_of(const EngineDev &e, u64 key) {
    return ((u64)slice_of(e, part_of(key)) << e.slot_bits) | (mix64(key) >> (64 - e.slot_bits));
}

// Programmatic dependent launch: inside the captured loop every kernel is launched with the
// programmatic-serialisation attribute, so its CTAs may become resident while the kernel before it
// still runs.  dep_release() lets the next kernel's CTAs be scheduled as soon as all CTAs of this
// one have started; dep_wait() returns when the kernel before this one has completed and its writes
// are visible.  Every thread executes dep_wait() before it touches global memory or returns (a
// kernel that ended without waiting would complete before its predecessor).  Launched without the
// attribute both are no-ops.
__device__ __forceinline__ void dep_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ bool better(u64 k1, i64 c1, u64 k2, i64 c2) {
    // (k1, c1) beats (k2, c2): larger count, ties to the smaller packed key
    // (gpu_tokenizer/trainers/bpe_gpu.py:106-127)
    return c1 > c2 || (c1 == c2 && k1 < k2);
}

__device__ __forceinline__ void mark_dirty(const EngineDev &e, u64 slot_index) {
    unsigned int blk = (unsigned int)(slot_index / STBPE_BLK);
    if (*(volatile unsigned int *)&e.dirty_flag[blk] == 0u) {
        if (atomicExch(&e.dirty_flag[blk], 1u) == 0u) {
            unsigned int i = atomicAdd(&e.st->n_dirty, 1u);
            if (i < e.n_blocks) e.dirty_list[i] = blk;
        }
    }
}

// add delta to key in the pair table, inserting the key when absent
__device__ __forceinline__ void table_add(const EngineDev &e, u64 key, i64 delta) {
    u64 h = slot_of(e, key);
    // the recorded maximum and the dirty flag of the block the key hashes to, fetched together with
    // the first probe (a key that was pushed into the next block re-reads them below)
    const u64 blk0 = h / STBPE_BLK;
    uint4 raw = __ldcg(reinterpret_cast<const uint4 *>(e.blockmax + blk0));
    unsigned int flagged = *(volatile unsigned int *)&e.dirty_flag[blk0];
    for (unsigned int probe = 0; probe < STBPE_MAX_PROBE; ++probe) {
        Slot *s = &e.table[h];
        u64 k = *(volatile u64 *)&s->key;
        if (k == STBPE_EMPTY) {
            u64 old = atomicCAS(&s->key, STBPE_EMPTY, key);
            if (old == STBPE_EMPTY) {
                atomicAdd(&e.st->n_keys, 1ull);
                k = key;
            } else {
                k = old;
            }
        }
        if (k == key) {
            const i64 now = (i64)atomicAdd((u64 *)&s->count, (u64)delta) + delta;
            // The maximum of the slot's block can only change if this key is the recorded maximum or
            // if its count now reaches it (the add that brings a key to its final count sees that
            // count, because the adds on one slot are serialised; the recorded maxima do not change
            // while deltas are applied).  Only those blocks are recomputed by refresh_kernel.
            if (h / STBPE_BLK != blk0) {
                raw = __ldcg(reinterpret_cast<const uint4 *>(e.blockmax + (h / STBPE_BLK)));
                flagged = 0u;
            }
            const u64 mk = ((u64)raw.y << 32) | raw.x;
            const i64 mc = (i64)(((u64)raw.w << 32) | raw.z);
            if (!flagged && (key == mk || now > mc || (now == mc && key < mk))) mark_dirty(e, h);
            return;
        }
        h = (h + 1) & e.mask;
    }
    atomicOr(&e.st->error, STBPE_DERR_TABLE_FULL);
}

// rank-local delta table (multi-GPU): same probing, first touch recorded for the drain
__device__ __forceinline__ void ltable_add(const EngineDev &e, u64 key, i64 delta) {
    u64 h = mix64(key * 0x9E3779B97F4A7C15ULL + 1) & e.lmask;
    for (unsigned int probe = 0; probe <= (unsigned int)e.lmask; ++probe) {
        Slot *s = &e.ltable[h];
        u64 k = *(volatile u64 *)&s->key;
        if (k == STBPE_EMPTY) {
            u64 old = atomicCAS(&s->key, STBPE_EMPTY, key);
            if (old == STBPE_EMPTY) {
                unsigned int i = atomicAdd(&e.st->n_ltouched, 1u);
                e.ltouched[i] = (unsigned int)h;  // i <= lmask: one entry per slot
                k = key;
            } else {
                k = old;
            }
        }
        if (k == key) {
            atomicAdd((u64 *)&s->count, (u64)delta);
            return;
        }
        h = (h + 1) & e.lmask;
    }
    atomicOr(&e.st->error, STBPE_DERR_LTABLE_FULL);
}

template <bool MG>
__device__ __forceinline__ void sink_add(const EngineDev &e, u64 key, i64 delta) {
    if (MG)
        ltable_add(e, key, delta);
    else
        table_add(e, key, delta);
}

// ---------------------------------------------------------------------------------------
// Per-CTA aggregation table in shared memory: key -> int32 delta.  Inserts that do not
// find a slot within a few probes go straight to the global sink.
// The table is addressed through the shared state space explicitly (ld/atom/red .shared):
// atomics issued through generic pointers to shared memory were measured at ~450 cycles each
// on this part, against ~10-20 for the .shared forms.
// ---------------------------------------------------------------------------------------
struct SmemTable {
    u64 *keys;
    int *vals;
    unsigned int mask;
};

__device__ __forceinline__ u64 lds_u64_volatile(const u64 *p) {
    u64 v;
    asm volatile("ld.volatile.shared.u64 %0, [%1];" : "=l"(v) : "r"((uint32_t)__cvta_generic_to_shared(p)) : "memory");
    return v;
}
__device__ __forceinline__ u64 atoms_cas_u64(u64 *p, u64 cmp, u64 val) {
    u64 old;
    asm volatile("atom.shared.cas.b64 %0, [%1], %2, %3;"
                 : "=l"(old)
                 : "r"((uint32_t)__cvta_generic_to_shared(p)), "l"(cmp), "l"(val)
                 : "memory");
    return old;
}
__device__ __forceinline__ void reds_add_s32(int *p, int v) {
    asm volatile("red.shared.add.s32 [%0], %1;" ::"r"((uint32_t)__cvta_generic_to_shared(p)), "r"(v) : "memory");
}

__device__ __forceinline__ void smem_table_clear(const SmemTable &t) {
    for (unsigned int i = threadIdx.x; i <= t.mask; i += blockDim.x) {
        t.keys[i] = STBPE_EMPTY;
        t.vals[i] = 0;
    }
}

__device__ __forceinline__ unsigned int hash32(u64 key) {
    unsigned int a = (unsigned int)(key >> 32), b = (unsigned int)key;
    unsigned int h = a * 0x9E3779B1u ^ (b * 0x85EBCA77u + 0x7F4A7C15u);
    h ^= h >> 15;
    h *= 0x2C1B3C6Du;
    h ^= h >> 13;
    return h;
}

// pair filter: the three rows of a pair key, and setting the pair's bits for a tile.  The filter is
// kept only while it pays: a merge with more matches than tiles visits nearly every tile anyway, and
// entering its new pairs costs more than the whole rewrite (measured: 37 of 61 ms on the first 20
// merges of a 1 GiB corpus), so the host lets the filter go stale for such merges and rebuilds it
// from the stream once the counts have fallen below the number of tiles.  With about a
// thousand distinct pairs in a full tile, three bits per pair over 16 384 rows leave a row about 17 %
// full and let through about 0.5 % of the tiles that do not hold the pair (two bits over 8 192 rows
// let through 5 %, which late in a run was most of the tiles a merge visited).
__device__ __forceinline__ void filter_rows(u64 key, unsigned int &r1, unsigned int &r2, unsigned int &r3) {
    // 32-bit arithmetic only (a 64-bit finaliser costs about three times the instructions, and the
    // merge kernel hashes two keys per match): two rows from disjoint bits of one mixed word, the
    // third from a second multiplicative mix of it
    const unsigned int h = hash32(key);
    unsigned int g = h * 0x9E3779B1u;
    g ^= g >> 15;
    r1 = h & (STBPE_PROWS - 1);
    r2 = (h >> 14) & (STBPE_PROWS - 1);
    r3 = (g >> 9) & (STBPE_PROWS - 1);
}
__device__ __forceinline__ void filter_set(const EngineDev &e, int tile, u64 key) {
    if (tile < 0) return;
    unsigned int r1, r2, r3;
    filter_rows(key, r1, r2, r3);
    const unsigned int w = (unsigned int)tile >> 5, bit = 1u << (tile & 31);
    unsigned int *p1 = e.presence + (size_t)r1 * e.presence_words + w;
    unsigned int *p2 = e.presence + (size_t)r2 * e.presence_words + w;
    unsigned int *p3 = e.presence + (size_t)r3 * e.presence_words + w;
    if (!(*(volatile unsigned int *)p1 & bit)) atomicOr(p1, bit);
    if (!(*(volatile unsigned int *)p2 & bit)) atomicOr(p2, bit);
    if (!(*(volatile unsigned int *)p3 & bit)) atomicOr(p3, bit);
}

// slow path: probe for the key, claim an empty slot, or give up after a few probes
template <bool MG>
__device__ __noinline__ void smem_table_add_probe(SmemTable t, const EngineDev *e, u64 key, int delta,
                                                  unsigned int h) {
#pragma unroll 1
    for (int probe = 0; probe < 8; ++probe) {
        u64 k = lds_u64_volatile(&t.keys[h]);
        if (k == STBPE_EMPTY) {
            const u64 old = atoms_cas_u64(&t.keys[h], STBPE_EMPTY, key);
            k = (old == STBPE_EMPTY) ? key : old;
        }
        if (k == key) {
            reds_add_s32(&t.vals[h], delta);
            return;
        }
        h = (h + 1) & t.mask;
    }
    sink_add<MG>(*e, key, (i64)delta);
}

// A key never leaves its slot once written, so a plain load that sees the key is final; any
// other value (empty or a different key) goes to the probing path.  Keeping the fast path free
// of volatile accesses lets several independent adds overlap.
__device__ __forceinline__ u64 lds_u64(const u64 *p) {
    u64 v;
    asm("ld.shared.u64 %0, [%1];" : "=l"(v) : "r"((uint32_t)__cvta_generic_to_shared(p)));
    return v;
}
template <bool MG>
__device__ __forceinline__ void smem_table_add(const SmemTable &t, const EngineDev &e, u64 key,
                                               int delta) {
    const unsigned int h = hash32(key) & t.mask;
    if (lds_u64(&t.keys[h]) == key)
        reds_add_s32(&t.vals[h], delta);
    else
        smem_table_add_probe<MG>(t, &e, key, delta, h);
}

template <bool MG>
__device__ __forceinline__ void smem_table_flush(const SmemTable &t, const EngineDev &e) {
    for (unsigned int i = threadIdx.x; i <= t.mask; i += blockDim.x) {
        u64 k = t.keys[i];
        int v = t.vals[i];
        if (k != STBPE_EMPTY && v != 0) sink_add<MG>(e, k, (i64)v);
    }
}

// ---------------------------------------------------------------------------------------
// Tile records
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ TileRec load_rec(const TileRec *p) {
    TileRec r;
    const uint4 *q = reinterpret_cast<const uint4 *>(p);
    uint4 x = q[0], y = q[1];
    r.ver = (int)x.x;
    r.len = (int)x.y;
    r.head[0] = x.z;
    r.head[1] = x.w;
    r.head[2] = y.x;
    r.tail = y.y;
    r.tail2 = y.z;
    r.pad = 0;
    return r;
}

// record of `tile` that was current before merge number m; returns its slot index
__device__ __forceinline__ int current_rec(const EngineDev &e, int tile, int m, TileRec &out) {
    TileRec r0 = load_rec(&e.recs[2 * tile]);
    TileRec r1 = load_rec(&e.recs[2 * tile + 1]);
    bool ok0 = r0.ver >= 0 && r0.ver < m;
    bool ok1 = r1.ver >= 0 && r1.ver < m;
    int s = (ok1 && (!ok0 || r1.ver > r0.ver)) ? 1 : 0;
    out = s ? r1 : r0;
    if (!ok0 && !ok1) out.len = 0;
    return s;
}

// Live tokens around a tile, in stream order: the last two live tokens before it and up to
// three live tokens after it (STBPE_NONE where the stream ends).  Walks records only.
// `before` / `after`: the records of tiles tile - 1 and tile + 1 when the caller has loaded them
// already (together with the tile's own, so that the three look-ups are one round trip).
__device__ __forceinline__ void gather_halo(const EngineDev &e, int tile, int m, uint32_t &prev,
                                            uint32_t &prev2, uint32_t nxt[3], int &next_tile, int &prev_tile,
                                            const TileRec *before = nullptr, const TileRec *after = nullptr) {
    next_tile = prev_tile = -1;
    prev = prev2 = STBPE_NONE;
    nxt[0] = nxt[1] = nxt[2] = STBPE_NONE;
    TileRec r;
    int back = 0;
    for (int t = tile - 1; t >= 0 && back < 2; --t) {
        if (before && t == tile - 1)
            r = *before;
        else
            current_rec(e, t, m, r);
        if (r.len > 0) {
            if (back == 0) {
                prev = r.tail;
                prev_tile = t;
                back = 1;
                if (r.len > 1) {
                    prev2 = r.tail2;
                    back = 2;
                }
            } else {
                prev2 = r.tail;
                back = 2;
            }
        }
    }
    int have = 0;
    for (int t = tile + 1; t < e.n_tiles && have < 3; ++t) {
        if (after && t == tile + 1)
            r = *after;
        else
            current_rec(e, t, m, r);
        int take = r.len < 3 ? r.len : 3;
        if (take > 0 && next_tile < 0) next_tile = t;
        for (int i = 0; i < take && have < 3; ++i) nxt[have++] = r.head[i];
    }
}
