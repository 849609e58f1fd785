// K2, wide path: first count of a fresh stream whose ids are all below 65 536 (a 16-bit vocabulary).
//
// The pair space is 2^32 keys and a Zipf-like id stream touches 10^8 of them, so a histogram kept in
// one place is bound by random memory accesses, not by the stream (one scattered reduction per token
// into a table in HBM ran at 37 G sector requests per second, 4 % of the stream rate).  Random
// reductions are six times faster while their target stays in L2 (measured on B200: 227 G per second
// into 64 MB, 21 G per second into 4 GB), so the count is split in two passes that never touch HBM at
// random:
//
//   pass 1  partition_pairs_kernel reads the stream once.  Pairs of two ids below 256 (44 % of a
//           Zipf(1.1) stream) go to 16-bit shared-memory counters as in the byte-level kernel.  Every
//           other pair becomes one 32-bit word, mix32((a << 16) | b), and is appended to the
//           partition named by the word's top 8 bits: per CTA a ring of 64 words per partition in
//           shared memory, flushed with coalesced stores after every batch of tokens into a region
//           of the partition that belongs to this CTA alone (no reservation, hence no atomic and no
//           round trip to memory in the loop; with one global cursor per partition the flush waited
//           for 256 dependent reservations per batch and the pass took 13.4 ms instead of 4).  The
//           mix is a bijection, so partitions are balanced whatever the ids, and the word still
//           identifies the pair.
//   pass 2  partition_table_kernel, one launch per partition: every word is turned back into its
//           pair (unmix32) and added to the pair table.  The slot index of a key starts with the
//           same 8 partition bits, so all adds of a launch fall into one slice of the table
//           (1/256 of it: 32 MB of an 8 GiB table), which stays in L2 while the launch runs; the
//           words are streamed past it with evict-first loads.  (An intermediate block of 2^24
//           directly indexed 32-bit counters per partition, 64 MB, was tried first: together with
//           the table slice it did not stay in L2 and the pass ran at the HBM rate, 43.5 ms.)
//
// An id of 65 536 or more, or a partition region that outgrows its buffer, raises
// STBPE_DERR_DENSE_OVERFLOW and the host recounts with the general kernel.
#pragma once
#include "common.cuh"

#define STBPE_PART_RING 64          // words per partition and CTA between two flushes
#define STBPE_PART_THREADS 1024
#define STBPE_PART_UNROLL 3         // uint4 loads per thread and batch: 12 288 tokens per CTA batch
static_assert(STBPE_PARTS == 8 * (STBPE_PART_THREADS / 32), "a warp of the first pass serves eight rings");
#define STBPE_PART_CACHE_BITS 12    // log2 of the entries of the per-CTA word cache of pass 2 (32 KB)
#define STBPE_PART_CACHE (1 << STBPE_PART_CACHE_BITS)
#define STBPE_PART_SHIFT (32 - STBPE_PART_BITS)
#define STBPE_PART_SMEM_BYTES (32768 * 4 + STBPE_PARTS * STBPE_PART_RING * 4 + 2 * STBPE_PARTS * 4)

struct PartBuffers {
    uint32_t *words;        // [partition][CTA of pass 1] regions of `cap` words
    unsigned int *fill;     // words in each region
    i64 cap;
    int n_cta;              // grid size of pass 1
};

// Several ranks: every rank partitions its own rows, then the owner of a partition (partition modulo
// the number of ranks) counts the partition's words out of every rank's regions with plain peer
// loads over NVLink, and sums the ranks' counters of the hot pairs it owns.  The buffers of a rank
// live in one allocation that its peers map: a header {cap, n_cta}, the region fills, the 65 536 hot
// counters, the regions.
#define STBPE_WIDE_HEADER_BYTES 256
struct WideHeader {
    i64 cap;
    int n_cta;
};
struct WidePeers {
    const unsigned char *block[STBPE_MAX_PEERS];  // every rank's allocation ([rank] = own)
    int world, rank;
};
__host__ __device__ __forceinline__ size_t wide_fill_bytes(int n_cta) {
    return (((size_t)STBPE_PARTS * n_cta * sizeof(unsigned int)) + 255) & ~(size_t)255;
}
__host__ __device__ __forceinline__ const unsigned int *wide_fill(const unsigned char *block) {
    return reinterpret_cast<const unsigned int *>(block + STBPE_WIDE_HEADER_BYTES);
}
__host__ __device__ __forceinline__ const u64 *wide_dense(const unsigned char *block, int n_cta) {
    return reinterpret_cast<const u64 *>(block + STBPE_WIDE_HEADER_BYTES + wide_fill_bytes(n_cta));
}
__host__ __device__ __forceinline__ const uint32_t *wide_words(const unsigned char *block, int n_cta) {
    return reinterpret_cast<const uint32_t *>(block + STBPE_WIDE_HEADER_BYTES + wide_fill_bytes(n_cta) +
                                              65536 * sizeof(u64));
}

__device__ __forceinline__ void part_append(const PartBuffers &pb, unsigned int *s_ring, unsigned int *s_cur,
                                            unsigned int *s_fill, unsigned int *derr, uint32_t word) {
    const unsigned int p = word >> STBPE_PART_SHIFT;
    const unsigned int pos = atomicAdd(&s_cur[p], 1u);
    if (pos < STBPE_PART_RING) {
        // rings fill at about the same pace, so slot `pos` of every ring would sit in the same bank:
        // rotate each ring by its partition number
        s_ring[p * STBPE_PART_RING + ((pos + p) & (STBPE_PART_RING - 1))] = word;
    } else {  // ring full before the flush (far out in the tail of the batch statistics): append directly
        const unsigned int g = atomicAdd(&s_fill[p], 1u);
        if ((i64)g < pb.cap)
            pb.words[((i64)p * pb.n_cta + blockIdx.x) * pb.cap + g] = word;
        else
            atomicOr(derr, STBPE_DERR_DENSE_OVERFLOW);
    }
}

__device__ __forceinline__ void part_pair(const PartBuffers &pb, unsigned int *s_tab, unsigned int *s_ring,
                                          unsigned int *s_cur, unsigned int *s_fill, u64 *g_dense,
                                          unsigned int *derr, uint32_t t0, uint32_t t1) {
    // the classes are worked out first and the two kinds of add follow one another, so that the lanes
    // of a warp, whose pairs fall into different classes, share the instructions of each kind
    t0 &= ~STBPE_FLAG;
    const uint32_t both = t0 | t1;             // bit 31 set: the right token starts a row or lies past the end
    const bool hot = both < 256u;
    const bool wide = !hot && both < 65536u;
    if (hot) dense_add(s_tab, g_dense, derr, t0, t1);
    if (wide) part_append(pb, s_ring, s_cur, s_fill, derr, mix32((t0 << 16) | t1));
    if (!hot && !wide && !(t1 & STBPE_FLAG)) atomicOr(derr, STBPE_DERR_DENSE_OVERFLOW);
}

__global__ void __launch_bounds__(STBPE_PART_THREADS, 1)
    partition_pairs_kernel(EngineDev e, i64 n_tokens, u64 *g_dense, PartBuffers pb) {
    extern __shared__ __align__(16) unsigned int s_all[];
    unsigned int *s_tab = s_all;                                  // 32 768 words of 16-bit counters
    unsigned int *s_ring = s_all + 32768;                         // STBPE_PARTS rings
    unsigned int *s_cur = s_ring + STBPE_PARTS * STBPE_PART_RING;  // ring fill
    unsigned int *s_fill = s_cur + STBPE_PARTS;                   // words this CTA has stored per partition
    for (int i = threadIdx.x; i < 32768; i += STBPE_PART_THREADS) s_tab[i] = 0u;
    for (int i = threadIdx.x; i < STBPE_PARTS; i += STBPE_PART_THREADS) s_cur[i] = s_fill[i] = 0u;
    __syncthreads();
    const uint32_t *tok = e.tiles;
    unsigned int *derr = &e.st->error;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const i64 span = (i64)STBPE_PART_THREADS * 4;
    uint4 v[STBPE_PART_UNROLL];
    uint32_t nx[STBPE_PART_UNROLL];
    // the loads of a batch are issued before the flush of the batch before it, so that their trip to
    // memory runs under the flush and its two CTA barriers
    auto load_batch = [&](i64 base) {
#pragma unroll
        for (int u = 0; u < STBPE_PART_UNROLL; ++u) {
            const i64 i = base + u * span + (i64)threadIdx.x * 4;
            if (i + 4 <= n_tokens) {
                v[u] = __ldcs(reinterpret_cast<const uint4 *>(tok + i));
            } else {
                v[u].x = i < n_tokens ? tok[i] : STBPE_NONE;
                v[u].y = i + 1 < n_tokens ? tok[i + 1] : STBPE_NONE;
                v[u].z = i + 2 < n_tokens ? tok[i + 2] : STBPE_NONE;
                v[u].w = i + 3 < n_tokens ? tok[i + 3] : STBPE_NONE;
            }
            nx[u] = (lane == 31) ? (i + 4 < n_tokens ? tok[i + 4] : STBPE_NONE) : 0u;
        }
    };
    const i64 step = (i64)gridDim.x * span * STBPE_PART_UNROLL;
    i64 base = (i64)blockIdx.x * span * STBPE_PART_UNROLL;
    if (base < n_tokens) load_batch(base);
    for (; base < n_tokens; base += step) {
#pragma unroll
        for (int u = 0; u < STBPE_PART_UNROLL; ++u) {
            uint32_t n0 = __shfl_down_sync(0xFFFFFFFFu, v[u].x, 1);
            if (lane == 31) n0 = nx[u];
            part_pair(pb, s_tab, s_ring, s_cur, s_fill, g_dense, derr, v[u].x, v[u].y);
            part_pair(pb, s_tab, s_ring, s_cur, s_fill, g_dense, derr, v[u].y, v[u].z);
            part_pair(pb, s_tab, s_ring, s_cur, s_fill, g_dense, derr, v[u].z, v[u].w);
            part_pair(pb, s_tab, s_ring, s_cur, s_fill, g_dense, derr, v[u].w, n0);
        }
        if (base + step < n_tokens) load_batch(base + step);
        __syncthreads();
        // flush into this CTA's regions: a warp serves its eight rings at once, four lanes per ring
        // (one ring at a time cost eight times the bookkeeping: the pass was bound by instruction
        // issue, 128 instructions per token, a third of them here)
        {
            const int p = warp * (STBPE_PARTS / (STBPE_PART_THREADS / 32)) + (lane >> 2);
            const unsigned int n = min(s_cur[p], (unsigned int)STBPE_PART_RING);
            const unsigned int g = s_fill[p];
            __syncwarp();
            if ((i64)g + n <= pb.cap) {
                uint32_t *dst = pb.words + ((i64)p * pb.n_cta + blockIdx.x) * pb.cap + g;
                for (unsigned int k = lane & 3; k < n; k += 4)
                    dst[k] = s_ring[p * STBPE_PART_RING + ((k + p) & (STBPE_PART_RING - 1))];
            } else if ((lane & 3) == 0) {
                atomicOr(derr, STBPE_DERR_DENSE_OVERFLOW);
            }
            if ((lane & 3) == 0) {
                s_fill[p] = g + n;
                s_cur[p] = 0u;
            }
        }
        __syncthreads();
    }
    for (int p = threadIdx.x; p < STBPE_PARTS; p += STBPE_PART_THREADS) {
        const unsigned int n = s_fill[p];
        pb.fill[(i64)p * pb.n_cta + blockIdx.x] = (i64)n < pb.cap ? n : (unsigned int)pb.cap;
    }
    for (int p = threadIdx.x; p < 32768; p += STBPE_PART_THREADS) {
        const unsigned int x = s_tab[p];
        const unsigned int w = (unsigned int)p ^ (((unsigned int)p >> 7) & 31u);  // inverse of dense_word
        if (x & 0xFFFFu) atomicAdd(&g_dense[2 * w], (u64)(x & 0xFFFFu));
        if (x >> 16) atomicAdd(&g_dense[2 * w + 1], (u64)(x >> 16));
    }
}

// Add n occurrences of a key to the pair table during the first count: no maxima to keep (a full
// refresh follows), and a key that is already there costs one load and one reduction without result.
__device__ __forceinline__ bool table_count_n(const EngineDev &e, u64 key, u64 h, u64 n, unsigned int &fresh) {
    for (unsigned int probe = 0; probe < STBPE_MAX_PROBE; ++probe) {
        Slot *s = &e.table[h];
        u64 k = __ldcg(&s->key);
        if (k == STBPE_EMPTY) {
            const u64 old = atomicCAS(&s->key, STBPE_EMPTY, key);
            if (old == STBPE_EMPTY) {
                ++fresh;
                k = key;
            } else {
                k = old;
            }
        }
        if (k == key) {
            atomicAdd((u64 *)&s->count, n);  // result unused: a reduction
            return true;
        }
        h = (h + 1) & e.mask;
    }
    atomicOr(&e.st->error, STBPE_DERR_TABLE_FULL);
    return false;
}

// `top`: the word's table slice shifted into place (every word of a pass-2 launch is of one partition)
__device__ __forceinline__ void part_word_to_table(const EngineDev &e, uint32_t x, u64 n, unsigned int &fresh, u64 top) {
    const uint32_t ab = unmix32(x);
    const u64 key = ((u64)(ab >> 16) << 32) | (u64)(ab & 0xFFFFu);
    const u64 h = top | (mix64(key) >> (64 - e.slot_bits));
    table_count_n(e, key, h, n, fresh);
}

// pass 2: the words of partition p (the regions of all pass-1 CTAs) into the table slice of p.
// Block b serves region b / per_region.  A frequent pair would otherwise be tens of thousands of
// reductions on one address, which L2 executes one after the other (the hottest pair of a partition
// alone took longer than everything else of its launch), so every block first collects its words in
// a direct-mapped cache in shared memory (word -> count; a word whose entry is taken by another
// goes straight to the table) and then adds each cached word once.
// One launch serves several partitions: consecutive groups of n_cta * per_region blocks take
// consecutive partitions, so the blocks resident at any time work on two or three slices.
__global__ void __launch_bounds__(1024) partition_table_kernel(EngineDev e, PartBuffers pb, int p_first, int per_region) {
    const int blocks_per_part = pb.n_cta * per_region;
    const int p = p_first + (int)(blockIdx.x / blocks_per_part);
    const int block = (int)(blockIdx.x % blocks_per_part);
    __shared__ uint32_t s_word[STBPE_PART_CACHE];
    __shared__ unsigned int s_cnt[STBPE_PART_CACHE];
    for (int i = threadIdx.x; i < STBPE_PART_CACHE; i += blockDim.x) {
        s_word[i] = 0xFFFFFFFFu;
        s_cnt[i] = 0u;
    }
    __syncthreads();
    const int region = block / per_region, part = block % per_region;
    const u64 top = (u64)slice_of(e, (unsigned int)p) << e.slot_bits;
    const i64 n = pb.fill[(i64)p * pb.n_cta + region];
    const uint32_t *w = pb.words + ((i64)p * pb.n_cta + region) * pb.cap;
    unsigned int fresh = 0;
    // (four words per thread and step, with their four table slots loaded before any is looked at,
    // was slower: 30 ms instead of 21 ms for the 256 launches on 2^31 ids)
    for (i64 i = (i64)part * blockDim.x + threadIdx.x; i < n; i += (i64)per_region * blockDim.x) {
        const uint32_t x = __ldcs(w + i);  // streamed once: keep it from displacing the table slice
        const unsigned int c = (x * 0x9E3779B1u) >> (32 - STBPE_PART_CACHE_BITS);
        uint32_t k = s_word[c];
        if (k == 0xFFFFFFFFu && x != 0xFFFFFFFFu) {
            const uint32_t old = atomicCAS(&s_word[c], 0xFFFFFFFFu, x);
            k = old == 0xFFFFFFFFu ? x : old;
        }
        if (k == x && x != 0xFFFFFFFFu)
            atomicAdd(&s_cnt[c], 1u);
        else
            part_word_to_table(e, x, 1ull, fresh, top);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < STBPE_PART_CACHE; i += blockDim.x) {
        const unsigned int c = s_cnt[i];
        if (c) part_word_to_table(e, s_word[i], (u64)c, fresh, top);
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) fresh += __shfl_down_sync(0xFFFFFFFFu, fresh, d);
    if ((threadIdx.x & 31) == 0 && fresh) atomicAdd(&e.st->n_keys, (u64)fresh);
}

// pass 2, several ranks: partition p, owned by this rank, out of the regions of every rank.  The grid
// is one wave of blocks whatever the number of ranks; a block walks over its share of the
// (source rank, region, half) units with one cache, which it adds to the table at the end.
__global__ void __launch_bounds__(1024)
    partition_table_peers_kernel(EngineDev e, WidePeers wp, int p_first, int p_step, int n_cta) {
    // consecutive groups of 2 * n_cta blocks take the partitions p_first, p_first + p_step, ...
    const int blocks_per_part = 2 * n_cta;
    const int p = p_first + (int)(blockIdx.x / blocks_per_part) * p_step;
    const int block = (int)(blockIdx.x % blocks_per_part);
    __shared__ uint32_t s_word[STBPE_PART_CACHE];
    __shared__ unsigned int s_cnt[STBPE_PART_CACHE];
    for (int i = threadIdx.x; i < STBPE_PART_CACHE; i += blockDim.x) {
        s_word[i] = 0xFFFFFFFFu;
        s_cnt[i] = 0u;
    }
    __syncthreads();
    unsigned int fresh = 0;
    const u64 top = (u64)slice_of(e, (unsigned int)p) << e.slot_bits;
    const int n_units = wp.world * n_cta * 2;
    for (int unit = block; unit < n_units; unit += blocks_per_part) {
        const int half = unit & 1, region = (unit >> 1) % n_cta, src = (unit >> 1) / n_cta;
        const unsigned char *blk = wp.block[src];
        const WideHeader hd = *reinterpret_cast<const WideHeader *>(blk);
        if (hd.n_cta != n_cta) {  // every rank runs the first pass with the same grid
            if (threadIdx.x == 0) atomicOr(&e.st->error, STBPE_DERR_DENSE_OVERFLOW);
            continue;
        }
        const i64 n = wide_fill(blk)[(i64)p * n_cta + region];
        const uint32_t *w = wide_words(blk, n_cta) + ((i64)p * n_cta + region) * hd.cap;
        // words come four at a time (16-byte loads; regions are 16-byte aligned): a peer's words
        // cross NVLink, and one word per load left the loop waiting for the link's latency
        const i64 n4 = n / 4;
        const uint4 *w4 = reinterpret_cast<const uint4 *>(w);
        for (i64 i = (i64)half * blockDim.x + threadIdx.x; i <= n4; i += 2 * (i64)blockDim.x) {
            uint32_t x[4];
            int m = 4;
            if (i < n4) {
                const uint4 q = __ldcs(w4 + i);
                x[0] = q.x, x[1] = q.y, x[2] = q.z, x[3] = q.w;
            } else {
                m = (int)(n - n4 * 4);
                for (int k = 0; k < 4; ++k) x[k] = k < m ? w[n4 * 4 + k] : 0u;
            }
            for (int k = 0; k < m; ++k) {
                const unsigned int c = (x[k] * 0x9E3779B1u) >> (32 - STBPE_PART_CACHE_BITS);
                uint32_t kk = s_word[c];
                if (kk == 0xFFFFFFFFu && x[k] != 0xFFFFFFFFu) {
                    const uint32_t old = atomicCAS(&s_word[c], 0xFFFFFFFFu, x[k]);
                    kk = old == 0xFFFFFFFFu ? x[k] : old;
                }
                if (kk == x[k] && x[k] != 0xFFFFFFFFu)
                    atomicAdd(&s_cnt[c], 1u);
                else
                    part_word_to_table(e, x[k], 1ull, fresh, top);
            }
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < STBPE_PART_CACHE; i += blockDim.x) {
        const unsigned int c = s_cnt[i];
        if (c) part_word_to_table(e, s_word[i], (u64)c, fresh, top);
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) fresh += __shfl_down_sync(0xFFFFFFFFu, fresh, d);
    if ((threadIdx.x & 31) == 0 && fresh) atomicAdd(&e.st->n_keys, (u64)fresh);
}

// hot pairs (both ids below 256) owned by this rank: the sum of every rank's counter
__global__ void dense_peers_to_table_kernel(EngineDev e, WidePeers wp, int n_cta) {
    const int k = blockIdx.x * blockDim.x + threadIdx.x;
    if (k >= 65536) return;
    const u64 key = ((u64)(k >> 8) << 32) | (u64)(k & 0xFF);
    if (owner_of(key, wp.world) != wp.rank) return;
    u64 c = 0;
    for (int r = 0; r < wp.world; ++r) c += __ldcg(wide_dense(wp.block[r], n_cta) + k);
    if (c) table_add(e, key, (i64)c);
}
