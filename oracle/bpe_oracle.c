/*
 * CPU oracle for the BPE merge loop.  TEST INFRASTRUCTURE ONLY: nothing on the
 * product path may link, import or execute this file.  It is used by tests/,
 * by the smoke check and by the bench's cpu_baseline / reference arm.
 *
 * It restates, in plain C, the integer algorithm of the reference trainer's
 * CPU ("recount") path.  Each function cites the reference file:line it follows
 * (paths relative to the reference project root).
 *
 * Parity status: PINNED.  The restatement is checked against (i) the reference's
 * own known-answer unit tests and (ii) outputs of the reference trainer itself,
 * imported and run in recount mode, stored as fixtures under tests/golden/.
 *
 * Two count implementations are provided:
 *   mode 0 ("literal")  gather packed int64 keys -> sort -> run-length encode,
 *                       exactly the dataflow of gpu_tokenizer/utils.py:558-635.
 *   mode 1 ("fast")     hash / dense-table recount, multi-threaded (OpenMP).
 *                       Same result (sorted unique keys, int64 counts); used for
 *                       the larger parity cases and as the timed CPU baseline.
 *
 * Build: gcc -O3 -fopenmp -shared -fPIC -o liborc.so bpe_oracle.c
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_EXPORT __attribute__((visibility("default")))

/* ------------------------------------------------------------------------- */
/* helpers                                                                    */
/* ------------------------------------------------------------------------- */

static inline uint64_t pack_key(int32_t a, int32_t b) {
    /* key = (a << 32) | b on int64, gpu_tokenizer/utils.py:595 */
    return ((uint64_t)(uint32_t)a << 32) | (uint64_t)(uint32_t)b;
}

/* LSD radix sort of 64-bit keys, 16-bit digits, skipping constant digits.
 * Stands in for torch.sort at gpu_tokenizer/utils.py:596. */
static int radix_sort_u64(uint64_t *keys, int64_t n) {
    if (n <= 1) return 0;
    uint64_t *tmp = (uint64_t *)malloc((size_t)n * sizeof(uint64_t));
    if (!tmp) return -1;
    size_t *hist = (size_t *)malloc(65536 * sizeof(size_t));
    if (!hist) { free(tmp); return -1; }
    uint64_t *src = keys, *dst = tmp;
    for (int pass = 0; pass < 4; ++pass) {
        int shift = pass * 16;
        memset(hist, 0, 65536 * sizeof(size_t));
        for (int64_t i = 0; i < n; ++i) hist[(src[i] >> shift) & 0xFFFF]++;
        if (hist[(src[0] >> shift) & 0xFFFF] == (size_t)n) continue; /* constant digit */
        size_t sum = 0;
        for (int d = 0; d < 65536; ++d) { size_t c = hist[d]; hist[d] = sum; sum += c; }
        for (int64_t i = 0; i < n; ++i) dst[hist[(src[i] >> shift) & 0xFFFF]++] = src[i];
        uint64_t *t = src; src = dst; dst = t;
    }
    if (src != keys) memcpy(keys, src, (size_t)n * sizeof(uint64_t));
    free(tmp); free(hist);
    return 0;
}

/* run-length encode sorted keys, gpu_tokenizer/utils.py:604-616 */
static int64_t rle_sorted(const uint64_t *sorted, int64_t n, uint64_t *keys_out,
                          int64_t *counts_out, int64_t cap) {
    int64_t u = 0;
    int64_t i = 0;
    while (i < n) {
        int64_t j = i + 1;
        while (j < n && sorted[j] == sorted[i]) ++j;
        if (u >= cap) return -1; /* "pair workspace capacity exceeded", utils.py:619-620 */
        keys_out[u] = sorted[i];
        counts_out[u] = j - i;
        ++u;
        i = j;
    }
    return u;
}

/* ------------------------------------------------------------------------- */
/* padded-row operators (the reference's operator seam)                       */
/* ------------------------------------------------------------------------- */

/* count_pairs -> _count_pairs_pytorch, gpu_tokenizer/utils.py:558-635.
 * tokens/valid are [B, L] row-major; a pair (i, i+1) counts when both positions
 * are valid (utils.py:586).  Output: unique keys ascending, int64 counts.
 * Returns the number of unique pairs, -1 when cap is exceeded, -2 on alloc failure. */
ORC_EXPORT int64_t orc_count_pairs_rows(const int32_t *tokens, const uint8_t *valid, int64_t B,
                                        int64_t L, uint64_t *keys_out, int64_t *counts_out,
                                        int64_t cap) {
    if (B <= 0 || L <= 1) return 0;
    int64_t n = 0;
    for (int64_t r = 0; r < B; ++r)
        for (int64_t i = 0; i + 1 < L; ++i)
            if (valid[r * L + i] && valid[r * L + i + 1]) ++n;
    if (n == 0) return 0;
    uint64_t *keys = (uint64_t *)malloc((size_t)n * sizeof(uint64_t));
    if (!keys) return -2;
    int64_t k = 0;
    for (int64_t r = 0; r < B; ++r)
        for (int64_t i = 0; i + 1 < L; ++i)
            if (valid[r * L + i] && valid[r * L + i + 1])
                keys[k++] = pack_key(tokens[r * L + i], tokens[r * L + i + 1]);
    if (radix_sort_u64(keys, n) != 0) { free(keys); return -2; }
    int64_t u = rle_sorted(keys, n, keys_out, counts_out, cap);
    free(keys);
    return u;
}

/* apply_merge_once (CPU branch) + compact_tokens_inplace,
 * gpu_tokenizer/utils.py:515-555 and :347-410.
 * The match mask is evaluated for all positions on the pre-merge row
 * (utils.py:520-527); then tok[i]=new, valid[i+1]=0, tok[i+1]=0 for every match
 * (utils.py:529-531); then a stable left compaction with a zero-filled tail
 * (utils.py:376-394).  span_out (may be NULL) is the [B, L-1] match mask in
 * pre-compaction coordinates.  lengths_out receives the surviving count per row. */
ORC_EXPORT void orc_apply_merge_rows(int32_t *tokens, uint8_t *valid, int64_t *lengths_out,
                                     int64_t B, int64_t L, int32_t a, int32_t b, int32_t new_id,
                                     uint8_t *span_out) {
    if (B <= 0 || L <= 0) return;
    uint8_t *mask = (uint8_t *)malloc((size_t)(L > 1 ? L - 1 : 1));
    for (int64_t r = 0; r < B; ++r) {
        int32_t *t = tokens + r * L;
        uint8_t *v = valid + r * L;
        for (int64_t i = 0; i + 1 < L; ++i)
            mask[i] = (uint8_t)(t[i] == a && t[i + 1] == b && v[i] && v[i + 1]);
        if (span_out) memcpy(span_out + r * (L - 1), mask, (size_t)(L - 1));
        for (int64_t i = 0; i + 1 < L; ++i)
            if (mask[i]) t[i] = new_id;
        for (int64_t i = 0; i + 1 < L; ++i)
            if (mask[i]) { v[i + 1] = 0; t[i + 1] = 0; }
        int64_t w = 0;
        for (int64_t i = 0; i < L; ++i) {
            if (v[i]) {
                int32_t val = t[i];
                /* destinations never overtake sources: w <= i */
                t[w] = val;
                v[w] = 1;
                ++w;
            }
        }
        for (int64_t i = w; i < L; ++i) { t[i] = 0; v[i] = 0; }
        if (lengths_out) lengths_out[r] = w;
    }
    free(mask);
}

/* select_best_pair, gpu_tokenizer/trainers/bpe_gpu.py:96-130: maximum count;
 * among equal counts the smallest packed key.  Keys need not be sorted.
 * Returns the index of the winner or -1 when there is no positive count. */
ORC_EXPORT int64_t orc_select_best(const uint64_t *keys, const int64_t *counts, int64_t n,
                                   uint64_t *best_key, int64_t *best_count) {
    int64_t bi = -1, bc = 0;
    uint64_t bk = 0;
    for (int64_t i = 0; i < n; ++i) {
        if (counts[i] > bc || (counts[i] == bc && bc > 0 && keys[i] < bk)) {
            bc = counts[i]; bk = keys[i]; bi = i;
        }
    }
    if (bi >= 0) { *best_key = bk; *best_count = bc; }
    return bi;
}

/* ------------------------------------------------------------------------- */
/* flat-stream operators (rows concatenated; off[r]..off[r+1] delimits row r) */
/* ------------------------------------------------------------------------- */

typedef struct {
    uint64_t *keys;
    int64_t *vals;
    uint64_t mask; /* capacity - 1 */
    int64_t used;
} orc_map;

#define ORC_EMPTY 0xFFFFFFFFFFFFFFFFull

static inline uint64_t mix64(uint64_t x) {
    x ^= x >> 33; x *= 0xff51afd7ed558ccdull; x ^= x >> 33;
    x *= 0xc4ceb9fe1a85ec53ull; x ^= x >> 33;
    return x;
}

static int map_init(orc_map *m, uint64_t cap_pow2) {
    m->keys = (uint64_t *)malloc(cap_pow2 * sizeof(uint64_t));
    m->vals = (int64_t *)calloc(cap_pow2, sizeof(int64_t));
    if (!m->keys || !m->vals) return -1;
    memset(m->keys, 0xFF, cap_pow2 * sizeof(uint64_t));
    m->mask = cap_pow2 - 1;
    m->used = 0;
    return 0;
}
static void map_free(orc_map *m) { free(m->keys); free(m->vals); m->keys = NULL; m->vals = NULL; }
static int map_add(orc_map *m, uint64_t key, int64_t delta);
static int map_grow(orc_map *m) {
    orc_map n;
    if (map_init(&n, (m->mask + 1) * 2) != 0) return -1;
    for (uint64_t i = 0; i <= m->mask; ++i)
        if (m->keys[i] != ORC_EMPTY) map_add(&n, m->keys[i], m->vals[i]);
    map_free(m);
    *m = n;
    return 0;
}
static int map_add(orc_map *m, uint64_t key, int64_t delta) {
    if ((uint64_t)m->used * 10 > (m->mask + 1) * 6)
        if (map_grow(m) != 0) return -1;
    uint64_t h = mix64(key) & m->mask;
    for (;;) {
        uint64_t k = m->keys[h];
        if (k == key) { m->vals[h] += delta; return 0; }
        if (k == ORC_EMPTY) { m->keys[h] = key; m->vals[h] = delta; m->used++; return 0; }
        h = (h + 1) & m->mask;
    }
}

/* Count every adjacent in-row pair of a flat stream.
 * mode 0: literal sort + RLE (utils.py:558-635).  mode 1: threaded table recount.
 * Output sorted ascending by key (as aggregate_pair_keys leaves it, utils.py:709-751).
 * Returns number of unique pairs; -1 capacity exceeded; -2 allocation failure. */
ORC_EXPORT int64_t orc_count_pairs_flat(const int32_t *ids, const int64_t *off, int64_t n_rows,
                                        int mode, uint64_t *keys_out, int64_t *counts_out,
                                        int64_t cap) {
    int64_t n_pairs = 0;
    for (int64_t r = 0; r < n_rows; ++r) {
        int64_t len = off[r + 1] - off[r];
        if (len > 1) n_pairs += len - 1;
    }
    if (n_pairs == 0) return 0;

    if (mode == 0) {
        uint64_t *keys = (uint64_t *)malloc((size_t)n_pairs * sizeof(uint64_t));
        if (!keys) return -2;
        int64_t k = 0;
        for (int64_t r = 0; r < n_rows; ++r)
            for (int64_t i = off[r]; i + 1 < off[r + 1]; ++i) keys[k++] = pack_key(ids[i], ids[i + 1]);
        if (radix_sort_u64(keys, n_pairs) != 0) { free(keys); return -2; }
        int64_t u = rle_sorted(keys, n_pairs, keys_out, counts_out, cap);
        free(keys);
        return u;
    }

    /* mode 1: per-thread hash maps over row ranges, merged, then sorted by key */
    int nt = 1;
#ifdef _OPENMP
    nt = omp_get_max_threads();
#endif
    if (n_pairs < 65536) nt = 1;
    orc_map *maps = (orc_map *)calloc((size_t)nt, sizeof(orc_map));
    int fail = 0;
    for (int t = 0; t < nt; ++t)
        if (map_init(&maps[t], 1u << 12) != 0) fail = 1;
    if (fail) return -2;
    int64_t total = off[n_rows];
#pragma omp parallel num_threads(nt)
    {
        int t = 0;
#ifdef _OPENMP
        t = omp_get_thread_num();
#endif
        /* split by token position; a thread owns pairs whose left token lies in its slice */
        int64_t lo = total * t / nt, hi = total * (t + 1) / nt;
        /* find the row containing lo by binary search */
        int64_t r0 = 0, r1 = n_rows;
        while (r0 < r1) { int64_t m = (r0 + r1) / 2; if (off[m + 1] <= lo) r0 = m + 1; else r1 = m; }
        int64_t r = r0;
        for (int64_t i = lo; i < hi; ++i) {
            while (r < n_rows && off[r + 1] <= i) ++r;
            if (r >= n_rows) break;
            if (i + 1 < off[r + 1])
                if (map_add(&maps[t], pack_key(ids[i], ids[i + 1]), 1) != 0) fail = 1;
        }
    }
    if (fail) { for (int t = 0; t < nt; ++t) map_free(&maps[t]); free(maps); return -2; }
    for (int t = 1; t < nt; ++t) {
        for (uint64_t i = 0; i <= maps[t].mask; ++i)
            if (maps[t].keys[i] != ORC_EMPTY) map_add(&maps[0], maps[t].keys[i], maps[t].vals[i]);
        map_free(&maps[t]);
    }
    int64_t u = maps[0].used;
    if (u > cap) { map_free(&maps[0]); free(maps); return -1; }
    /* sort unique keys, then look the counts up */
    int64_t k = 0;
    for (uint64_t i = 0; i <= maps[0].mask; ++i)
        if (maps[0].keys[i] != ORC_EMPTY) keys_out[k++] = maps[0].keys[i];
    if (radix_sort_u64(keys_out, u) != 0) { map_free(&maps[0]); free(maps); return -2; }
    for (int64_t i = 0; i < u; ++i) {
        uint64_t h = mix64(keys_out[i]) & maps[0].mask;
        while (maps[0].keys[h] != keys_out[i]) h = (h + 1) & maps[0].mask;
        counts_out[i] = maps[0].vals[h];
    }
    map_free(&maps[0]);
    free(maps);
    return u;
}

/* Apply one merge to a flat stream in place and update the row offsets.
 * Same rule as orc_apply_merge_rows (utils.py:515-555, :347-410): with
 * M = { i : t[i]=a, t[i+1]=b, both in the row } on the pre-merge row, position i
 * becomes new_id when i is in M and is dropped when i-1 is in M.
 * Returns the number of matches |M| summed over rows. */
ORC_EXPORT int64_t orc_apply_merge_flat(int32_t *ids, int64_t *off, int64_t n_rows, int32_t a,
                                        int32_t b, int32_t new_id) {
    int64_t w = 0, matches = 0;
    int64_t row_begin = off[0];
    for (int64_t r = 0; r < n_rows; ++r) {
        int64_t end = off[r + 1];
        int64_t new_begin = w;
        int32_t prev = 0;
        for (int64_t i = row_begin; i < end; ++i) {
            int32_t cur = ids[i];
            int dropped = (i > row_begin) && prev == a && cur == b;
            int match = (i + 1 < end) && cur == a && ids[i + 1] == b;
            prev = cur;
            matches += match;
            if (dropped) continue;
            ids[w++] = match ? new_id : cur; /* w <= i, ids[i+1] not yet overwritten */
        }
        row_begin = end;
        off[r] = new_begin;
    }
    off[n_rows] = w;
    return matches;
}

/* The merge loop in recount mode, gpu_tokenizer/bpe_trainer.py:4193-4517:
 *   count (utils.py:558-635) -> aggregate (utils.py:709-751)
 *   -> select max count / min key (bpe_gpu.py:96-130)
 *   -> "no pairs" stop (bpe_trainer.py:4304-4308) / "count < 2" gate (:2491-2494, :4361-4364)
 *   -> new_id = vocab_size (:4365) -> apply (utils.py:413-555).
 * merges_out holds 2*target int32 (a, b); counts_out target int64.
 * *reason: 0 target reached, 1 no pairs left at all, 2 best count below 2.
 * Random padding after reason 2 (bpe_trainer.py:4347-4353) is host-side Python
 * and not part of this function.  Returns merges done, or <0 on failure. */
ORC_EXPORT int64_t orc_train_flat(int32_t *ids, int64_t *off, int64_t n_rows, int32_t base_vocab,
                                  int64_t target, int mode, int32_t *merges_out,
                                  int64_t *counts_out, int32_t *reason) {
    int64_t done = 0;
    *reason = 0;
    int64_t cap = off[n_rows] - off[0];
    if (cap < 1) cap = 1;
    uint64_t *keys = (uint64_t *)malloc((size_t)cap * sizeof(uint64_t));
    int64_t *cnts = (int64_t *)malloc((size_t)cap * sizeof(int64_t));
    if (!keys || !cnts) { free(keys); free(cnts); return -2; }
    int32_t vocab = base_vocab;
    while (done < target) {
        int64_t u = orc_count_pairs_flat(ids, off, n_rows, mode, keys, cnts, cap);
        if (u < 0) { free(keys); free(cnts); return u; }
        if (u == 0) { *reason = 1; break; }
        uint64_t bk = 0; int64_t bc = 0;
        orc_select_best(keys, cnts, u, &bk, &bc);
        if (bc < 2) { *reason = 2; break; }
        int32_t a = (int32_t)(bk >> 32), b = (int32_t)(bk & 0xFFFFFFFFull);
        merges_out[2 * done] = a;
        merges_out[2 * done + 1] = b;
        counts_out[done] = bc;
        orc_apply_merge_flat(ids, off, n_rows, a, b, vocab);
        ++vocab;
        ++done;
    }
    free(keys); free(cnts);
    return done;
}

/* Number of threads of the threaded recount (launchers such as torch.distributed.run export
 * OMP_NUM_THREADS=1 to their children, which would otherwise time a single-threaded baseline). */
ORC_EXPORT void orc_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

ORC_EXPORT int orc_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
