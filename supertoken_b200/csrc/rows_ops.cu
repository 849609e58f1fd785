// Stateless operators on padded [B, L] batches, with the reference's operator signatures
// (gpu_tokenizer/utils.py:691-706 count_pairs, :413-555 apply_merge_once).
#include <cub/device/device_radix_sort.cuh>
#include <cuda_runtime.h>

#include <cstdio>
#include <mutex>
#include <string>

#include "../../include/stbpe.h"
#include "common.cuh"

#define STBPE_VISIBLE __attribute__((visibility("default")))
#define ROWS_NT 256
#define ROWS_IPT 8
#define ROWS_CHUNK (ROWS_NT * ROWS_IPT)

namespace {

struct RowsTable {
    Slot *table;
    u64 mask;
    unsigned int *error;
    u64 *n_keys;
};

__device__ __forceinline__ void rows_table_add(const RowsTable &t, u64 key) {
    u64 h = mix64(key) & t.mask;
    for (u64 probe = 0; probe <= t.mask; ++probe) {
        Slot *s = &t.table[h];
        u64 k = *(volatile u64 *)&s->key;
        if (k == STBPE_EMPTY) {
            u64 old = atomicCAS(&s->key, STBPE_EMPTY, key);
            if (old == STBPE_EMPTY) {
                atomicAdd(t.n_keys, 1ull);
                k = key;
            } else {
                k = old;
            }
        }
        if (k == key) {
            atomicAdd((u64 *)&s->count, 1ull);
            return;
        }
        h = (h + 1) & t.mask;
    }
    atomicOr(t.error, 1u);
}

__global__ void rows_clear_kernel(RowsTable t) {
    for (u64 i = (u64)blockIdx.x * blockDim.x + threadIdx.x; i <= t.mask; i += (u64)gridDim.x * blockDim.x) {
        Slot s;
        s.key = STBPE_EMPTY;
        s.count = 0;
        t.table[i] = s;
    }
}

// a pair (i, i+1) counts when both positions are valid (gpu_tokenizer/utils.py:586)
__global__ void rows_count_kernel(const int32_t *__restrict__ tokens, const uint8_t *__restrict__ valid,
                                  i64 B, i64 L, RowsTable t) {
    const i64 width = L - 1, total = B * width;
    for (i64 i = (i64)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (i64)gridDim.x * blockDim.x) {
        const i64 r = i / width, c = i - r * width;
        const i64 p = r * L + c;
        if (valid[p] && valid[p + 1])
            rows_table_add(t, ((u64)(uint32_t)tokens[p] << 32) | (u64)(uint32_t)tokens[p + 1]);
    }
}

__global__ void rows_export_kernel(RowsTable t, u64 *keys, i64 *counts, u64 *n_out, i64 cap) {
    for (u64 i = (u64)blockIdx.x * blockDim.x + threadIdx.x; i <= t.mask; i += (u64)gridDim.x * blockDim.x) {
        const Slot s = t.table[i];
        if (s.key != STBPE_EMPTY) {
            const u64 j = atomicAdd(n_out, 1ull);
            if ((i64)j < cap) {
                keys[j] = s.key;
                counts[j] = s.count;
            }
        }
    }
}

// unique (a, b) rows ascending, unused rows -1 / 0, length (gpu_tokenizer/utils.py:622-635)
__global__ void rows_write_kernel(const u64 *__restrict__ keys, const i64 *__restrict__ counts, i64 n,
                                  int32_t *pair_keys, i64 *pair_counts, i64 cap, i64 *length) {
    for (i64 i = (i64)blockIdx.x * blockDim.x + threadIdx.x; i < cap; i += (i64)gridDim.x * blockDim.x) {
        if (i < n) {
            pair_keys[2 * i] = (int32_t)(keys[i] >> 32);
            pair_keys[2 * i + 1] = (int32_t)(keys[i] & 0xFFFFFFFFull);
            pair_counts[i] = counts[i];
        } else {
            pair_keys[2 * i] = -1;
            pair_keys[2 * i + 1] = -1;
            pair_counts[i] = 0;
        }
    }
    if (blockIdx.x == 0 && threadIdx.x == 0 && length) *length = n;
}

// One CTA per row, walking the row in chunks with a running output offset.  Writes never
// overtake reads (the output is a left compaction), so the row is rewritten in place.
//   mask[i] = tok[i]==a && tok[i+1]==b && valid[i] && valid[i+1]   on the pre-merge row
//   tok[i] = new where mask[i]; position i+1 is dropped where mask[i]   (utils.py:520-531)
//   stable compaction of the remaining valid positions, zero-filled tail (utils.py:347-410)
__global__ void __launch_bounds__(ROWS_NT)
    rows_merge_kernel(int32_t *tokens, uint8_t *valid, int32_t *lengths, i64 B, i64 L, int32_t a,
                      int32_t b, int32_t new_id, uint8_t *spans) {
    __shared__ int32_t s_tok[ROWS_CHUNK + 2];
    __shared__ uint8_t s_val[ROWS_CHUNK + 2];
    __shared__ int32_t s_out[ROWS_CHUNK];
    __shared__ int s_wcnt[ROWS_IPT * (ROWS_NT / 32)];
    __shared__ int s_total;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    constexpr int NW = ROWS_NT / 32;
    for (i64 row = blockIdx.x; row < B; row += gridDim.x) {
        int32_t *t = tokens + row * L;
        uint8_t *v = valid + row * L;
        uint8_t *sp = spans ? spans + row * (L - 1) : nullptr;
        i64 w = 0;  // output length so far (uniform across the CTA)
        int32_t carry_tok = 0;
        uint8_t carry_val = 0;  // pre-merge token / valid just before the chunk
        for (i64 base = 0; base < L; base += ROWS_CHUNK) {
            const int n = (int)((L - base) < ROWS_CHUNK ? (L - base) : ROWS_CHUNK);
            // s_tok[1 + i] = position base + i; s_tok[0] = carry; s_tok[n + 1] = lookahead
            for (int i = tid; i < n + 1; i += ROWS_NT) {
                const i64 p = base + i;
                s_tok[1 + i] = p < L ? t[p] : 0;
                s_val[1 + i] = p < L ? v[p] : 0;
            }
            if (tid == 0) {
                s_tok[0] = carry_tok;
                s_val[0] = base > 0 ? carry_val : 0;
            }
            __syncthreads();
            int32_t outv[ROWS_IPT];
            unsigned int surv = 0;
#pragma unroll
            for (int j = 0; j < ROWS_IPT; ++j) {
                const int i = j * ROWS_NT + tid;
                outv[j] = 0;
                if (i < n) {
                    const int32_t tm1 = s_tok[i], t0 = s_tok[i + 1], t1 = s_tok[i + 2];
                    const bool vm1 = s_val[i], v0 = s_val[i + 1], v1 = s_val[i + 2];
                    const bool M0 = t0 == a && t1 == b && v0 && v1 && (base + i + 1 < L);
                    const bool D0 = tm1 == a && t0 == b && vm1 && v0;
                    if (sp && base + i < L - 1) sp[base + i] = (uint8_t)M0;
                    outv[j] = M0 ? new_id : t0;
                    if (v0 && !D0) surv |= 1u << j;
                }
            }
            const int32_t next_carry_tok = s_tok[n];
            const uint8_t next_carry_val = s_val[n];
            unsigned int bal[ROWS_IPT];
#pragma unroll
            for (int j = 0; j < ROWS_IPT; ++j) {
                bal[j] = __ballot_sync(0xFFFFFFFFu, (surv >> j) & 1u);
                if (lane == 0) s_wcnt[j * NW + warp] = __popc(bal[j]);
            }
            __syncthreads();
            if (warp == 0) {
                // exclusive scan of IPT*NW (=64) counts, 2 per lane
                int v0c = s_wcnt[lane * 2], v1c = s_wcnt[lane * 2 + 1];
                int sum = v0c + v1c, incl = sum;
#pragma unroll
                for (int d = 1; d < 32; d <<= 1) {
                    int o = __shfl_up_sync(0xFFFFFFFFu, incl, d);
                    if (lane >= d) incl += o;
                }
                s_wcnt[lane * 2] = incl - sum;
                s_wcnt[lane * 2 + 1] = incl - sum + v0c;
                if (lane == 31) s_total = incl;
            }
            __syncthreads();
            const unsigned int lt = (1u << lane) - 1u;
#pragma unroll
            for (int j = 0; j < ROWS_IPT; ++j)
                if ((surv >> j) & 1u) s_out[s_wcnt[j * NW + warp] + __popc(bal[j] & lt)] = outv[j];
            __syncthreads();
            const int produced = s_total;
            for (int i = tid; i < produced; i += ROWS_NT) {
                t[w + i] = s_out[i];
                v[w + i] = 1;
            }
            w += produced;
            carry_tok = next_carry_tok;
            carry_val = next_carry_val;
            __syncthreads();
        }
        for (i64 i = w + tid; i < L; i += ROWS_NT) {
            t[i] = 0;
            v[i] = 0;
        }
        if (tid == 0 && lengths) lengths[row] = (int32_t)w;
        __syncthreads();
    }
}

thread_local std::string g_rows_err;

}  // namespace

#define RCK(call)                                                        \
    do {                                                                 \
        cudaError_t c_ = (call);                                         \
        if (c_ != cudaSuccess) {                                         \
            g_rows_err = std::string(#call) + ": " + cudaGetErrorString(c_); \
            cudaGetLastError();                                          \
            return STBPE_E_CUDA;                                         \
        }                                                                \
    } while (0)

extern "C" {

STBPE_VISIBLE int stbpe_rows_count_pairs(const int32_t *tokens, const uint8_t *valid, int64_t B, int64_t L,
                                         int32_t *pair_keys, int64_t *pair_counts, int64_t cap,
                                         int64_t *length_dev, void *stream) {
    cudaStream_t s = (cudaStream_t)stream;
    if (B < 0 || L < 0 || cap < 0) return STBPE_E_BADARG;
    const i64 total = (B > 0 && L > 1) ? B * (L - 1) : 0;
    u64 *keys = nullptr, *skeys = nullptr, *meta = nullptr;
    i64 *counts = nullptr, *scounts = nullptr;
    Slot *table = nullptr;
    i64 n = 0;
    int rc = STBPE_OK;
    if (total > 0) {
        u64 slots = 1024;
        while (slots < (u64)total * 2 && slots < (1ull << 28)) slots <<= 1;
        RCK(cudaMallocAsync((void **)&table, slots * sizeof(Slot), s));
        RCK(cudaMallocAsync((void **)&meta, 2 * sizeof(u64), s));
        RCK(cudaMemsetAsync(meta, 0, 2 * sizeof(u64), s));
        RowsTable t;
        t.table = table;
        t.mask = slots - 1;
        t.n_keys = meta;
        t.error = reinterpret_cast<unsigned int *>(meta + 1);
        rows_clear_kernel<<<592, 256, 0, s>>>(t);
        i64 blocks = (total + 255) / 256;
        if (blocks > 148 * 32) blocks = 148 * 32;
        rows_count_kernel<<<(unsigned int)blocks, 256, 0, s>>>(tokens, valid, B, L, t);
        RCK(cudaGetLastError());
        u64 hmeta[2];
        RCK(cudaMemcpyAsync(hmeta, meta, sizeof(hmeta), cudaMemcpyDeviceToHost, s));
        RCK(cudaStreamSynchronize(s));
        n = (i64)hmeta[0];
        if ((hmeta[1] & 0xFFFFFFFFull) != 0 || n > cap) {
            rc = STBPE_E_CAPACITY;  // "pair workspace capacity exceeded" (utils.py:619-620)
            n = 0;
        } else if (n > 0) {
            RCK(cudaMallocAsync((void **)&keys, n * sizeof(u64), s));
            RCK(cudaMallocAsync((void **)&counts, n * sizeof(i64), s));
            RCK(cudaMallocAsync((void **)&skeys, n * sizeof(u64), s));
            RCK(cudaMallocAsync((void **)&scounts, n * sizeof(i64), s));
            RCK(cudaMemsetAsync(meta, 0, sizeof(u64), s));
            rows_export_kernel<<<592, 256, 0, s>>>(t, keys, counts, meta, n);
            size_t tmp_bytes = 0;
            cub::DeviceRadixSort::SortPairs(nullptr, tmp_bytes, keys, skeys, counts, scounts, (int)n, 0, 64, s);
            void *tmp = nullptr;
            RCK(cudaMallocAsync(&tmp, tmp_bytes ? tmp_bytes : 16, s));
            cub::DeviceRadixSort::SortPairs(tmp, tmp_bytes, keys, skeys, counts, scounts, (int)n, 0, 64, s);
            RCK(cudaGetLastError());
            RCK(cudaFreeAsync(tmp, s));
        }
        RCK(cudaFreeAsync(table, s));
        RCK(cudaFreeAsync(meta, s));
    }
    if (rc == STBPE_OK && cap > 0) {
        i64 blocks = (cap + 255) / 256;
        if (blocks > 148 * 32) blocks = 148 * 32;
        rows_write_kernel<<<(unsigned int)blocks, 256, 0, s>>>(skeys, scounts, n, pair_keys, (i64 *)pair_counts, cap, (i64 *)length_dev);
        RCK(cudaGetLastError());
    } else if (rc == STBPE_OK && length_dev) {
        RCK(cudaMemsetAsync(length_dev, 0, sizeof(i64), s));
    }
    if (keys) RCK(cudaFreeAsync(keys, s));
    if (counts) RCK(cudaFreeAsync(counts, s));
    if (skeys) RCK(cudaFreeAsync(skeys, s));
    if (scounts) RCK(cudaFreeAsync(scounts, s));
    RCK(cudaStreamSynchronize(s));
    return rc;
}

STBPE_VISIBLE int stbpe_rows_apply_merge(int32_t *tokens, uint8_t *valid, int32_t *lengths, int64_t B,
                                         int64_t L, int32_t a, int32_t b, int32_t new_id, uint8_t *spans,
                                         void *stream) {
    cudaStream_t s = (cudaStream_t)stream;
    if (B < 0 || L < 0) return STBPE_E_BADARG;
    if (B == 0 || L == 0) return STBPE_OK;
    i64 grid = B < 148 * 8 ? B : 148 * 8;
    rows_merge_kernel<<<(unsigned int)grid, ROWS_NT, 0, s>>>(tokens, valid, lengths, B, L, a, b, new_id, spans);
    RCK(cudaGetLastError());
    return STBPE_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------------------
// Pair counting for callers that must not allocate.
//
// stbpe_rows_count_pairs above takes its hash table, staging arrays and sort workspace from
// the stream-ordered allocator on every call.  Two kinds of caller of this library cannot
// afford that.  The reference's trainer sizes its batches to fill device memory (its
// --target-util flag) and hands every byte to preallocated workspaces before the merge loop
// starts, so an allocation made in the middle of the loop is the one that fails; and it
// overlaps copies and kernels on three streams per device, which a cudaMalloc / cudaFree
// stalls, because those calls synchronise the whole device.
//
// This variant works out of one fixed scratch block that is part of the library image: a
// file-scope __device__ array.  Every GPU on which the library is loaded holds the block
// (STBPE_STATIC_SCRATCH_BYTES, about 5.3 MB) from load to exit.  In host code the array's
// name is only a handle for the runtime, not a device address, so the entry point asks
// cudaGetSymbolAddress for the address once per device, with that device current, and hands
// the returned pointer to the kernels.  That look-up happens inside the first call made on
// each device; make that first call outside any stream capture.
//
// All calls share the block and it keeps what the last call left there: the table and the
// counters are cleared at the start of every call, and two calls that overlap on the GPU
// (different streams, or different host threads) race on it -- serialise them.
// ---------------------------------------------------------------------------------------
#define STBPE_STATIC_MAX_POSITIONS (1 << 16)  /* largest B*(L-1) accepted */
#define STBPE_STATIC_TABLE_SLOTS (1 << 17)
#define STBPE_STATIC_SORT_BYTES (1 << 20)
#define STBPE_STATIC_SCRATCH_BYTES                                                              \
    ((size_t)STBPE_STATIC_TABLE_SLOTS * sizeof(Slot) + (size_t)4 * STBPE_STATIC_MAX_POSITIONS * 8 + \
     256 + (size_t)STBPE_STATIC_SORT_BYTES)

static __device__ __align__(256) unsigned char g_static_scratch[STBPE_STATIC_SCRATCH_BYTES];

namespace {
std::mutex g_static_mu;
unsigned char *g_static_ptr[64] = {};

// device address of the scratch block on the current device (looked up once per device)
int static_scratch(unsigned char **out, char *err, size_t err_len) {
    int dev = -1;
    cudaError_t c = cudaGetDevice(&dev);
    if (c != cudaSuccess || dev < 0 || dev >= 64) {
        if (err) snprintf(err, err_len, "cudaGetDevice failed or device ordinal out of range: %s", cudaGetErrorString(c));
        return STBPE_E_CUDA;
    }
    std::lock_guard<std::mutex> lock(g_static_mu);
    if (g_static_ptr[dev]) {
        // a cudaDeviceReset since the look-up gives the block a new address: ask again if the cached
        // one is no longer device memory of this device (a query, no allocation)
        cudaPointerAttributes at;
        if (cudaPointerGetAttributes(&at, g_static_ptr[dev]) != cudaSuccess || at.type != cudaMemoryTypeDevice ||
            at.device != dev) {
            cudaGetLastError();
            g_static_ptr[dev] = nullptr;
        }
    }
    if (!g_static_ptr[dev]) {
        void *p = nullptr;
        c = cudaGetSymbolAddress(&p, g_static_scratch);
        if (c != cudaSuccess || !p) {
            if (err) snprintf(err, err_len, "cudaGetSymbolAddress(scratch) failed: %s", cudaGetErrorString(c));
            cudaGetLastError();
            return STBPE_E_CUDA;
        }
        g_static_ptr[dev] = static_cast<unsigned char *>(p);
    }
    *out = g_static_ptr[dev];
    return STBPE_OK;
}
}  // namespace

#define SCK(call)                                                                         \
    do {                                                                                  \
        cudaError_t c_ = (call);                                                          \
        if (c_ != cudaSuccess) {                                                          \
            if (err) snprintf(err, err_len, "%s: %s", #call, cudaGetErrorString(c_));     \
            cudaGetLastError();                                                           \
            return STBPE_E_CUDA;                                                          \
        }                                                                                 \
    } while (0)

extern "C" STBPE_VISIBLE int stbpe_rows_count_pairs_noalloc(const int32_t *tokens, const uint8_t *valid,
                                                            int64_t B, int64_t L, int32_t *pair_keys,
                                                            int64_t *pair_counts, int64_t cap,
                                                            int64_t *length_dev, void *stream, char *err,
                                                            size_t err_len) {
    cudaStream_t s = (cudaStream_t)stream;
    if (err && err_len) err[0] = 0;
    if (B < 0 || L < 0 || cap < 0) {
        if (err) snprintf(err, err_len, "negative size");
        return STBPE_E_BADARG;
    }
    const i64 total = (B > 0 && L > 1) ? B * (L - 1) : 0;
    if (total > STBPE_STATIC_MAX_POSITIONS) {
        if (err)
            snprintf(err, err_len,
                     "batch too large for the fixed scratch block: B*(L-1) = %lld pair positions, limit %d "
                     "(use stbpe_rows_count_pairs, which allocates)",
                     (long long)total, STBPE_STATIC_MAX_POSITIONS);
        return STBPE_E_CAPACITY;
    }
    unsigned char *base = nullptr;
    int rc = static_scratch(&base, err, err_len);
    if (rc != STBPE_OK) return rc;
    // carve the block: table | keys | counts | sorted keys | sorted counts | counters | sort workspace
    Slot *table = reinterpret_cast<Slot *>(base);
    u64 *keys = reinterpret_cast<u64 *>(base + (size_t)STBPE_STATIC_TABLE_SLOTS * sizeof(Slot));
    i64 *counts = reinterpret_cast<i64 *>(keys + STBPE_STATIC_MAX_POSITIONS);
    u64 *skeys = reinterpret_cast<u64 *>(counts + STBPE_STATIC_MAX_POSITIONS);
    i64 *scounts = reinterpret_cast<i64 *>(skeys + STBPE_STATIC_MAX_POSITIONS);
    u64 *meta = reinterpret_cast<u64 *>(scounts + STBPE_STATIC_MAX_POSITIONS);
    void *sort_ws = reinterpret_cast<unsigned char *>(meta) + 256;
    const u64 *sorted_keys = skeys;
    const i64 *sorted_counts = scounts;
    i64 n = 0;
    if (total > 0) {
        RowsTable t;
        t.table = table;
        t.mask = STBPE_STATIC_TABLE_SLOTS - 1;
        t.n_keys = meta;
        t.error = reinterpret_cast<unsigned int *>(meta + 1);
        // the block still holds the previous call's table and counters: start from zero
        SCK(cudaMemsetAsync(meta, 0, 256, s));
        rows_clear_kernel<<<256, 256, 0, s>>>(t);
        i64 blocks = (total + 255) / 256;
        rows_count_kernel<<<(unsigned int)blocks, 256, 0, s>>>(tokens, valid, B, L, t);
        SCK(cudaGetLastError());
        u64 hmeta[2] = {0, 0};
        SCK(cudaMemcpyAsync(hmeta, meta, sizeof(hmeta), cudaMemcpyDeviceToHost, s));
        SCK(cudaStreamSynchronize(s));
        n = (i64)hmeta[0];
        if ((hmeta[1] & 0xFFFFFFFFull) != 0 || n > cap) {
            if (err) snprintf(err, err_len, "pair workspace capacity exceeded (%lld unique pairs, cap %lld)", (long long)n, (long long)cap);
            return STBPE_E_CAPACITY;
        }
        if (n > 0) {
            // Sort through double buffers: the two key arrays and the two count arrays of the block are
            // the sort's ping-pong buffers, so its own workspace holds only digit counters (without
            // them it would ask for a second copy of keys and counts, 1 MiB at the size limit).  The
            // workspace size is checked before anything else is queued on the shared block.
            cub::DoubleBuffer<u64> dk(keys, skeys);
            cub::DoubleBuffer<i64> dc(counts, scounts);
            size_t need = 0;
            cub::DeviceRadixSort::SortPairs(nullptr, need, dk, dc, (int)n, 0, 64, s);
            if (need > (size_t)STBPE_STATIC_SORT_BYTES) {
                if (err) snprintf(err, err_len, "sort workspace of %zu bytes exceeds the reserved %d", need, STBPE_STATIC_SORT_BYTES);
                return STBPE_E_CAPACITY;
            }
            SCK(cudaMemsetAsync(meta, 0, sizeof(u64), s));
            rows_export_kernel<<<256, 256, 0, s>>>(t, keys, counts, meta, n);
            cub::DeviceRadixSort::SortPairs(sort_ws, need, dk, dc, (int)n, 0, 64, s);
            SCK(cudaGetLastError());
            sorted_keys = dk.Current();
            sorted_counts = dc.Current();
        }
    }
    if (cap > 0) {
        i64 blocks = (cap + 255) / 256;
        if (blocks > 148 * 32) blocks = 148 * 32;
        rows_write_kernel<<<(unsigned int)blocks, 256, 0, s>>>(sorted_keys, sorted_counts, n, pair_keys, (i64 *)pair_counts, cap, (i64 *)length_dev);
        SCK(cudaGetLastError());
    } else if (length_dev) {
        SCK(cudaMemsetAsync(length_dev, 0, sizeof(i64), s));
    }
    SCK(cudaStreamSynchronize(s));
    return STBPE_OK;
}
